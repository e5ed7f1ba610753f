// The message model exchanged between nodes: Node, Control, Meta, Message.
//
// Field names and enum values follow the reference (include/ps/internal/message.h:13-229)
// because they are part of the public API and, through meta.proto, of the wire contract.
// Additions: bf16/fp16 element tags appended after OTHER, and a JOINT node role for
// processes that are worker and server at once.
#ifndef PS_INTERNAL_MESSAGE_H_
#define PS_INTERNAL_MESSAGE_H_
#include <climits>
#include <cstdint>
#include <string>
#include <type_traits>
#include <vector>

#include "ps/sarray.h"

namespace ps {

// Element type tags carried in Meta::data_type (one per data frame).
enum DataType {
  CHAR, INT8, INT16, INT32, INT64,
  UINT8, UINT16, UINT32, UINT64,
  FLOAT, DOUBLE, OTHER,
  BFLOAT16, FLOAT16  // not in the reference; appended so that older tags keep their values
};

static const char* const DataTypeName[] = {
    "CHAR", "INT8", "INT16", "INT32", "INT64", "UINT8", "UINT16", "UINT32", "UINT64",
    "FLOAT", "DOUBLE", "OTHER", "BFLOAT16", "FLOAT16"};

// Opaque 16-bit storage types so that KVWorker<bfloat16_t> maps to the BFLOAT16 tag.
struct bfloat16_t { uint16_t bits; };
struct float16_t { uint16_t bits; };

// True when V without const/volatile is W (source compatibility: the reference exposes it).
template <typename V, typename W>
inline bool SameType() {
  return std::is_same<typename std::remove_cv<V>::type, W>::value;
}

template <typename V>
constexpr DataType GetDataType() {
  if (std::is_same<V, bfloat16_t>::value) return BFLOAT16;
  if (std::is_same<V, float16_t>::value) return FLOAT16;
  if (std::is_same<typename std::remove_cv<V>::type, char>::value) return CHAR;
  if (std::is_same<V, int8_t>::value) return INT8;
  if (std::is_same<V, int16_t>::value) return INT16;
  if (std::is_same<V, int32_t>::value) return INT32;
  if (std::is_same<V, int64_t>::value) return INT64;
  if (std::is_same<V, uint8_t>::value) return UINT8;
  if (std::is_same<V, uint16_t>::value) return UINT16;
  if (std::is_same<V, uint32_t>::value) return UINT32;
  if (std::is_same<V, uint64_t>::value) return UINT64;
  if (std::is_same<V, float>::value) return FLOAT;
  if (std::is_same<V, double>::value) return DOUBLE;
  return OTHER;
}

// "no value" marker for integer meta fields.
static const int kEmptyField = INT_MAX;

struct Node {
  static const int kEmpty;
  // JOINT: the process hosts a server node id and a worker node id (one per GPU).
  enum Role { SERVER, WORKER, SCHEDULER, JOINT };

  Node() : role(SERVER), id(kEmptyField), customer_id(0), port(kEmptyField),
           is_recovery(false) {}
  std::string DebugString() const;
  std::string ShortDebugString() const;

  Role role;
  int id;
  int customer_id;
  std::string hostname;
  int port;
  bool is_recovery;
};

struct Control {
  enum Command { EMPTY, TERMINATE, ADD_NODE, BARRIER, ACK, HEARTBEAT };

  Control() : cmd(EMPTY), barrier_group(0), msg_sig(0) {}
  bool empty() const { return cmd == EMPTY; }
  std::string DebugString() const;

  Command cmd;
  std::vector<Node> node;
  int barrier_group;
  uint64_t msg_sig;
};

struct Meta {
  static const int kEmpty;

  Meta() : head(kEmptyField), app_id(kEmptyField), customer_id(kEmptyField),
           timestamp(kEmptyField), sender(kEmptyField), recver(kEmptyField),
           request(false), push(false), pull(false), simple_app(false),
           data_size(0), priority(0) {}
  std::string DebugString() const;

  int head;
  int app_id;
  int customer_id;
  int timestamp;
  int sender;   // node id; supplied by the transport, not serialised in PBMeta
  int recver;   // node id; supplied by the transport, not serialised in PBMeta
  bool request;
  bool push;
  bool pull;
  bool simple_app;
  std::string body;
  std::vector<DataType> data_type;
  Control control;
  int data_size;
  int priority;
};

struct Message {
  Meta meta;
  std::vector<SArray<char>> data;

  // Append a typed array as a data frame (zero-copy) and record its element type.
  template <typename V>
  void AddData(const SArray<V>& val) {
    CHECK_EQ(data.size(), meta.data_type.size());
    meta.data_type.push_back(GetDataType<V>());
    SArray<char> bytes(val);
    meta.data_size += static_cast<int>(bytes.size());
    data.push_back(bytes);
  }
  std::string DebugString() const;
};

}  // namespace ps
#endif  // PS_INTERNAL_MESSAGE_H_
