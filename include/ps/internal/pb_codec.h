// Hand-written encoder/decoder for the protobuf messages of the wire contract.
//
// The reference serialises Meta through protoc-generated classes of src/meta.proto:8-60
// (Van::PackMeta / UnpackMeta, src/van.cc:477-557).  This codec produces and accepts the
// same bytes without a protobuf dependency:
//
//   PBNode    : 1 role int32 | 2 id int32 | 3 hostname string | 4 port int32
//               | 5 is_recovery bool | 10 customer_id int32
//   PBControl : 1 cmd int32 | 2 node repeated PBNode | 3 barrier_group int32 | 4 msg_sig uint64
//   PBMeta    : 1 head int32 | 2 body bytes | 3 control PBControl | 4 request bool
//               | 5 push bool | 6 simple_app bool | 7 app_id int32 | 8 timestamp int32
//               | 9 data_type repeated int32 [packed] | 10 customer_id int32
//               | 11 data_size int32 | 12 pull bool | 13 priority int32
//
// Presence rules on encode (those of PackMeta): head, request, push, pull, simple_app,
// customer_id and priority are always written; app_id and timestamp only when set; body
// only when non-empty; control only for control messages, with barrier_group only for
// BARRIER and msg_sig only for ACK; data_size is never written.  Fields are written in
// field-number order; negative int32 values take ten bytes, as protobuf encodes them.
// Decode accepts fields in any order, packed or unpacked data_type, and skips unknown
// fields of any wire type.
#ifndef PS_INTERNAL_PB_CODEC_H_
#define PS_INTERNAL_PB_CODEC_H_
#include <string>

#include "ps/internal/message.h"

namespace ps {
namespace pb {

// Appends the PBMeta encoding of `meta` to `out`.
void EncodeMeta(const Meta& meta, std::string* out);
// Parses a PBMeta; returns false on malformed input.  sender/recver are left untouched.
bool DecodeMeta(const char* buf, size_t len, Meta* meta);

// Building blocks, exposed for tests and for other codecs.
void EncodeNode(const Node& node, std::string* out);
bool DecodeNode(const char* buf, size_t len, Node* node);
void PutVarint(uint64_t v, std::string* out);
// Reads a varint at *pos; advances *pos; false if truncated or longer than 10 bytes.
bool GetVarint(const char* buf, size_t len, size_t* pos, uint64_t* v);

}  // namespace pb
}  // namespace ps
#endif  // PS_INTERNAL_PB_CODEC_H_
