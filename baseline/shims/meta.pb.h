// Stand-in for the protoc output of the reference's src/meta.proto, for building the
// reference where protoc and the protobuf C++ runtime are not installed.  It provides the
// three message classes with exactly the accessors that the reference's src/van.cc calls
// (:445-557) and serialises them in the proto2 wire format of that schema (fields written
// in field-number order, presence tracked per field), so the bytes on the wire are the ones
// the generated code would produce.  Self-contained: depends on nothing but the C++ library.
#ifndef BASELINE_SHIM_META_PB_H_
#define BASELINE_SHIM_META_PB_H_
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>

namespace ps {
namespace pbshim {
inline void PutVarint(std::string* o, uint64_t v) {
  while (v >= 0x80) { o->push_back(static_cast<char>((v & 0x7f) | 0x80)); v >>= 7; }
  o->push_back(static_cast<char>(v));
}
inline void PutTag(std::string* o, int field, int wt) { PutVarint(o, (uint64_t(field) << 3) | wt); }
inline void PutI32(std::string* o, int f, int32_t v) { PutTag(o, f, 0); PutVarint(o, uint64_t(int64_t(v))); }
inline void PutBool(std::string* o, int f, bool v) { PutTag(o, f, 0); o->push_back(v ? 1 : 0); }
inline void PutBytes(std::string* o, int f, const std::string& s) { PutTag(o, f, 2); PutVarint(o, s.size()); o->append(s); }
struct Reader {
  const char* p; size_t n; size_t i;
  Reader(const char* p_, size_t n_) : p(p_), n(n_), i(0) {}
  bool done() const { return i >= n; }
  bool varint(uint64_t* v) {
    uint64_t a = 0;
    for (int s = 0; s < 70; s += 7) {
      if (i >= n) return false;
      uint8_t b = uint8_t(p[i++]);
      if (s < 64) a |= uint64_t(b & 0x7f) << s;
      if (!(b & 0x80)) { *v = a; return true; }
    }
    return false;
  }
  bool bytes(const char** q, size_t* l) {
    uint64_t len;
    if (!varint(&len) || len > n - i) return false;
    *q = p + i; *l = size_t(len); i += *l; return true;
  }
  bool skip(int wt) {
    uint64_t v; const char* q; size_t l;
    if (wt == 0) return varint(&v);
    if (wt == 1) { if (n - i < 8) return false; i += 8; return true; }
    if (wt == 2) return bytes(&q, &l);
    if (wt == 5) { if (n - i < 4) return false; i += 4; return true; }
    return false;
  }
};
}  // namespace pbshim

#define PS_PB_FIELD(type, name)                                  \
 public:                                                         \
  void set_##name(type v) { name##_ = v; has_##name##_ = true; } \
  type name() const { return name##_; }                          \
  bool has_##name() const { return has_##name##_; }              \
 private:                                                        \
  type name##_ = type();                                         \
  bool has_##name##_ = false;

class PBNode {
  PS_PB_FIELD(int32_t, role)
  PS_PB_FIELD(int32_t, id)
  PS_PB_FIELD(int32_t, port)
  PS_PB_FIELD(bool, is_recovery)
  PS_PB_FIELD(int32_t, customer_id)
 public:
  void set_hostname(const std::string& s) { hostname_ = s; has_hostname_ = true; }
  const std::string& hostname() const { return hostname_; }
  void Encode(std::string* o) const {
    using namespace pbshim;
    if (has_role_) PutI32(o, 1, role_);
    if (has_id_) PutI32(o, 2, id_);
    if (has_hostname_) PutBytes(o, 3, hostname_);
    if (has_port_) PutI32(o, 4, port_);
    if (has_is_recovery_) PutBool(o, 5, is_recovery_);
    if (has_customer_id_) PutI32(o, 10, customer_id_);
  }
  bool Decode(const char* p, size_t n) {
    pbshim::Reader r{p, n};
    while (!r.done()) {
      uint64_t t, v; if (!r.varint(&t)) return false;
      int f = int(t >> 3), wt = int(t & 7);
      if (wt == 0 && (f == 1 || f == 2 || f == 4 || f == 5 || f == 10)) {
        if (!r.varint(&v)) return false;
        if (f == 1) set_role(int32_t(v)); else if (f == 2) set_id(int32_t(v));
        else if (f == 4) set_port(int32_t(v)); else if (f == 5) set_is_recovery(v != 0);
        else set_customer_id(int32_t(v));
      } else if (f == 3 && wt == 2) {
        const char* q; size_t l; if (!r.bytes(&q, &l)) return false;
        set_hostname(std::string(q, l));
      } else if (!r.skip(wt)) return false;
    }
    return true;
  }
 private:
  std::string hostname_;
  bool has_hostname_ = false;
};

class PBControl {
  PS_PB_FIELD(int32_t, cmd)
  PS_PB_FIELD(int32_t, barrier_group)
  PS_PB_FIELD(uint64_t, msg_sig)
 public:
  PBNode* add_node() { node_.emplace_back(); return &node_.back(); }
  int node_size() const { return int(node_.size()); }
  const PBNode& node(int i) const { return node_[i]; }
  void Encode(std::string* o) const {
    using namespace pbshim;
    if (has_cmd_) PutI32(o, 1, cmd_);
    for (const auto& n : node_) { std::string t; n.Encode(&t); PutBytes(o, 2, t); }
    if (has_barrier_group_) PutI32(o, 3, barrier_group_);
    if (has_msg_sig_) { PutTag(o, 4, 0); PutVarint(o, msg_sig_); }
  }
  bool Decode(const char* p, size_t n) {
    pbshim::Reader r{p, n};
    while (!r.done()) {
      uint64_t t, v; if (!r.varint(&t)) return false;
      int f = int(t >> 3), wt = int(t & 7);
      if (wt == 0 && (f == 1 || f == 3 || f == 4)) {
        if (!r.varint(&v)) return false;
        if (f == 1) set_cmd(int32_t(v)); else if (f == 3) set_barrier_group(int32_t(v)); else set_msg_sig(v);
      } else if (f == 2 && wt == 2) {
        const char* q; size_t l; if (!r.bytes(&q, &l)) return false;
        if (!add_node()->Decode(q, l)) return false;
      } else if (!r.skip(wt)) return false;
    }
    return true;
  }
 private:
  std::vector<PBNode> node_;
};

class PBMeta {
  PS_PB_FIELD(int32_t, head)
  PS_PB_FIELD(bool, request)
  PS_PB_FIELD(bool, push)
  PS_PB_FIELD(bool, simple_app)
  PS_PB_FIELD(int32_t, app_id)
  PS_PB_FIELD(int32_t, timestamp)
  PS_PB_FIELD(int32_t, customer_id)
  PS_PB_FIELD(int32_t, data_size)
  PS_PB_FIELD(bool, pull)
  PS_PB_FIELD(int32_t, priority)
 public:
  void set_body(const std::string& s) { body_ = s; has_body_ = true; }
  const std::string& body() const { return body_; }
  void add_data_type(int32_t d) { data_type_.push_back(d); }
  int data_type_size() const { return int(data_type_.size()); }
  int32_t data_type(int i) const { return data_type_[i]; }
  PBControl* mutable_control() { has_control_ = true; return &control_; }
  bool has_control() const { return has_control_; }
  const PBControl& control() const { return control_; }

  std::string SerializeAsString() const {
    using namespace pbshim;
    std::string o;
    if (has_head_) PutI32(&o, 1, head_);
    if (has_body_) PutBytes(&o, 2, body_);
    if (has_control_) { std::string t; control_.Encode(&t); PutBytes(&o, 3, t); }
    if (has_request_) PutBool(&o, 4, request_);
    if (has_push_) PutBool(&o, 5, push_);
    if (has_simple_app_) PutBool(&o, 6, simple_app_);
    if (has_app_id_) PutI32(&o, 7, app_id_);
    if (has_timestamp_) PutI32(&o, 8, timestamp_);
    if (!data_type_.empty()) {
      std::string t;
      for (int32_t d : data_type_) PutVarint(&t, uint64_t(int64_t(d)));
      PutBytes(&o, 9, t);
    }
    if (has_customer_id_) PutI32(&o, 10, customer_id_);
    if (has_data_size_) PutI32(&o, 11, data_size_);
    if (has_pull_) PutBool(&o, 12, pull_);
    if (has_priority_) PutI32(&o, 13, priority_);
    return o;
  }
  int ByteSize() const { return int(SerializeAsString().size()); }
  bool SerializeToArray(void* data, int size) const {
    std::string s = SerializeAsString();
    if (int(s.size()) > size) return false;
    memcpy(data, s.data(), s.size());
    return true;
  }
  bool ParseFromArray(const void* data, int size) {
    *this = PBMeta();
    pbshim::Reader r{static_cast<const char*>(data), size_t(size)};
    while (!r.done()) {
      uint64_t t, v; if (!r.varint(&t)) return false;
      int f = int(t >> 3), wt = int(t & 7);
      if (wt == 0) {
        if (!r.varint(&v)) return false;
        switch (f) {
          case 1: set_head(int32_t(v)); break;
          case 4: set_request(v != 0); break;
          case 5: set_push(v != 0); break;
          case 6: set_simple_app(v != 0); break;
          case 7: set_app_id(int32_t(v)); break;
          case 8: set_timestamp(int32_t(v)); break;
          case 9: add_data_type(int32_t(v)); break;
          case 10: set_customer_id(int32_t(v)); break;
          case 11: set_data_size(int32_t(v)); break;
          case 12: set_pull(v != 0); break;
          case 13: set_priority(int32_t(v)); break;
          default: break;
        }
      } else if (wt == 2) {
        const char* q; size_t l; if (!r.bytes(&q, &l)) return false;
        if (f == 2) set_body(std::string(q, l));
        else if (f == 3) { if (!mutable_control()->Decode(q, l)) return false; }
        else if (f == 9) {
          pbshim::Reader pr{q, l};
          while (!pr.done()) { if (!pr.varint(&v)) return false; add_data_type(int32_t(v)); }
        }
      } else if (!r.skip(wt)) return false;
    }
    return true;
  }
 private:
  std::string body_;
  bool has_body_ = false;
  std::vector<int32_t> data_type_;
  PBControl control_;
  bool has_control_ = false;
};
#undef PS_PB_FIELD

}  // namespace ps
#endif  // BASELINE_SHIM_META_PB_H_
