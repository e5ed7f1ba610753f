#include "ps/internal/pb_codec.h"

namespace ps {
namespace pb {
namespace {

enum WireType { kVarint = 0, kFixed64 = 1, kBytes = 2, kFixed32 = 5 };

inline void PutTag(int field, WireType wt, std::string* out) {
  PutVarint((static_cast<uint64_t>(field) << 3) | wt, out);
}
// int32 fields: negative values are sign-extended to 64 bits before encoding.
inline void PutInt32(int field, int32_t v, std::string* out) {
  PutTag(field, kVarint, out);
  PutVarint(static_cast<uint64_t>(static_cast<int64_t>(v)), out);
}
inline void PutBool(int field, bool v, std::string* out) {
  PutTag(field, kVarint, out);
  out->push_back(v ? 1 : 0);
}
inline void PutBytes(int field, const std::string& s, std::string* out) {
  PutTag(field, kBytes, out);
  PutVarint(s.size(), out);
  out->append(s);
}

// Cursor over an encoded message.
struct Reader {
  const char* buf;
  size_t len;
  size_t pos = 0;
  bool done() const { return pos >= len; }
  bool tag(int* field, int* wt) {
    uint64_t t;
    if (!GetVarint(buf, len, &pos, &t)) return false;
    *field = static_cast<int>(t >> 3);
    *wt = static_cast<int>(t & 7);
    return *field > 0;
  }
  bool varint(uint64_t* v) { return GetVarint(buf, len, &pos, v); }
  bool bytes(const char** p, size_t* n) {
    uint64_t l;
    if (!varint(&l) || l > len - pos) return false;
    *p = buf + pos;
    *n = static_cast<size_t>(l);
    pos += *n;
    return true;
  }
  bool skip(int wt) {
    uint64_t v;
    const char* p;
    size_t n;
    switch (wt) {
      case kVarint: return varint(&v);
      case kFixed64: if (len - pos < 8) return false; pos += 8; return true;
      case kBytes: return bytes(&p, &n);
      case kFixed32: if (len - pos < 4) return false; pos += 4; return true;
      default: return false;  // groups are not used by this schema
    }
  }
};

void EncodeControl(const Control& c, std::string* out) {
  PutInt32(1, static_cast<int32_t>(c.cmd), out);
  std::string tmp;
  for (const Node& n : c.node) {
    tmp.clear();
    EncodeNode(n, &tmp);
    PutBytes(2, tmp, out);
  }
  if (c.cmd == Control::BARRIER) PutInt32(3, c.barrier_group, out);
  if (c.cmd == Control::ACK) {
    PutTag(4, kVarint, out);
    PutVarint(c.msg_sig, out);
  }
}

bool DecodeControl(const char* buf, size_t len, Control* c) {
  Reader r{buf, len};
  *c = Control();
  while (!r.done()) {
    int f, wt;
    if (!r.tag(&f, &wt)) return false;
    uint64_t v;
    if (f == 1 && wt == kVarint) {
      if (!r.varint(&v)) return false;
      // a command outside the enumeration makes the message undecodable, not undefined
      const int32_t cmd = static_cast<int32_t>(v);
      if (cmd < 0 || cmd > static_cast<int32_t>(Control::HEARTBEAT)) return false;
      c->cmd = static_cast<Control::Command>(cmd);
    } else if (f == 2 && wt == kBytes) {
      const char* p;
      size_t n;
      if (!r.bytes(&p, &n)) return false;
      Node node;
      if (!DecodeNode(p, n, &node)) return false;
      c->node.push_back(node);
    } else if (f == 3 && wt == kVarint) {
      if (!r.varint(&v)) return false;
      c->barrier_group = static_cast<int32_t>(v);
    } else if (f == 4 && wt == kVarint) {
      if (!r.varint(&v)) return false;
      c->msg_sig = v;
    } else if (!r.skip(wt)) {
      return false;
    }
  }
  return true;
}

}  // namespace

void PutVarint(uint64_t v, std::string* out) {
  while (v >= 0x80) {
    out->push_back(static_cast<char>((v & 0x7f) | 0x80));
    v >>= 7;
  }
  out->push_back(static_cast<char>(v));
}

bool GetVarint(const char* buf, size_t len, size_t* pos, uint64_t* v) {
  uint64_t acc = 0;
  for (int shift = 0; shift < 70; shift += 7) {
    if (*pos >= len) return false;
    const uint8_t b = static_cast<uint8_t>(buf[(*pos)++]);
    if (shift < 64) acc |= static_cast<uint64_t>(b & 0x7f) << shift;
    if (!(b & 0x80)) {
      *v = acc;
      return true;
    }
  }
  return false;
}

void EncodeNode(const Node& n, std::string* out) {
  PutInt32(1, static_cast<int32_t>(n.role), out);
  PutInt32(2, n.id, out);
  PutBytes(3, n.hostname, out);
  PutInt32(4, n.port, out);
  PutBool(5, n.is_recovery, out);
  PutInt32(10, n.customer_id, out);
}

bool DecodeNode(const char* buf, size_t len, Node* n) {
  Reader r{buf, len};
  *n = Node();
  while (!r.done()) {
    int f, wt;
    if (!r.tag(&f, &wt)) return false;
    uint64_t v;
    if (wt == kVarint && (f == 1 || f == 2 || f == 4 || f == 5 || f == 10)) {
      if (!r.varint(&v)) return false;
      const int32_t x = static_cast<int32_t>(v);
      switch (f) {
        case 1:
          if (x < 0 || x > static_cast<int32_t>(Node::JOINT)) return false;
          n->role = static_cast<Node::Role>(x);
          break;
        case 2: n->id = x; break;
        case 4: n->port = x; break;
        case 5: n->is_recovery = (v != 0); break;
        case 10: n->customer_id = x; break;
      }
    } else if (f == 3 && wt == kBytes) {
      const char* p;
      size_t l;
      if (!r.bytes(&p, &l)) return false;
      n->hostname.assign(p, l);
    } else if (!r.skip(wt)) {
      return false;
    }
  }
  return true;
}

void EncodeMeta(const Meta& m, std::string* out) {
  PutInt32(1, m.head, out);
  if (!m.body.empty()) PutBytes(2, m.body, out);
  if (!m.control.empty()) {
    std::string tmp;
    EncodeControl(m.control, &tmp);
    PutBytes(3, tmp, out);
  }
  PutBool(4, m.request, out);
  PutBool(5, m.push, out);
  PutBool(6, m.simple_app, out);
  if (m.app_id != Meta::kEmpty) PutInt32(7, m.app_id, out);
  if (m.timestamp != Meta::kEmpty) PutInt32(8, m.timestamp, out);
  if (!m.data_type.empty()) {
    std::string packed;
    for (DataType d : m.data_type)
      PutVarint(static_cast<uint64_t>(static_cast<int64_t>(static_cast<int32_t>(d))), &packed);
    PutBytes(9, packed, out);
  }
  PutInt32(10, m.customer_id, out);
  PutBool(12, m.pull, out);
  PutInt32(13, m.priority, out);
}

// A type tag from the wire; values outside the enumeration (a newer or a corrupt sender)
// become OTHER instead of an out-of-range enum value.
static DataType ToDataType(int32_t x) {
  return (x >= 0 && x <= static_cast<int32_t>(FLOAT16)) ? static_cast<DataType>(x) : OTHER;
}

bool DecodeMeta(const char* buf, size_t len, Meta* m) {
  Reader r{buf, len};
  const int sender = m->sender, recver = m->recver;
  *m = Meta();
  m->sender = sender;
  m->recver = recver;
  while (!r.done()) {
    int f, wt;
    if (!r.tag(&f, &wt)) return false;
    uint64_t v;
    if (wt == kVarint) {
      if (!r.varint(&v)) return false;
      const int32_t x = static_cast<int32_t>(v);
      switch (f) {
        case 1: m->head = x; break;
        case 4: m->request = (v != 0); break;
        case 5: m->push = (v != 0); break;
        case 6: m->simple_app = (v != 0); break;
        case 7: m->app_id = x; break;
        case 8: m->timestamp = x; break;
        case 9: m->data_type.push_back(ToDataType(x)); break;  // unpacked form
        case 10: m->customer_id = x; break;
        case 11: m->data_size = x; break;
        case 12: m->pull = (v != 0); break;
        case 13: m->priority = x; break;
        default: break;
      }
    } else if (wt == kBytes) {
      const char* p;
      size_t n;
      if (!r.bytes(&p, &n)) return false;
      if (f == 2) {
        m->body.assign(p, n);
      } else if (f == 3) {
        if (!DecodeControl(p, n, &m->control)) return false;
      } else if (f == 9) {
        size_t q = 0;
        while (q < n) {
          if (!GetVarint(p, n, &q, &v)) return false;
          m->data_type.push_back(ToDataType(static_cast<int32_t>(v)));
        }
      }
    } else if (!r.skip(wt)) {
      return false;
    }
  }
  return true;
}

}  // namespace pb
}  // namespace ps
