// Single-process unit tests of the host runtime's building blocks.
#include <cstdio>
#include <cstring>
#include <random>
#include <thread>

#include "ps/internal/parallel_kv_match.h"
#include "ps/internal/parallel_sort.h"
#include "ps/internal/pb_codec.h"
#include "ps/internal/resender.h"
#include "ps/internal/threadsafe_pqueue.h"
#include "ps/internal/threadsafe_queue.h"
#include "ps/ps.h"

using namespace ps;

static void TestSArray() {
  SArray<int> a(10, 3);
  CHECK_EQ(a.size(), (size_t)10);
  for (int v : a) CHECK_EQ(v, 3);
  SArray<int> b = a;  // shares storage
  b[0] = 7;
  CHECK_EQ(a[0], 7);
  SArray<char> bytes(a);  // reinterpret
  CHECK_EQ(bytes.size(), (size_t)40);
  SArray<int> back(bytes);
  CHECK_EQ(back.size(), (size_t)10);
  CHECK_EQ(back.data(), a.data());
  SArray<int> seg = a.segment(2, 5);
  CHECK_EQ(seg.size(), (size_t)3);
  seg[0] = 42;
  CHECK_EQ(a[2], 42);
  a.resize(20, 9);
  CHECK_EQ(a.size(), (size_t)20);
  CHECK_EQ(a[19], 9);
  CHECK_EQ(a[2], 42);
  a.resize(4);
  CHECK_EQ(a.size(), (size_t)4);
  SArray<int> c;
  for (int i = 0; i < 1000; ++i) c.push_back(i);
  CHECK_EQ(c.size(), (size_t)1000);
  CHECK_EQ(c.back(), 999);
  c.pop_back();
  CHECK_EQ(c.back(), 998);
  SArray<int> d({1, 2, 3});
  d.append(SArray<int>({4, 5}));
  CHECK_EQ(d.size(), (size_t)5);
  CHECK_EQ(d[4], 5);
  std::vector<float> vec = {1.f, 2.f};
  SArray<float> e(vec);
  vec[0] = 5.f;
  CHECK_EQ(e[0], 1.f);  // copied
  auto sp = std::make_shared<std::vector<float>>(3, 2.5f);
  SArray<float> f(sp);
  (*sp)[1] = 8.f;
  CHECK_EQ(f[1], 8.f);  // shared
  float raw[3] = {1, 2, 3};
  {
    SArray<float> g(raw, 3);  // not owned
    g[1] = 9;
  }
  CHECK_EQ(raw[1], 9.f);
  SArray<float> h;
  h.CopyFrom(raw, 3);
  raw[0] = -1;
  CHECK_EQ(h[0], 1.f);
  h.clear();
  CHECK(h.empty());
  bool freed = false;
  {
    SArray<int> k;
    k.reset(new int[4], 4, [&freed](int* p) { delete[] p; freed = true; });
    SArray<int> k2 = k.segment(1, 2);
    k.clear();
    CHECK(!freed);  // the segment keeps the owner alive
  }
  CHECK(freed);
  SArray<Key> keys({1, 5, 9, 12, 20});
  Range r = FindRange(keys, (Key)5, (Key)13);
  CHECK_EQ(r.begin(), (uint64_t)1);
  CHECK_EQ(r.end(), (uint64_t)4);
  int devmem[4];
  SArray<int> dv = SArray<int>::FromDevice(devmem, 4);
  CHECK(dv.mem_kind() == MemKind::kDevice);
  CHECK(dv.segment(1, 3).mem_kind() == MemKind::kDevice);
  std::ostringstream os;
  os << d;
  CHECK(os.str().find("[5]") != std::string::npos);
}

static void TestEnv() {
  Environment::Init({{"PSB_TEST_KEY", "17"}});
  CHECK_EQ(GetEnv("PSB_TEST_KEY", 0), 17);
  CHECK_EQ(GetEnv("PSB_TEST_ABSENT", 5), 5);
  setenv("PSB_TEST_OS", "abc", 1);
  CHECK_EQ(GetEnv("PSB_TEST_OS", std::string("x")), std::string("abc"));
  Environment::Get()->set("PSB_TEST_OS", "override");
  CHECK_EQ(GetEnv("PSB_TEST_OS", std::string("x")), std::string("override"));
}

static void TestQueues() {
  ThreadsafeQueue<int> q;
  std::thread t([&q] { for (int i = 0; i < 100; ++i) q.Push(i); });
  for (int i = 0; i < 100; ++i) {
    int v;
    q.WaitAndPop(&v);
    CHECK_EQ(v, i);
  }
  t.join();
  int v;
  CHECK(!q.WaitAndPopFor(&v, 10));
  ThreadsafePQueue pq;
  int prios[] = {1, 5, 5, 0, 9, 5};
  for (int i = 0; i < 6; ++i) {
    Message m;
    m.meta.priority = prios[i];
    m.meta.timestamp = i;
    pq.Push(m);
  }
  int want_ts[] = {4, 1, 2, 5, 0, 3};  // highest priority first, ties in arrival order
  for (int i = 0; i < 6; ++i) {
    Message m;
    pq.WaitAndPop(&m);
    CHECK_EQ(m.meta.timestamp, want_ts[i]);
  }
}

static std::string Hex(const std::string& s) {
  static const char* d = "0123456789abcdef";
  std::string o;
  for (unsigned char c : s) { o.push_back(d[c >> 4]); o.push_back(d[c & 15]); }
  return o;
}

static void TestCodec() {
  // golden bytes: a data request as PackMeta of the reference would emit it
  Meta m;
  m.head = 3;
  m.app_id = 0;
  m.customer_id = 1;
  m.timestamp = 7;
  m.request = true;
  m.push = true;
  m.data_type = {UINT64, FLOAT};
  m.priority = 2;
  std::string out;
  pb::EncodeMeta(m, &out);
  CHECK_EQ(Hex(out), std::string("0803200128013000380040074a020809500160006802"))
      << Hex(out);
  Meta back;
  CHECK(pb::DecodeMeta(out.data(), out.size(), &back));
  CHECK_EQ(back.head, 3);
  CHECK_EQ(back.timestamp, 7);
  CHECK_EQ(back.customer_id, 1);
  CHECK(back.request && back.push && !back.pull && !back.simple_app);
  CHECK_EQ(back.data_type.size(), (size_t)2);
  CHECK_EQ((int)back.data_type[1], (int)FLOAT);
  CHECK_EQ(back.priority, 2);

  // "empty" ints are INT_MAX and still written; negative ints take ten bytes
  Meta e;
  e.priority = -1;
  out.clear();
  pb::EncodeMeta(e, &out);
  Meta e2;
  CHECK(pb::DecodeMeta(out.data(), out.size(), &e2));
  CHECK_EQ(e2.head, Meta::kEmpty);
  CHECK_EQ(e2.customer_id, Meta::kEmpty);
  CHECK_EQ(e2.app_id, Meta::kEmpty);
  CHECK_EQ(e2.timestamp, Meta::kEmpty);
  CHECK_EQ(e2.priority, -1);
  CHECK(Hex(out).find("68ffffffffffffffffff01") != std::string::npos) << Hex(out);

  // control message with nodes
  Meta c;
  c.control.cmd = Control::ADD_NODE;
  Node n;
  n.role = Node::WORKER;
  n.id = 9;
  n.hostname = "10.0.0.1";
  n.port = 5555;
  n.customer_id = 2;
  n.is_recovery = true;
  c.control.node = {n, n};
  c.control.node[1].id = Node::kEmpty;
  c.body = std::string("b\0dy", 4);
  out.clear();
  pb::EncodeMeta(c, &out);
  Meta c2;
  CHECK(pb::DecodeMeta(out.data(), out.size(), &c2));
  CHECK_EQ((int)c2.control.cmd, (int)Control::ADD_NODE);
  CHECK_EQ(c2.control.node.size(), (size_t)2);
  CHECK_EQ(c2.control.node[0].hostname, std::string("10.0.0.1"));
  CHECK_EQ(c2.control.node[0].port, 5555);
  CHECK_EQ(c2.control.node[0].id, 9);
  CHECK(c2.control.node[0].is_recovery);
  CHECK_EQ(c2.control.node[0].customer_id, 2);
  CHECK_EQ(c2.control.node[1].id, Node::kEmpty);
  CHECK_EQ(c2.body.size(), (size_t)4);
  // barrier group and ack signature
  Meta b;
  b.control.cmd = Control::BARRIER;
  b.control.barrier_group = 7;
  out.clear();
  pb::EncodeMeta(b, &out);
  Meta b2;
  CHECK(pb::DecodeMeta(out.data(), out.size(), &b2));
  CHECK_EQ(b2.control.barrier_group, 7);
  Meta a;
  a.control.cmd = Control::ACK;
  a.control.msg_sig = 0xfedcba9876543210ull;
  out.clear();
  pb::EncodeMeta(a, &out);
  Meta a2;
  CHECK(pb::DecodeMeta(out.data(), out.size(), &a2));
  CHECK_EQ(a2.control.msg_sig, 0xfedcba9876543210ull);

  // unknown fields of every wire type are skipped; unpacked data_type is accepted
  std::string ext = out;
  ext += std::string("\xa0\x06\x05", 3);                          // field 100 varint
  ext += std::string("\xa9\x06", 2) + std::string(8, '\x01');     // field 101 fixed64
  ext += std::string("\xb2\x06\x03" "abc", 6);                    // field 102 bytes
  ext += std::string("\xbd\x06", 2) + std::string(4, '\x02');     // field 103 fixed32
  ext += std::string("\x48\x09", 2);                              // data_type unpacked: FLOAT
  Meta x;
  CHECK(pb::DecodeMeta(ext.data(), ext.size(), &x));
  CHECK_EQ(x.control.msg_sig, 0xfedcba9876543210ull);
  CHECK_EQ(x.data_type.size(), (size_t)1);

  // truncated or random input never crashes and is mostly rejected
  for (size_t cut = 0; cut + 1 < out.size(); ++cut) {
    Meta t;
    pb::DecodeMeta(out.data(), cut, &t);
  }
  std::mt19937 rng(5);
  for (int it = 0; it < 20000; ++it) {
    std::string junk(rng() % 64, '\0');
    for (auto& ch : junk) ch = static_cast<char>(rng());
    Meta t;
    pb::DecodeMeta(junk.data(), junk.size(), &t);
  }
  // round trip of random metas
  for (int it = 0; it < 2000; ++it) {
    Meta r;
    r.head = static_cast<int>(rng());
    r.app_id = rng() % 3 ? static_cast<int>(rng() % 100) : Meta::kEmpty;
    r.customer_id = static_cast<int>(rng() % 10);
    r.timestamp = rng() % 3 ? static_cast<int>(rng() % 100000) : Meta::kEmpty;
    r.request = rng() & 1; r.push = rng() & 1; r.pull = rng() & 1; r.simple_app = rng() & 1;
    r.priority = static_cast<int>(rng()) % 1000;
    r.body.assign(rng() % 20, 'x');
    for (unsigned k = 0; k < rng() % 4; ++k)
      r.data_type.push_back(static_cast<DataType>(rng() % 14));
    std::string s;
    pb::EncodeMeta(r, &s);
    Meta q;
    CHECK(pb::DecodeMeta(s.data(), s.size(), &q));
    CHECK_EQ(q.head, r.head); CHECK_EQ(q.app_id, r.app_id); CHECK_EQ(q.timestamp, r.timestamp);
    CHECK_EQ(q.priority, r.priority); CHECK_EQ(q.body, r.body);
    CHECK_EQ(q.data_type.size(), r.data_type.size());
    CHECK_EQ(q.request, r.request); CHECK_EQ(q.pull, r.pull);
  }
}

// Mutated encodings (flipped, inserted, removed bytes, truncations) must either decode into
// something that can be printed and encoded again, or be refused; never anything undefined.
static void TestCodecFuzz() {
  std::mt19937_64 rng(42);
  Meta m;
  m.head = 7; m.app_id = 1; m.customer_id = 2; m.timestamp = 99; m.request = true; m.push = true;
  m.body = "hello world";
  m.data_type = {UINT64, FLOAT, INT32};
  m.priority = 5;
  m.data_size = 123;
  m.control.cmd = Control::ADD_NODE;
  m.control.barrier_group = 7;
  m.control.msg_sig = 0x1234567890ull;
  for (int i = 0; i < 3; ++i) {
    Node n;
    n.role = Node::WORKER; n.id = 9 + 2 * i; n.hostname = "10.0.0.1"; n.port = 1000 + i;
    n.customer_id = i;
    m.control.node.push_back(n);
  }
  std::string good;
  pb::EncodeMeta(m, &good);
  size_t accepted = 0;
  for (int it = 0; it < 200000; ++it) {
    std::string s = good;
    const int edits = 1 + static_cast<int>(rng() % 4);
    for (int k = 0; k < edits; ++k) {
      switch (rng() % 4) {
        case 0: s[rng() % s.size()] = static_cast<char>(rng()); break;
        case 1: s.resize(rng() % (s.size() + 1)); break;
        case 2: s.insert(rng() % s.size(), 1, static_cast<char>(rng())); break;
        default: s.erase(rng() % s.size(), 1); break;
      }
      if (s.empty()) s = "x";
    }
    Meta out;
    if (pb::DecodeMeta(s.data(), s.size(), &out)) {
      ++accepted;
      std::string again;
      pb::EncodeMeta(out, &again);
      Message msg;
      msg.meta = out;
      CHECK(!msg.DebugString().empty());
    }
  }
  CHECK_GT(accepted, (size_t)0);
}

static void TestMisc() {
  CHECK_EQ(Postoffice::WorkerRankToID(3), 15);
  CHECK_EQ(Postoffice::ServerRankToID(3), 14);
  CHECK_EQ(Postoffice::IDtoRank(15), 3);
  CHECK_EQ(Postoffice::IDtoRank(14), 3);
  CHECK_EQ(Postoffice::IDtoRank(1), 0);
  CHECK(Postoffice::IsServerID(8) && !Postoffice::IsServerID(9) && !Postoffice::IsServerID(2));
  CHECK_EQ((int)GetDataType<float>(), (int)FLOAT);
  CHECK_EQ((int)GetDataType<uint64_t>(), (int)UINT64);
  CHECK_EQ((int)GetDataType<bfloat16_t>(), (int)BFLOAT16);
  CHECK_EQ((int)GetDataType<Range>(), (int)OTHER);
  Message m1, m2;
  m1.meta.app_id = m2.meta.app_id = 0;
  m1.meta.sender = 9; m1.meta.recver = 8; m1.meta.timestamp = 5; m1.meta.request = true;
  m2 = m1; m2.meta.request = false;
  CHECK_NE(Resender::Signature(m1), Resender::Signature(m2));
  m2 = m1; m2.meta.sender = 265;  // differs from 9 only above bit 8
  CHECK_NE(Resender::Signature(m1), Resender::Signature(m2));
  Message d;
  d.AddData(SArray<Key>({1, 2}));
  d.AddData(SArray<float>({1.f, 2.f}));
  CHECK_EQ(d.meta.data_size, static_cast<int>(2 * sizeof(Key) + 2 * sizeof(float)));
  CHECK(d.DebugString().find(sizeof(Key) == 8 ? "UINT64" : "UINT32") != std::string::npos);
  bool threw = false;
  try { CHECK_EQ(1, 2) << "boom"; } catch (const dmlc::Error& e) {
    threw = std::string(e.what()).find("boom") != std::string::npos;
  }
  CHECK(threw);
  Range r(5, 9);
  CHECK_EQ(r.size(), (uint64_t)4);
}

static void TestSortAndMatch() {
  std::mt19937_64 rng(3);
  SArray<Key> a(200000);
  for (auto& v : a) v = rng();
  std::vector<Key> ref(a.begin(), a.end());
  std::sort(ref.begin(), ref.end());
  ParallelSort(&a, 4);
  for (size_t i = 0; i < ref.size(); ++i) CHECK_EQ(a[static_cast<int>(i)], ref[i]);
  SArray<Key> sk, dk;
  SArray<float> sv;
  for (Key i = 0; i < 30000; i += 3) { sk.push_back(i); sv.push_back(1.f); sv.push_back(2.f); }
  for (Key i = 0; i < 30000; i += 2) dk.push_back(i);
  SArray<float> dv(dk.size() * 2, 10.f);
  size_t n = ParallelOrderedMatch(sk, sv, dk, &dv, 2, PLUS, 4);
  CHECK_EQ(n, (size_t)5000);
  for (size_t j = 0; j < dk.size(); ++j) {
    const bool hit = dk[static_cast<int>(j)] % 3 == 0;
    CHECK_EQ(dv[static_cast<int>(2 * j)], hit ? 11.f : 10.f);
    CHECK_EQ(dv[static_cast<int>(2 * j + 1)], hit ? 12.f : 10.f);
  }
  int x = 12;
  AssignFunc(10, XOR, &x);
  CHECK_EQ(x, 6);
}

int main() {
  TestSortAndMatch();
  TestSArray();
  TestEnv();
  TestQueues();
  TestCodec();
  TestCodecFuzz();
  TestMisc();
  printf("UNIT_OK\n");
  return 0;
}
