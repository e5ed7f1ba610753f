// Shared-memory payload frames (DMLC_LOCAL=1): large arrays travel between processes of one
// host as a file descriptor plus (offset, length) instead of bytes.
//
// Without arguments: single-process checks of the pool (allocation, recycling, a shared view
// keeps its contents, a segment that comes back to its owner is recognised).
// With "job" under the launcher: every worker pushes three generations of a large tensor; the
// server keeps the received arrays WITHOUT copying them; the worker's buffers are freed and
// recycled in between.  A later pull must return every generation intact, which fails if a
// segment were reused while the server still held a view of it.
#include <unistd.h>

#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "ps/internal/shm_pool.h"
#include "ps/ps.h"

using namespace ps;

namespace {

constexpr size_t kN = 1 << 20;  // floats per push: 4 MiB, far above the shared-memory threshold

int UnitChecks() {
  setenv("PS_SHM", "1", 1);
  CHECK(shm::Enabled());
  const shm::Stats s0 = shm::GetStats();
  char* a = shm::ArrayAlloc(1 << 20);
  memset(a, 7, 1 << 20);
  int fd = -1;
  uint64_t off = 0, seg = 0;
  CHECK(!shm::Share(a, 100, &fd, &off, &seg)) << "small ranges go through the socket";
  CHECK(shm::Share(a + 4096, 1 << 19, &fd, &off, &seg));
  CHECK_EQ(off, (uint64_t)(4096 + 4096));
  // the peer's side, played by this process: the segment is recognised by its inode
  char* base = shm::Import(dup(fd), seg);
  CHECK(base != nullptr);
  CHECK_EQ(static_cast<int>(base[off]), 7);
  CHECK_EQ(base + 4096, a) << "own segment must not be mapped a second time";
  // freed by its owner while a view is still out: must not be handed out again
  shm::ArrayFree(a);
  char* b = shm::ArrayAlloc(1 << 20);
  CHECK(b != a);
  CHECK_EQ(static_cast<int>(base[off]), 7) << "the view lost its contents";
  shm::Release(base);
  shm::ArrayFree(b);
  // now both are idle: the next request of that size recycles one of them
  char* c = shm::ArrayAlloc(1 << 20);
  CHECK(c == a || c == b);
  shm::ArrayFree(c);
  const shm::Stats s1 = shm::GetStats();
  CHECK_GE(s1.segments_reused, s0.segments_reused + 1);
  CHECK_EQ(s1.bytes_live, s0.bytes_live);
  // arrays draw from the pool and give back to it
  {
    SArray<float> x(kN, 1.5f);
    CHECK(shm::Share(x.data(), kN * sizeof(float), &fd, &off, &seg));
    shm::Unshare(x.data());
    SArray<float> y;
    y.CopyFrom(x);
    CHECK_EQ(y[kN - 1], 1.5f);
  }
  CHECK_EQ(shm::GetStats().bytes_live, s0.bytes_live);
  shm::Trim();
  CHECK_EQ(shm::GetStats().bytes_pooled, (uint64_t)0);
  // small arrays stay on the heap
  char* small = shm::ArrayAlloc(100);
  CHECK(!shm::Share(small, 100, &fd, &off, &seg));
  shm::ArrayFree(small);
  fprintf(stderr, "SHM_UNIT_OK\n");
  return 0;
}

// Keeps every pushed array as received (no copy) and answers pulls from them.
struct KeepHandle {
  std::map<Key, SArray<float>> kept;
  void operator()(const KVMeta& m, const KVPairs<float>& d, KVServer<float>* s) {
    KVPairs<float> res;
    if (m.push) {
      CHECK_EQ(d.keys.size(), (size_t)1);
      kept[d.keys[0]] = d.vals;  // shares the transport buffer, i.e. the sender's pages
    } else {
      CHECK_EQ(d.keys.size(), (size_t)1);
      res.keys = d.keys;
      res.vals = kept.at(d.keys[0]);
    }
    s->Response(m, res);
  }
};

float Pattern(int rank, int gen, size_t i) {
  return static_cast<float>((rank + 1) * 1000 + gen * 10) + static_cast<float>(i % 7);
}

int Job() {
  Start(0);
  KVServer<float>* server = nullptr;
  if (IsServer()) {
    server = new KVServer<float>(0);
    server->set_request_handle(KeepHandle());
    RegisterExitCallback([server]() { delete server; });
  }
  if (IsWorker()) {
    KVWorker<float> kv(0, 0);
    const int rank = MyRank();
    const int gens = 3;
    for (int g = 0; g < gens; ++g) {
      // one key per (worker, generation), all in server 0's range
      std::vector<Key> keys = {static_cast<Key>(100 + rank * 10 + g)};
      std::vector<float> vals(kN);
      for (size_t i = 0; i < kN; ++i) vals[i] = Pattern(rank, g, i);
      kv.Wait(kv.Push(keys, vals));  // the copy made by Push is freed here and may be recycled
    }
    const shm::Stats st = shm::GetStats();
    CHECK_GE(st.segments_created, (uint64_t)gens) << "a kept view must not be recycled";
    for (int g = 0; g < gens; ++g) {
      std::vector<Key> keys = {static_cast<Key>(100 + rank * 10 + g)};
      std::vector<float> out;
      kv.Wait(kv.Pull(keys, &out));
      CHECK_EQ(out.size(), kN);
      for (size_t i = 0; i < kN; i += 997) CHECK_EQ(out[i], Pattern(rank, g, i)) << g << " " << i;
    }
    fprintf(stdout, "SHM_JOB_OK %d created=%llu reused=%llu\n", rank,
            (unsigned long long)st.segments_created, (unsigned long long)st.segments_reused);
    fflush(stdout);
  }
  Finalize(0, true);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc > 1 && std::string(argv[1]) == "job") return Job();
  return UnitChecks();
}
