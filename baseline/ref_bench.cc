// Dense push+pull benchmark written against the reference library's own public API
// (ps::Start/Finalize, KVWorker::ZPush/ZPull/Wait, KVServer with a request handle).  It is
// compiled and linked against the unmodified reference sources.  Shape: every worker pushes
// one tensor of `n` floats as S key-value pairs (key j in server j's range, n/S values each,
// dynamic lengths); the server handle sums the workers' pushes and, once all W arrived,
// applies SGD (lr 0.01) to its master copy and answers; every worker then pulls the tensor.
// Usage: ref_bench <n_floats> <steps> <warmup>; each worker prints "REF_SECONDS <s>".
#include <chrono>
#include <cstdlib>
#include <unordered_map>

#include "ps/ps.h"

using namespace ps;

struct SumSgdHandle {
  struct Slot {
    std::vector<float> master, acc;
    int arrived = 0;
    std::vector<KVMeta> waiting;
  };
  std::unordered_map<Key, Slot> store;
  void operator()(const KVMeta& m, const KVPairs<float>& d, KVServer<float>* s) {
    if (m.push) {
      size_t off = 0;
      for (size_t i = 0; i < d.keys.size(); ++i) {
        const size_t len = d.lens.size() ? d.lens[i] : d.vals.size() / d.keys.size();
        Slot& slot = store[d.keys[i]];
        if (slot.master.empty()) { slot.master.assign(len, 0.f); slot.acc.assign(len, 0.f); }
        const float* v = d.vals.data() + off;
        for (size_t j = 0; j < len; ++j) slot.acc[j] += v[j];
        off += len;
        slot.waiting.push_back(m);
        if (++slot.arrived == NumWorkers()) {
          for (size_t j = 0; j < len; ++j) {
            slot.master[j] -= 0.01f * slot.acc[j];
            slot.acc[j] = 0.f;
          }
          slot.arrived = 0;
          for (const KVMeta& w : slot.waiting) s->Response(w);
          slot.waiting.clear();
        }
      }
      return;
    }
    KVPairs<float> res;
    res.keys = d.keys;
    res.lens.resize(d.keys.size());
    for (size_t i = 0; i < d.keys.size(); ++i) {
      const Slot& slot = store[d.keys[i]];
      res.lens[i] = static_cast<int>(slot.master.size());
      const size_t old = res.vals.size();
      res.vals.resize(old + slot.master.size());
      memcpy(res.vals.data() + old, slot.master.data(), slot.master.size() * sizeof(float));
    }
    s->Response(m, res);
  }
};

int main(int argc, char* argv[]) {
  const size_t n = argc > 1 ? strtoull(argv[1], nullptr, 10) : (1u << 20);
  const int steps = argc > 2 ? atoi(argv[2]) : 10;
  const int warmup = argc > 3 ? atoi(argv[3]) : 3;
  Start(0);
  KVServer<float>* server = nullptr;
  if (IsServer()) {
    server = new KVServer<float>(0);
    server->set_request_handle(SumSgdHandle());
    RegisterExitCallback([server]() { delete server; });
  }
  if (IsWorker()) {
    KVWorker<float> kv(0, 0);
    const int S = NumServers();
    const size_t per = n / S;
    SArray<Key> keys(S);
    SArray<int> lens(S);
    for (int j = 0; j < S; ++j) { keys[j] = kMaxKey / S * j + 1; lens[j] = static_cast<int>(per); }
    SArray<float> vals(per * S);
    unsigned seed = 1234u + MyRank();
    for (size_t i = 0; i < vals.size(); ++i) vals[i] = (rand_r(&seed) % 2001 - 1000) * 1e-3f;
    SArray<float> out(per * S);
    SArray<int> out_lens(S);
    auto round = [&]() {
      kv.Wait(kv.ZPush(keys, vals, lens));
      kv.Wait(kv.ZPull(keys, &out, &out_lens));
    };
    for (int i = 0; i < warmup; ++i) round();
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    const auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < steps; ++i) round();
    const double sec = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    fprintf(stdout, "REF_SECONDS %.6f %zu\n", sec, per * S);
    fflush(stdout);
  }
  Finalize(0, true);
  return 0;
}
