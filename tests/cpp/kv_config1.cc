// Correctness run shaped like the reference's test_kv_app: every worker pushes the same
// N = 100000 keys k_i = i * floor((2^64-1)/N), one float ~U(-1,1) each from a fixed seed,
// ten times; after a worker barrier a pull must return 10 * num_workers * val.  Runs in any
// role layout: separate scheduler/servers/workers, or joint processes.
#include <cmath>
#include <random>

#include "ps/ps.h"

using namespace ps;

int main(int argc, char* argv[]) {
  Start(0);
  KVServer<float>* server = nullptr;
  if (IsServer()) {
    server = new KVServer<float>(0);
    server->set_request_handle(KVServerDefaultHandle<float>());
  }
  if (IsWorker()) {
    KVWorker<float> kv(0, 0);
    const int N = 100000;
    const Key stride = kMaxKey / N;
    std::vector<Key> keys(N);
    std::vector<float> vals(N);
    std::mt19937 rng(2024);
    std::uniform_real_distribution<float> uni(-1.f, 1.f);
    for (int i = 0; i < N; ++i) {
      keys[i] = stride * static_cast<Key>(i);
      vals[i] = uni(rng);
    }
    const int rounds = 10;
    for (int r = 0; r < rounds; ++r) kv.Wait(kv.Push(keys, vals));
    Postoffice::Get()->Barrier(0, kWorkerGroup);  // every worker's pushes have landed
    std::vector<float> got;
    kv.Wait(kv.Pull(keys, &got));
    CHECK_EQ(got.size(), vals.size());
    double err = 0;
    const float scale = static_cast<float>(rounds * NumWorkers());
    for (int i = 0; i < N; ++i) err += std::fabs(got[i] - scale * vals[i]);
    CHECK_LT(err / N, 1e-5 * scale) << "mean abs error " << err / N;
    LOG(INFO) << "CONFIG1_OK rank " << MyRank() << " mean abs error " << err / N;
  }
  Finalize(0, true);
  delete server;
  return 0;
}
