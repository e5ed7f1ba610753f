// Whole runtime in one process (DMLC_PS_VAN_TYPE=loop): scheduler, server 0 and worker 0.
#include <cmath>

#include "ps/ps.h"

using namespace ps;

int main() {
  Environment::Init({{"DMLC_PS_VAN_TYPE", "loop"}});
  for (int round = 0; round < 2; ++round) {  // Start/Finalize can be repeated in-process
    Start(0);
    CHECK(IsWorker() && IsServer() && IsScheduler());
    CHECK_EQ(NumWorkers(), 1);
    CHECK_EQ(NumServers(), 1);
    auto* server = new KVServer<float>(0);
    server->set_request_handle(KVServerDefaultHandle<float>());
    RegisterExitCallback([server]() { delete server; });
    {
      KVWorker<float> kv(0, 0);
      std::vector<Key> keys = {1, 3, 1000, kMaxKey - 7};
      std::vector<float> vals = {1, 2, 3, 4, 5, 6, 7, 8};  // width 2
      for (int i = 0; i < 5; ++i) kv.Wait(kv.Push(keys, vals));
      std::vector<float> got;
      kv.Wait(kv.Pull(keys, &got));
      CHECK_EQ(got.size(), (size_t)8);
      for (int i = 0; i < 8; ++i) CHECK_LT(std::fabs(got[i] - 5 * vals[i]), 1e-6f);
      std::vector<float> outs;
      kv.Wait(kv.PushPull(keys, vals, &outs));
      for (int i = 0; i < 8; ++i) CHECK_LT(std::fabs(outs[i] - 6 * vals[i]), 1e-6f);
      // many requests: the tracker forgets completed ones beyond a window, timestamps keep
      // counting, and waiting for a forgotten request returns at once
      std::vector<int> stamps;
      for (int i = 0; i < 10000; ++i) stamps.push_back(kv.Push(keys, vals));
      CHECK_EQ(stamps.back() - stamps.front(), 9999);
      kv.Wait(stamps.back());
      for (int ts : {stamps[0], stamps[5000], stamps[9999]}) kv.Wait(ts);
      kv.Wait(kv.Pull(keys, &got));
      for (int i = 0; i < 8; ++i) CHECK_LT(std::fabs(got[i] - 10006 * vals[i]), 1e-3f * 10006);
      const auto& ranges = Postoffice::Get()->GetServerKeyRanges();
      CHECK_EQ(ranges.size(), (size_t)1);
      CHECK_EQ(ranges[0].begin(), (uint64_t)0);
      Postoffice::Get()->Barrier(0, kWorkerGroup + kServerGroup + kScheduler);
    }
    Finalize(0, true);
  }
  LOG(INFO) << "LOOP_OK";
  return 0;
}
