// One worker process with two customer threads (DMLC_NUM_WORKER=2), like the reference's
// test_kv_app_multi_workers: each thread calls Start/Finalize with its own customer id.
#include <cmath>
#include <cstring>
#include <thread>

#include "ps/ps.h"

using namespace ps;

static void Worker(int cid) {
  Start(cid);
  KVWorker<float> kv(0, cid);
  const int n = 1000;
  std::vector<Key> keys(n);
  std::vector<float> vals(n);
  for (int i = 0; i < n; ++i) {
    keys[i] = kMaxKey / n * i + cid;  // the two threads use disjoint keys
    vals[i] = static_cast<float>(i % 7 + cid);
  }
  const int repeat = 20 + 30 * cid;  // the threads finish at different times
  for (int r = 0; r < repeat; ++r) kv.Wait(kv.Push(keys, vals));
  std::vector<float> got;
  kv.Wait(kv.Pull(keys, &got));
  for (int i = 0; i < n; ++i) CHECK_LT(std::fabs(got[i] - repeat * vals[i]), 1e-3f);
  LOG(INFO) << "CUSTOMER_OK " << cid;
  Finalize(cid, true);
}

int main(int argc, char* argv[]) {
  const char* role = getenv("DMLC_ROLE");
  if (strcmp(role, "worker") != 0) {
    Start(0);
    KVServer<float>* server = nullptr;
    if (IsServer()) {
      server = new KVServer<float>(0);
      server->set_request_handle(KVServerDefaultHandle<float>());
    }
    Finalize(0, true);
    delete server;
    return 0;
  }
  std::thread t0(Worker, 0), t1(Worker, 1);
  t0.join();
  t1.join();
  return 0;
}
