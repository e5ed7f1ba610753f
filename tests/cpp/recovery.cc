// Failure detection and recovery registration, driven from outside:
//   * every node sends heartbeats (PS_HEARTBEAT_INTERVAL=1);
//   * a worker started with PSB_TEST_DIE=1 exits abruptly after the start barrier;
//   * the scheduler polls GetDeadNodes(PS_HEARTBEAT_TIMEOUT) and prints DEAD <id>;
//   * a replacement worker (started by the test once DEAD was printed) registers, is given
//     the dead node's id with is_recovery set, and prints RECOVERED <id>;
//   * the surviving nodes learn the new address (they print nothing; the test checks that
//     the replacement can push to the servers and pull the sum back).
// No barrier is used after the failure: a dead node cannot enter one.
#include <unistd.h>

#include <chrono>
#include <cmath>
#include <thread>

#include "ps/ps.h"

using namespace ps;

int main() {
  const bool die = GetEnv("PSB_TEST_DIE", 0) != 0;
  const bool replacement = GetEnv("PSB_TEST_REPLACEMENT", 0) != 0;
  if (replacement) StartAsync(0); else Start(0);
  KVServer<float>* server = nullptr;
  if (IsServer()) {
    server = new KVServer<float>(0);
    server->set_request_handle(KVServerDefaultHandle<float>());
  }
  if (IsWorker()) {
    if (die) _exit(0);  // abrupt death: no Finalize, sockets just close
    KVWorker<float> kv(0, 0);
    std::vector<Key> keys = {10, kMaxKey / 2 + 10};
    std::vector<float> vals = {1.f, 2.f};
    if (replacement) {
      CHECK(Postoffice::Get()->is_recovery());
      fprintf(stderr, "RECOVERED %d\n", Postoffice::Get()->van()->my_node().id);
    }
    kv.Wait(kv.Push(keys, vals));
    std::vector<float> got;
    kv.Wait(kv.Pull(keys, &got));
    CHECK_GE(got[0], 1.f);
    if (!replacement) {
      // stay alive (and heartbeating) until the replacement's push shows up in the store
      for (int i = 0; i < 400 && got[0] < 2.f; ++i) {
        std::this_thread::sleep_for(std::chrono::milliseconds(100));
        kv.Wait(kv.Pull(keys, &got));
      }
      CHECK_GE(got[0], 2.f) << "the replacement never pushed";
    }
    fprintf(stderr, "WORKER_DONE %d %.1f\n", Postoffice::Get()->van()->my_node().id, got[0]);
  }
  if (IsScheduler()) {
    const int timeout = GetEnv("PS_HEARTBEAT_TIMEOUT", 3);
    bool reported = false;
    for (int i = 0; i < 300 && !reported; ++i) {
      std::this_thread::sleep_for(std::chrono::milliseconds(100));
      for (int id : Postoffice::Get()->GetDeadNodes(timeout)) {
        fprintf(stderr, "DEAD %d\n", id);
        reported = true;
      }
    }
    CHECK(reported) << "no dead node detected";
  }
  // leave without a global barrier; give in-flight traffic a moment
  std::this_thread::sleep_for(std::chrono::milliseconds(IsWorker() ? 200 : 4000));
  Finalize(0, false);
  delete server;
  return 0;
}
