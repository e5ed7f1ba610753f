// Worker processes with two customer threads each; every thread calls
// Barrier(kWorkerGroup) several times, and in every other process the second thread arrives
// late.  Each customer's k-th call must pass exactly the k-th round: a late caller that opened
// a round of its own would leave a half-counted round at the scheduler and hang.
// (The reference counts every customer's call once: src/postoffice.cc:142-167.)
#include <atomic>
#include <chrono>
#include <cstring>
#include <thread>

#include "ps/ps.h"

using namespace ps;

static std::atomic<int> g_rounds{0};

static void Worker(int cid) {
  Start(cid);
  const int stagger_ms = (cid == 1 && (MyRank() / 2) % 2 == 0) ? 300 : 0;
  for (int round = 0; round < 4; ++round) {
    if (stagger_ms) std::this_thread::sleep_for(std::chrono::milliseconds(stagger_ms));
    Postoffice::Get()->Barrier(cid, kWorkerGroup);
    ++g_rounds;
  }
  Finalize(cid, true);
}

int main(int argc, char* argv[]) {
  const char* role = getenv("DMLC_ROLE");
  if (strcmp(role, "worker") != 0) {
    Start(0);
    Finalize(0, true);
    return 0;
  }
  std::thread t0(Worker, 0), t1(Worker, 1);
  t0.join();
  t1.join();
  CHECK_EQ(g_rounds.load(), 8);
  LOG(INFO) << "BARRIER_ROUNDS_OK";
  return 0;
}
