// Host-plane checkpoint: servers save their shard on a group request, lose later updates on a
// load, and the files of two saves of the same state are identical.
// Usage (under the launcher): checkpoint <directory>
#include <atomic>
#include <cmath>
#include <fstream>
#include <iterator>

#include "ps/kv_checkpoint.h"
#include "ps/ps.h"

using namespace ps;

static std::string Slurp(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  return std::string(std::istreambuf_iterator<char>(f), std::istreambuf_iterator<char>());
}

int main(int argc, char** argv) {
  CHECK_GE(argc, 2) << "usage: checkpoint <directory>";
  const std::string dir = argv[1];
  Start(0);
  KVServer<float>* server = nullptr;
  CheckpointableHandle<float> handle;
  if (IsServer()) {
    server = new KVServer<float>(0);
    server->set_request_handle(handle);
    EnableCheckpointCommands(server, handle);
  }
  // nobody sends a command before every server obeys it
  Postoffice::Get()->Barrier(0, kScheduler + kServerGroup + kWorkerGroup);
  if (IsWorker()) {
    KVWorker<float> kv(0, 0);
    std::atomic<int> ok{0}, failed{0};
    kv.SimpleApp::set_response_handle([&](const SimpleData& d, SimpleApp*) {
      if (d.body == "ok") ++ok;
      if (d.body == "failed") ++failed;
    });
    const int W = NumWorkers(), S = NumServers();
    const int n = 1000, k = 3;
    std::vector<Key> keys(n);
    std::vector<float> vals(n * k), out;
    for (int i = 0; i < n; ++i) {
      keys[i] = kMaxKey / n * i + 5;
      for (int j = 0; j < k; ++j) vals[i * k + j] = static_cast<float>(i % 17 + j);
    }
    // pulling the initial values before anything was pushed is a normal pattern: one zero per
    // key comes back and the first wide push afterwards must find no narrow slot in its way
    kv.Wait(kv.Pull(keys, &out));
    CHECK_EQ(out.size(), static_cast<size_t>(n));
    for (int i = 0; i < n; ++i) CHECK_EQ(out[i], 0.f);
    out.clear();
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    kv.Wait(kv.Push(keys, vals));
    Postoffice::Get()->Barrier(0, kWorkerGroup);  // every worker's push is in
    if (MyRank() == 0) {
      kv.Wait(kv.Request(kCheckpointSave, dir, kServerGroup));
      CHECK_EQ(ok.load(), S);
      std::vector<std::string> first;
      for (int s = 0; s < S; ++s) first.push_back(Slurp(CheckpointFile(dir, s)));
      kv.Wait(kv.Request(kCheckpointSave, dir, kServerGroup));
      for (int s = 0; s < S; ++s) {
        CHECK(!first[s].empty());
        CHECK(first[s] == Slurp(CheckpointFile(dir, s))) << "saves of one state differ";
      }
    }
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    kv.Wait(kv.Push(keys, vals));                 // updates that the load will discard
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    kv.Wait(kv.Pull(keys, &out));
    for (int i = 0; i < n * k; ++i) CHECK_LT(std::fabs(out[i] - 2 * W * vals[i]), 1e-4f);
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    if (MyRank() == 0) {
      ok = 0;
      kv.Wait(kv.Request(kCheckpointLoad, dir, kServerGroup));
      CHECK_EQ(ok.load(), S);
      kv.Wait(kv.Request(kCheckpointLoad, dir + "/does-not-exist", kServerGroup));
      CHECK_EQ(failed.load(), S) << "a missing file must be reported, the store kept";
    }
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    kv.Wait(kv.Pull(keys, &out));
    for (int i = 0; i < n * k; ++i) CHECK_LT(std::fabs(out[i] - W * vals[i]), 1e-4f);
    LOG(INFO) << "CHECKPOINT_OK rank " << MyRank();
  }
  Finalize(0, true);
  delete server;
  return 0;
}
