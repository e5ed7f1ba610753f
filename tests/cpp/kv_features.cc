// Multi-process feature test: dynamic-length values, wide fixed-length values, zero-copy
// calls with completion callbacks, a request handle that defers its response until every
// worker has pushed (bulk-synchronous update), the cmd field, priorities, a custom slicer,
// and SimpleApp group requests.
#include <atomic>
#include <cmath>
#include <map>

#include "ps/ps.h"

using namespace ps;

// Server handle with three behaviours selected by cmd:
//   cmd 0: accumulate variable-length values per key (lens required on push)
//   cmd 1: bulk-synchronous: hold the push responses until all workers pushed this key set
//   cmd 2: return "priority seen" bookkeeping
struct Handle {
  std::map<Key, std::vector<float>> store;
  std::vector<KVMeta> waiting;
  void operator()(const KVMeta& m, const KVPairs<float>& d, KVServer<float>* s) {
    if (m.cmd == 1 && m.push) {
      size_t off = 0;
      for (size_t i = 0; i < d.keys.size(); ++i) {
        auto& v = store[d.keys[i]];
        if (v.empty()) v.assign(1, 0.f);
        v[0] += d.vals[off++];
      }
      waiting.push_back(m);
      if (static_cast<int>(waiting.size()) == NumWorkers()) {
        for (const auto& w : waiting) s->Response(w);
        waiting.clear();
      }
      return;
    }
    KVPairs<float> res;
    size_t off = 0;
    for (size_t i = 0; i < d.keys.size(); ++i) {
      const Key k = d.keys[i];
      if (m.push) {
        const int len = d.lens.empty() ? static_cast<int>(d.vals.size() / d.keys.size())
                                       : d.lens[i];
        auto& v = store[k];
        if (v.empty()) v.assign(len, 0.f);
        CHECK_EQ((int)v.size(), len);
        for (int j = 0; j < len; ++j) v[j] += d.vals[off + j];
        off += len;
      }
      if (m.pull) {
        const auto& v = store[k];
        res.keys.push_back(k);
        res.lens.push_back(static_cast<int>(v.size()));
        for (float x : v) res.vals.push_back(x);
      }
    }
    s->Response(m, res);
  }
};

int main() {
  Start(0);
  KVServer<float>* server = nullptr;
  if (IsServer()) {
    server = new KVServer<float>(0);
    server->set_request_handle(Handle());
  }
  std::atomic<int> simple_seen{0};
  SimpleApp app(1, 0);
  app.set_request_handle([&simple_seen](const SimpleData& d, SimpleApp* a) {
    CHECK_EQ(d.head, 42);
    CHECK_EQ(d.body, std::string("hello"));
    ++simple_seen;
    a->Response(d, "ack");
  });
  std::atomic<int> responses{0};
  app.set_response_handle([&responses](const SimpleData& d, SimpleApp*) {
    CHECK_EQ(d.body, std::string("ack"));
    ++responses;
  });
  // a request that arrives before the handles above are installed would be answered by the
  // default handle: nobody sends one before everybody is here
  Postoffice::Get()->Barrier(0, kScheduler + kServerGroup + kWorkerGroup);

  if (IsWorker()) {
    KVWorker<float> kv(0, 0);
    const int W = NumWorkers();
    // keys spread over the whole key space so that every server gets some
    const int n = 64;
    SArray<Key> keys(n);
    SArray<int> lens(n);
    size_t total = 0;
    for (int i = 0; i < n; ++i) {
      keys[i] = kMaxKey / n * i + 17;
      lens[i] = 1 + i % 5;
      total += lens[i];
    }
    SArray<float> vals(total);
    for (size_t i = 0; i < total; ++i) vals[i] = static_cast<float>(i % 13) - 6.f;
    // (1) dynamic lengths, zero-copy push with callback, then barrier and pull with lens
    std::atomic<bool> cb_ran{false};
    int ts = kv.ZPush(keys, vals, lens, 0, [&cb_ran]() { cb_ran = true; }, /*priority=*/3);
    kv.Wait(ts);
    CHECK(cb_ran.load()) << "callback must have finished when Wait returns";
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    SArray<float> got;
    SArray<int> got_lens;
    kv.Wait(kv.ZPull(keys, &got, &got_lens));
    CHECK_EQ(got.size(), total);
    CHECK_EQ(got_lens.size(), (size_t)n);
    for (int i = 0; i < n; ++i) CHECK_EQ(got_lens[i], lens[i]);
    for (size_t i = 0; i < total; ++i) CHECK_LT(std::fabs(got[i] - W * vals[i]), 1e-4f);

    // (2) bulk-synchronous push: the response arrives only after all workers pushed
    std::vector<Key> k2 = {kMaxKey / 3, kMaxKey / 3 * 2};
    std::vector<float> v2 = {1.f, 2.f};
    kv.Wait(kv.Push(k2, v2, {}, /*cmd=*/1));
    std::vector<float> g2;
    kv.Wait(kv.Pull(k2, &g2));
    CHECK_EQ(g2.size(), (size_t)2);
    CHECK_LT(std::fabs(g2[0] - W * 1.f), 1e-5f) << "all pushes are visible after a BSP push";
    CHECK_LT(std::fabs(g2[1] - W * 2.f), 1e-5f);

    // (3) PushPull with a custom slicer that sends everything to the owner of the first key
    Postoffice::Get()->Barrier(0, kWorkerGroup);
    std::vector<Key> k3 = {5, 6, 7};
    std::vector<float> v3 = {1.f, 1.f, 1.f}, o3;
    int calls = 0;
    kv.set_slicer([&calls](const KVPairs<float>& send, const std::vector<Range>& ranges,
                           KVWorker<float>::SlicedKVs* sliced) {
      ++calls;
      sliced->assign(ranges.size(), std::make_pair(false, KVPairs<float>()));
      (*sliced)[0].first = true;
      (*sliced)[0].second = send;
    });
    kv.Wait(kv.PushPull(k3, v3, &o3));
    CHECK_GE(calls, 1);
    CHECK_EQ(o3.size(), (size_t)3);
    CHECK_GE(o3[0], 1.f);
    CHECK_LE(o3[0], (float)W);

    // (4) an empty request completes at once and still runs its callback
    std::atomic<bool> empty_cb{false};
    kv.Wait(kv.ZPush(SArray<Key>(), SArray<float>(), {}, 0, [&empty_cb]() { empty_cb = true; }));
    CHECK(empty_cb.load());
    LOG(INFO) << "FEATURES_OK rank " << MyRank();
  }
  if (IsScheduler()) {
    // (5) group request: everyone (scheduler included) handles it and answers
    int ts = app.Request(42, "hello", kScheduler + kServerGroup + kWorkerGroup);
    app.Wait(ts);
    CHECK_EQ(responses.load(), NumWorkers() + NumServers() + 1);
  }
  Finalize(0, true);
  if (!IsScheduler() || true) CHECK_GE(simple_seen.load(), 1);
  delete server;
  return 0;
}
