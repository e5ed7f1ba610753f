// The device plane driven through the ordinary API: ps::Start, KVWorker push / pull /
// push-pull with timestamps, callbacks and Wait, Finalize -- and nothing else (no collective
// library).  Runs with the CPU stand-in of the plane (PlaneOptions::device = -1), in one
// process under the loop van or as several joint processes, so the handle exchange over the
// control plane, the key -> shard mapping, the routing in KVWorker and the completion through
// the Customer tracker are checked where no GPU exists.  Built with -DPLANE_DEVICE=0 the same
// program runs on GPUs (tests/test_kvstore_gpu.py, tests/test_multi_gpu.py).
// Reference behaviour checked: include/ps/kv_app.h:54-372 (timestamps, Wait, callback before
// Wait returns, zero-copy Z* calls).
#include <atomic>
#include <cmath>
#include <cstring>

#include "ps/device/plane.h"
#include "ps/ps.h"

using namespace ps;
using device::Plane;

#ifndef PLANE_DEVICE
#define PLANE_DEVICE -1
#endif

static psdev_opt_t Sgd(float lr) {
  psdev_opt_t o{};
  o.kind = PSDEV_OPT_SGD;
  o.scale = 1.f;
  o.lr = lr;
  return o;
}

int main(int argc, char** argv) {
  Start(0);
  if (!IsWorker()) {  // scheduler (or a pure server): nothing to do on the device plane
    Finalize(0, true);
    return 0;
  }
  device::PlaneOptions po;
  po.heap_bytes = PLANE_DEVICE < 0 ? (64u << 20) : (96u << 20);
  po.slice_bytes = 1u << 20;  // several slices per request, with the ramp at both ends
  po.device = PLANE_DEVICE < 0 ? -1 : MyRank();
  po.timeout_ns = 1500000000ull;
  Plane* plane = Plane::Get();
  plane->Start(po);
  const int W = plane->world(), R = plane->rank();
  CHECK_EQ(W, NumWorkers());

  // control-plane collectives
  auto all = plane->AllGather("rank-" + std::to_string(R));
  CHECK_EQ(all.size(), (size_t)W);
  for (int r = 0; r < W; ++r) CHECK_EQ(all[r], "rank-" + std::to_string(r));

  const int64_t n = 600000 + 8 * W + 3;  // not a multiple of anything convenient
  const uint64_t kTensor = 7;
  const device::DenseInfo& d =
      plane->DeclareDense(0, kTensor, n, PSDEV_F32, PSDEV_F32, Sgd(0.5f));
  const std::vector<Key> keys = plane->DenseKeys(kTensor);
  CHECK_EQ(keys.size(), (size_t)W);
  {
    const auto& ranges = plane->KeyRanges();
    for (int j = 0; j < W; ++j) CHECK_EQ(keys[j], ranges[j].begin() + kTensor);
  }
  KVWorker<float> kv(0, 0);

  auto val_of = [](int rank, int64_t i) { return static_cast<float>((i % 13) - 6 + rank); };
  std::vector<float> vals(n), expect(n, 0.f);
  for (int64_t i = 0; i < n; ++i) vals[i] = val_of(R, i);
  auto sum_of = [&](int64_t i) {
    float s = 0.f;
    for (int r = 0; r < W; ++r) s += val_of(r, i);
    return s;
  };

  // 1. Push (copies), then Pull into empty vectors: sizes and per-key lengths come back
  int last_ts = -1;
  for (int rep = 0; rep < 3; ++rep) {
    const int ts = kv.Push(keys, vals);
    CHECK_GT(ts, last_ts);
    last_ts = ts;
    kv.Wait(ts);
    for (int64_t i = 0; i < n; ++i) expect[i] -= 0.5f * sum_of(i);
  }
  std::vector<float> got;
  std::vector<int> lens;
  kv.Wait(kv.Pull(keys, &got, &lens));
  CHECK_EQ(got.size(), (size_t)n);
  CHECK_EQ(lens.size(), (size_t)W);
  int64_t total = 0;
  for (int j = 0; j < W; ++j) total += lens[j];
  CHECK_EQ(total, n);
  for (int64_t i = 0; i < n; ++i) CHECK_LT(std::fabs(got[i] - expect[i]), 1e-4f) << "at " << i;

  // 2. ZPushPull with explicit lens and a callback that has run when Wait returns
  std::atomic<int> called{0};
  SArray<Key> skeys(keys);
  SArray<float> svals(vals), souts(n, 0.f);
  SArray<int> slens(lens);
  kv.Wait(kv.ZPushPull(skeys, svals, &souts, &slens, 0, [&called]() { ++called; }));
  CHECK_EQ(called.load(), 1);
  for (int64_t i = 0; i < n; ++i) {
    expect[i] -= 0.5f * sum_of(i);
    CHECK_LT(std::fabs(souts[i] - expect[i]), 1e-4f) << "at " << i;
  }

  // 2b. a request that nobody waits for, by a worker that goes away: Plane::Drain returns when
  // the request has completed (callback run, tracker credited); the worker may then be deleted
  {
    KVWorker<float> brief(0, 7);
    std::atomic<int> fired{0};
    brief.ZPush(skeys, svals, slens, 0, [&fired]() { ++fired; });
    plane->Drain();
    CHECK_EQ(fired.load(), 1);
  }
  for (int64_t i = 0; i < n; ++i) expect[i] -= 0.5f * sum_of(i);
  kv.Wait(kv.Pull(keys, &got));
  for (int64_t i = 0; i < n; ++i) CHECK_LT(std::fabs(got[i] - expect[i]), 1e-4f) << "at " << i;

  // 3. a subset of the keys touches only those shards' values
  if (W > 1) {
    const int j = W - 1;
    const int64_t lo = j * d.share, hi = std::min<int64_t>(lo + d.share, n);
    std::vector<float> part(vals.begin() + lo, vals.begin() + hi), part_out;
    kv.Wait(kv.PushPull({keys[j]}, part, &part_out));
    CHECK_EQ(part_out.size(), (size_t)(hi - lo));
    for (int64_t i = lo; i < hi; ++i) {
      expect[i] -= 0.5f * sum_of(i);
      CHECK_LT(std::fabs(part_out[i - lo] - expect[i]), 1e-4f);
    }
    kv.Wait(kv.Pull(keys, &got));
    for (int64_t i = 0; i < n; ++i) CHECK_LT(std::fabs(got[i] - expect[i]), 1e-4f) << "at " << i;
  }

  // 4. zero copy: values written straight into the tensor's gradient buffer in the arena and
  // pulled straight into its weight buffer
#if PLANE_DEVICE < 0
  {
    float* g = static_cast<float*>(d.grad);
    for (int64_t i = 0; i < n; ++i) g[i] = 1.f;
    SArray<float> dev_vals = SArray<float>::FromDevice(g, n);
    SArray<float> dev_out = SArray<float>::FromDevice(static_cast<float*>(d.weight), n);
    kv.Wait(kv.ZPushPull(skeys, dev_vals, &dev_out));
    const float* w = static_cast<const float*>(d.weight);
    for (int64_t i = 0; i < n; ++i) {
      expect[i] -= 0.5f * W;
      CHECK_LT(std::fabs(w[i] - expect[i]), 1e-4f);
    }
  }
#endif

  // 5. a peer that never issues the matching request: the wait runs out on the device side
  // (a flag that nothing sets) and Wait reports it instead of hanging; afterwards the channel
  // works again
  if (W > 1) {
    plane->Barrier();
    if (R == 0) {
      bool threw = false;
      const int ts = kv.Push(keys, vals);
      try {
        kv.Wait(ts);
      } catch (const Error& e) {
        threw = strstr(e.what(), "did not arrive") != nullptr;
      }
      CHECK(threw) << "a request that no peer matched must fail, not hang or succeed";
    }
    plane->ClearStatus(0, kTensor);  // collective
    // rank 0's gradients of the failed round were applied nowhere
    kv.Wait(kv.Push(keys, vals));
    for (int64_t i = 0; i < n; ++i) expect[i] -= 0.5f * sum_of(i);
    kv.Wait(kv.Pull(keys, &got));
    for (int64_t i = 0; i < n; ++i) CHECK_LT(std::fabs(got[i] - expect[i]), 1e-4f) << "at " << i;
  }

  // 6. keyed (sparse) requests: key array in device memory -> the app's keyed table.  Every
  // worker pushes the same sorted keys with value (rank + 1) per element; the sum handle then
  // holds W(W+1)/2 per element after one push, and a pull-only request reads it back.
  {
    const int kApp = 3, width = 2;
    const int64_t nk = 5000;
    const uint64_t key_space = 1u << 20;
    const device::SparseInfo& sp =
        plane->DeclareSparse(kApp, key_space, nk, width, /*sum*/ 0, 0.f, 0.f, 0.f, 0.f, 0.f);
    KVWorker<float> skv(kApp, 1);
    std::vector<Key> hkeys(nk);
    for (int64_t i = 0; i < nk; ++i) hkeys[i] = static_cast<Key>(i) * (key_space / nk) + 7;
    std::vector<float> hvals(nk * width, static_cast<float>(R + 1));
    // device copies: scratch from the symmetric heap (any device memory would do)
    const int64_t koff = plane->Alloc(nk * 8), voff = plane->Alloc(nk * width * 4),
                  ooff = plane->Alloc(nk * width * 4);
    CHECK(koff >= 0 && voff >= 0 && ooff >= 0);
    Key* dkeys = static_cast<Key*>(plane->Local(koff));
    float* dvals = static_cast<float*>(plane->Local(voff));
    float* dout = static_cast<float*>(plane->Local(ooff));
    plane->Memcpy(dkeys, hkeys.data(), nk * 8);
    plane->Memcpy(dvals, hvals.data(), nk * width * 4);
    SArray<Key> sk = SArray<Key>::FromDevice(dkeys, nk);
    SArray<float> sv = SArray<float>::FromDevice(dvals, nk * width);
    SArray<float> so = SArray<float>::FromDevice(dout, nk * width);
    std::atomic<int> done{0};
    skv.Wait(skv.ZPushPull(sk, sv, &so, nullptr, 0, [&done]() { ++done; }));
    CHECK_EQ(done.load(), 1);
    std::vector<float> back(nk * width);
    plane->Memcpy(back.data(), dout, nk * width * 4);
    const float want = 0.5f * W * (W + 1);
    for (size_t i = 0; i < back.size(); ++i) CHECK_EQ(back[i], want) << "at " << i;
    skv.Wait(skv.ZPush(sk, sv));                       // push only
    skv.Wait(skv.ZPull(sk, &so));                      // pull only
    plane->Memcpy(back.data(), dout, nk * width * 4);
    for (size_t i = 0; i < back.size(); ++i) CHECK_EQ(back[i], 2 * want) << "at " << i;
    CHECK(&sp == plane->FindSparse(kApp));
  }

  // 7. keyed requests with per-key lengths: key i carries 1 + i % 3 elements, packed back to
  // back.  A push names the lengths; a pull-only request learns them from the owners and gets
  // values and lengths back.
  {
    const int kApp = 4, width = 3;
    const int64_t nk = 3000;
    const uint64_t key_space = 1u << 18;
    plane->DeclareSparse(kApp, key_space, nk, width, /*sum*/ 0, 0.f, 0.f, 0.f, 0.f, 0.f,
                         /*var_len=*/true);
    KVWorker<float> skv(kApp, 2);
    std::vector<Key> hkeys(nk);
    std::vector<int> hlens(nk);
    int64_t total = 0;
    for (int64_t i = 0; i < nk; ++i) {
      hkeys[i] = static_cast<Key>(i) * (key_space / nk) + 3;
      hlens[i] = 1 + static_cast<int>(i % 3);
      total += hlens[i];
    }
    std::vector<float> hvals(total);
    for (int64_t i = 0, o = 0; i < nk; ++i)
      for (int j = 0; j < hlens[i]; ++j) hvals[o++] = static_cast<float>((R + 1) * (j + 1));
    const int64_t koff = plane->Alloc(nk * 8), voff = plane->Alloc(total * 4),
                  ooff = plane->Alloc(nk * width * 4), loff = plane->Alloc(nk * 4),
                  l2off = plane->Alloc(nk * 4);
    CHECK(koff >= 0 && voff >= 0 && ooff >= 0 && loff >= 0 && l2off >= 0);
    Key* dkeys = static_cast<Key*>(plane->Local(koff));
    float* dvals = static_cast<float*>(plane->Local(voff));
    float* dout = static_cast<float*>(plane->Local(ooff));
    int* dlens = static_cast<int*>(plane->Local(loff));
    int* dlens_back = static_cast<int*>(plane->Local(l2off));
    plane->Memcpy(dkeys, hkeys.data(), nk * 8);
    plane->Memcpy(dvals, hvals.data(), total * 4);
    plane->Memcpy(dlens, hlens.data(), nk * 4);
    SArray<Key> sk = SArray<Key>::FromDevice(dkeys, nk);
    SArray<float> sv = SArray<float>::FromDevice(dvals, total);
    SArray<int> sl = SArray<int>::FromDevice(dlens, nk);
    skv.Wait(skv.ZPush(sk, sv, sl));
    // pull only: the caller sizes the output for the widest case and names no lengths
    SArray<float> so = SArray<float>::FromDevice(dout, nk * width);
    SArray<int> slb = SArray<int>::FromDevice(dlens_back, nk);
    skv.Wait(skv.ZPull(sk, &so, &slb));
    std::vector<int> lens_back(nk);
    std::vector<float> back(total);
    plane->Memcpy(lens_back.data(), dlens_back, nk * 4);
    plane->Memcpy(back.data(), dout, total * 4);
    const float tri = 0.5f * W * (W + 1);
    for (int64_t i = 0, o = 0; i < nk; ++i) {
      CHECK_EQ(lens_back[i], hlens[i]) << "length of key " << i;
      for (int j = 0; j < hlens[i]; ++j, ++o) CHECK_EQ(back[o], tri * (j + 1)) << "key " << i;
    }
    // push + pull in one request, lengths named
    SArray<float> so2 = SArray<float>::FromDevice(dout, total);
    skv.Wait(skv.ZPushPull(sk, sv, &so2, &sl));
    plane->Memcpy(back.data(), dout, total * 4);
    for (int64_t i = 0, o = 0; i < nk; ++i)
      for (int j = 0; j < hlens[i]; ++j, ++o) CHECK_EQ(back[o], 2 * tri * (j + 1)) << "key " << i;
  }

  // 8. keyed table with the FTRL-proximal handle (three numbers per value, kept side by side):
  // every worker pushes gradient 1 for the same keys; from zero state the summed gradient W gives
  // z = W, n = W^2 and w = -(z - l1) / ((beta + sqrt(n)) / alpha + l2).
  {
    const int kApp = 5, width = 2;
    const int64_t nk = 1000;
    const uint64_t key_space = 1u << 16;
    const float alpha = 0.1f, beta = 1.f, l1 = 0.5f, l2 = 0.1f;
    plane->DeclareSparse(kApp, key_space, nk, width, /*ftrl*/ 2, 0.f, alpha, beta, l1, l2);
    KVWorker<float> skv(kApp, 3);
    std::vector<Key> hkeys(nk);
    for (int64_t i = 0; i < nk; ++i) hkeys[i] = static_cast<Key>(i) * (key_space / nk) + 1;
    std::vector<float> hvals(nk * width, 1.f);
    const int64_t koff = plane->Alloc(nk * 8), voff = plane->Alloc(nk * width * 4),
                  ooff = plane->Alloc(nk * width * 4);
    CHECK(koff >= 0 && voff >= 0 && ooff >= 0);
    Key* dkeys = static_cast<Key*>(plane->Local(koff));
    float* dvals = static_cast<float*>(plane->Local(voff));
    float* dout = static_cast<float*>(plane->Local(ooff));
    plane->Memcpy(dkeys, hkeys.data(), nk * 8);
    plane->Memcpy(dvals, hvals.data(), nk * width * 4);
    SArray<Key> sk = SArray<Key>::FromDevice(dkeys, nk);
    SArray<float> sv = SArray<float>::FromDevice(dvals, nk * width);
    SArray<float> so = SArray<float>::FromDevice(dout, nk * width);
    skv.Wait(skv.ZPushPull(sk, sv, &so));
    std::vector<float> back(nk * width);
    plane->Memcpy(back.data(), dout, nk * width * 4);
    const float g = static_cast<float>(W);
    const float want = -(g - l1) / ((beta + std::sqrt(g * g)) / alpha + l2);
    for (size_t i = 0; i < back.size(); ++i)
      CHECK_LT(std::fabs(back[i] - want), 1e-6f) << "at " << i << ": " << back[i] << " vs " << want;
  }

  CHECK_GT(plane->launches(), (uint64_t)0);
  LOG(INFO) << "DEVICE_PLANE_OK rank " << R << " of " << W << " backend " << plane->backend();
  plane->Stop();
  Finalize(0, true);
  return 0;
}
