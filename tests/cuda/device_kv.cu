// GPU test of DeviceKVWorker (include/ps/device/kv_device.h): timestamps, callbacks, Wait,
// and the error path when a peer never arrives (a flag that nothing sets).
#include <atomic>
#include <cstdio>
#include <vector>

#include "ps/device/kv_device.h"

#define CK(x)                                                           \
  do {                                                                  \
    auto _e = (x);                                                      \
    if (_e != 0) {                                                      \
      printf("FAILED %s = %d line %d\n", #x, (int)_e, __LINE__);        \
      return 1;                                                         \
    }                                                                   \
  } while (0)

int main() {
  const int64_t n = 1 << 16;
  void *heap0 = nullptr, *heap1 = nullptr;
  CK(psdev_heap_create(4 << 20, &heap0, nullptr));
  CK(psdev_heap_create(4 << 20, &heap1, nullptr));
  float *master = nullptr;
  CK(cudaMalloc(&master, n * sizeof(float)));
  CK(cudaMemset(master, 0, n * sizeof(float)));
  psdev_table_t t{};
  t.grad_off = PSDEV_CTRL_BYTES;
  t.weight_off = PSDEV_CTRL_BYTES + n * sizeof(float);
  t.n = n;
  t.blk = n;
  t.master = master;
  t.grad_dtype = PSDEV_F32;
  t.out_dtype = PSDEV_F32;
  psdev_opt_t opt{};
  opt.kind = PSDEV_OPT_SUM;
  opt.scale = 1.f;
  std::vector<float> ones(n, 1.f);
  CK(cudaMemcpy((char*)heap0 + t.grad_off, ones.data(), n * sizeof(float), cudaMemcpyHostToDevice));
  cudaStream_t s;
  CK(cudaStreamCreate(&s));
  {
    psdev_world_t w{};
    w.rank = 0;
    w.world = 1;
    w.peer_base[0] = heap0;
    ps::DeviceKVWorker kv(w, t, opt, /*channel=*/2);
    std::atomic<int> cbs{0};
    std::vector<int> ts;
    for (int i = 0; i < 3; ++i) ts.push_back(kv.PushPull(0, n, s, [&cbs] { ++cbs; }));
    if (ts[0] != 0 || ts[2] != 2) { printf("FAILED timestamps\n"); return 1; }
    kv.Wait(ts[2]);
    if (cbs.load() != 3) { printf("FAILED callbacks %d\n", cbs.load()); return 1; }
    std::vector<float> out(n);
    CK(cudaMemcpy(out.data(), (char*)heap0 + t.weight_off, n * sizeof(float),
                  cudaMemcpyDeviceToHost));
    for (int64_t i = 0; i < n; ++i)
      if (out[i] != 3.f) { printf("FAILED value %f at %lld\n", out[i], (long long)i); return 1; }
    kv.Wait(kv.Pull(0, n, s));
  }
  {
    // two ranks, but only rank 0 ever launches: its wait for rank 1 must run out
    psdev_world_t w{};
    w.rank = 0;
    w.world = 2;
    w.peer_base[0] = heap0;
    w.peer_base[1] = heap1;
    ps::DeviceKVWorker kv(w, t, opt, /*channel=*/5, /*timeout_ns=*/200000000ull);
    bool threw = false;
    try {
      kv.Wait(kv.PushPull(0, n, s));
    } catch (const ps::Error&) {
      threw = true;
    }
    if (!threw) { printf("FAILED: no error after a peer never arrived\n"); return 1; }
  }
  printf("DEVICE_KV_OK\n");
  return 0;
}
