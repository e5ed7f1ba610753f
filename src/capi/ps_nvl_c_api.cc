#include "capi/ps_nvl_c_api.h"

#include <cstring>
#include <string>

#include "capi/ps_c_api.h"
#include "ps/device/plane.h"
#include "ps/ps.h"

using namespace ps;
using ps::device::Plane;

// error text shared with ps_c_api.cc
extern "C" void ps_capi_set_error(const char* text);

namespace {
template <typename F>
auto Guard(F&& f) -> decltype(f()) {
  try {
    return f();
  } catch (const std::exception& e) {
    ps_capi_set_error(e.what());
    return static_cast<decltype(f())>(-1);
  }
}
}  // namespace

extern "C" {

int psnvl_start(uint64_t heap_bytes, int device, const char* backend, int multicast,
                const char* device_lib, uint64_t slice_bytes, uint64_t timeout_ns) {
  return Guard([&] {
    device::PlaneOptions o;
    o.heap_bytes = heap_bytes;
    o.device = device;
    if (backend && *backend) o.backend = backend;
    o.multicast = multicast;
    if (device_lib) o.device_lib = device_lib;
    if (slice_bytes) o.slice_bytes = slice_bytes;
    if (timeout_ns) o.timeout_ns = timeout_ns;
    Plane::Get()->Start(o);
    return 0;
  });
}
int psnvl_stop(void) {
  return Guard([] {
    Plane::Get()->Stop();
    return 0;
  });
}
int psnvl_started(void) { return Plane::Get()->started() ? 1 : 0; }
int psnvl_rank(void) { return Plane::Get()->rank(); }
int psnvl_world(void) { return Plane::Get()->world(); }
int psnvl_world_struct(psdev_world_t* out) {
  *out = Plane::Get()->world_struct();
  return 0;
}
const char* psnvl_backend(void) { return Plane::Get()->backend().c_str(); }
int psnvl_barrier(void) {
  return Guard([] {
    Plane::Get()->Barrier();
    return 0;
  });
}
long psnvl_allgather(const void* mine, size_t n, void* out, size_t cap, size_t* sizes) {
  return Guard([&]() -> long {
    const auto all = Plane::Get()->AllGather(std::string(static_cast<const char*>(mine), n));
    size_t total = 0;
    for (const auto& s : all) total += s.size();
    if (total <= cap) {
      char* at = static_cast<char*>(out);
      for (size_t r = 0; r < all.size(); ++r) {
        memcpy(at, all[r].data(), all[r].size());
        at += all[r].size();
      }
    }
    for (size_t r = 0; r < all.size(); ++r) sizes[r] = all[r].size();
    return static_cast<long>(total);
  });
}
int64_t psnvl_alloc(uint64_t bytes, uint64_t align) {
  return Guard([&]() -> int64_t { return Plane::Get()->Alloc(bytes, align ? align : 256); });
}
int psnvl_free(int64_t offset) {
  return Guard([&] {
    Plane::Get()->Free(offset);
    return 0;
  });
}
uint64_t psnvl_heap_in_use(void) { return Plane::Get()->heap_in_use(); }
int psnvl_new_channel(void) {
  return Guard([] { return Plane::Get()->NewChannel(); });
}
int psnvl_register_dense(int app_id, uint64_t tensor_id, int64_t n_user, const psdev_table_t* t,
                         const psdev_opt_t* opt, int channel, int nvls, int num_ctas) {
  return Guard([&] {
    Plane::Get()->RegisterDense(app_id, tensor_id, n_user, *t, *opt, channel, nvls != 0, num_ctas);
    return 0;
  });
}
int psnvl_unregister_dense(int app_id, uint64_t tensor_id) {
  return Guard([&] {
    Plane::Get()->UnregisterDense(app_id, tensor_id);
    return 0;
  });
}
int psnvl_set_optimizer(int app_id, uint64_t tensor_id, const psdev_opt_t* opt) {
  return Guard([&] {
    Plane::Get()->SetOptimizer(app_id, tensor_id, *opt);
    return 0;
  });
}
int psnvl_dense_keys(uint64_t tensor_id, uint64_t* keys) {
  return Guard([&] {
    const auto k = Plane::Get()->DenseKeys(tensor_id);
    for (size_t i = 0; i < k.size(); ++i) keys[i] = k[i];
    return static_cast<int>(k.size());
  });
}
int psnvl_set_stream(void* stream) {
  Plane::Get()->SetStream(stream);
  return 0;
}
int psnvl_set_slice_bytes(uint64_t bytes) {
  return Guard([&] {
    Plane::Get()->SetSliceBytes(bytes);
    return 0;
  });
}
int psnvl_clear_status(int app_id, uint64_t tensor_id) {
  return Guard([&] {
    Plane::Get()->ClearStatus(app_id, tensor_id);
    return 0;
  });
}
uint64_t psnvl_launches(void) { return Plane::Get()->launches(); }
int psnvl_drain(void) {
  return Guard([&] {
    Plane::Get()->Drain();
    return 0;
  });
}

// ---- byte worker ----
void* ps_capi_bworker_new(int app_id, int customer_id) {
  try {
    return new KVWorker<char>(app_id, customer_id);
  } catch (const std::exception& e) {
    ps_capi_set_error(e.what());
    return nullptr;
  }
}
int ps_capi_bworker_delete(void* worker) {
  return Guard([&] {
    delete static_cast<KVWorker<char>*>(worker);
    return 0;
  });
}
int ps_capi_bworker_request(void* worker, int push, int pull, const uint64_t* keys, size_t nkeys,
                            const void* vals, size_t vals_bytes, void* outs, size_t outs_bytes,
                            int cmd, int priority) {
  return Guard([&] {
    auto* kv = static_cast<KVWorker<char>*>(worker);
    SArray<Key> k;
    k.CopyFrom(reinterpret_cast<const Key*>(keys), nkeys);  // a handful of keys per tensor
    SArray<char> v(const_cast<char*>(static_cast<const char*>(vals)), vals_bytes, false);
    if (push && pull) {
      // the output view lives until the request has completed
      auto* o = new SArray<char>(static_cast<char*>(outs), outs_bytes, false);
      return kv->ZPushPull(k, v, o, nullptr, cmd, [o]() { delete o; }, priority);
    }
    if (push) return kv->ZPush(k, v, {}, cmd, nullptr, priority);
    auto* o = new SArray<char>(static_cast<char*>(outs), outs_bytes, false);
    return kv->ZPull(k, o, nullptr, cmd, [o]() { delete o; }, priority);
  });
}
int ps_capi_bworker_wait(void* worker, int timestamp) {
  return Guard([&] {
    static_cast<KVWorker<char>*>(worker)->Wait(timestamp);
    return 0;
  });
}

int psnvl_declare_sparse(int app_id, uint64_t key_space, int64_t max_keys, int width, int kind,
                         float lr, float alpha, float beta, float l1, float l2, int var_len) {
  return Guard([&] {
    Plane::Get()->DeclareSparse(app_id, key_space, max_keys, width, kind, lr, alpha, beta, l1, l2,
                                var_len != 0);
    return 0;
  });
}

int ps_capi_bworker_keyed_request(void* worker, int push, int pull, const uint64_t* keys_dev,
                                  size_t nkeys, const void* vals_dev, size_t vals_bytes,
                                  void* outs_dev, size_t outs_bytes, const int* lens_dev,
                                  int* lens_out_dev, int cmd) {
  return Guard([&] {
    auto* kv = static_cast<KVWorker<char>*>(worker);
    SArray<Key> k = SArray<Key>::FromDevice(
        const_cast<Key*>(reinterpret_cast<const Key*>(keys_dev)), nkeys);
    SArray<char> v = SArray<char>::FromDevice(
        const_cast<char*>(static_cast<const char*>(vals_dev)), vals_bytes);
    SArray<int> l;
    if (lens_dev) l = SArray<int>::FromDevice(const_cast<int*>(lens_dev), nkeys);
    if (push && !pull) return kv->ZPush(k, v, l, cmd);
    // output views live until the request has completed
    auto* o = new SArray<char>(SArray<char>::FromDevice(static_cast<char*>(outs_dev), outs_bytes));
    if (push) {
      auto* lp = lens_dev ? new SArray<int>(l) : nullptr;
      return kv->ZPushPull(k, v, o, lp, cmd, [o, lp]() { delete o; delete lp; });
    }
    auto* lo = lens_out_dev ? new SArray<int>(SArray<int>::FromDevice(lens_out_dev, nkeys))
                            : nullptr;
    return kv->ZPull(k, o, lo, cmd, [o, lo]() { delete o; delete lo; });
  });
}

}  // extern "C"
