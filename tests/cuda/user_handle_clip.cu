// Example of a user-defined server handle on the device: SGD on a clipped gradient.
//
//     g <- clamp(scale * sum over workers, -c, +c),   w <- w - lr * g,   c = opt.user[0]
//
// Built by tests/test_user_handle_gpu.py into a shared object that links libpsb200_device.so;
// loading the object registers the handle as kind 100.  This is the device form of installing
// a request handle on a KVServer (reference: include/ps/kv_app.h:414-420).
#include "ps/device/user_handle.cuh"

struct ClippedSgd {
  static constexpr int kStates = 0;
  __device__ static __forceinline__ void apply(float& w, float g, float&, float&,
                                               const psdev_opt_t& o) {
    const float c = o.user[0];
    g = fminf(fmaxf(g, -c), c);
    w = fmaf(-o.lr, g, w);
  }
};

PSDEV_REGISTER_DENSE_HANDLE(100, ClippedSgd)
