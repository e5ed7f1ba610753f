#include "van/nvl_host_sim.h"

#include <sched.h>

#include <chrono>
#include <cmath>
#include <cstring>

#include "ps/device/ctrl_layout.h"

namespace ps {
namespace device {
namespace sim {
namespace {

inline psdev_ctrl_t* CtrlOf(void* base) { return static_cast<psdev_ctrl_t*>(base); }

inline float Bf16ToF32(uint16_t h) {
  uint32_t u = static_cast<uint32_t>(h) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
inline uint16_t F32ToBf16(float f) {  // round to nearest even, like __float2bfloat16_rn
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return static_cast<uint16_t>(u >> 16);
}

bool WaitGe(const unsigned long long* flag, unsigned long long want, uint64_t timeout_ns) {
  const auto t0 = std::chrono::steady_clock::now();
  for (unsigned spin = 0;; ++spin) {
    if (__atomic_load_n(flag, __ATOMIC_ACQUIRE) >= want) return true;
    if ((spin & 63) == 63) {
      const auto dt = std::chrono::steady_clock::now() - t0;
      if (static_cast<uint64_t>(
              std::chrono::duration_cast<std::chrono::nanoseconds>(dt).count()) > timeout_ns)
        return false;
      sched_yield();
    }
  }
}

void Fail(psdev_ctrl_t* my, int channel, int code, int late_rank) {
  __atomic_fetch_or(&my->late_mask[channel], 1u << late_rank, __ATOMIC_RELAXED);
  int cur = __atomic_load_n(&my->status[channel], __ATOMIC_RELAXED);
  while (code < cur &&
         !__atomic_compare_exchange_n(&my->status[channel], &cur, code, false, __ATOMIC_RELAXED,
                                      __ATOMIC_RELAXED)) {
  }
}

void Apply(const psdev_opt_t& o, float& w, float g, float* m, float* v) {
  switch (o.kind) {
    case PSDEV_OPT_SUM: w += g; break;
    case PSDEV_OPT_ASSIGN: w = g; break;
    case PSDEV_OPT_SGD:
      g = std::fma(o.weight_decay, w, g);
      w = std::fma(-o.lr, g, w);
      break;
    case PSDEV_OPT_MOMENTUM:
      g = std::fma(o.weight_decay, w, g);
      *m = std::fma(o.momentum, *m, g);
      w = std::fma(-o.lr, *m, w);
      break;
    case PSDEV_OPT_ADAM: {
      if (o.decoupled_wd) w *= (1.f - o.lr * o.weight_decay);
      else g = std::fma(o.weight_decay, w, g);
      *m = std::fma(o.beta1, *m, (1.f - o.beta1) * g);
      *v = std::fma(o.beta2, *v, (1.f - o.beta2) * g * g);
      const float denom = std::sqrt(*v) / o.bias2 + o.eps;
      w -= (o.lr / o.bias1) * (*m / denom);
      break;
    }
    default: break;
  }
}

}  // namespace

int DenseOp(const psdev_world_t* w, const psdev_table_t* t, int op, int64_t begin, int64_t end,
            const psdev_opt_t* opt, int channel, uint64_t timeout_ns, int sync) {
  if (!w || !t || !opt || w->world < 1 || w->world > PSDEV_MAX_RANKS || channel < 0 ||
      channel >= PSDEV_NUM_CHANNELS || begin < 0 || end > t->n || begin > end || t->blk <= 0)
    return PSDEV_ERR_ARG;
  if (t->grad_dtype == PSDEV_I8) return PSDEV_ERR_UNSUPPORTED;
  const int W = w->world, R = w->rank;
  psdev_ctrl_t* my = CtrlOf(w->peer_base[R]);
  unsigned long long e = 1;
  bool ok = true;
  if ((sync & 1) && __atomic_load_n(&my->status[channel], __ATOMIC_RELAXED) != 0) {
    ok = false;  // out of service until the status has been cleared
  } else if (sync & 1) {
    e = my->epoch[channel] + 1ull;
    for (int p = 0; p < W; ++p)
      __atomic_store_n(&CtrlOf(w->peer_base[p])->flag_in[channel][R], e, __ATOMIC_RELEASE);
    for (int p = 0; p < W; ++p) {
      if (!WaitGe(&my->flag_in[channel][p], e, timeout_ns)) {
        Fail(my, channel, PSDEV_ERR_TIMEOUT_ENTRY, p);
        ok = false;
      }
    }
  }
  const bool reduce = (op & PSDEV_OP_PUSH) != 0;
  const bool bcast = (op & PSDEV_OP_PULL) != 0;
  const bool publish = (op & PSDEV_OP_PUBLISH) != 0;
  if (ok) {
    for (int64_t j = R; j * t->blk < end; j += W) {
      int64_t lo = j * t->blk, hi = lo + t->blk;
      if (hi <= begin) continue;
      if (lo < begin) lo = begin;
      if (hi > end) hi = end;
      const int64_t st_base = (j / W) * t->blk - j * t->blk;
      for (int64_t i = lo; i < hi; ++i) {
        const int64_t si = st_base + i;
        float wv = t->master[si];
        if (reduce) {
          float g = 0.f;
          for (int p = 0; p < W; ++p) {
            const char* gb = static_cast<const char*>(w->peer_base[p]) + t->grad_off;
            g += t->grad_dtype == PSDEV_F32 ? reinterpret_cast<const float*>(gb)[i]
                                            : Bf16ToF32(reinterpret_cast<const uint16_t*>(gb)[i]);
          }
          float* m = t->state1 ? t->state1 + si : nullptr;
          float* v = t->state2 ? t->state2 + si : nullptr;
          float zero1 = 0.f, zero2 = 0.f;
          Apply(*opt, wv, g * opt->scale, m ? m : &zero1, v ? v : &zero2);
          t->master[si] = wv;
        }
        if (bcast || publish) {
          for (int pp = 0; pp < W; ++pp) {
            const int p = (R + pp) % W;
            if (!bcast && p != R) continue;
            char* wb = static_cast<char*>(w->peer_base[p]) + t->weight_off;
            if (t->out_dtype == PSDEV_F32) reinterpret_cast<float*>(wb)[i] = wv;
            else reinterpret_cast<uint16_t*>(wb)[i] = F32ToBf16(wv);
          }
        }
      }
    }
  }
  if (sync & 1) {
    const bool healthy = ok && __atomic_load_n(&my->status[channel], __ATOMIC_RELAXED) == 0;
    if (healthy) {
      for (int p = 0; p < W; ++p)
        __atomic_store_n(&CtrlOf(w->peer_base[p])->flag_out[channel][R], e, __ATOMIC_RELEASE);
      for (int p = 0; p < W; ++p) {
        if (!WaitGe(&my->flag_out[channel][p], e, timeout_ns))
          Fail(my, channel, PSDEV_ERR_TIMEOUT_EXIT, p);
      }
    }
    if (ok) my->epoch[channel] = e;
  }
  return 0;
}

int ChannelStatus(void* local_base, int channel, int32_t* status, uint64_t* epoch) {
  if (!local_base || channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  psdev_ctrl_t* c = CtrlOf(local_base);
  if (status) *status = __atomic_load_n(&c->status[channel], __ATOMIC_ACQUIRE);
  if (epoch) *epoch = c->epoch[channel];
  return 0;
}

int ChannelClear(void* local_base, int channel) {
  if (!local_base || channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  psdev_ctrl_t* c = CtrlOf(local_base);
  c->status[channel] = 0;
  c->late_mask[channel] = 0;
  return 0;
}

}  // namespace sim
}  // namespace device
}  // namespace ps
