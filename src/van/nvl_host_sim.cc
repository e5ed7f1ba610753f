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

// ---- keyed tables ------------------------------------------------------------------------------
namespace {

// First half of a rendezvous: announce this rank, wait for every rank.  Returns the epoch of the
// round, or 0 when the channel is out of service or a rank did not arrive.
unsigned long long Enter(const psdev_world_t* w, int channel, uint64_t timeout_ns) {
  const int W = w->world, R = w->rank;
  psdev_ctrl_t* my = CtrlOf(w->peer_base[R]);
  if (__atomic_load_n(&my->status[channel], __ATOMIC_RELAXED) != 0) return 0;
  const unsigned long long e = my->epoch[channel] + 1ull;
  for (int p = 0; p < W; ++p)
    __atomic_store_n(&CtrlOf(w->peer_base[p])->flag_in[channel][R], e, __ATOMIC_RELEASE);
  bool ok = true;
  for (int p = 0; p < W; ++p) {
    if (!WaitGe(&my->flag_in[channel][p], e, timeout_ns)) {
      Fail(my, channel, PSDEV_ERR_TIMEOUT_ENTRY, p);
      ok = false;
    }
  }
  return ok ? e : 0;
}

// Second half: announce that this rank is done, wait for every rank, advance the epoch.
void Leave(const psdev_world_t* w, int channel, uint64_t timeout_ns, unsigned long long e) {
  const int W = w->world, R = w->rank;
  psdev_ctrl_t* my = CtrlOf(w->peer_base[R]);
  if (e == 0 || __atomic_load_n(&my->status[channel], __ATOMIC_RELAXED) != 0) return;
  for (int p = 0; p < W; ++p)
    __atomic_store_n(&CtrlOf(w->peer_base[p])->flag_out[channel][R], e, __ATOMIC_RELEASE);
  for (int p = 0; p < W; ++p) {
    if (!WaitGe(&my->flag_out[channel][p], e, timeout_ns))
      Fail(my, channel, PSDEV_ERR_TIMEOUT_EXIT, p);
  }
  my->epoch[channel] = e;
}

inline char* Heap(const psdev_world_t* w, int rank) {
  return static_cast<char*>(w->peer_base[rank]);
}

bool SparseOk(const psdev_world_t* w, const psdev_sparse_t* t) {
  return w && t && w->world >= 1 && w->world <= PSDEV_MAX_RANKS && t->range != 0 && t->w &&
         t->capacity == 0 && t->width >= 1 && t->channel >= 0 &&
         t->channel < PSDEV_NUM_CHANNELS && (t->kind != 2 || (t->z && t->n)) &&
         (t->lens_off == 0 || (t->offs_off != 0 && t->klen));
}

// Length and value offset of request entry i of worker r.
void ValueSpan(const psdev_world_t* w, const psdev_sparse_t* t, int r, int64_t i, int64_t* off,
               int* len) {
  if (t->lens_off == 0) {
    *off = i * t->width;
    *len = t->width;
    return;
  }
  int l = reinterpret_cast<const int32_t*>(Heap(w, r) + t->lens_off)[i];
  if (l < 0) l = 0;
  if (l > t->width) l = t->width;
  *off = reinterpret_cast<const int64_t*>(Heap(w, r) + t->offs_off)[i];
  *len = l;
}

void AtomicAddF32(float* p, float v) {
  uint32_t* u = reinterpret_cast<uint32_t*>(p);
  uint32_t cur = __atomic_load_n(u, __ATOMIC_RELAXED);
  for (;;) {
    float f;
    memcpy(&f, &cur, 4);
    f += v;
    uint32_t want;
    memcpy(&want, &f, 4);
    if (__atomic_compare_exchange_n(u, &cur, want, false, __ATOMIC_RELAXED, __ATOMIC_RELAXED))
      return;
  }
}

uint64_t TimeoutOf(const psdev_sparse_t* t) {
  return t->timeout_ns ? t->timeout_ns : 20000000000ull;
}

}  // namespace

int KeyShardLookup(const uint64_t* keys, int64_t n, uint64_t range, int world, int64_t* pos) {
  if (world < 1 || world > PSDEV_MAX_RANKS || range == 0 || !pos || (n > 0 && !keys))
    return PSDEV_ERR_ARG;
  for (int s = 0; s <= world; ++s) {
    const uint64_t bound = range * static_cast<uint64_t>(s);
    int64_t lo = 0, hi = n;
    while (lo < hi) {
      const int64_t m = (lo + hi) >> 1;
      if (keys[m] < bound) lo = m + 1; else hi = m;
    }
    pos[s] = lo;
  }
  pos[world + 1] = n;
  return 0;
}

int LensToOffsets(const int32_t* lens, int64_t n, int64_t* offs) {
  if (!lens || !offs || n < 0) return PSDEV_ERR_ARG;
  int64_t run = 0;
  for (int64_t i = 0; i < n; ++i) {
    offs[i] = run;
    run += lens[i] > 0 ? lens[i] : 0;
  }
  offs[n] = run;
  return 0;
}

int SparseScatter(const psdev_world_t* w, const psdev_sparse_t* t, int64_t n) {
  if (!SparseOk(w, t) || n < 0 || n > t->max_n) return PSDEV_ERR_ARG;
  const int W = w->world, R = w->rank;
  char* mine = Heap(w, R);
  const uint64_t* keys = reinterpret_cast<const uint64_t*>(mine + t->keys_off);
  if (t->lens_off)
    LensToOffsets(reinterpret_cast<const int32_t*>(mine + t->lens_off), n,
                  reinterpret_cast<int64_t*>(mine + t->offs_off));
  KeyShardLookup(keys, n, t->range, W, reinterpret_cast<int64_t*>(mine + t->pos_off));
  const float* grads = reinterpret_cast<const float*>(mine + t->grads_off);
  for (int64_t i = 0; i < n; ++i) {
    const uint64_t s = keys[i] / t->range;
    if (s >= static_cast<uint64_t>(W)) continue;  // outside every range: dropped
    const int64_t idx = static_cast<int64_t>(keys[i] - s * t->range);
    if (idx >= t->slots) continue;
    int64_t off;
    int len;
    ValueSpan(w, t, R, i, &off, &len);
    if (off < 0 || off + len > t->max_vals) continue;
    float* acc = reinterpret_cast<float*>(Heap(w, static_cast<int>(s)) + t->acc_off);
    for (int j = 0; j < len; ++j) AtomicAddF32(acc + idx * t->width + j, grads[off + j]);
  }
  // the cut points and the additions are visible before this rank announces itself
  __atomic_thread_fence(__ATOMIC_RELEASE);
  return 0;
}

int SparseApply(const psdev_world_t* w, const psdev_sparse_t* t, int sync) {
  if (!SparseOk(w, t)) return PSDEV_ERR_ARG;
  const int W = w->world, R = w->rank;
  if (sync && Enter(w, t->channel, TimeoutOf(t)) == 0) return 0;
  float* acc = reinterpret_cast<float*>(Heap(w, R) + t->acc_off);
  for (int r = 0; r < W; ++r) {
    const int64_t* pos = reinterpret_cast<const int64_t*>(Heap(w, r) + t->pos_off);
    const int64_t lo = pos[R], hi = pos[R + 1];
    if (lo < 0 || hi < lo || hi > t->max_n) continue;
    const uint64_t* keys = reinterpret_cast<const uint64_t*>(Heap(w, r) + t->keys_off);
    for (int64_t i = lo; i < hi; ++i) {
      const int64_t idx = static_cast<int64_t>(keys[i] - static_cast<uint64_t>(R) * t->range);
      if (idx < 0 || idx >= t->slots) continue;
      if (t->klen && t->lens_off) {
        int64_t off;
        int len;
        ValueSpan(w, t, r, i, &off, &len);
        if (len > 0) t->klen[idx] = len;
      }
      const int64_t stride = t->state_stride > 1 ? t->state_stride : 1;
      for (int j = 0; j < t->width; ++j) {
        const int64_t ea = idx * t->width + j;
        const float g = acc[ea];
        if (g == 0.f) continue;  // applied for another worker already, or nothing pushed
        acc[ea] = 0.f;
        const int64_t el = ea * stride;  // the value's place in the state arrays
        if (t->kind == 0) {
          t->w[el] += g;
        } else if (t->kind == 1) {
          t->w[el] -= t->lr * g;
        } else {
          const float wv = t->w[el], nv = t->n[el];
          const float n2 = nv + g * g;
          const float sigma = (std::sqrt(n2) - std::sqrt(nv)) / t->alpha;
          const float z = t->z[el] + g - sigma * wv;
          t->z[el] = z;
          t->n[el] = n2;
          if (std::fabs(z) <= t->l1) {
            t->w[el] = 0.f;
          } else {
            const float sgn = z > 0.f ? 1.f : -1.f;
            t->w[el] = -(z - sgn * t->l1) / ((t->beta + std::sqrt(n2)) / t->alpha + t->l2);
          }
        }
      }
    }
  }
  return 0;
}

int SparseRespond(const psdev_world_t* w, const psdev_sparse_t* t, int sync) {
  if (!SparseOk(w, t)) return PSDEV_ERR_ARG;
  const int W = w->world, R = w->rank;
  psdev_ctrl_t* my = CtrlOf(w->peer_base[R]);
  const bool healthy = !sync || __atomic_load_n(&my->status[t->channel], __ATOMIC_RELAXED) == 0;
  const int64_t stride = t->state_stride > 1 ? t->state_stride : 1;
  if (healthy) {
    for (int rr = 0; rr < W; ++rr) {
      const int r = (R + rr) % W;
      const int64_t* pos = reinterpret_cast<const int64_t*>(Heap(w, r) + t->pos_off);
      const int64_t lo = pos[R], hi = pos[R + 1];
      if (lo < 0 || hi < lo || hi > t->max_n) continue;
      const uint64_t* keys = reinterpret_cast<const uint64_t*>(Heap(w, r) + t->keys_off);
      float* out = reinterpret_cast<float*>(Heap(w, r) + t->out_off);
      for (int64_t i = lo; i < hi; ++i) {
        int64_t off;
        int len;
        ValueSpan(w, t, r, i, &off, &len);
        if (off < 0 || off + len > t->max_vals) continue;
        const int64_t idx = static_cast<int64_t>(keys[i] - static_cast<uint64_t>(R) * t->range);
        for (int j = 0; j < len; ++j)
          out[off + j] = (idx >= 0 && idx < t->slots) ? t->w[(idx * t->width + j) * stride] : 0.f;
      }
    }
  }
  if (sync) {
    // the round that the apply call entered: one ahead of the last completed one
    const unsigned long long e = healthy ? my->epoch[t->channel] + 1ull : 0ull;
    Leave(w, t->channel, TimeoutOf(t), e);
  }
  return 0;
}

int SparseLens(const psdev_world_t* w, const psdev_sparse_t* t) {
  if (!SparseOk(w, t) || !t->lens_off || !t->klen) return PSDEV_ERR_ARG;
  const int W = w->world, R = w->rank;
  for (int r = 0; r < W; ++r) {
    const int64_t* pos = reinterpret_cast<const int64_t*>(Heap(w, r) + t->pos_off);
    const int64_t lo = pos[R], hi = pos[R + 1];
    if (lo < 0 || hi < lo || hi > t->max_n) continue;
    const uint64_t* keys = reinterpret_cast<const uint64_t*>(Heap(w, r) + t->keys_off);
    int32_t* lens = reinterpret_cast<int32_t*>(Heap(w, r) + t->lens_off);
    for (int64_t i = lo; i < hi; ++i) {
      const int64_t idx = static_cast<int64_t>(keys[i] - static_cast<uint64_t>(R) * t->range);
      lens[i] = (idx >= 0 && idx < t->slots) ? t->klen[idx] : 0;
    }
  }
  return 0;
}

int DeviceBarrier(const psdev_world_t* w, int channel, uint64_t timeout_ns) {
  if (!w || w->world < 1 || w->world > PSDEV_MAX_RANKS || channel < 0 ||
      channel >= PSDEV_NUM_CHANNELS)
    return PSDEV_ERR_ARG;
  Leave(w, channel, timeout_ns, Enter(w, channel, timeout_ns));
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
