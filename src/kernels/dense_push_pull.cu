// Host dispatch for the fused dense push / pull kernel (see ps/device/push_pull.cuh).
#include <cuda_runtime.h>

#include <atomic>
#include <cstdlib>

#include <map>
#include <mutex>

#include "ps/device/user_handle.cuh"

namespace psdev {
std::atomic<uint64_t> g_launches{0};
int dense_dispatch_f32_f32(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_bf16_bf16(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_bf16_f32(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_f32_bf16(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_i8_f32(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_i8_bf16(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_ll_dispatch_f32_f32(const LLArgs& a, cudaStream_t s);
int dense_ll_dispatch_bf16_bf16(const LLArgs& a, cudaStream_t s);
int dense_ll_dispatch_bf16_f32(const LLArgs& a, cudaStream_t s);
int dense_ll_dispatch_f32_bf16(const LLArgs& a, cudaStream_t s);
}  // namespace psdev

// ---- user-defined handles -------------------------------------------------------------------
namespace {
struct UserHandle {
  int num_states;
  psdev_user_dense_fn dense;
  psdev_user_ll_fn ll;
};
std::mutex g_user_mu;
std::map<int, UserHandle>& user_handles() {
  static std::map<int, UserHandle>* m = new std::map<int, UserHandle>;  // used by static ctors
  return *m;
}
bool find_user(int kind, UserHandle* out) {
  std::lock_guard<std::mutex> lk(g_user_mu);
  auto it = user_handles().find(kind);
  if (it == user_handles().end()) return false;
  *out = it->second;
  return true;
}
}  // namespace

extern "C" int psdev_register_dense_handle(int kind, int num_states, psdev_user_dense_fn dense,
                                           psdev_user_ll_fn ll) {
  if (kind < PSDEV_OPT_USER || num_states < 0 || num_states > 2 || !dense) return PSDEV_ERR_ARG;
  std::lock_guard<std::mutex> lk(g_user_mu);
  if (user_handles().count(kind)) return PSDEV_ERR_ARG;
  user_handles()[kind] = UserHandle{num_states, dense, ll};
  return 0;
}

extern "C" int psdev_handle_states(int kind) {
  switch (kind) {
    case PSDEV_OPT_SUM: case PSDEV_OPT_SGD: case PSDEV_OPT_ASSIGN: return 0;
    case PSDEV_OPT_MOMENTUM: return 1;
    case PSDEV_OPT_ADAM: return 2;
    default: break;
  }
  UserHandle h;
  return find_user(kind, &h) ? h.num_states : -1;
}

extern "C" void psdev_count_launch(void) {
  psdev::g_launches.fetch_add(1, std::memory_order_relaxed);
}

// ---- P3 slice schedule (device side) ----------------------------------------------------------
// Orders the slices of one launch by priority (highest first, ties in submission order -- the
// order of the reference's priority send queue, src/p3_van.h:40-50, with FIFO ties) and
// numbers this rank's tiles across the ordered slices, so that the CTAs of the push/pull
// kernel, which take tiles in increasing number, work on the most urgent slice first.
namespace psdev {
constexpr int kMaxSegs = 1024;

__global__ void p3_slice_schedule_kernel(const long long* segs, int nseg, long long blk, int W,
                                         int R, long long tiles_per_blk, SchedEntry* out) {
  __shared__ int order[kMaxSegs];
  __shared__ long long scan[kMaxSegs];
  const int i = threadIdx.x;
  if (i < nseg) {
    const long long pri = segs[3 * i + 2];
    int rank = 0;
    for (int j = 0; j < nseg; ++j) {
      const long long pj = segs[3 * j + 2];
      rank += (pj > pri) || (pj == pri && j < i);
    }
    order[rank] = i;
  }
  __syncthreads();
  SchedEntry e{};
  long long tiles = 0;
  if (i < nseg) {
    const int s = order[i];
    e.begin = segs[3 * s];
    e.end = segs[3 * s + 1];
    if (e.end > e.begin) {
      const long long jb = e.begin / blk, je = (e.end - 1) / blk;
      const long long first = jb + ((R - jb % W) + W) % W;
      if (first <= je) {
        e.first_owned = first;
        e.n_owned = (je - first) / W + 1;
      }
    }
    tiles = e.n_owned * tiles_per_blk;
  }
  scan[i] = tiles;
  __syncthreads();
  for (int off = 1; off < kMaxSegs; off <<= 1) {
    const long long t = i >= off ? scan[i - off] : 0;
    __syncthreads();
    scan[i] += t;
    __syncthreads();
  }
  if (i < nseg) {
    e.tile_begin = scan[i] - tiles;
    out[i] = e;
  }
  if (i == nseg - 1) {
    SchedEntry last{};
    last.tile_begin = scan[i];
    out[nseg] = last;
  }
}

void launch_p3_schedule(const long long* segs, int nseg, long long blk, int world, int rank,
                        long long tiles_per_blk, SchedEntry* out, cudaStream_t s) {
  p3_slice_schedule_kernel<<<1, kMaxSegs, 0, s>>>(segs, nseg, blk, world, rank, tiles_per_blk, out);
  g_launches.fetch_add(1, std::memory_order_relaxed);
}
}  // namespace psdev

using namespace psdev;

static int dense_op_impl(const psdev_world_t* w, const psdev_table_t* t, int op, int64_t begin,
                         int64_t end, const psdev_opt_t* opt, int channel, int num_ctas,
                         uint64_t timeout_ns, int sync, void* stream, const int64_t* segs,
                         int nseg, void* sched);

extern "C" int psdev_dense_op(const psdev_world_t* w, const psdev_table_t* t, int op,
                              int64_t begin, int64_t end, const psdev_opt_t* opt, int channel,
                              int num_ctas, uint64_t timeout_ns, int sync, void* stream) {
  return dense_op_impl(w, t, op, begin, end, opt, channel, num_ctas, timeout_ns, sync, stream,
                       nullptr, 0, nullptr);
}

// Several slices in one launch and one rendezvous.  `segs` is device memory holding nseg
// triples (begin, end, priority), begin/end multiples of 8 inside the table; `sched` is device
// scratch of psdev_sched_bytes(nseg) bytes.  The slices are consumed in priority order.
extern "C" int psdev_dense_op_multi(const psdev_world_t* w, const psdev_table_t* t, int op,
                                    const int64_t* segs, int nseg, void* sched,
                                    const psdev_opt_t* opt, int channel, int num_ctas,
                                    uint64_t timeout_ns, int sync, void* stream) {
  if (!segs || !sched || nseg < 1 || nseg > kMaxSegs) return PSDEV_ERR_ARG;
  return dense_op_impl(w, t, op, 0, t ? t->n : 0, opt, channel, num_ctas, timeout_ns, sync,
                       stream, segs, nseg, sched);
}

extern "C" size_t psdev_ll_bytes(int world, int64_t ll_cap) {
  if (world < 1 || ll_cap <= 0) return 0;
  return kLLHeaderBytes + (size_t)(world + 1) * (size_t)ll_cap * 8;
}

// PSB200_LL=0 keeps every request on the general kernel (read once).
static bool ll_enabled() {
  static const bool on = [] {
    const char* e = getenv("PSB200_LL");
    return !(e && e[0] == '0');
  }();
  return on;
}

// Whether a request of `bytes` gradient bytes should take the NVSwitch multicast path when the
// arena has a multicast alias.  Measured: with 4 ranks multicast wins up to 4 MiB (one flag-free
// reduce-load and one store per vector instead of three of each) and loses from 16 MiB up, where
// the peer path keeps both directions of every link busy (883 against 860 GB/s per GPU at 256
// MiB); with 8 ranks it wins up to 256 MiB (855 against 741) and loses at 1 GiB.
// PSB200_NVLS_MAX_BYTES overrides the limit.
extern "C" int psdev_multicast_pays(int world, uint64_t bytes) {
  static const long long env = [] {
    const char* e = getenv("PSB200_NVLS_MAX_BYTES");
    return e ? atoll(e) : -1ll;
  }();
  if (world < 2) return 0;
  const uint64_t cap = env >= 0 ? (uint64_t)env : (world > 4 ? 512ull << 20 : 4ull << 20);
  return bytes <= cap ? 1 : 0;
}

extern "C" size_t psdev_sched_bytes(int nseg) { return sizeof(SchedEntry) * (size_t)(nseg + 1); }

static int dense_op_impl(const psdev_world_t* w, const psdev_table_t* t, int op, int64_t begin,
                         int64_t end, const psdev_opt_t* opt, int channel, int num_ctas,
                         uint64_t timeout_ns, int sync, void* stream, const int64_t* segs,
                         int nseg, void* sched) {
  if (!w || !t || w->world < 1 || w->world > PSDEV_MAX_RANKS || w->rank < 0 ||
      w->rank >= w->world)
    return PSDEV_ERR_ARG;
  if (channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  if (begin < 0 || end > t->n || begin > end || (begin & 7) || (end & 7) || t->blk <= 0 ||
      (t->blk & 7))
    return PSDEV_ERR_ARG;
  if ((op & PSDEV_OP_PUSH) && !opt) return PSDEV_ERR_ARG;
  if (!t->master) return PSDEV_ERR_ARG;
  if (w->heap_bytes) {
    // every buffer of the table must lie inside the arena, behind the control region
    const uint64_t gsz = t->grad_dtype == PSDEV_F32 ? 4 : (t->grad_dtype == PSDEV_BF16 ? 2 : 1);
    const uint64_t osz = t->out_dtype == PSDEV_F32 ? 4 : 2;
    const uint64_t n = static_cast<uint64_t>(t->n);
    auto inside = [&](uint64_t off, uint64_t bytes) {
      return off >= PSDEV_CTRL_BYTES && off <= w->heap_bytes && bytes <= w->heap_bytes - off;
    };
    if (!inside(t->grad_off, n * gsz) || !inside(t->weight_off, n * osz)) return PSDEV_ERR_BOUNDS;
    if (t->grad_dtype == PSDEV_I8 &&
        !inside(t->gscale_off, (n + kInt8Group - 1) / kInt8Group * sizeof(float)))
      return PSDEV_ERR_BOUNDS;
  }
  const int W = w->world, R = w->rank;
  DenseArgs a{};
  for (int p = 0; p < W; ++p) {
    if (!w->peer_base[p]) return PSDEV_ERR_ARG;
    a.base[p] = w->peer_base[p];
  }
  a.rank = R;
  a.world = W;
  a.grad_off = t->grad_off;
  a.weight_off = t->weight_off;
  a.blk = t->blk;
  a.begin = begin;
  a.end = end;
  a.master = t->master;
  a.s1 = t->state1;
  a.s2 = t->state2;
  if (opt) a.opt = *opt;
  a.channel = channel;
  // one rank has nobody to meet: no flag round and none of the system-scope fences that go
  // with it (they are slow while copy engines are busy, which is when a staged request runs)
  a.sync = (sync & 1) && W > 1;
  a.mc_base = (sync & 2) ? w->mc_base : nullptr;  // bit 1: use the NVSwitch multicast alias
  if (op == (PSDEV_OP_PUSH | PSDEV_OP_PUBLISH)) {
    // push, and store the new values of the owned blocks into this rank's own weight
    // buffer, where a later fused pull finds them
    op = PSDEV_OP_PUSHPULL;
    a.self_only = 1;
    a.mc_base = nullptr;
  }
  a.timeout_ns = timeout_ns;
  a.heap_bytes = w->heap_bytes;
  a.n_total = t->n;
  {
    // blocks owned by this rank: j = R, R + W, ... below ceil(n / blk)
    const int64_t nblocks = (t->n + t->blk - 1) / t->blk;
    const int64_t owned = nblocks > R ? (nblocks - R + W - 1) / W : 0;
    a.local_len = owned * t->blk;
  }
#ifdef PSDEV_CHECKS
  // Test hook of the checks build: pretend that the table is shorter than it is, so that the
  // kernel's own index check has something to refuse while every address stays valid.
  if (const char* shrink = getenv("PSDEV_CHECKS_TEST_SHRINK")) {
    const long long by = atoll(shrink);
    if (by > 0 && by < a.n_total) a.n_total -= by;
  }
#endif
  a.segs_in = reinterpret_cast<const long long*>(segs);
  a.nseg = nseg;
  a.sched = static_cast<const SchedEntry*>(sched);
  // owned blocks meeting [begin, end): indices j in [jb, je] with j % W == R
  a.n_owned = 0;
  a.first_owned = 0;
  if (end > begin) {
    const int64_t jb = begin / t->blk, je = (end - 1) / t->blk;
    int64_t first = jb + ((R - jb % W) + W) % W;
    if (first <= je) {
      a.first_owned = first;
      a.n_owned = (je - first) / W + 1;
    }
  }
  const int ctas = num_ctas;
  cudaStream_t s = (cudaStream_t)stream;
  const bool gbf = t->grad_dtype == PSDEV_BF16, obf = t->out_dtype == PSDEV_BF16;
  if (op == PSDEV_OP_PUSHPULL && !a.self_only && (sync & 1) && W > 1 && nseg == 0 &&
      t->ll_cap > 0 && end - begin <= t->ll_cap && end > begin && t->grad_dtype != PSDEV_I8 &&
      ll_enabled()) {
    // small request: one sequence-numbered exchange instead of two flag rendezvous
    if (w->heap_bytes) {
      const uint64_t need = psdev_ll_bytes(W, t->ll_cap);
      if (t->ll_off < PSDEV_CTRL_BYTES || t->ll_off > w->heap_bytes ||
          need > w->heap_bytes - t->ll_off)
        return PSDEV_ERR_BOUNDS;
    }
    LLArgs l{};
    for (int p = 0; p < W; ++p) l.base[p] = a.base[p];
    l.rank = R;
    l.world = W;
    l.grad_off = t->grad_off;
    l.weight_off = t->weight_off;
    l.ll_off = t->ll_off;
    l.ll_cap = t->ll_cap;
    l.blk = t->blk;
    l.begin = begin;
    l.end = end;
    l.master = t->master;
    l.s1 = t->state1;
    l.s2 = t->state2;
    l.opt = a.opt;
    l.channel = channel;
    l.timeout_ns = timeout_ns;
    l.n_total = a.n_total;
    l.local_len = a.local_len;
    if (a.opt.kind >= PSDEV_OPT_USER) {
      UserHandle h;
      if (!find_user(a.opt.kind, &h)) return PSDEV_ERR_UNSUPPORTED;
      if (h.ll) return h.ll(&l, stream, t->grad_dtype, t->out_dtype);
    } else {
      if (gbf && obf) return dense_ll_dispatch_bf16_bf16(l, s);
      if (gbf && !obf) return dense_ll_dispatch_bf16_f32(l, s);
      if (!gbf && obf) return dense_ll_dispatch_f32_bf16(l, s);
      return dense_ll_dispatch_f32_f32(l, s);
    }
  }
  if ((op & PSDEV_OP_PUSH) && a.opt.kind >= PSDEV_OPT_USER) {
    // a handle that the application compiled and registered (ps/device/user_handle.cuh)
    UserHandle h;
    if (!find_user(a.opt.kind, &h)) return PSDEV_ERR_UNSUPPORTED;
    return h.dense(op, &a, ctas, stream, t->grad_dtype, t->out_dtype);
  }
  if (t->grad_dtype == PSDEV_I8) {
    // int8 block-scale gradients: 16 values per vector, ranges aligned to 16, no multicast
    // reduction (the switch cannot apply per-block scales)
    if ((begin & 15) || (end & 15) || (t->blk & 15) || (t->blk % 256) != 0) return PSDEV_ERR_ARG;
    a.gscale_off = t->gscale_off;
    if (op & PSDEV_OP_PUSH) a.mc_base = nullptr;
    return obf ? dense_dispatch_i8_bf16(op, a, ctas, s) : dense_dispatch_i8_f32(op, a, ctas, s);
  }
  if (gbf && obf) return dense_dispatch_bf16_bf16(op, a, ctas, s);
  if (gbf && !obf) return dense_dispatch_bf16_f32(op, a, ctas, s);
  if (!gbf && obf) return dense_dispatch_f32_bf16(op, a, ctas, s);
  return dense_dispatch_f32_f32(op, a, ctas, s);
}

extern "C" uint64_t psdev_launch_count(void) { return g_launches.load(); }

// ---- flag-only device barrier -----------------------------------------------------------
namespace psdev {
struct BarrierArgs {
  void* base[PSDEV_MAX_RANKS];
  int rank, world, channel;
  unsigned long long timeout_ns;
};
__global__ void barrier_kernel(const __grid_constant__ BarrierArgs a) {
  __shared__ unsigned long long s_epoch;
  __shared__ int s_err, s_last;
  unsigned long long e =
      channel_enter(a.base, a.rank, a.world, a.channel, a.timeout_ns, &s_epoch, &s_err);
  channel_leave(a.base, a.rank, a.world, a.channel, e, a.timeout_ns, &s_last);
}

__global__ void link_copy_kernel(uint4* dst, const uint4* src, size_t n16) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n16;
       i += (size_t)gridDim.x * blockDim.x)
    st_v4(dst + i, ld_sys_v4(src + i));
}
}  // namespace psdev

extern "C" int psdev_device_barrier(const psdev_world_t* w, int channel, uint64_t timeout_ns,
                                    void* stream) {
  if (!w || w->world < 1 || w->world > PSDEV_MAX_RANKS || channel < 0 ||
      channel >= PSDEV_NUM_CHANNELS)
    return PSDEV_ERR_ARG;
  BarrierArgs a{};
  for (int p = 0; p < w->world; ++p) a.base[p] = w->peer_base[p];
  a.rank = w->rank;
  a.world = w->world;
  a.channel = channel;
  a.timeout_ns = timeout_ns;
  barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

extern "C" int psdev_link_copy(void* dst, const void* src, size_t bytes, int num_ctas,
                                void* stream) {
  if ((bytes & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)src & 15)) return PSDEV_ERR_ARG;
  link_copy_kernel<<<num_ctas > 0 ? num_ctas : 296, 512, 0, (cudaStream_t)stream>>>(
      (uint4*)dst, (const uint4*)src, bytes / 16);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}
