// Host dispatch for the fused dense push / pull kernel (see ps/device/push_pull.cuh).
#include <cuda_runtime.h>

#include <atomic>

#include "ps/device/push_pull.cuh"

namespace psdev {
std::atomic<uint64_t> g_launches{0};
int dense_dispatch_f32_f32(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_bf16_bf16(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_bf16_f32(int op, const DenseArgs& a, int ctas, cudaStream_t s);
int dense_dispatch_f32_bf16(int op, const DenseArgs& a, int ctas, cudaStream_t s);
}  // namespace psdev

using namespace psdev;

extern "C" int psdev_dense_op(const psdev_world_t* w, const psdev_table_t* t, int op,
                              int64_t begin, int64_t end, const psdev_opt_t* opt, int channel,
                              int num_ctas, uint64_t timeout_ns, int sync, void* stream) {
  if (!w || !t || w->world < 1 || w->world > PSDEV_MAX_RANKS || w->rank < 0 ||
      w->rank >= w->world)
    return PSDEV_ERR_ARG;
  if (channel < 0 || channel >= PSDEV_NUM_CHANNELS) return PSDEV_ERR_ARG;
  if (begin < 0 || end > t->n || begin > end || (begin & 7) || (end & 7) || t->blk <= 0 ||
      (t->blk & 7))
    return PSDEV_ERR_ARG;
  if ((op & PSDEV_OP_PUSH) && !opt) return PSDEV_ERR_ARG;
  if (!t->master) return PSDEV_ERR_ARG;
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
  a.sync = sync & 1;
  a.mc_base = (sync & 2) ? w->mc_base : nullptr;  // bit 1: use the NVSwitch multicast alias
  if (op == (PSDEV_OP_PUSH | PSDEV_OP_PUBLISH)) {
    // push, and store the new values of the owned blocks into this rank's own weight
    // buffer, where a later fused pull finds them
    op = PSDEV_OP_PUSHPULL;
    a.self_only = 1;
    a.mc_base = nullptr;
  }
  a.timeout_ns = timeout_ns;
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

__global__ void copy_probe_kernel(uint4* dst, const uint4* src, size_t n16) {
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

extern "C" int psdev_copy_probe(void* dst, const void* src, size_t bytes, int num_ctas,
                                void* stream) {
  if ((bytes & 15) || ((uintptr_t)dst & 15) || ((uintptr_t)src & 15)) return PSDEV_ERR_ARG;
  copy_probe_kernel<<<num_ctas > 0 ? num_ctas : 296, 512, 0, (cudaStream_t)stream>>>(
      (uint4*)dst, (const uint4*)src, bytes / 16);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}
