// Instantiations of the fused dense kernel for one (gradient dtype, weight dtype) pair.
// Included by the dense_inst_*.cu files so that the pairs compile in parallel.
#include <cuda_runtime.h>

#include <atomic>

#include "ps/device/push_pull.cuh"

namespace psdev {
extern std::atomic<uint64_t> g_launches;
void launch_p3_schedule(const long long* segs, int nseg, long long blk, int world, int rank,
                        long long tiles_per_blk, SchedEntry* out, cudaStream_t s);

template <typename GT, typename OT, class Opt, bool RED, bool BC, int WMAX>
static int launch_w(DenseArgs a, int num_ctas, cudaStream_t s) {
  constexpr int tile = DenseTile<GT, OT, RED, WMAX>::kElems;
  a.tiles_per_blk = (a.blk + tile - 1) / tile;
  const long long ntiles = a.n_owned * a.tiles_per_blk;
  int ctas = num_ctas > 0 ? num_ctas : 2 * 148;
  if (a.nseg > 0) {
    // device-side schedule: slices ordered by priority, tiles numbered across slices
    launch_p3_schedule(a.segs_in, a.nseg, a.blk, a.world, a.rank, a.tiles_per_blk,
                       const_cast<SchedEntry*>(a.sched), s);
  } else if (ntiles < ctas) {
    ctas = ntiles > 0 ? (int)ntiles : 1;
  }
  dense_kernel<GT, OT, Opt, RED, BC, WMAX><<<ctas, kDenseThreads, 0, s>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

template <typename GT, typename OT, class Opt, bool RED, bool BC>
static int launch_mc(DenseArgs a, int num_ctas, cudaStream_t s) {
  constexpr int tile = DenseTile<GT, OT, RED, 1>::kElems;
  a.tiles_per_blk = (a.blk + tile - 1) / tile;
  const long long ntiles = a.n_owned * a.tiles_per_blk;
  int ctas = num_ctas > 0 ? num_ctas : 2 * 148;
  if (a.nseg > 0) {
    launch_p3_schedule(a.segs_in, a.nseg, a.blk, a.world, a.rank, a.tiles_per_blk,
                       const_cast<SchedEntry*>(a.sched), s);
  } else if (ntiles < ctas) {
    ctas = ntiles > 0 ? (int)ntiles : 1;
  }
  dense_kernel<GT, OT, Opt, RED, BC, 1, true><<<ctas, kDenseThreads, 0, s>>>(a);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return (int)cudaGetLastError();
}

template <typename GT, typename OT, class Opt, bool RED, bool BC>
static int launch(const DenseArgs& a, int ctas, cudaStream_t s) {
  if (a.mc_base && a.world > 1) return launch_mc<GT, OT, Opt, RED, BC>(a, ctas, s);
  if (a.world == 1) return launch_w<GT, OT, Opt, RED, BC, 1>(a, ctas, s);
  if (a.world == 2) return launch_w<GT, OT, Opt, RED, BC, 2>(a, ctas, s);
  if (a.world <= 4) return launch_w<GT, OT, Opt, RED, BC, 4>(a, ctas, s);
  return launch_w<GT, OT, Opt, RED, BC, 8>(a, ctas, s);
}

template <typename GT, typename OT, bool RED, bool BC>
static int by_opt(const DenseArgs& a, int ctas, cudaStream_t s) {
  if (!RED) return launch<GT, OT, OptSum, RED, BC>(a, ctas, s);
  switch (a.opt.kind) {
    case PSDEV_OPT_SUM: return launch<GT, OT, OptSum, RED, BC>(a, ctas, s);
    case PSDEV_OPT_ASSIGN: return launch<GT, OT, OptAssign, RED, BC>(a, ctas, s);
    case PSDEV_OPT_SGD: return launch<GT, OT, OptSgd, RED, BC>(a, ctas, s);
    case PSDEV_OPT_MOMENTUM:
      if (!a.s1) return PSDEV_ERR_ARG;
      return launch<GT, OT, OptMomentum, RED, BC>(a, ctas, s);
    case PSDEV_OPT_ADAM:
      if (!a.s1 || !a.s2) return PSDEV_ERR_ARG;
      return launch<GT, OT, OptAdam, RED, BC>(a, ctas, s);
    default: return PSDEV_ERR_UNSUPPORTED;
  }
}

int PSDEV_DENSE_FN(int op, const DenseArgs& a, int ctas, cudaStream_t s) {
  using GT = PSDEV_DENSE_GT;
  using OT = PSDEV_DENSE_OT;
  switch (op) {
    case PSDEV_OP_PUSH: return by_opt<GT, OT, true, false>(a, ctas, s);
    case PSDEV_OP_PUSHPULL: return by_opt<GT, OT, true, true>(a, ctas, s);
    case PSDEV_OP_PULL: return by_opt<GT, OT, false, true>(a, ctas, s);
    default: return PSDEV_ERR_ARG;
  }
}
}  // namespace psdev
