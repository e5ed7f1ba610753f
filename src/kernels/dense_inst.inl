// Instantiations of the fused dense kernel for one (gradient dtype, weight dtype) pair.
// Included by the dense_inst_*.cu files so that the pairs compile in parallel.
#include <cuda_runtime.h>

#include "ps/device/dense_launch.cuh"
#include "ps/device/user_handle.cuh"

namespace psdev {

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
    default: return PSDEV_ERR_UNSUPPORTED;  // user-defined kinds are dispatched by the caller
  }
}

#ifdef PSDEV_DENSE_LL_FN
int PSDEV_DENSE_LL_FN(const LLArgs& a, cudaStream_t s) {
  using GT = PSDEV_DENSE_GT;
  using OT = PSDEV_DENSE_OT;
  switch (a.opt.kind) {
    case PSDEV_OPT_SUM: return launch_ll<GT, OT, OptSum>(a, s);
    case PSDEV_OPT_ASSIGN: return launch_ll<GT, OT, OptAssign>(a, s);
    case PSDEV_OPT_SGD: return launch_ll<GT, OT, OptSgd>(a, s);
    case PSDEV_OPT_MOMENTUM:
      if (!a.s1) return PSDEV_ERR_ARG;
      return launch_ll<GT, OT, OptMomentum>(a, s);
    case PSDEV_OPT_ADAM:
      if (!a.s1 || !a.s2) return PSDEV_ERR_ARG;
      return launch_ll<GT, OT, OptAdam>(a, s);
    default: return PSDEV_ERR_UNSUPPORTED;
  }
}
#endif

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
