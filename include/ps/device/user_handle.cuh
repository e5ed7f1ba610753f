// User-defined server handles on the device.
//
// In the reference a server's behaviour is whatever function the application installs with
// KVServer::set_request_handle (include/ps/kv_app.h:414-420).  On the device plane the handle
// runs inside the fused push kernel, so it is compiled: an application writes a struct with
// the static interface of the built-in handles (push_pull.cuh: OptSum, OptSgd, ...),
//
//     struct ClippedSgd {
//       static constexpr int kStates = 0;            // fp32 state arrays used: 0, 1 or 2
//       __device__ static void apply(float& w, float g, float& s1, float& s2,
//                                    const psdev_opt_t& o) { ... }
//     };
//     PSDEV_REGISTER_DENSE_HANDLE(100, ClippedSgd)    // kinds >= PSDEV_OPT_USER are free
//
// in a .cu file of its own, compiles it for sm_100a into a shared object that links
// libpsb200_device.so, and loads that object into the process.  The macro instantiates the
// fused kernels (push, push+pull, the low-latency small-request form; every supported pair of
// gradient and weight dtypes; peer and NVSwitch-multicast paths) for the struct and registers
// them under the kind; psdev_opt_t::kind = 100 then selects the handle in every call that
// takes a psdev_opt_t, and psdev_opt_t::user[] carries its extra hyper-parameters.
// tests/cuda/user_handle_clip.cu is a complete example.
#pragma once
#include "ps/device/dense_launch.cuh"

// Entry points that a registered handle supplies (filled in by the macro).
typedef int (*psdev_user_dense_fn)(int op, const psdev::DenseArgs* a, int ctas, void* stream,
                                   int grad_dtype, int out_dtype);
typedef int (*psdev_user_ll_fn)(const psdev::LLArgs* a, void* stream, int grad_dtype,
                                int out_dtype);
// Registers the handle of `kind` (>= PSDEV_OPT_USER) with `num_states` state arrays; returns 0,
// or PSDEV_ERR_ARG when the kind is reserved or taken.
extern "C" int psdev_register_dense_handle(int kind, int num_states, psdev_user_dense_fn dense,
                                           psdev_user_ll_fn ll);

namespace psdev {

template <class Opt, typename GT, typename OT>
inline int user_dense_by_op(int op, const DenseArgs& a, int ctas, cudaStream_t s) {
  switch (op) {
    case PSDEV_OP_PUSH: return launch<GT, OT, Opt, true, false>(a, ctas, s);
    case PSDEV_OP_PUSHPULL: return launch<GT, OT, Opt, true, true>(a, ctas, s);
    default: return PSDEV_ERR_ARG;  // a pull runs no handle
  }
}

template <class Opt>
inline int user_dense_dispatch(int op, const DenseArgs* a, int ctas, void* stream, int gdt,
                               int odt) {
  cudaStream_t s = (cudaStream_t)stream;
  if (Opt::kStates >= 1 && !a->s1) return PSDEV_ERR_ARG;
  if (Opt::kStates >= 2 && !a->s2) return PSDEV_ERR_ARG;
  const bool gbf = gdt == PSDEV_BF16, obf = odt == PSDEV_BF16;
  if (gdt == PSDEV_I8) return PSDEV_ERR_UNSUPPORTED;
  if (gbf && obf) return user_dense_by_op<Opt, __nv_bfloat16, __nv_bfloat16>(op, *a, ctas, s);
  if (gbf) return user_dense_by_op<Opt, __nv_bfloat16, float>(op, *a, ctas, s);
  if (obf) return user_dense_by_op<Opt, float, __nv_bfloat16>(op, *a, ctas, s);
  return user_dense_by_op<Opt, float, float>(op, *a, ctas, s);
}

template <class Opt>
inline int user_ll_dispatch(const LLArgs* a, void* stream, int gdt, int odt) {
  cudaStream_t s = (cudaStream_t)stream;
  if (Opt::kStates >= 1 && !a->s1) return PSDEV_ERR_ARG;
  if (Opt::kStates >= 2 && !a->s2) return PSDEV_ERR_ARG;
  const bool gbf = gdt == PSDEV_BF16, obf = odt == PSDEV_BF16;
  if (gbf && obf) return launch_ll<__nv_bfloat16, __nv_bfloat16, Opt>(*a, s);
  if (gbf) return launch_ll<__nv_bfloat16, float, Opt>(*a, s);
  if (obf) return launch_ll<float, __nv_bfloat16, Opt>(*a, s);
  return launch_ll<float, float, Opt>(*a, s);
}

}  // namespace psdev

// Instantiates the kernels for `OptStruct` and registers them under `KIND` when the object
// that contains this line is loaded.
#define PSDEV_REGISTER_DENSE_HANDLE(KIND, OptStruct)                                        \
  namespace {                                                                               \
  struct PsdevRegister_##OptStruct {                                                        \
    PsdevRegister_##OptStruct() {                                                           \
      psdev_register_dense_handle(KIND, OptStruct::kStates,                                 \
                                  &psdev::user_dense_dispatch<OptStruct>,                   \
                                  &psdev::user_ll_dispatch<OptStruct>);                     \
    }                                                                                       \
  } psdev_register_instance_##OptStruct;                                                    \
  }
