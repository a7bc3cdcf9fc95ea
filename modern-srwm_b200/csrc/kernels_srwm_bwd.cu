// Instantiations of the SRWM backward kernels for every compiled configuration (configs.h).
// Built twice: -DSRWM_TIO_BF16=0 (fp32 streams) and -DSRWM_TIO_BF16=1 (bf16 streams).
#include "configs.h"
#include "launch.h"

namespace srwm {
namespace {

#if SRWM_TIO_BF16
typedef __nv_bfloat16 TIO;
#else
typedef float TIO;
#endif

// The layer-level form of a call runs the LAYER instantiation of a configuration.
constexpr unsigned EXT_FLAGS = F_INPUT_SOFTMAX | F_BASE | F_REDUCE;

template <int E, int V, int P, int R, int T, bool PK, int MINB, int LAYER>
int run(const SrwmBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & EXT_FLAGS) {
    if constexpr (LAYER) {
      constexpr int smem = SrwmBwdSmem<TIO, E, P, T, true>::TOTAL;
      if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_ext = 0;
      return launch_kernel(srwm_bwd_kernel<TIO, E, P, R, T, PK, MINB, true>, p, grid, P, smem, s, &dev_mask_ext,
                           cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = SrwmBwdSmem<TIO, E, P, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_bwd_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

// second formulation: one instantiation serves the plain and the layer-level form
template <int E, int V, int P, int R, int T, int MINB, int OPT>
int run2(const SrwmBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  constexpr int smem = SrwmBwd2Smem<TIO, E, P, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_bwd2_kernel<TIO, E, P, R, T, MINB, OPT>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

}  // namespace

#if SRWM_TIO_BF16
int dispatch_srwm_bwd_bf16(
#else
int dispatch_srwm_bwd_f32(
#endif
    int E, int variant, const SrwmBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err, int sms) {
  (void)sms;
  if (variant == 0) variant = 1;   // one configuration per head size serves every grid
#define X(E_, V_, P_, R_, T_, PK_, MINB_, LAYER_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_, LAYER_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_BWD_CONFIGS(X)
#undef X
#define Z(E_, V_, P_, R_, T_, MINB_, OPT_) \
  if (E == E_ && variant == V_) return run2<E_, V_, P_, R_, T_, MINB_, OPT_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_BWD2_CONFIGS(Z)
#undef Z
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace srwm
