// Instantiations of srwm_bwd_kernel for every compiled configuration (configs.h).
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

// The extended form of a call runs the EXT instantiation of the default configuration.
constexpr unsigned EXT_FLAGS = F_INPUT_SOFTMAX | F_BASE;

template <int E, int V, int P, int R, int T, bool PK, int MINB>
int run(const SrwmBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  // (at E = 64 the EXT instantiation also serves plain calls: it reads x as fp32 rows converted once
  // per chunk, which leaves the step loop fewer conversions and fewer spilled registers; measured
  // 5 % faster with bf16 streams, equal with fp32 streams)
  if ((p.flags & EXT_FLAGS) || (E == 64 && V == 0)) {
    if constexpr (V == 0) {
      constexpr int smem = SrwmBwdSmem<TIO, E, P, T, true>::TOTAL;
      if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_ext = 0;
      return launch_kernel(srwm_bwd_kernel<TIO, E, P, R, T, PK, MINB, true>, p, grid, P, smem, s, &dev_mask_ext,
                           cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = SrwmBwdSmem<TIO, E, P, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_bwd_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

}  // namespace

#if SRWM_TIO_BF16
int dispatch_srwm_bwd_bf16(
#else
int dispatch_srwm_bwd_f32(
#endif
    int E, int variant, const SrwmBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err) {
#define X(E_, V_, P_, R_, T_, PK_, MINB_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_BWD_CONFIGS(X)
#undef X
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace srwm
