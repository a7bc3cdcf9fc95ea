// Instantiations of srwm_bwd_det_kernel (backward with the state detached at every step).
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

template <int E, int V, int P, int R, int T, bool PK, int MINB>
int run(const SrwmBwdDetParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  constexpr int smem = SrwmBwdDetSmem<TIO, E, P, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_bwd_det_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

}  // namespace

#if SRWM_TIO_BF16
int dispatch_srwm_bwd_det_bf16(
#else
int dispatch_srwm_bwd_det_f32(
#endif
    int E, int variant, const SrwmBwdDetParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err, int sms) {
  (void)sms;
  if (variant == 0) variant = 1;
#define X(E_, V_, P_, R_, T_, PK_, MINB_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_BWD_DET_CONFIGS(X)
#undef X
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace srwm
