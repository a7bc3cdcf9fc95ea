// Instantiations of delta_fwd_kernel for every compiled configuration (configs.h).
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

// The packed (layer-level) form of a call runs the PACKED instantiation of the default
// configuration; the plain form keeps its own, unchanged code.
template <int E, int V, int P, int R, int T, bool PK, int MINB>
int run(const DeltaFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & F_PACKED) {
    if constexpr (V == (E == 64 ? 6 : 0)) {
      constexpr int smem = DeltaFwdSmem<TIO, E, T, true>::TOTAL;
      if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_pk = 0;
      return launch_kernel(delta_fwd_kernel<TIO, E, P, R, T, PK, MINB, true>, p, grid, P, smem, s, &dev_mask_pk, cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = DeltaFwdSmem<TIO, E, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(delta_fwd_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

template <int E, int P, int T, bool PK, int MINB, int NRP>
int run_col(const DeltaFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & F_PACKED) {
    if constexpr (E == 64 && NRP == 1 && P == 32) {   // the packed form of the default configuration
      constexpr int smem = DeltaFwdColSmem<TIO, E, T, true>::TOTAL;
      if (info) { info->P = P; info->R = E / NRP; info->T = T; info->smem = smem; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_pk = 0;
      return launch_kernel(delta_fwd_col_kernel<TIO, E, P, T, PK, MINB, NRP, true>, p, grid, P, smem, s, &dev_mask_pk,
                           cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = DeltaFwdColSmem<TIO, E, T>::TOTAL;
  if (info) { info->P = P; info->R = E / NRP; info->T = T; info->smem = smem; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(delta_fwd_col_kernel<TIO, E, P, T, PK, MINB, NRP>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

}  // namespace

#if SRWM_TIO_BF16
int dispatch_delta_fwd_bf16(
#else
int dispatch_delta_fwd_f32(
#endif
    int E, int variant, const DeltaFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err) {
  // the packed (layer-level) form at E = 64: column kernel (variant 0) when the grid fills the SMs,
  // register tiles (variant 6) otherwise
  if ((p.flags & F_PACKED) && E == 64 && variant == 0 && !describe_only && grid < 592) variant = 6;
  // default at E = 64: one warp per sequence when the grid can fill the SMs; with fewer sequences the
  // per-step latency of a single warp shows, and two warps per sequence (variant 8) are faster
  // (measured: 256 sequences 201 vs 261 us, 1184 sequences 900 vs 814 us)
  if (!(p.flags & F_PACKED) && E == 64 && variant == 0 && !describe_only && grid < 592) variant = 8;
#define X(E_, V_, P_, R_, T_, PK_, MINB_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_>(p, grid, s, info, describe_only, cuda_err);
  DELTA_FWD_CONFIGS(X)
#undef X
#define Y(E_, V_, P_, T_, PK_, MINB_, NRP_) \
  if (E == E_ && variant == V_) return run_col<E_, P_, T_, PK_, MINB_, NRP_>(p, grid, s, info, describe_only, cuda_err);
  DELTA_FWD_COL_CONFIGS(Y)
#undef Y
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace srwm
