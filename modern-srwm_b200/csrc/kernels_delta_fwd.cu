// Instantiations of the delta-rule forward kernels for every compiled configuration (configs.h).
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

// The packed (layer-level) form of a call runs the LAYER instantiation of a configuration.
template <int E, int V, int P, int R, int T, bool PK, int MINB, int LAYER>
int run(const DeltaFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & F_PACKED) {
    if constexpr (LAYER) {
      constexpr int smem = DeltaFwdSmem<TIO, E, T, true>::TOTAL;
      if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_pk = 0;
      return launch_kernel(delta_fwd_kernel<TIO, E, P, R, T, PK, MINB, true>, p, grid, P, smem, s, &dev_mask_pk, cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = DeltaFwdSmem<TIO, E, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(delta_fwd_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

template <int E, int V, int P, int T, bool PK, int MINB, int NRP, int LAYER, int UNR>
int run_col(const DeltaFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & F_PACKED) {
    if constexpr (LAYER) {
      constexpr int smem = DeltaFwdColSmem<TIO, E, T, true>::TOTAL;
      if (info) { info->P = P; info->R = E / NRP; info->T = T; info->smem = smem; info->id = V; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_pk = 0;
      return launch_kernel(delta_fwd_col_kernel<TIO, E, P, T, PK, MINB, NRP, true, UNR>, p, grid, P, smem, s, &dev_mask_pk,
                           cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = DeltaFwdColSmem<TIO, E, T>::TOTAL;
  if (info) { info->P = P; info->R = E / NRP; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(delta_fwd_col_kernel<TIO, E, P, T, PK, MINB, NRP, false, UNR>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

// Automatic choice at E = 64 (measured on B200, 2048-step sequences).  One warp per sequence keeps eight
// sequences resident per multiprocessor and has the best throughput once the grid offers more than
// about four per multiprocessor; with fewer, a lone warp's step latency is exposed and four warps per
// sequence (16-step chunks, step loop unrolled twice) are faster (432 sequences: 0.90 against 1.16 ms;
// 256: 0.74 against 1.16 ms).
inline int auto_variant(int E, unsigned flags, int grid, int sms) {
  if (E != 64) return 1;
  if (flags & F_PACKED) return grid < 4 * sms ? 4 : 1;
  return grid <= 4 * sms ? 3 : 1;
}

}  // namespace

#if SRWM_TIO_BF16
int dispatch_delta_fwd_bf16(
#else
int dispatch_delta_fwd_f32(
#endif
    int E, int variant, const DeltaFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err, int sms) {
  if (variant == 0) variant = auto_variant(E, p.flags, grid, current_sms(sms, describe_only));
#define X(E_, V_, P_, R_, T_, PK_, MINB_, LAYER_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_, LAYER_>(p, grid, s, info, describe_only, cuda_err);
  DELTA_FWD_CONFIGS(X)
#undef X
#define Y(E_, V_, P_, T_, PK_, MINB_, NRP_, LAYER_, UNR_) \
  if (E == E_ && variant == V_)                            \
    return run_col<E_, V_, P_, T_, PK_, MINB_, NRP_, LAYER_, UNR_>(p, grid, s, info, describe_only, cuda_err);
  DELTA_FWD_COL_CONFIGS(Y)
#undef Y
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace srwm
