// Instantiations of the SRWM forward kernels for every compiled configuration (configs.h).
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

// The layer-level form of a call (flag bits above the ABI's three) runs the LAYER instantiation
// of a configuration; the plain form keeps its own code.
constexpr unsigned EXT_FLAGS = F_INPUT_SOFTMAX | F_BASE | F_SHIFT_IN | F_DONE;

template <int E, int V, int P, int R, int T, bool PK, int MINB, int LAYER>
int run(const SrwmFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & EXT_FLAGS) {
    if constexpr (LAYER) {
      constexpr int smem = SrwmFwdSmem<TIO, E, T, true>::TOTAL;
      if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_ext = 0;
      return launch_kernel(srwm_fwd_kernel<TIO, E, P, R, T, PK, MINB, true>, p, grid, P, smem, s, &dev_mask_ext,
                           cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = SrwmFwdSmem<TIO, E, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_fwd_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

template <int E, int V, int T, bool PK, int MINB, bool DPRE, int NRP, int LAYER>
int run_col(const SrwmFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & EXT_FLAGS) {
    if constexpr (LAYER) {
      constexpr int smem = SrwmFwdColSmem<TIO, E, T, true>::TOTAL;
      if (info) { info->P = 96; info->R = E / NRP; info->T = T; info->smem = smem; info->id = V; }
      if (describe_only) return 0;
      if (p.flags & F_DONE) {
        static unsigned long long dev_mask_rst = 0;
        return launch_kernel(srwm_fwd_col_kernel<TIO, E, T, PK, MINB, DPRE, NRP, true, true>, p, grid, 96, smem, s,
                             &dev_mask_rst, cuda_err);
      }
      static unsigned long long dev_mask_ext = 0;
      return launch_kernel(srwm_fwd_col_kernel<TIO, E, T, PK, MINB, DPRE, NRP, true, false>, p, grid, 96, smem, s,
                           &dev_mask_ext, cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = SrwmFwdColSmem<TIO, E, T>::TOTAL;
  if (info) { info->P = 96; info->R = E / NRP; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_fwd_col_kernel<TIO, E, T, PK, MINB, DPRE, NRP>, p, grid, 96, smem, s, &dev_mask, cuda_err);
}

template <int E, int V, int T, int MINB>
int run_warp(const SrwmFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  constexpr int SPW = 32 / E;                     // sequences per warp (= per CTA of 32 threads)
  const int ctas = (grid + SPW - 1) / SPW;
  if (p.flags & EXT_FLAGS) {
    constexpr int smem = SPW * SrwmFwdWarpSmem<TIO, E, T, true>::TOTAL;
    if (info) { info->P = E; info->R = E; info->T = T; info->smem = smem; info->id = V; }
    if (describe_only) return 0;
    if (p.flags & F_DONE) {
      static unsigned long long dev_mask_rst = 0;
      return launch_kernel(srwm_fwd_warp_kernel<TIO, E, T, MINB, true, true>, p, ctas, 32, smem, s, &dev_mask_rst, cuda_err);
    }
    static unsigned long long dev_mask_ext = 0;
    return launch_kernel(srwm_fwd_warp_kernel<TIO, E, T, MINB, true, false>, p, ctas, 32, smem, s, &dev_mask_ext, cuda_err);
  }
  constexpr int smem = SPW * SrwmFwdWarpSmem<TIO, E, T, false>::TOTAL;
  if (info) { info->P = E; info->R = E; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(srwm_fwd_warp_kernel<TIO, E, T, MINB, false, false>, p, ctas, 32, smem, s, &dev_mask, cuda_err);
}

}  // namespace

#if SRWM_TIO_BF16
int dispatch_srwm_fwd_bf16(
#else
int dispatch_srwm_fwd_f32(
#endif
    int E, int variant, const SrwmFwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err, int sms) {
  // E = 32: one warp per sequence once the grid offers more than eight sequences per multiprocessor
  // (fewer instructions per step, but a longer step for a lone sequence) -- unless its last wave of
  // twelve sequences per multiprocessor would be mostly empty (2048 sequences on 148 multiprocessors
  // are 1.15 waves: no gain over the column layout there)
  if (variant == 0) {
    variant = 1;
    if (E == 32) {
      const int n_sm = current_sms(sms, describe_only), slots = 12 * n_sm;
      const int full = grid / slots, rest = grid - full * slots;
      if (grid > 8 * n_sm && (rest == 0 || full >= 3 || rest * 20 >= slots * 13)) variant = 2;
    }
  }
#define X(E_, V_, P_, R_, T_, PK_, MINB_, LAYER_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_, LAYER_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_FWD_CONFIGS(X)
#undef X
#define Y(E_, V_, T_, PK_, MINB_, DPRE_, NRP_, LAYER_) \
  if (E == E_ && variant == V_)                         \
    return run_col<E_, V_, T_, PK_, MINB_, DPRE_, NRP_, LAYER_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_FWD_COL_CONFIGS(Y)
#undef Y
#define V(E_, V_, T_, MINB_) \
  if (E == E_ && variant == V_) return run_warp<E_, V_, T_, MINB_>(p, grid, s, info, describe_only, cuda_err);
  SRWM_FWD_WARP_CONFIGS(V)
#undef V
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace srwm
