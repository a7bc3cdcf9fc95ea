// Instantiations of delta_bwd_kernel for every compiled configuration (configs.h).
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
int run(const DeltaBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only, int* cuda_err) {
  if (p.flags & F_PACKED) {
    if constexpr (LAYER) {
      constexpr int smem = DeltaBwdSmem<TIO, E, P, T, true>::TOTAL;
      if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
      if (describe_only) return 0;
      static unsigned long long dev_mask_pk = 0;
      return launch_kernel(delta_bwd_kernel<TIO, E, P, R, T, PK, MINB, true>, p, grid, P, smem, s, &dev_mask_pk, cuda_err);
    } else {
      return -6;
    }
  }
  constexpr int smem = DeltaBwdSmem<TIO, E, P, T>::TOTAL;
  if (info) { info->P = P; info->R = R; info->T = T; info->smem = smem; info->id = V; }
  if (describe_only) return 0;
  static unsigned long long dev_mask = 0;
  return launch_kernel(delta_bwd_kernel<TIO, E, P, R, T, PK, MINB>, p, grid, P, smem, s, &dev_mask, cuda_err);
}

int by_id(int E, int variant, const DeltaBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
          int* cuda_err) {
#define X(E_, V_, P_, R_, T_, PK_, MINB_, LAYER_) \
  if (E == E_ && variant == V_) return run<E_, V_, P_, R_, T_, PK_, MINB_, LAYER_>(p, grid, s, info, describe_only, cuda_err);
  DELTA_BWD_CONFIGS(X)
#undef X
  return (E == 8 || E == 16 || E == 32 || E == 64) ? -6 : -3;
}

}  // namespace

// Automatic choice at E = 64.  Configuration 1 (64 threads per sequence) keeps four sequences resident
// per multiprocessor and has the best throughput on full waves, but a sequence takes the same time
// whether its multiprocessor holds four sequences or three: a partial last wave costs a whole one.  So
// the call is split: whole waves on configuration 1, the sequences of the remainder on a configuration
// with twice the threads per sequence (shorter step latency; 432 sequences: 1.84 against 2.09 ms),
// launched behind them on the same stream.  (Four times the threads was measured too: slower at every
// grid size.)
#if SRWM_TIO_BF16
int dispatch_delta_bwd_bf16(
#else
int dispatch_delta_bwd_f32(
#endif
    int E, int variant, const DeltaBwdParams& p, int grid, cudaStream_t s, KernelInfo* info, int describe_only,
    int* cuda_err, int sms) {
  if (variant != 0 || E != 64 || (p.flags & F_PACKED))
    return by_id(E, variant == 0 ? 1 : variant, p, grid, s, info, describe_only, cuda_err);
  const int n_sm = current_sms(sms, describe_only);
  const int wave = 4 * n_sm;                       // sequences resident at once with configuration 1
  int full = (grid / wave) * wave, rest = grid - full;
  // Beyond a few waves the multiprocessors drift apart and a single launch fills the gaps by itself
  // (8192 sequences: 13.5 ms in one launch, 13.7 ms split); a remainder that nearly fills a wave is
  // left with the whole waves as well.
  if (grid > 3 * wave || rest * 10 > wave * 9) { full = grid; rest = 0; }
  constexpr int tail_id = 2;                       // 128 threads per sequence
  if (describe_only) return by_id(E, full > 0 ? 1 : tail_id, p, grid, s, info, 1, cuda_err);
  if (full > 0) {
    const int rc = by_id(E, 1, p, full, s, info, 0, cuda_err);
    if (rc != 0 || rest == 0) return rc;
  }
  DeltaBwdParams q = p;
  q.seq0 = p.seq0 + full;
  return by_id(E, tail_id, q, rest, s, full > 0 ? nullptr : info, 0, cuda_err);
}

}  // namespace srwm
