// Host-side launch plumbing shared by the kernel translation units and the C ABI.
#pragma once
#include <cuda_runtime.h>
#include "delta.cuh"
#include "srwm.cuh"
#include "srwm_bwd2.cuh"
#include "srwm_fwd_warp.cuh"

namespace srwm {

enum Op { OP_SRWM_FWD = 0, OP_SRWM_BWD = 1, OP_DELTA_FWD = 2, OP_DELTA_BWD = 3, OP_SRWM_BWD_DET = 4 };

// What a (op, E, dtype, variant) combination resolves to.
struct KernelInfo {
  int P, R, T, smem;
  int id;   // the configuration id that was resolved
};

// Dispatchers, one per (operator, stream element type); defined in kernels_*.cu.
// variant 0 = automatic choice by head size and grid; ids >= 1 name one compiled configuration.
// `sms` = number of multiprocessors the automatic choice plans for (<= 0: ask the current device
// when launching, assume DEFAULT_SMS when only describing).
// Return 0 launched (or described), -3 head dim not compiled, -6 variant not compiled,
// -7 CUDA error (code stored through *cuda_err).  describe_only != 0: fill *info with the
// configuration that `grid` sequences would run on and return without touching CUDA.
#define SRWM_DECL_DISPATCH(op, Params)                                                            \
  int dispatch_##op##_f32(int E, int variant, const Params& p, int grid, cudaStream_t s,          \
                          KernelInfo* info, int describe_only, int* cuda_err, int sms);           \
  int dispatch_##op##_bf16(int E, int variant, const Params& p, int grid, cudaStream_t s,         \
                           KernelInfo* info, int describe_only, int* cuda_err, int sms);
SRWM_DECL_DISPATCH(srwm_fwd, SrwmFwdParams)
SRWM_DECL_DISPATCH(srwm_bwd, SrwmBwdParams)
SRWM_DECL_DISPATCH(srwm_bwd_det, SrwmBwdDetParams)
SRWM_DECL_DISPATCH(delta_fwd, DeltaFwdParams)
SRWM_DECL_DISPATCH(delta_bwd, DeltaBwdParams)
#undef SRWM_DECL_DISPATCH

constexpr int DEFAULT_SMS = 148;

// Multiprocessor count of the current device (cached per device ordinal).
inline int current_sms(int hint, int describe_only) {
  if (hint > 0) return hint;
  if (describe_only) return DEFAULT_SMS;
  static int cache[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return DEFAULT_SMS; }
  int& c = cache[dev & 63];
  int v = __atomic_load_n(&c, __ATOMIC_RELAXED);
  if (v <= 0) {
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) {
      (void)cudaGetLastError();
      v = DEFAULT_SMS;
    }
    __atomic_store_n(&c, v, __ATOMIC_RELAXED);
  }
  return v;
}

// Launch helper: raises the kernel's dynamic shared-memory limit once per device, then
// launches on the caller's stream.  Thread-safe (the attribute call is idempotent).
template <typename Kernel, typename Params>
inline int launch_kernel(Kernel kern, const Params& p, int grid, int block, int smem, cudaStream_t s,
                         unsigned long long* dev_mask, int* cuda_err) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *cuda_err = (int)e; return -7; }
  const unsigned long long bit = 1ull << (dev & 63);
  if (!(__atomic_load_n(dev_mask, __ATOMIC_ACQUIRE) & bit)) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) { *cuda_err = (int)e; (void)cudaGetLastError(); return -7; }
    __atomic_fetch_or(dev_mask, bit, __ATOMIC_RELEASE);
  }
  kern<<<grid, block, smem, s>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) { *cuda_err = (int)e; return -7; }
  return 0;
}

}  // namespace srwm
