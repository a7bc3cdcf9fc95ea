// Shared device-side building blocks of the SRWM / delta-rule recurrence kernels (sm_100a).
//
// Design in one paragraph.  One CTA owns one (batch, head) sequence for the whole call.
// Its weight state lives in REGISTERS as a 2-D tile per thread: the CTA's P threads form a
// grid of NRG row-groups x NCG column-groups over each E x E block; thread (rg, cg) owns
// rows [rg*R, rg*R+R) and columns [cg*C, cg*C+C).  Lanes that share a column group are
// adjacent (tid = cg*NRG + rg), so a "column" reduction (out[m] = sum_e v[e] W[e][m]) is a
// few xor-shuffles, and a "row" reduction (sum over m) is shuffles across the column
// groups of a warp plus one shared-memory combine across warps.  Register tiles are held as
// row PAIRS (64-bit registers) so that every multiply-add on the state is a packed
// fma.rn.f32x2 (two fp32 FMAs per issue slot on sm_100).  The activation streams are
// staged through shared memory a time chunk ahead with 16-byte cp.async copies and
// written back a chunk at a time with 16-byte stores.
#pragma once

#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace srwm {

typedef unsigned long long u64;

// ---------------------------------------------------------------------------------------
// Tiling of an E x E block over P threads with R rows per thread.
// ---------------------------------------------------------------------------------------
template <int E_, int P_, int R_>
struct Tiling {
  static constexpr int E = E_;
  static constexpr int P = P_;
  static constexpr int R = R_;              // rows per thread (even)
  static constexpr int NRG = E / R;         // row groups (adjacent lanes)
  static constexpr int NCG = P / NRG;       // column groups
  static constexpr int C = E / NCG;         // columns per thread
  static constexpr int NWARP = P / 32;
  static constexpr int CGW = 32 / NRG;      // column groups per warp
  static constexpr int BETA_CG_STEP = NCG / 4;  // column group j*STEP handles w_b column j
  static_assert(R % 2 == 0, "rows per thread must be even (row pairs)");
  static_assert(E % R == 0 && P % 32 == 0, "bad tiling");
  static_assert((NRG & (NRG - 1)) == 0 && NRG <= 32, "row groups must be a power of two <= 32");
  static_assert(NCG * NRG == P && NCG * C == E && C >= 1, "bad tiling");
  static_assert(NCG >= 4 && NCG % 4 == 0, "need at least 4 column groups");
};

// ---------------------------------------------------------------------------------------
// Packed fp32x2 arithmetic.  PK=true uses the sm_100 packed instructions; PK=false the
// scalar equivalents (bitwise identical results: both are IEEE fma per component).
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ u64 pack2(float lo, float hi) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 dup2(float v) { return pack2(v, v); }
__device__ __forceinline__ float hsum2(u64 v) {
  float lo, hi;
  unpack2(v, lo, hi);
  return lo + hi;
}

template <bool PK>
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
  if constexpr (PK) {
    u64 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
  } else {
    float a0, a1, b0, b1, c0, c1;
    unpack2(a, a0, a1);
    unpack2(b, b0, b1);
    unpack2(c, c0, c1);
    return pack2(fmaf(a0, b0, c0), fmaf(a1, b1, c1));
  }
}
__device__ __forceinline__ u64 neg2(u64 a) { return a ^ 0x8000000080000000ull; }

// ---------------------------------------------------------------------------------------
// Shared-memory vector loads / stores of N consecutive values (N in {1,2,4,8,16,32,64}),
// with conversion from / to the streamed element type.  Addresses are N*sizeof(T) aligned.
// ---------------------------------------------------------------------------------------
template <int N>
__device__ __forceinline__ void ld_vec(const float* p, float (&v)[N]) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i) {
      float4 t = reinterpret_cast<const float4*>(p)[i];
      v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
    }
  } else if constexpr (N == 2) {
    float2 t = *reinterpret_cast<const float2*>(p);
    v[0] = t.x; v[1] = t.y;
  } else {
    static_assert(N == 1, "unsupported vector length");
    v[0] = p[0];
  }
}
__device__ __forceinline__ void bf16x2_to_f32(uint32_t w, float& lo, float& hi) {
  lo = __uint_as_float(w << 16);
  hi = __uint_as_float(w & 0xffff0000u);
}
template <int N>
__device__ __forceinline__ void ld_vec(const __nv_bfloat16* p, float (&v)[N]) {
  if constexpr (N % 8 == 0) {
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
      uint4 t = reinterpret_cast<const uint4*>(p)[i];
      bf16x2_to_f32(t.x, v[8 * i], v[8 * i + 1]);
      bf16x2_to_f32(t.y, v[8 * i + 2], v[8 * i + 3]);
      bf16x2_to_f32(t.z, v[8 * i + 4], v[8 * i + 5]);
      bf16x2_to_f32(t.w, v[8 * i + 6], v[8 * i + 7]);
    }
  } else if constexpr (N == 4) {
    uint2 t = *reinterpret_cast<const uint2*>(p);
    bf16x2_to_f32(t.x, v[0], v[1]);
    bf16x2_to_f32(t.y, v[2], v[3]);
  } else if constexpr (N == 2) {
    uint32_t t = *reinterpret_cast<const uint32_t*>(p);
    bf16x2_to_f32(t, v[0], v[1]);
  } else {
    static_assert(N == 1, "unsupported vector length");
    v[0] = __bfloat162float(p[0]);
  }
}

template <int N>
__device__ __forceinline__ void st_vec(float* p, const float (&v)[N]) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N / 4; ++i)
      reinterpret_cast<float4*>(p)[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  } else if constexpr (N == 2) {
    *reinterpret_cast<float2*>(p) = make_float2(v[0], v[1]);
  } else {
    static_assert(N == 1, "unsupported vector length");
    p[0] = v[0];
  }
}
__device__ __forceinline__ uint32_t f32x2_to_bf16x2(float lo, float hi) {
  __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);   // .x = lo (low 16 bits)
  return *reinterpret_cast<uint32_t*>(&t);
}
template <int N>
__device__ __forceinline__ void st_vec(__nv_bfloat16* p, const float (&v)[N]) {
  if constexpr (N % 8 == 0) {
#pragma unroll
    for (int i = 0; i < N / 8; ++i) {
      uint4 t;
      t.x = f32x2_to_bf16x2(v[8 * i], v[8 * i + 1]);
      t.y = f32x2_to_bf16x2(v[8 * i + 2], v[8 * i + 3]);
      t.z = f32x2_to_bf16x2(v[8 * i + 4], v[8 * i + 5]);
      t.w = f32x2_to_bf16x2(v[8 * i + 6], v[8 * i + 7]);
      reinterpret_cast<uint4*>(p)[i] = t;
    }
  } else if constexpr (N == 4) {
    uint2 t;
    t.x = f32x2_to_bf16x2(v[0], v[1]);
    t.y = f32x2_to_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(p) = t;
  } else if constexpr (N == 2) {
    *reinterpret_cast<uint32_t*>(p) = f32x2_to_bf16x2(v[0], v[1]);
  } else {
    static_assert(N == 1, "unsupported vector length");
    p[0] = __float2bfloat16_rn(v[0]);
  }
}

// ---------------------------------------------------------------------------------------
// Row mapping of a tile.  A thread's R local rows are not one contiguous run: local row i
// of row group rg is global row
//     (i/4) * (4*NRG) + rg*4 + i%4          (R a multiple of 4)
// i.e. quads of 4 consecutive rows, quad q of all row groups side by side.  The lanes of a
// column group then read a row vector (k, q, x ...) from shared memory as 16-byte pieces
// at a 16-byte stride -- bank-conflict free -- instead of at a 4*R-byte stride.
// ---------------------------------------------------------------------------------------
template <int R, int NRG>
__device__ __forceinline__ int row_of(int rg, int i) {
  if constexpr (R % 4 == 0) return (i / 4) * (4 * NRG) + rg * 4 + (i % 4);
  else return rg * R + i;
}
template <int R, int NRG, typename T>
__device__ __forceinline__ void ld_rows(const T* base, int rg, float (&v)[R]) {
  if constexpr (R % 4 == 0) {
#pragma unroll
    for (int q = 0; q < R / 4; ++q) {
      float t[4];
      ld_vec<4>(base + q * 4 * NRG + rg * 4, t);
      v[4 * q] = t[0]; v[4 * q + 1] = t[1]; v[4 * q + 2] = t[2]; v[4 * q + 3] = t[3];
    }
  } else {
    ld_vec<R>(base + rg * R, v);
  }
}
// store S consecutive local rows starting at local row i0 (S <= 4 stays inside one quad)
template <int S, int R, int NRG, int NV>
__device__ __forceinline__ void st_rows_piece(float* base, int rg, int i0, const float (&v)[NV]) {
  static_assert(S <= NV, "piece larger than its source");
  if constexpr (R % 4 == 0) {
    if constexpr (S <= 4) {
      float t[S];
#pragma unroll
      for (int i = 0; i < S; ++i) t[i] = v[i];
      st_vec<S>(base + (i0 / 4) * (4 * NRG) + rg * 4 + (i0 % 4), t);
    } else {
      static_assert(S % 4 == 0, "pieces longer than a quad are whole quads");
#pragma unroll
      for (int q = 0; q < S / 4; ++q) {
        float t[4] = {v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]};
        st_vec<4>(base + (i0 / 4 + q) * (4 * NRG) + rg * 4, t);
      }
    }
  } else {
    float t[S];
#pragma unroll
    for (int i = 0; i < S; ++i) t[i] = v[i];
    st_vec<S>(base + rg * R + i0, t);
  }
}
template <int R, int NRG>
__device__ __forceinline__ void st_rows(float* base, int rg, const float (&v)[R]) {
  st_rows_piece<R, R, NRG>(base, rg, 0, v);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ void from_f32(float& d, float v) { d = v; }
__device__ __forceinline__ void from_f32(__nv_bfloat16& d, float v) { d = __float2bfloat16_rn(v); }

// ---------------------------------------------------------------------------------------
// Warp reductions over the two lane axes of the tiling.
// ---------------------------------------------------------------------------------------
template <int NRG>
__device__ __forceinline__ float allreduce_rows(float v) {   // over the row groups of a column group
#pragma unroll
  for (int off = 1; off < NRG; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
template <int NRG>
__device__ __forceinline__ float allreduce_rows_max(float v) {
#pragma unroll
  for (int off = 1; off < NRG; off <<= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, off));
  return v;
}
// over the NP row parts of the column layouts: part p of a warp is its lanes [p*32/NP, (p+1)*32/NP)
// (a broadcast operand load then sees one address per half / quarter warp, which the shared-memory
// pipe serves in as many wavefronts as there are parts; interleaved parts cost twice that)
template <int NP>
__device__ __forceinline__ float allreduce_parts(float v) {
#pragma unroll
  for (int off = 32 / NP; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
template <int NRG>
__device__ __forceinline__ float allreduce_cols(float v) {   // over the column groups of this warp
#pragma unroll
  for (int off = NRG; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}
__device__ __forceinline__ float allreduce_warp(float v) {
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

// Reduce-scatter of v[0..N) across the K lanes {lane ^ (m*STRIDE)}, m < K (K a power of two
// dividing N).  On return the lane whose index along that axis is a = (lane/STRIDE) % K
// holds in v[0..N/K) the sums of elements [a*N/K, (a+1)*N/K).  N*(1-1/K) shuffles instead of
// the N*log2(K) of a butterfly all-reduce.
template <int N, int K, int STRIDE, int NV>
__device__ __forceinline__ void reduce_scatter(float (&v)[NV], int lane) {
  static_assert(N % K == 0 && N <= NV, "bad reduce_scatter shape");
  if constexpr (K > 1) {
    constexpr int n = N / 2, k = K / 2;
    const bool up = ((lane / STRIDE) & k) != 0;
#pragma unroll
    for (int i = 0; i < n; ++i) {
      const float send = up ? v[i] : v[i + n];
      const float keep = up ? v[i + n] : v[i];
      v[i] = keep + __shfl_xor_sync(0xffffffffu, send, k * STRIDE);
    }
    reduce_scatter<n, k, STRIDE, NV>(v, lane);
  }
}

// ---------------------------------------------------------------------------------------
// Asynchronous global -> shared staging of `nrows` rows of ROWBYTES bytes each (16-byte
// pieces, cp.async.cg: bypasses L1), and the matching shared -> global flush.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int ROWBYTES, int P>
__device__ __forceinline__ void stage_rows(void* smem_dst, const void* gsrc_row0, long long row_stride_bytes,
                                           int nrows, int tid) {
  static_assert(ROWBYTES % 16 == 0, "rows are staged in 16-byte pieces");
  constexpr int PPR = ROWBYTES / 16;
  const char* src = reinterpret_cast<const char*>(gsrc_row0);
  char* dst = reinterpret_cast<char*>(smem_dst);
  for (int p = tid; p < nrows * PPR; p += P) {
    const int row = p / PPR, off = p % PPR;
    cp_async16(dst + row * ROWBYTES + off * 16, src + row * row_stride_bytes + off * 16);
  }
}
template <int ROWBYTES, int P>
__device__ __forceinline__ void flush_rows(void* gdst_row0, long long row_stride_bytes, const void* smem_src,
                                           int nrows, int tid) {
  static_assert(ROWBYTES % 16 == 0, "rows are flushed in 16-byte pieces");
  constexpr int PPR = ROWBYTES / 16;
  char* dst = reinterpret_cast<char*>(gdst_row0);
  const char* src = reinterpret_cast<const char*>(smem_src);
  for (int p = tid; p < nrows * PPR; p += P) {
    const int row = p / PPR, off = p % PPR;
    const uint4 v = *reinterpret_cast<const uint4*>(src + row * ROWBYTES + off * 16);
    *reinterpret_cast<uint4*>(dst + row * row_stride_bytes + off * 16) = v;
  }
}

// Fast transcendental helpers (ex2.approx / rcp.approx based; relative error ~1e-7..1e-6,
// far inside the 1e-4 forward tolerance, and the backward consumes the SAVED results).
__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

// Debug build (-DSRWM_DEBUG_CHECKS): every staged / flushed chunk of rows is checked against the
// sequence length before any address is formed.  A violation is recorded once in a status word
// (bit 63 set | site id << 48 | CTA index (24 bits) << 24 | first row (24 bits)) and the access is
// skipped; nothing traps.  The C ABI returns the word (srwm_b200_debug_status).  In the ordinary
// build the check compiles to nothing.
#ifdef SRWM_DEBUG_CHECKS
__device__ __forceinline__ bool bad_rows(unsigned long long* dbg, int site, int t0, int nt, int L, int T) {
  if (t0 >= 0 && nt >= 0 && nt <= T && t0 + nt <= L) return false;
  if (dbg != nullptr && threadIdx.x == 0) {
    const unsigned long long w = (1ull << 63) | ((unsigned long long)(site & 0xff) << 48) |
                                 ((unsigned long long)(blockIdx.x & 0xffffffu) << 24) |
                                 (unsigned long long)((unsigned)t0 & 0xffffffu);
    atomicCAS(dbg, 0ull, w);
  }
  return true;
}
#define SRWM_BAD_ROWS(dbg, site, t0, nt, L, T) ::srwm::bad_rows(dbg, site, t0, nt, L, T)
#else
#define SRWM_BAD_ROWS(dbg, site, t0, nt, L, T) false
#endif

// A sequence view with byte strides, as passed to the kernels.
struct SeqView {
  char* base;
  long long sn, sh, sl;   // bytes
  __device__ __forceinline__ char* row(int n, int h, int t) const {
    return base + (long long)n * sn + (long long)h * sh + (long long)t * sl;
  }
};
struct StateView {
  float* base;
  long long sn, sh;       // elements
  __device__ __forceinline__ float* mat(int n, int h) const { return base + (long long)n * sn + (long long)h * sh; }
};

// Flag bits of the kernels' `flags` word (the first three are the ABI's; the rest are set by
// the C layer from the extension block of a call).
constexpr unsigned F_NO_SAVE = 1u, F_STATE_GRAD_IN = 2u, F_RESTORE = 4u, F_INPUT_SOFTMAX = 8u, F_BASE = 16u,
                   F_SHIFT_IN = 32u, F_DONE = 64u;

__device__ __forceinline__ float warp_max(float v) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, 0xffffffff;" : "=f"(r) : "f"(v));
  return r;
}

// Streamed rows to fp32 rows in shared memory (nt rows of E values).
template <typename TIO, int E, int P>
__device__ __forceinline__ void convert_rows(const TIO* src, float* dst, int nt, int tid) {
  for (int i = tid; i < nt * E / 2; i += P) {
    float v[2];
    ld_vec<2>(src + 2 * i, v);
    st_vec<2>(dst + 2 * i, v);
  }
}

// Row-wise softmax of nt (<= T) staged rows: dst[t][:] = softmax(src[t][:]) in fp32.  A row is
// handled by E/4 adjacent lanes with 4 values each, so a warp works on 128/E rows at once, and
// the rows a thread takes part in are independent chains the compiler can overlap.  dst may
// be the same memory as src when the streamed type is float (a lane rewrites exactly what it
// read).
template <typename TIO, int E, int P, int T>
__device__ __forceinline__ void softmax_rows(const TIO* src, float* dst, int nt, int tid) {
  constexpr int LPR = E / 4;                 // lanes per row
  constexpr int NG = P / LPR;                // rows in flight per pass over the block
  constexpr int K = (T + NG - 1) / NG;       // passes
  const int grp = tid / LPR, l = tid % LPR;
#pragma unroll
  for (int kk = 0; kk < K; ++kk) {
    const int t = grp + kk * NG;
    const int tc = min(t, nt - 1);           // lanes past the end redo the last row and do not store
    float v[4];
    ld_vec<4>(src + tc * E + l * 4, v);
    float m = fmaxf(fmaxf(v[0], v[1]), fmaxf(v[2], v[3]));
#pragma unroll
    for (int off = 1; off < LPR; off <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, off));
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __expf(v[i] - m);
      sum += v[i];
    }
#pragma unroll
    for (int off = 1; off < LPR; off <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    const float inv = __fdividef(1.f, sum);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= inv;
    if (t < nt) st_vec<4>(dst + t * E + l * 4, v);
  }
}

// Backward of that softmax, applied to finished gradient rows on their way out:
// out[t][e] = x[t][e] (g[t][e] - sum_e' g[t][e'] x[t][e']), rows of g `gstride` floats apart,
// written as streamed type to global rows `row_stride_bytes` apart.
template <typename TIO, int E, int P, int T>
__device__ __forceinline__ void softmax_bwd_rows(const float* xs, const float* g, int gstride, char* grow0,
                                                 long long row_stride_bytes, int nt, int tid) {
  constexpr int LPR = E / 4;
  constexpr int NG = P / LPR;
  constexpr int K = (T + NG - 1) / NG;
  const int grp = tid / LPR, l = tid % LPR;
#pragma unroll
  for (int kk = 0; kk < K; ++kk) {
    const int t = grp + kk * NG;
    const int tc = min(t, nt - 1);
    float xv[4], gv[4];
    ld_vec<4>(xs + tc * E + l * 4, xv);
    ld_vec<4>(g + tc * gstride + l * 4, gv);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) dot = fmaf(xv[i], gv[i], dot);
#pragma unroll
    for (int off = 1; off < LPR; off <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
#pragma unroll
    for (int i = 0; i < 4; ++i) gv[i] = xv[i] * (gv[i] - dot);
    if (t < nt) st_vec<4>(reinterpret_cast<TIO*>(grow0 + t * row_stride_bytes) + l * 4, gv);
  }
}

}  // namespace srwm
