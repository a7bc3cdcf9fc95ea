// Self-referential weight matrix (SRWM) recurrence, forward and reverse-time backward,
// for sm_100a.
//
// Semantics follow the reference's ground-truth loop
// (supervised_learning/self_ref_v0/__init__.py:310-356) plus what its kernel saves and
// leaves behind (supervised_learning/self_ref_v0/self_ref_v0.cu:317-431): per step t
//   [y, q~, k~, b~] = x_t.[W_y | W_q | W_k | w_b]          (y is the output, pre-update)
//   q = softmax(q~), k = softmax(k~), beta = sigmoid(b~) = (b_y, b_q, b_k, b_b)
//   d_Z = (q - k).W_Z ;  W_Z += k^T (b_Z d_Z)               for Z in {y, q, k, b}
// and the update is applied at every step, the last one included.
//
// Kernels in this file: srwm_fwd_kernel (register tiles; head sizes up to 16),
// srwm_fwd_col_kernel (one warp per block W_y / W_q / W_k, whole columns per lane; head sizes
// 32 and 64), srwm_bwd_kernel (register tiles, reverse time) and srwm_bwd_det_kernel (the
// gradient with the state detached at every step).  In the tile kernels the three E x E blocks
// share one register tiling (common.cuh); the small E x 4 block w_b lives transposed in shared
// memory, one column per designated column group, or -- in the backward -- in registers spread
// evenly over the lanes.  One block-wide barrier per time step, placed where the softmax needs all
// of q~ / k~ (forward) or where the row sums of the backward have to cross warps.
#pragma once
#include "common.cuh"

namespace srwm {

// The extended (layer-level) form of a call, selected by flag bits (common.cuh):
//   F_INPUT_SOFTMAX  x holds raw activations; the kernels apply softmax over the head dimension
//                    (supervised_learning/layer.py:162-163, reinforcement_learning/torchbeast/layer.py:383)
//                    and the backward returns the gradient with respect to the raw values
//   F_BASE           the state is base + shift, base being the un-repeated slow weights
//                    ([1,H,E,.], batch stride 0): W_* then receive the final SHIFT W_L - base
//                    (the subtraction of layer.py:412-415 / :200-204), and the backward reads W_L as
//                    base + W_*
//   F_SHIFT_IN       with F_BASE: the initial shift comes from s* (else it is zero)
//   F_DONE           with F_BASE: done[n, t] != 0 resets the shift of sample n to zero before step t
//                    (reinforcement_learning/torchbeast_procgen/model.py:1180-1194)
struct SrwmFwdParams {
  int N, H, L;
  unsigned flags;
  unsigned long long* dbg;   // status word of the debug build (null otherwise)
  SeqView x, out, q, k, beta, yd, qd, kd, bd;
  StateView Wy, Wq, Wk, wb;
  StateView bWy, bWq, bWk, bwb;   // slow weights
  StateView sWy, sWq, sWk, swb;   // initial shift
  const unsigned char* done;      // [N, L] bytes
  long long done_sn, done_sl;
};

// Batch reduction fused into the backward (F_REDUCE): the slow-weight gradient is the sum over the
// batch of the per-sample dL/dW_0 -- the backward of the callers' `W.repeat(bsz, 1, 1, 1)`
// (supervised_learning/layer.py:174-177).  The CTAs of one head form groups of `gs` consecutive
// samples; whichever CTA of a group finishes last (an atomic counter tells it; nobody waits) adds the
// group's per-sample gradients in sample order into a partial, and whichever group of a head finishes
// last adds the partials in group order into the output.  The order of every addition is fixed, so the
// result does not depend on timing.  `cnt` ([H][ng+1] counters) must be zero on entry and is zero again
// on exit; `part` holds [H][ng] partial states (not used when ng == 1).
constexpr unsigned F_REDUCE = 128u;
struct SrwmReduce {
  StateView oWy, oWq, oWk, owb;   // [1,H,E,.] outputs
  float* part;
  unsigned* cnt;
  int gs, ng, accumulate;
};

struct SrwmBwdParams {
  int N, H, L;
  unsigned flags;
  unsigned long long* dbg;   // status word of the debug build (null otherwise)
  SeqView x, q, k, beta, yd, qd, kd, bd, gout, gx;
  StateView Wy, Wq, Wk, wb, gWy, gWq, gWk, gwb;
  StateView bWy, bWq, bWk, bwb;   // slow weights
  SrwmReduce red;
};

__device__ __forceinline__ void add4g(float4& a, const float* src) {
  const float4 v = __ldcg(reinterpret_cast<const float4*>(src));   // written by other CTAs: read through L2
  a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
}

// Epilogue of the backward kernels for F_REDUCE (all P threads of the CTA of sample n, head h call it
// after storing their per-sample gradients).
template <int E, int P>
__device__ void reduce_epilogue(const SrwmBwdParams& p, int n, int h, int tid) {
  __shared__ int s_last;
  const SrwmReduce& r = p.red;
  constexpr int STATE = 3 * E * E + 4 * E;
  const int g = n / r.gs, n0 = g * r.gs;
  const int members = min(r.gs, p.N - n0);
  unsigned* cnt = r.cnt + (long long)h * (r.ng + 1);
  __threadfence();   // this CTA's per-sample gradients are visible device-wide before it is counted
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&cnt[g], 1u) == (unsigned)(members - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const bool single = r.ng == 1;
  float* part = r.part + ((long long)h * r.ng + g) * STATE;
#pragma unroll 1
  for (int z = 0; z < 4; ++z) {
    const StateView& src = z == 0 ? p.gWy : (z == 1 ? p.gWq : (z == 2 ? p.gWk : p.gwb));
    const StateView& out = z == 0 ? r.oWy : (z == 1 ? r.oWq : (z == 2 ? r.oWk : r.owb));
    const int count = z < 3 ? E * E : 4 * E;
    float* dst = single ? out.mat(0, h) : part + z * E * E;
    for (int i = tid * 4; i < count; i += P * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (single && r.accumulate) acc = *reinterpret_cast<const float4*>(dst + i);
      for (int m = 0; m < members; ++m) add4g(acc, src.mat(n0 + m, h) + i);
      *reinterpret_cast<float4*>(dst + i) = acc;
    }
  }
  if (single) {
    if (tid == 0) cnt[0] = 0u;
    return;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) s_last = atomicAdd(&cnt[r.ng], 1u) == (unsigned)(r.ng - 1);
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  const float* parts = r.part + (long long)h * r.ng * STATE;
#pragma unroll 1
  for (int z = 0; z < 4; ++z) {
    const StateView& out = z == 0 ? r.oWy : (z == 1 ? r.oWq : (z == 2 ? r.oWk : r.owb));
    const int count = z < 3 ? E * E : 4 * E;
    float* dst = out.mat(0, h);
    for (int i = tid * 4; i < count; i += P * 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      if (r.accumulate) acc = *reinterpret_cast<const float4*>(dst + i);
      for (int g2 = 0; g2 < r.ng; ++g2) add4g(acc, parts + (long long)g2 * STATE + z * E * E + i);
      *reinterpret_cast<float4*>(dst + i) = acc;
    }
  }
  for (int i = tid; i <= r.ng; i += P) cnt[i] = 0u;
}

template <int E, int C, int R, int NRG>
__device__ __forceinline__ void load_tile(const float* g, int rg, int cg, u64 (&W)[R / 2][C]) {
#pragma unroll
  for (int i2 = 0; i2 < R / 2; ++i2) {
    float a[C], b[C];
    ld_vec<C>(g + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    ld_vec<C>(g + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
#pragma unroll
    for (int j = 0; j < C; ++j) W[i2][j] = pack2(a[j], b[j]);
  }
}
// W = a + b (b may be null)
template <int E, int C, int R, int NRG>
__device__ __forceinline__ void load_tile_sum(const float* ga, const float* gb, int rg, int cg, u64 (&W)[R / 2][C]) {
#pragma unroll
  for (int i2 = 0; i2 < R / 2; ++i2) {
    float a[C], b[C];
    ld_vec<C>(ga + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    ld_vec<C>(ga + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
    if (gb) {
      float a1[C], b1[C];
      ld_vec<C>(gb + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a1);
      ld_vec<C>(gb + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b1);
#pragma unroll
      for (int j = 0; j < C; ++j) { a[j] += a1[j]; b[j] += b1[j]; }
    }
#pragma unroll
    for (int j = 0; j < C; ++j) W[i2][j] = pack2(a[j], b[j]);
  }
}
// g = W - base (base may be null)
template <int E, int C, int R, int NRG>
__device__ __forceinline__ void store_tile_diff(float* g, const float* gbase, int rg, int cg, const u64 (&W)[R / 2][C]) {
#pragma unroll
  for (int i2 = 0; i2 < R / 2; ++i2) {
    float a[C], b[C];
#pragma unroll
    for (int j = 0; j < C; ++j) unpack2(W[i2][j], a[j], b[j]);
    if (gbase) {
      float a1[C], b1[C];
      ld_vec<C>(gbase + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a1);
      ld_vec<C>(gbase + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b1);
#pragma unroll
      for (int j = 0; j < C; ++j) { a[j] -= a1[j]; b[j] -= b1[j]; }
    }
    st_vec<C>(g + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    st_vec<C>(g + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
  }
}
template <int E, int C, int R, int NRG>
__device__ __forceinline__ void store_tile(float* g, int rg, int cg, const u64 (&W)[R / 2][C]) {
#pragma unroll
  for (int i2 = 0; i2 < R / 2; ++i2) {
    float a[C], b[C];
#pragma unroll
    for (int j = 0; j < C; ++j) unpack2(W[i2][j], a[j], b[j]);
    st_vec<C>(g + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    st_vec<C>(g + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
  }
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
template <typename TIO, int E, int T, bool EXT = false>
struct SrwmFwdSmem {
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int IN_BYTES = T * ROW_IO;                       // x of one buffer
  static constexpr int XF_BYTES = (EXT && sizeof(TIO) != 4) ? T * ROW_F : 0;   // softmax(x) in fp32
  static constexpr int OUT_BYTES = T * ROW_IO + 5 * T * ROW_F + 2 * T * 16;  // y | q k yd qd kd | beta bd
  static constexpr int XCHG_BYTES = 2 * 2 * ROW_F + 2 * 16;         // q~,k~ (x2 parity) + beta (x2)
  static constexpr int WB_BYTES = 4 * ROW_F;                        // w_b transposed [4][E]
  static constexpr int DONE_BYTES = EXT ? ((T + 15) / 16) * 16 : 0; // reset flags of the chunk
  static constexpr int TOTAL = 2 * IN_BYTES + XF_BYTES + OUT_BYTES + XCHG_BYTES + WB_BYTES + DONE_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB, bool EXT = false>
__global__ void __launch_bounds__(P, MINB) srwm_fwd_kernel(const SrwmFwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = SrwmFwdSmem<TIO, E, T, EXT>;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const bool save = !(p.flags & 1u);
  // w_b column handled by this thread's column group (-1: none)
  const int jb = (cg % TL::BETA_CG_STEP == 0) ? cg / TL::BETA_CG_STEP : -1;

  extern __shared__ __align__(16) unsigned char smem[];
  float* xf32 = reinterpret_cast<float*>(smem + 2 * SM::IN_BYTES);   // EXT, bf16 streams only
  unsigned char* s_o = smem + 2 * SM::IN_BYTES + SM::XF_BYTES;
  TIO* sy = reinterpret_cast<TIO*>(s_o);
  float* sq = reinterpret_cast<float*>(s_o + T * SM::ROW_IO);
  float* sk = sq + T * E;
  float* syd = sk + T * E;
  float* sqd = syd + T * E;
  float* skd = sqd + T * E;
  float* sbeta = skd + T * E;          // [T][4]
  float* sbd = sbeta + T * 4;          // [T][4]
  float* xq = sbd + T * 4;             // [2][2][E]  pre-softmax q~ / k~, double buffered
  float* xbeta = xq + 4 * E;           // [2][4]
  float* wbT = xbeta + 8;              // [4][E]
  unsigned char* sdone = reinterpret_cast<unsigned char*>(wbT + 4 * E);   // [T] (EXT)

  const bool smx = EXT && (p.flags & F_INPUT_SOFTMAX);
  const bool has_base = EXT && (p.flags & F_BASE);
  const bool has_done = EXT && (p.flags & F_DONE);

  u64 Wy[R2][C], Wq[R2][C], Wk[R2][C];
  float* gWy = p.Wy.mat(n, h);
  float* gWq = p.Wq.mat(n, h);
  float* gWk = p.Wk.mat(n, h);
  float* gwb = p.wb.mat(n, h);
  if (has_base) {
    const bool sh = (p.flags & F_SHIFT_IN) != 0;
    load_tile_sum<E, C, R, NRG>(p.bWy.mat(n, h), sh ? p.sWy.mat(n, h) : nullptr, rg, cg, Wy);
    load_tile_sum<E, C, R, NRG>(p.bWq.mat(n, h), sh ? p.sWq.mat(n, h) : nullptr, rg, cg, Wq);
    load_tile_sum<E, C, R, NRG>(p.bWk.mat(n, h), sh ? p.sWk.mat(n, h) : nullptr, rg, cg, Wk);
    const float* bb = p.bwb.mat(n, h);
    const float* sb = sh ? p.swb.mat(n, h) : nullptr;
    for (int i = tid; i < 4 * E; i += P) wbT[(i % 4) * E + i / 4] = bb[i] + (sb ? sb[i] : 0.f);
  } else {
    load_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
    load_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
    load_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
    for (int i = tid; i < 4 * E; i += P) wbT[(i % 4) * E + i / 4] = gwb[i];   // [E][4] -> [4][E]
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return reinterpret_cast<TIO*>(smem + b * SM::IN_BYTES); };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 1, t0, nt, L, T)) return;
    stage_rows<SM::ROW_IO, P>(in_buf(c & 1), p.x.row(n, h, t0), p.x.sl, nt, tid);
  };
  stage_chunk(0);
  cp_async_commit();
  // reset flags travel one chunk ahead in a register
  int dn_next = 0;
  if (has_done && tid < min(T, L)) dn_next = p.done[(long long)n * p.done_sn + (long long)tid * p.done_sl];

  int par = 0;
  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 1, t0, nt, L, T)) break;
    if (c + 1 < nchunks) stage_chunk(c + 1);
    cp_async_commit();
    if (has_done) {
      if (tid < T) sdone[tid] = (unsigned char)dn_next;
      if (tid < min(T, L - t0 - T))
        dn_next = p.done[(long long)n * p.done_sn + (long long)(t0 + T + tid) * p.done_sl];
    }
    cp_async_wait<1>();
    __syncthreads();   // chunk c (and, first time, w_b) visible; output stage free again
    const TIO* sx = in_buf(c & 1);
    const float* sxs = nullptr;   // softmax(x) of this chunk, when the kernel applies it
    if constexpr (EXT) {
      if (smx) {
        float* d = sizeof(TIO) == 4 ? reinterpret_cast<float*>(in_buf(c & 1)) : xf32;
        softmax_rows<TIO, E, P, T>(sx, d, nt, tid);
        __syncthreads();
        sxs = d;
      }
    }
    // reset flags of the chunk as a bit mask (one ballot per chunk instead of a load per step)
    const unsigned dmask = has_done ? __ballot_sync(0xffffffffu, (tid % 32) < nt && sdone[tid % 32] != 0) : 0u;

    #pragma unroll 1

    for (int t = 0; t < nt; ++t, par ^= 1) {
      if constexpr (EXT) {
        if ((dmask >> t) & 1u) {   // episode boundary: the shift goes back to zero
          load_tile<E, C, R, NRG>(p.bWy.mat(n, h), rg, cg, Wy);
          load_tile<E, C, R, NRG>(p.bWq.mat(n, h), rg, cg, Wq);
          load_tile<E, C, R, NRG>(p.bWk.mat(n, h), rg, cg, Wk);
          if (jb >= 0) {
            const float* bb = p.bwb.mat(n, h);
            float wr0[R];
#pragma unroll
            for (int i = 0; i < R; ++i) wr0[i] = bb[row_of<R, NRG>(rg, i) * 4 + jb];
            st_rows<R, NRG>(wbT + jb * E, rg, wr0);
          }
        }
      }
      // ---- pass 1: [y, q~, k~, b~] = x.W ------------------------------------------------
      float xr[R];
      if (EXT && sxs) ld_rows<R, NRG>(sxs + t * E, rg, xr);
      else ld_rows<R, NRG>(sx + t * E, rg, xr);
      u64 ay[C], aq[C], ak[C];
#pragma unroll
      for (int j = 0; j < C; ++j) { ay[j] = 0ull; aq[j] = 0ull; ak[j] = 0ull; }
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        const u64 x2 = pack2(xr[2 * i2], xr[2 * i2 + 1]);
#pragma unroll
        for (int j = 0; j < C; ++j) {
          ay[j] = fma2<PK>(x2, Wy[i2][j], ay[j]);
          aq[j] = fma2<PK>(x2, Wq[i2][j], aq[j]);
          ak[j] = fma2<PK>(x2, Wk[i2][j], ak[j]);
        }
      }
      float pb = 0.f;
      if (jb >= 0) {
        float wr[R];
        ld_rows<R, NRG>(wbT + jb * E, rg, wr);
#pragma unroll
        for (int i = 0; i < R; ++i) pb = fmaf(xr[i], wr[i], pb);
      }
      float y[C], qp[C], kp[C];
#pragma unroll
      for (int j = 0; j < C; ++j) {
        y[j] = allreduce_rows<NRG>(hsum2(ay[j]));
        qp[j] = allreduce_rows<NRG>(hsum2(aq[j]));
        kp[j] = allreduce_rows<NRG>(hsum2(ak[j]));
      }
      pb = allreduce_rows<NRG>(pb);
      float* xq_cur = xq + par * 2 * E;
      if (rg == 0) {
        st_vec<C>(sy + t * E + cg * C, y);
        st_vec<C>(xq_cur + cg * C, qp);
        st_vec<C>(xq_cur + E + cg * C, kp);
        if (jb >= 0) {
          const float b = fast_sigmoid(pb);
          xbeta[par * 4 + jb] = b;
          sbeta[t * 4 + jb] = b;
        }
      }
      __syncthreads();

      // ---- softmax of q~ and k~ on this thread's rows ------------------------------------
      float qr[R], kr[R];
      ld_rows<R, NRG>(xq_cur, rg, qr);
      ld_rows<R, NRG>(xq_cur + E, rg, kr);
      float mq = qr[0], mk = kr[0];
#pragma unroll
      for (int i = 1; i < R; ++i) { mq = fmaxf(mq, qr[i]); mk = fmaxf(mk, kr[i]); }
      mq = allreduce_rows_max<NRG>(mq);
      mk = allreduce_rows_max<NRG>(mk);
      float sumq = 0.f, sumk = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        qr[i] = __expf(qr[i] - mq);
        kr[i] = __expf(kr[i] - mk);
        sumq += qr[i];
        sumk += kr[i];
      }
      sumq = allreduce_rows<NRG>(sumq);
      sumk = allreduce_rows<NRG>(sumk);
      const float iq = __fdividef(1.f, sumq), ik = __fdividef(1.f, sumk);
#pragma unroll
      for (int i = 0; i < R; ++i) { qr[i] *= iq; kr[i] *= ik; }
      if (save && cg == 0) {
        st_rows<R, NRG>(sq + t * E, rg, qr);
        st_rows<R, NRG>(sk + t * E, rg, kr);
      }
      float beta[4];
      ld_vec<4>(xbeta + par * 4, beta);

      // ---- pass 2: d_Z = (q - k).W_Z ------------------------------------------------------
      u64 k2[R2];
#pragma unroll
      for (int j = 0; j < C; ++j) { ay[j] = 0ull; aq[j] = 0ull; ak[j] = 0ull; }
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
        const u64 d2 = pack2(qr[2 * i2] - kr[2 * i2], qr[2 * i2 + 1] - kr[2 * i2 + 1]);
#pragma unroll
        for (int j = 0; j < C; ++j) {
          ay[j] = fma2<PK>(d2, Wy[i2][j], ay[j]);
          aq[j] = fma2<PK>(d2, Wq[i2][j], aq[j]);
          ak[j] = fma2<PK>(d2, Wk[i2][j], ak[j]);
        }
      }
      float db = 0.f;
      float wr[R];
      if (jb >= 0) {
        ld_rows<R, NRG>(wbT + jb * E, rg, wr);
#pragma unroll
        for (int i = 0; i < R; ++i) db = fmaf(qr[i] - kr[i], wr[i], db);
      }
      float dy[C], dq[C], dk[C];
#pragma unroll
      for (int j = 0; j < C; ++j) {
        dy[j] = allreduce_rows<NRG>(hsum2(ay[j]));
        dq[j] = allreduce_rows<NRG>(hsum2(aq[j]));
        dk[j] = allreduce_rows<NRG>(hsum2(ak[j]));
      }
      db = allreduce_rows<NRG>(db);
      if (save && rg == 0) {
        st_vec<C>(syd + t * E + cg * C, dy);
        st_vec<C>(sqd + t * E + cg * C, dq);
        st_vec<C>(skd + t * E + cg * C, dk);
        if (jb >= 0) sbd[t * 4 + jb] = db;
      }

      // ---- rank-1 update of all four blocks ---------------------------------------------
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 iy = dup2(beta[0] * dy[j]);
        const u64 iq2 = dup2(beta[1] * dq[j]);
        const u64 ik2 = dup2(beta[2] * dk[j]);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          Wy[i2][j] = fma2<PK>(k2[i2], iy, Wy[i2][j]);
          Wq[i2][j] = fma2<PK>(k2[i2], iq2, Wq[i2][j]);
          Wk[i2][j] = fma2<PK>(k2[i2], ik2, Wk[i2][j]);
        }
      }
      if (jb >= 0) {
        const float ib = beta[3] * db;
#pragma unroll
        for (int i = 0; i < R; ++i) wr[i] = fmaf(kr[i], ib, wr[i]);
        st_rows<R, NRG>(wbT + jb * E, rg, wr);   // only this thread ever touches these entries
      }
    }

    __syncthreads();   // output stage of this chunk complete
    flush_rows<SM::ROW_IO, P>(p.out.row(n, h, t0), p.out.sl, sy, nt, tid);
    if (save) {
      flush_rows<SM::ROW_F, P>(p.q.row(n, h, t0), p.q.sl, sq, nt, tid);
      flush_rows<SM::ROW_F, P>(p.k.row(n, h, t0), p.k.sl, sk, nt, tid);
      flush_rows<SM::ROW_F, P>(p.yd.row(n, h, t0), p.yd.sl, syd, nt, tid);
      flush_rows<SM::ROW_F, P>(p.qd.row(n, h, t0), p.qd.sl, sqd, nt, tid);
      flush_rows<SM::ROW_F, P>(p.kd.row(n, h, t0), p.kd.sl, skd, nt, tid);
      flush_rows<16, P>(p.beta.row(n, h, t0), p.beta.sl, sbeta, nt, tid);
      flush_rows<16, P>(p.bd.row(n, h, t0), p.bd.sl, sbd, nt, tid);
    }
  }

  if (has_base) {   // W_* receive the shift W_L - base
    store_tile_diff<E, C, R, NRG>(gWy, p.bWy.mat(n, h), rg, cg, Wy);
    store_tile_diff<E, C, R, NRG>(gWq, p.bWq.mat(n, h), rg, cg, Wq);
    store_tile_diff<E, C, R, NRG>(gWk, p.bWk.mat(n, h), rg, cg, Wk);
  } else {
    store_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
    store_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
    store_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
  }
  __syncthreads();
  {
    const float* bb = has_base ? p.bwb.mat(n, h) : nullptr;
    for (int i = tid; i < 4 * E; i += P) gwb[i] = wbT[(i % 4) * E + i / 4] - (bb ? bb[i] : 0.f);
  }
}

// ---------------------------------------------------------------------------------------
// Forward, column layout (E = 32 or 64; 96 threads).  Warp 0 owns W_y, warp 1 W_q, warp 2
// W_k; lane l holds E/32 whole columns (all E rows) of its block as row pairs.  Both
// matvec passes and the rank-1 update are then thread-local -- no shuffle reductions --
// with the operand vector (x, q-k, k) read from shared memory as 16-byte broadcasts.  The
// q~ / k~ values of a step land 2 per lane in the warp that owns the block, exactly the
// shape of a warp-level softmax (one redux.sync max, one shuffle-tree sum), and warp 0
// meanwhile handles the four w_b columns (lane = column j x an eighth of the rows).
// One block-wide barrier per step (q, k, beta published through the output staging rows).
// ---------------------------------------------------------------------------------------
template <typename TIO, int E, int T, bool EXT = false>
struct SrwmFwdColSmem {
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int IN_BYTES = T * ROW_IO;
  static constexpr int XF_BYTES = sizeof(TIO) == 4 ? 0 : T * ROW_F;   // x converted to fp32
  static constexpr int OUT_BYTES = T * ROW_IO + 5 * T * ROW_F + 2 * T * 16;
  static constexpr int WB_BYTES = 4 * ROW_F;
  static constexpr int DQ_BYTES = 2 * ROW_F;                          // q - k, double buffered
  static constexpr int DONE_BYTES = EXT ? ((T + 15) / 16) * 16 : 0;   // reset flags of the chunk
  static constexpr int TOTAL = 2 * IN_BYTES + XF_BYTES + OUT_BYTES + WB_BYTES + DQ_BYTES + DONE_BYTES;
};

// RST: the in-loop episode resets (F_DONE) are compiled in; the layer-level form without resets keeps
// the plain step loop (the reset path costs registers in a kernel that already spills at E = 64).
template <typename TIO, int E, int T, bool PK, int MINB, bool DPRE, int NRP, bool EXT = false, bool RST = EXT>
__global__ void __launch_bounds__(96, MINB) srwm_fwd_col_kernel(const SrwmFwdParams p) {
  static_assert(E == 16 || E == 32 || E == 64, "column layout: one warp per block");
  static_assert(T <= 32, "reset flags of a chunk travel as one 32-bit mask");
  // Lane (cq, rp) of a warp holds CPL adjacent columns x RL rows (row part rp of NRP) of the
  // warp's block.  NRP = 1 is the pure column layout; NRP > 1 trades a log2(NRP)-stage
  // shuffle per pass for 1/NRP of the broadcast operand loads (the shared-memory data pipe
  // is the busiest unit of this kernel).
  using SM = SrwmFwdColSmem<TIO, E, T, EXT>;
  // At E = 16 a block has only 16 columns: NRP = 2 with one column per lane, and the two
  // row-part lanes of a column both end up holding its (duplicated) pre-activation (DUP).
  constexpr int P = 96, CPL = (E * NRP) / 32, RL = E / NRP, RL2 = RL / 2, RB = E / 8;
  constexpr bool DUP = CPL < NRP;
  constexpr int VPL = DUP ? CPL : CPL / NRP;
  static_assert(NRP == 1 || NRP == 2 || NRP == 4, "row parts per column group");
  static_assert(CPL >= 1 && (CPL * 32) == E * NRP && RL % 4 == 0 && (DUP || CPL % NRP == 0), "bad column-layout shape");
  const int tid = threadIdx.x;
  const int warp = tid / 32, lane = tid % 32;
  constexpr int LPP = 32 / NRP;   // lanes per row part: part rp is lanes [rp*LPP, (rp+1)*LPP) of the warp
  const int rp = lane / LPP, c0 = (lane % LPP) * CPL;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const bool save = !(p.flags & 1u);
  const int jb = lane / 8, r8 = lane % 8;   // warp 0: w_b column / row eighth of this lane

  extern __shared__ __align__(16) unsigned char smem[];
  float* xf32 = reinterpret_cast<float*>(smem + 2 * SM::IN_BYTES);
  unsigned char* s_o = smem + 2 * SM::IN_BYTES + SM::XF_BYTES;
  TIO* sy = reinterpret_cast<TIO*>(s_o);
  float* sq = reinterpret_cast<float*>(s_o + T * SM::ROW_IO);
  float* sk = sq + T * E;
  float* syd = sk + T * E;
  float* sqd = syd + T * E;
  float* skd = sqd + T * E;
  float* sbeta = skd + T * E;   // [T][4]
  float* sbd = sbeta + T * 4;   // [T][4]
  float* wbT = sbd + T * 4;     // [4][E]
  float* sdq = wbT + 4 * E;     // [2][E]  q - k of the current step (DPRE)
  unsigned char* sdone = reinterpret_cast<unsigned char*>(sdq + 2 * E);   // [T] (EXT)
  float* sdz = warp == 0 ? syd : (warp == 1 ? sqd : skd);

  const bool smx = EXT && (p.flags & F_INPUT_SOFTMAX);
  const bool has_base = EXT && (p.flags & F_BASE);
  const bool has_done = EXT && RST && (p.flags & F_DONE);

  u64 W[RL2][CPL];
  float* gW = (warp == 0 ? p.Wy : (warp == 1 ? p.Wq : p.Wk)).mat(n, h);
  float* gwb = p.wb.mat(n, h);
  // slow weights / initial shift of this warp's block (extended form)
  const float* gB = has_base ? (warp == 0 ? p.bWy : (warp == 1 ? p.bWq : p.bWk)).mat(n, h) : nullptr;
  const float* gS = (has_base && (p.flags & F_SHIFT_IN)) ? (warp == 0 ? p.sWy : (warp == 1 ? p.sWq : p.sWk)).mat(n, h)
                                                         : nullptr;
  // local row r of row part rp is global row ((r/4)*NRP + rp)*4 + r%4: quads of rows are
  // interleaved over the row parts, so the lanes of a warp read an operand vector as adjacent
  // 16-byte pieces (no shared-memory bank conflict between row parts)
  auto grow = [&](int r) { return ((r / 4) * NRP + rp) * 4 + (r % 4); };
  // W = ga + gb (gb may be null)
  auto load_state = [&](const float* ga, const float* gb) {
#pragma unroll
    for (int e2 = 0; e2 < RL2; ++e2) {
      float a[CPL], b[CPL];
      ld_vec<CPL>(ga + grow(2 * e2) * E + c0, a);
      ld_vec<CPL>(ga + grow(2 * e2 + 1) * E + c0, b);
      if (EXT && gb) {
        float a1[CPL], b1[CPL];
        ld_vec<CPL>(gb + grow(2 * e2) * E + c0, a1);
        ld_vec<CPL>(gb + grow(2 * e2 + 1) * E + c0, b1);
#pragma unroll
        for (int c = 0; c < CPL; ++c) { a[c] += a1[c]; b[c] += b1[c]; }
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) W[e2][c] = pack2(a[c], b[c]);
    }
  };
  if (has_base) {
    load_state(gB, gS);
    const float* bb = p.bwb.mat(n, h);
    const float* sb = gS ? p.swb.mat(n, h) : nullptr;
    for (int i = tid; i < 4 * E; i += P) wbT[(i % 4) * E + i / 4] = bb[i] + (sb ? sb[i] : 0.f);
  } else {
    load_state(gW, nullptr);
    for (int i = tid; i < 4 * E; i += P) wbT[(i % 4) * E + i / 4] = gwb[i];
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return reinterpret_cast<TIO*>(smem + b * SM::IN_BYTES); };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 2, t0, nt, L, T)) return;
    stage_rows<SM::ROW_IO, P>(in_buf(c & 1), p.x.row(n, h, t0), p.x.sl, nt, tid);
  };
  stage_chunk(0);
  cp_async_commit();
  const u64 neg1 = pack2(-1.f, -1.f);
  int par = 0;
  // reset flags travel one chunk ahead in a register
  int dn_next = 0;
  if (has_done && tid < min(T, L)) dn_next = p.done[(long long)n * p.done_sn + (long long)tid * p.done_sl];

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 2, t0, nt, L, T)) break;
    if (c + 1 < nchunks) stage_chunk(c + 1);
    cp_async_commit();
    if (has_done) {
      if (tid < T) sdone[tid] = (unsigned char)dn_next;
      if (tid < min(T, L - t0 - T))
        dn_next = p.done[(long long)n * p.done_sn + (long long)(t0 + T + tid) * p.done_sl];
    }
    cp_async_wait<1>();
    __syncthreads();
    const float* sxf;
    if constexpr (sizeof(TIO) == 4) {
      float* xs = reinterpret_cast<float*>(in_buf(c & 1));
      if (smx) {
        softmax_rows<TIO, E, P, T>(xs, xs, nt, tid);
        __syncthreads();
      }
      sxf = xs;
    } else {
      if (smx) softmax_rows<TIO, E, P, T>(in_buf(c & 1), xf32, nt, tid);
      else convert_rows<TIO, E, P>(in_buf(c & 1), xf32, nt, tid);
      __syncthreads();
      sxf = xf32;
    }
    // reset flags of the chunk as a bit mask (one ballot per chunk instead of a load per step)
    const unsigned dmask = has_done ? __ballot_sync(0xffffffffu, lane < nt && sdone[lane] != 0) : 0u;

    #pragma unroll 1

    for (int t = 0; t < nt; ++t, par ^= 1) {
      if constexpr (EXT && RST) {
        if ((dmask >> t) & 1u) {   // episode boundary: the shift goes back to zero
          load_state(gB, nullptr);
          if (warp == 0) {
            const float* bb = p.bwb.mat(n, h);
#pragma unroll
            for (int i = 0; i < RB; ++i) wbT[jb * E + r8 * RB + i] = bb[(r8 * RB + i) * 4 + jb];
          }
        }
      }
      const float* xr = sxf + t * E;
      const float* qr = sq + t * E;
      const float* kr = sk + t * E;
      float* dq = sdq + par * E;
      // ---- pass 1: this lane's part of x.W --------------------------------------------------
      u64 a0[CPL], a1[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) { a0[cc] = 0ull; a1[cc] = 0ull; }
#pragma unroll
      for (int e4 = 0; e4 < RL / 4; ++e4) {
        const float4 xv = reinterpret_cast<const float4*>(xr)[e4 * NRP + rp];
        const u64 p0 = pack2(xv.x, xv.y), p1 = pack2(xv.z, xv.w);
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) {
          a0[cc] = fma2<PK>(p0, W[2 * e4][cc], a0[cc]);
          a1[cc] = fma2<PK>(p1, W[2 * e4 + 1][cc], a1[cc]);
        }
      }
      float v[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) v[cc] = hsum2(a0[cc]) + hsum2(a1[cc]);
      float vs[VPL];
      int cs;
      if constexpr (DUP) {
#pragma unroll
        for (int i = 0; i < CPL; ++i) vs[i] = allreduce_parts<NRP>(v[i]);   // every row-part lane gets the column
        cs = c0;
      } else {
        reduce_scatter<CPL, NRP, LPP>(v, lane);   // lane rp keeps columns c0 + rp*VPL .. + VPL
#pragma unroll
        for (int i = 0; i < VPL; ++i) vs[i] = v[i];
        cs = c0 + rp * VPL;
      }
      const bool writer = !DUP || rp == 0;
      if (warp == 0) {
        if (writer) st_vec<VPL>(sy + t * E + cs, vs);
        float xrow[RB], wrow[RB];
        ld_vec<RB>(xr + r8 * RB, xrow);
        ld_vec<RB>(wbT + jb * E + r8 * RB, wrow);
        float pb = 0.f;
#pragma unroll
        for (int i = 0; i < RB; ++i) pb = fmaf(xrow[i], wrow[i], pb);
        pb = allreduce_rows<8>(pb);
        if (r8 == 0) sbeta[t * 4 + jb] = fast_sigmoid(pb);
      } else {
        float m = vs[0];
#pragma unroll
        for (int i = 1; i < VPL; ++i) m = fmaxf(m, vs[i]);
        m = warp_max(m);
        float ssum = 0.f;
#pragma unroll
        for (int i = 0; i < VPL; ++i) { vs[i] = __expf(vs[i] - m); ssum += vs[i]; }
        ssum = allreduce_warp(ssum);
        const float inv = __fdividef(DUP ? (float)NRP : 1.f, ssum);   // duplicated columns were summed NRP times
#pragma unroll
        for (int i = 0; i < VPL; ++i) vs[i] *= inv;
        if (writer) st_vec<VPL>((warp == 1 ? sq : sk) + t * E + cs, vs);
        if constexpr (DPRE) {
          // the k warp publishes q - k once for everybody: it needs q from the q warp,
          // handed over through a two-warp named barrier
          asm volatile("bar.sync 1, 64;" ::: "memory");
          if (warp == 2 && writer) {
            float qv[VPL];
            ld_vec<VPL>(qr + cs, qv);
#pragma unroll
            for (int i = 0; i < VPL; ++i) qv[i] -= vs[i];
            st_vec<VPL>(dq + cs, qv);
          }
        }
      }
      __syncthreads();

      // ---- pass 2: d_Z = (q - k).W_Z --------------------------------------------------------
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) { a0[cc] = 0ull; a1[cc] = 0ull; }
#pragma unroll
      for (int e4 = 0; e4 < RL / 4; ++e4) {
        u64 d0, d1;
        if constexpr (DPRE) {
          const float4 dv = reinterpret_cast<const float4*>(dq)[e4 * NRP + rp];
          d0 = pack2(dv.x, dv.y);
          d1 = pack2(dv.z, dv.w);
        } else {
          const float4 qv = reinterpret_cast<const float4*>(qr)[e4 * NRP + rp];
          const float4 kv = reinterpret_cast<const float4*>(kr)[e4 * NRP + rp];
          d0 = fma2<PK>(pack2(kv.x, kv.y), neg1, pack2(qv.x, qv.y));
          d1 = fma2<PK>(pack2(kv.z, kv.w), neg1, pack2(qv.z, qv.w));
        }
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) {
          a0[cc] = fma2<PK>(d0, W[2 * e4][cc], a0[cc]);
          a1[cc] = fma2<PK>(d1, W[2 * e4 + 1][cc], a1[cc]);
        }
      }
      const float bz = sbeta[t * 4 + warp];
      u64 ins2[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) {
        v[cc] = allreduce_parts<NRP>(hsum2(a0[cc]) + hsum2(a1[cc]));
        ins2[cc] = dup2(bz * v[cc]);
      }
      if (rp == 0) st_vec<CPL>(sdz + t * E + c0, v);
      if (warp == 0) {   // w_b column jb, rows of this lane
        float qrow[RB], krow[RB], wrow[RB];
        ld_vec<RB>(qr + r8 * RB, qrow);
        ld_vec<RB>(kr + r8 * RB, krow);
        ld_vec<RB>(wbT + jb * E + r8 * RB, wrow);
        float db = 0.f;
#pragma unroll
        for (int i = 0; i < RB; ++i) db = fmaf(qrow[i] - krow[i], wrow[i], db);
        db = allreduce_rows<8>(db);
        if (r8 == 0) sbd[t * 4 + jb] = db;
        const float ib = sbeta[t * 4 + 3] * db;
#pragma unroll
        for (int i = 0; i < RB; ++i) wrow[i] = fmaf(krow[i], ib, wrow[i]);
        st_vec<RB>(wbT + jb * E + r8 * RB, wrow);
      }
      // ---- rank-1 update -------------------------------------------------------------------
#pragma unroll
      for (int e4 = 0; e4 < RL / 4; ++e4) {
        const float4 kv = reinterpret_cast<const float4*>(kr)[e4 * NRP + rp];
        const u64 k0 = pack2(kv.x, kv.y), k1 = pack2(kv.z, kv.w);
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) {
          W[2 * e4][cc] = fma2<PK>(k0, ins2[cc], W[2 * e4][cc]);
          W[2 * e4 + 1][cc] = fma2<PK>(k1, ins2[cc], W[2 * e4 + 1][cc]);
        }
      }
    }

    __syncthreads();
    flush_rows<SM::ROW_IO, P>(p.out.row(n, h, t0), p.out.sl, sy, nt, tid);
    if (save) {
      flush_rows<SM::ROW_F, P>(p.q.row(n, h, t0), p.q.sl, sq, nt, tid);
      flush_rows<SM::ROW_F, P>(p.k.row(n, h, t0), p.k.sl, sk, nt, tid);
      flush_rows<SM::ROW_F, P>(p.yd.row(n, h, t0), p.yd.sl, syd, nt, tid);
      flush_rows<SM::ROW_F, P>(p.qd.row(n, h, t0), p.qd.sl, sqd, nt, tid);
      flush_rows<SM::ROW_F, P>(p.kd.row(n, h, t0), p.kd.sl, skd, nt, tid);
      flush_rows<16, P>(p.beta.row(n, h, t0), p.beta.sl, sbeta, nt, tid);
      flush_rows<16, P>(p.bd.row(n, h, t0), p.bd.sl, sbd, nt, tid);
    }
  }

#pragma unroll
  for (int e2 = 0; e2 < RL2; ++e2) {
    float a[CPL], b[CPL];
#pragma unroll
    for (int cc = 0; cc < CPL; ++cc) unpack2(W[e2][cc], a[cc], b[cc]);
    if (EXT && gB) {   // W_* receive the shift W_L - base
      float a1[CPL], b1[CPL];
      ld_vec<CPL>(gB + grow(2 * e2) * E + c0, a1);
      ld_vec<CPL>(gB + grow(2 * e2 + 1) * E + c0, b1);
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) { a[cc] -= a1[cc]; b[cc] -= b1[cc]; }
    }
    st_vec<CPL>(gW + grow(2 * e2) * E + c0, a);
    st_vec<CPL>(gW + grow(2 * e2 + 1) * E + c0, b);
  }
  __syncthreads();
  {
    const float* bb = has_base ? p.bwb.mat(n, h) : nullptr;
    for (int i = tid; i < 4 * E; i += P) gwb[i] = wbT[(i % 4) * E + i / 4] - (bb ? bb[i] : 0.f);
  }
}

// ---------------------------------------------------------------------------------------
// Backward (reverse time).  With G_Z = dL/dW_Z after the update of step t, g = dL/dy_t:
//   ins_Z = b_Z d_Z ;  W_Z -= k^T ins_Z                       (rebuilds W(t-1))
//   r_Z = k.G_Z ; gd_Z = b_Z r_Z ; gb~_Z = b_Z(1-b_Z) r_Z.d_Z
//   gk = sum_Z G_Z ins_Z - u ,  gq = u ,  u = sum_Z W_Z(t-1) gd_Z ;  G_Z += (q-k)^T gd_Z
//   gq~ = q (gq - gq.q) ; gk~ = k (gk - gk.k) ; pre = [g | gq~ | gk~ | gb~]
//   gx = W(t-1) pre ;  G += x^T pre
// (the arithmetic of self_ref_v0.cu:694-1187).  Phase 1 runs up to the row sums (gq, gk and
// the six scalars), which cross warps through shared memory and the step's single
// barrier; phase 2 finishes the step.  gx is an output only: its per-warp partials are
// parked in shared memory and summed when the chunk is written out.
// ---------------------------------------------------------------------------------------
template <typename TIO, int E, int P, int T, bool EXT = false>
struct SrwmBwdSmem {
  static constexpr int NWARP = P / 32;
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  // x, gout (io) | q, k, yd, qd, kd (f32) | beta, bd ([T][4] f32)
  static constexpr int IN_BYTES = 2 * T * ROW_IO + 5 * T * ROW_F + 2 * T * 16;
  static constexpr int GX_BYTES = T * NWARP * ROW_F;             // per-warp partial gx
  static constexpr int XROW_BYTES = 2 * NWARP * 2 * ROW_F;       // [2 parity][NWARP][gq,gk][E]
  static constexpr int XSC_BYTES = 2 * NWARP * 8 * 4;            // [2][NWARP][8] scalars
  static constexpr int WB_BYTES = 2 * 4 * ROW_F;                 // w_b^T and its gradient
  static constexpr int XF_BYTES = (EXT && sizeof(TIO) != 4) ? T * ROW_F : 0;   // x (or softmax(x)) in fp32
  static constexpr int TOTAL = 2 * IN_BYTES + GX_BYTES + XROW_BYTES + XSC_BYTES + WB_BYTES + XF_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB, bool EXT = false>
__global__ void __launch_bounds__(P, MINB) srwm_bwd_kernel(const SrwmBwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = SrwmBwdSmem<TIO, E, P, T, EXT>;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2, NWARP = TL::NWARP, CGW = TL::CGW;
  // Row sums and scalars leave the warp through reduce-scatters when the tile shape allows
  // it (every lane ends up with a distinct piece); otherwise through butterfly all-reduces.
  constexpr bool SCATTER = (CGW >= 2) && (R % CGW == 0) && (8 % NRG == 0);
  constexpr int S_ROW = SCATTER ? (2 * R) / CGW : R;   // [u | gk] values per lane after the scatter
  constexpr int S_GX = SCATTER ? R / CGW : R;
  constexpr int S_SC = SCATTER ? 8 / NRG : 8;
  // column sums (3C+1 values over the NRG row-group lanes): padded to a power of two
  constexpr int NVC = 3 * C + 1;
  constexpr int PADN = NVC <= 4 ? 4 : (NVC <= 8 ? 8 : 16);
  constexpr int S_COL = PADN / NRG > 0 ? PADN / NRG : 1;
  // (at E = 64 the state already fills the register file and the scatter's staging array spills:
  // measured slower there, faster at E <= 32)
  constexpr bool RSCAT = (E <= 32) && (NRG >= 2) && (PADN % NRG == 0) && (PADN >= NRG) && (C % S_COL == 0) &&
                         (NVC <= 16);
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int warp = tid / 32, lane = tid % 32;
  const int cgl = lane / NRG;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  // The E x 4 block w_b and its gradient.  WBREG: every warp owns 4/NWARP of the four columns and
  // every lane one row pair of one column, in registers -- the work and the row reduction are
  // spread evenly over the block (left to the column groups 0..3, i.e. to warp 0, it put a
  // tenth more instructions on the one warp the step's barrier then waits for).  Otherwise the
  // columns live transposed in shared memory and column groups 0..3 handle one each.
  constexpr int CPW = NWARP <= 4 ? 4 / NWARP : 0;
  constexpr bool WBREG = (NWARP <= 4) && (CGW == CPW * R2);
  const int wi2 = cgl % R2;                                   // WBREG: row pair of this lane
  const int wrow = row_of<R, NRG>(rg, 2 * wi2);               // its first row (the second is wrow + 1)
  const int jb = WBREG ? warp * CPW + cgl / R2 : (cg < 4 ? cg : -1);
  float wbr[2] = {0.f, 0.f}, gbr[2] = {0.f, 0.f};

  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* s_o = smem + 2 * SM::IN_BYTES;
  float* sgx = reinterpret_cast<float*>(s_o);                               // [T][NWARP][E]
  float* xrow = reinterpret_cast<float*>(s_o + SM::GX_BYTES);               // [2][NWARP][2][E]
  float* xsc = reinterpret_cast<float*>(s_o + SM::GX_BYTES + SM::XROW_BYTES);  // [2][NWARP][8]
  float* wbT = xsc + 2 * NWARP * 8;                                         // [4][E]
  float* gbT = wbT + 4 * E;                                                 // [4][E]
  float* xf32 = gbT + 4 * E;                                                // [T][E] (EXT, bf16 streams)

  const bool smx = EXT && (p.flags & F_INPUT_SOFTMAX);
  const bool has_base = EXT && (p.flags & F_BASE);

  u64 Wy[R2][C], Wq[R2][C], Wk[R2][C], Gy[R2][C], Gq[R2][C], Gk[R2][C];
  float* gWy = p.Wy.mat(n, h);
  float* gWq = p.Wq.mat(n, h);
  float* gWk = p.Wk.mat(n, h);
  float* gwb = p.wb.mat(n, h);
  if (has_base) {   // W_* hold the final shift: W_L = base + shift
    load_tile_sum<E, C, R, NRG>(gWy, p.bWy.mat(n, h), rg, cg, Wy);
    load_tile_sum<E, C, R, NRG>(gWq, p.bWq.mat(n, h), rg, cg, Wq);
    load_tile_sum<E, C, R, NRG>(gWk, p.bWk.mat(n, h), rg, cg, Wk);
  } else {
    load_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
    load_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
    load_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
  }
  const bool gin = (p.flags & 2u) != 0;
  if (gin) {
    load_tile<E, C, R, NRG>(p.gWy.mat(n, h), rg, cg, Gy);
    load_tile<E, C, R, NRG>(p.gWq.mat(n, h), rg, cg, Gq);
    load_tile<E, C, R, NRG>(p.gWk.mat(n, h), rg, cg, Gk);
  } else {
#pragma unroll
    for (int i2 = 0; i2 < R2; ++i2)
#pragma unroll
      for (int j = 0; j < C; ++j) { Gy[i2][j] = 0ull; Gq[i2][j] = 0ull; Gk[i2][j] = 0ull; }
  }
  {
    const float* ggwb = p.gwb.mat(n, h);
    const float* bb = has_base ? p.bwb.mat(n, h) : nullptr;
    if constexpr (WBREG) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = (wrow + u) * 4 + jb;
        wbr[u] = gwb[i] + (bb ? bb[i] : 0.f);
        gbr[u] = gin ? ggwb[i] : 0.f;
      }
    } else {
      for (int i = tid; i < 4 * E; i += P) {
        wbT[(i % 4) * E + i / 4] = gwb[i] + (bb ? bb[i] : 0.f);
        gbT[(i % 4) * E + i / 4] = gin ? ggwb[i] : 0.f;
      }
    }
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 3, t0, nt, L, T)) return;
    unsigned char* ib = in_buf(c & 1);
    stage_rows<SM::ROW_IO, P>(ib, p.x.row(n, h, t0), p.x.sl, nt, tid);
    stage_rows<SM::ROW_IO, P>(ib + T * SM::ROW_IO, p.gout.row(n, h, t0), p.gout.sl, nt, tid);
    unsigned char* fb = ib + 2 * T * SM::ROW_IO;
    stage_rows<SM::ROW_F, P>(fb, p.q.row(n, h, t0), p.q.sl, nt, tid);
    stage_rows<SM::ROW_F, P>(fb + 1 * T * SM::ROW_F, p.k.row(n, h, t0), p.k.sl, nt, tid);
    stage_rows<SM::ROW_F, P>(fb + 2 * T * SM::ROW_F, p.yd.row(n, h, t0), p.yd.sl, nt, tid);
    stage_rows<SM::ROW_F, P>(fb + 3 * T * SM::ROW_F, p.qd.row(n, h, t0), p.qd.sl, nt, tid);
    stage_rows<SM::ROW_F, P>(fb + 4 * T * SM::ROW_F, p.kd.row(n, h, t0), p.kd.sl, nt, tid);
    unsigned char* bb = fb + 5 * T * SM::ROW_F;
    stage_rows<16, P>(bb, p.beta.row(n, h, t0), p.beta.sl, nt, tid);
    stage_rows<16, P>(bb + T * 16, p.bd.row(n, h, t0), p.bd.sl, nt, tid);
  };
  if (nchunks > 0) stage_chunk(nchunks - 1);   // (an empty sequence has nothing to stage: dL/dW_0 = dL/dW_L)
  cp_async_commit();

  int par = 0;
  for (int c = nchunks - 1; c >= 0; --c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 3, t0, nt, L, T)) break;
    if (c > 0) stage_chunk(c - 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    unsigned char* ib = in_buf(c & 1);
    const TIO* sx = reinterpret_cast<const TIO*>(ib);
    // in the extended form x is read as fp32 rows: softmax(x) when the kernel applies it
    const float* sxs = reinterpret_cast<const float*>(ib);
    if constexpr (EXT) {
      if constexpr (sizeof(TIO) == 4) {
        if (smx) {
          softmax_rows<TIO, E, P, T>(sx, reinterpret_cast<float*>(ib), nt, tid);
          __syncthreads();
        }
      } else {
        if (smx) softmax_rows<TIO, E, P, T>(sx, xf32, nt, tid);
        else convert_rows<TIO, E, P>(sx, xf32, nt, tid);
        __syncthreads();
        sxs = xf32;
      }
    }
    const TIO* sg = reinterpret_cast<const TIO*>(ib + T * SM::ROW_IO);
    const float* sq = reinterpret_cast<const float*>(ib + 2 * T * SM::ROW_IO);
    const float* sk = sq + T * E;
    const float* syd = sk + T * E;
    const float* sqd = syd + T * E;
    const float* skd = sqd + T * E;
    const float* sbeta = skd + T * E;
    const float* sbd = sbeta + T * 4;

    #pragma unroll 1

    for (int t = nt - 1; t >= 0; --t, par ^= 1) {
      // ================= phase 1 =================
      float beta[4];
      ld_vec<4>(sbeta + t * 4, beta);
      u64 k2[R2], gkr2[R2];
      {
        float kr[R];
        ld_rows<R, NRG>(sk + t * E, rg, kr);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
          gkr2[i2] = 0ull;
        }
      }
      // per block: undo the update, r = k.G (column partial), gk partial += G ins (row partial)
      float rcol[3][C];
      auto blk1 = [&](u64 (&W)[R2][C], u64 (&G)[R2][C], const float* sd, float bz, float (&rz)[C]) {
        float dz[C];
        ld_vec<C>(sd + t * E + cg * C, dz);
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 nins = dup2(-bz * dz[j]);   // minus the inserted value: undoes the update; gkr2 collects -G.ins
          u64 ar = 0ull;
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) {
            W[i2][j] = fma2<PK>(k2[i2], nins, W[i2][j]);
            ar = fma2<PK>(k2[i2], G[i2][j], ar);
            gkr2[i2] = fma2<PK>(G[i2][j], nins, gkr2[i2]);
          }
          rz[j] = hsum2(ar);
        }
      };
      blk1(Wy, Gy, syd, beta[0], rcol[0]);
      blk1(Wq, Gq, sqd, beta[1], rcol[1]);
      blk1(Wk, Gk, skd, beta[2], rcol[2]);
      float gkr[R], ur[R];   // gkr holds MINUS the row partial of G.ins until the subtraction of u below
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(gkr2[i2], gkr[2 * i2], gkr[2 * i2 + 1]);
      // w_b column jb: same three operations on shared-memory state
      float rb = 0.f, bdj = 0.f;
      if constexpr (WBREG) {
        float kp0 = 0.f, kp1 = 0.f;
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2)
          if (i2 == wi2) unpack2(k2[i2], kp0, kp1);
        bdj = sbd[t * 4 + jb];
        const float insb = beta[3] * bdj;
        wbr[0] = fmaf(-kp0, insb, wbr[0]);
        wbr[1] = fmaf(-kp1, insb, wbr[1]);
        rb = fmaf(kp1, gbr[1], kp0 * gbr[0]);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2)
          if (i2 == wi2) {
            gkr[2 * i2] = fmaf(-gbr[0], insb, gkr[2 * i2]);
            gkr[2 * i2 + 1] = fmaf(-gbr[1], insb, gkr[2 * i2 + 1]);
          }
#pragma unroll
        for (int off = 1; off < NRG * R2; off <<= 1) rb += __shfl_xor_sync(0xffffffffu, rb, off);   // all rows of the column
      } else if (jb >= 0) {
        float kr[R], wr[R], gr[R];
        ld_rows<R, NRG>(sk + t * E, rg, kr);
        ld_rows<R, NRG>(wbT + jb * E, rg, wr);
        ld_rows<R, NRG>(gbT + jb * E, rg, gr);
        bdj = sbd[t * 4 + jb];
        const float insb = beta[3] * bdj;
#pragma unroll
        for (int i = 0; i < R; ++i) {
          wr[i] = fmaf(-kr[i], insb, wr[i]);
          rb = fmaf(kr[i], gr[i], rb);
          gkr[i] = fmaf(-gr[i], insb, gkr[i]);
        }
        st_rows<R, NRG>(wbT + jb * E, rg, wr);
      }
      // complete r over the row groups; gd = b r; scalar partials r.d
      float sc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float gdb;
      if constexpr (RSCAT) {
        // reduce-scatter the 3C+1 column sums over the row-group lanes, let each lane finish its
        // S of them (all of one block, since S divides C), then hand every lane all of gd
        float v[PADN];
#pragma unroll
        for (int i = 0; i < PADN; ++i) v[i] = 0.f;
#pragma unroll
        for (int z = 0; z < 3; ++z)
#pragma unroll
          for (int j = 0; j < C; ++j) v[z * C + j] = rcol[z][j];
        if constexpr (!WBREG) v[3 * C] = rb;   // (WBREG: the column sum of w_b is already complete)
        reduce_scatter<PADN, NRG, 1>(v, lane);
        const int g0 = rg * S_COL;
        const int zl = min(g0 / C, 3);                     // block of this lane's values (3: the w_b column)
        const float bz = sbeta[t * 4 + zl];
        float fin[S_COL], sbl = 0.f;
#pragma unroll
        for (int i = 0; i < S_COL; ++i) {
          const int g = g0 + i;
          float dzv;
          if (zl < 3) dzv = syd[zl * T * E + t * E + cg * C + (g % C)];   // y_diff, q_diff, k_diff rows are adjacent
          else dzv = (g == 3 * C && jb >= 0) ? sbd[t * 4 + jb] : 0.f;
          sbl = fmaf(v[i], dzv, sbl);
          fin[i] = bz * v[i];
        }
#pragma unroll
        for (int zz = 0; zz < 4; ++zz) sc8[zz] = (zl == zz) ? sbl : 0.f;
        const int base = lane & ~(NRG - 1);
#pragma unroll
        for (int z = 0; z < 3; ++z)
#pragma unroll
          for (int j = 0; j < C; ++j)
            rcol[z][j] = __shfl_sync(0xffffffffu, fin[(z * C + j) % S_COL], base + (z * C + j) / S_COL);   // now gd
        if constexpr (WBREG) {
          gdb = beta[3] * rb;
          sc8[3] += (rg == 0 && wi2 == 0) ? rb * bdj : 0.f;
        } else {
          gdb = __shfl_sync(0xffffffffu, fin[(3 * C) % S_COL], base + (3 * C) / S_COL);
        }
      } else {
#pragma unroll
        for (int z = 0; z < 3; ++z) {
          float dz[C];
          ld_vec<C>((z == 0 ? syd : (z == 1 ? sqd : skd)) + t * E + cg * C, dz);
#pragma unroll
          for (int j = 0; j < C; ++j) {
            const float r = allreduce_rows<NRG>(rcol[z][j]);
            sc8[z] = fmaf(r, dz[j], sc8[z]);
            rcol[z][j] = beta[z] * r;   // now gd
          }
        }
        if constexpr (!WBREG) rb = allreduce_rows<NRG>(rb);
        gdb = beta[3] * rb;
        sc8[3] = rb * bdj;
        if (rg != 0) { sc8[0] = 0.f; sc8[1] = 0.f; sc8[2] = 0.f; sc8[3] = 0.f; }   // count each column once
        if constexpr (WBREG)
          if (wi2 != 0) sc8[3] = 0.f;
      }
      // G += (q-k)^T gd ; u = W(t-1) gd (row partial)
      u64 d2[R2], u2[R2];
      {
        float kr[R], qr[R];
        ld_rows<R, NRG>(sk + t * E, rg, kr);
        ld_rows<R, NRG>(sq + t * E, rg, qr);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          d2[i2] = pack2(qr[2 * i2] - kr[2 * i2], qr[2 * i2 + 1] - kr[2 * i2 + 1]);
          u2[i2] = 0ull;
        }
      }
      auto blk2 = [&](u64 (&W)[R2][C], u64 (&G)[R2][C], const float (&gd)[C]) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 g2 = dup2(gd[j]);
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) {
            G[i2][j] = fma2<PK>(d2[i2], g2, G[i2][j]);
            u2[i2] = fma2<PK>(W[i2][j], g2, u2[i2]);
          }
        }
      };
      blk2(Wy, Gy, rcol[0]);
      blk2(Wq, Gq, rcol[1]);
      blk2(Wk, Gk, rcol[2]);
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(u2[i2], ur[2 * i2], ur[2 * i2 + 1]);
      if constexpr (WBREG) {
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2)
          if (i2 == wi2) {
            float da, db;
            unpack2(d2[i2], da, db);
            gbr[0] = fmaf(da, gdb, gbr[0]);
            gbr[1] = fmaf(db, gdb, gbr[1]);
            ur[2 * i2] = fmaf(wbr[0], gdb, ur[2 * i2]);
            ur[2 * i2 + 1] = fmaf(wbr[1], gdb, ur[2 * i2 + 1]);
          }
      } else if (jb >= 0) {
        float wr[R], gr[R];
        ld_rows<R, NRG>(wbT + jb * E, rg, wr);
        ld_rows<R, NRG>(gbT + jb * E, rg, gr);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          float da, db;
          unpack2(d2[i2], da, db);
          gr[2 * i2] = fmaf(da, gdb, gr[2 * i2]);
          gr[2 * i2 + 1] = fmaf(db, gdb, gr[2 * i2 + 1]);
          ur[2 * i2] = fmaf(wr[2 * i2], gdb, ur[2 * i2]);
          ur[2 * i2 + 1] = fmaf(wr[2 * i2 + 1], gdb, ur[2 * i2 + 1]);
        }
        st_rows<R, NRG>(gbT + jb * E, rg, gr);
      }
      // row partials: gq = u, gk = G ins - u ; their dot products with q, k
      {
        float kr[R], qr[R];
        ld_rows<R, NRG>(sk + t * E, rg, kr);
        ld_rows<R, NRG>(sq + t * E, rg, qr);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          gkr[i] = -gkr[i] - ur[i];
          sc8[4] = fmaf(qr[i], ur[i], sc8[4]);
          sc8[5] = fmaf(kr[i], gkr[i], sc8[5]);
        }
      }
      float* xr_cur = xrow + (par * NWARP + warp) * 2 * E;
      float* xs_cur = xsc + (par * NWARP + warp) * 8;
      if constexpr (SCATTER) {
        float v[2 * R];
#pragma unroll
        for (int i = 0; i < R; ++i) { v[i] = ur[i]; v[R + i] = gkr[i]; }
        reduce_scatter<2 * R, CGW, NRG>(v, lane);
        float piece[S_ROW];
#pragma unroll
        for (int i = 0; i < S_ROW; ++i) piece[i] = v[i];
        // lanes of the lower half of the column groups hold pieces of u, the upper half of gk
        const int which = cgl >= CGW / 2 ? 1 : 0;
        st_rows_piece<S_ROW, R, NRG>(xr_cur + which * E, rg, (cgl % (CGW / 2)) * S_ROW, piece);
        reduce_scatter<8, NRG, 1>(sc8, lane);
        float sp[S_SC];
#pragma unroll
        for (int i = 0; i < S_SC; ++i) sp[i] = allreduce_cols<NRG>(sc8[i]);
        if (cgl == 0) st_vec<S_SC>(xs_cur + rg * S_SC, sp);
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          ur[i] = allreduce_cols<NRG>(ur[i]);
          gkr[i] = allreduce_cols<NRG>(gkr[i]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) sc8[i] = allreduce_warp(sc8[i]);
        if (lane < NRG) {
          st_rows<R, NRG>(xr_cur, rg, ur);
          st_rows<R, NRG>(xr_cur + E, rg, gkr);
        }
        if (lane == 0) st_vec<8>(xs_cur, sc8);
      }
      __syncthreads();

      // ================= phase 2 =================
      // The 2C values gq~ / gk~ of this column group are needed by all its NRG lanes.  Each lane
      // finishes a share of them (sum of the per-warp partials, softmax backward) and the
      // lanes exchange the results with shuffles, instead of every lane redoing all of them.
      constexpr int VPLN = (2 * C + NRG - 1) / NRG;   // values finished per lane
      float mine[VPLN];
#pragma unroll
      for (int u = 0; u < VPLN; ++u) {
        const int v = rg + u * NRG;                   // 0..C-1: gq~ of column v ; C..2C-1: gk~ of column v-C
        const int which = (v >= C) ? 1 : 0;
        const int col = cg * C + (which ? v - C : v);
        float acc = 0.f, dot = 0.f;
        if (v < 2 * C) {
#pragma unroll
          for (int w = 0; w < NWARP; ++w) {
            acc += xrow[(par * NWARP + w) * 2 * E + which * E + col];
            dot += xsc[(par * NWARP + w) * 8 + 4 + which];
          }
          const float sm_val = (which ? sk : sq)[t * E + col];
          acc = sm_val * (acc - dot);
        }
        mine[u] = acc;
      }
      float pre[3][C];
      ld_vec<C>(sg + t * E + cg * C, pre[0]);
#pragma unroll
      for (int j = 0; j < C; ++j) {
        pre[1][j] = __shfl_sync(0xffffffffu, mine[j / NRG], (lane & ~(NRG - 1)) + (j % NRG));
        pre[2][j] = __shfl_sync(0xffffffffu, mine[(C + j) / NRG], (lane & ~(NRG - 1)) + ((C + j) % NRG));
      }
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
      if (jb >= 0) {
#pragma unroll
        for (int w = 0; w < NWARP; ++w) sc[0] += xsc[(par * NWARP + w) * 8 + jb];
      }
      float xr[R];
      if constexpr (EXT) ld_rows<R, NRG>(sxs + t * E, rg, xr);
      else ld_rows<R, NRG>(sx + t * E, rg, xr);
      u64 gx2[R2], x2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        gx2[i2] = 0ull;
        x2[i2] = pack2(xr[2 * i2], xr[2 * i2 + 1]);
      }
      auto blk3 = [&](u64 (&W)[R2][C], u64 (&G)[R2][C], const float (&pz)[C]) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 pd = dup2(pz[j]);
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) {
            gx2[i2] = fma2<PK>(W[i2][j], pd, gx2[i2]);
            G[i2][j] = fma2<PK>(x2[i2], pd, G[i2][j]);
          }
        }
      };
      blk3(Wy, Gy, pre[0]);
      blk3(Wq, Gq, pre[1]);
      blk3(Wk, Gk, pre[2]);
      float gxr[R];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(gx2[i2], gxr[2 * i2], gxr[2 * i2 + 1]);
      if constexpr (WBREG) {
        const float b = sbeta[t * 4 + jb];
        const float pb = sc[0] * b * (1.f - b);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2)
          if (i2 == wi2) {
            gxr[2 * i2] = fmaf(wbr[0], pb, gxr[2 * i2]);
            gxr[2 * i2 + 1] = fmaf(wbr[1], pb, gxr[2 * i2 + 1]);
            gbr[0] = fmaf(xr[2 * i2], pb, gbr[0]);
            gbr[1] = fmaf(xr[2 * i2 + 1], pb, gbr[1]);
          }
      } else if (jb >= 0) {
        float wr[R], gr[R];
        ld_rows<R, NRG>(wbT + jb * E, rg, wr);
        ld_rows<R, NRG>(gbT + jb * E, rg, gr);
        const float b = sbeta[t * 4 + jb];
        const float pb = sc[0] * b * (1.f - b);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          gxr[i] = fmaf(wr[i], pb, gxr[i]);
          gr[i] = fmaf(xr[i], pb, gr[i]);
        }
        st_rows<R, NRG>(gbT + jb * E, rg, gr);
      }
      if constexpr (SCATTER) {
        reduce_scatter<R, CGW, NRG>(gxr, lane);
        float piece[S_GX];
#pragma unroll
        for (int i = 0; i < S_GX; ++i) piece[i] = gxr[i];
        st_rows_piece<S_GX, R, NRG>(sgx + (t * NWARP + warp) * E, rg, cgl * S_GX, piece);
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) gxr[i] = allreduce_cols<NRG>(gxr[i]);
        if (lane < NRG) st_rows<R, NRG>(sgx + (t * NWARP + warp) * E, rg, gxr);
      }
    }

    __syncthreads();
    // gx of this chunk: sum the per-warp partials, convert, store
    for (int idx = tid; idx < nt * (E / 4); idx += P) {
      const int e4 = idx % (E / 4), t = idx / (E / 4);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < NWARP; ++w) {
        float v[4];
        ld_vec<4>(sgx + (t * NWARP + w) * E + e4 * 4, v);
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] += v[u];
      }
      if (EXT && smx) st_vec<4>(sgx + (t * NWARP) * E + e4 * 4, acc);   // finished below, through the softmax
      else st_vec<4>(reinterpret_cast<TIO*>(p.gx.row(n, h, t0 + t)) + e4 * 4, acc);
    }
    if constexpr (EXT) {
      if (smx) {
        __syncthreads();
        softmax_bwd_rows<TIO, E, P, T>(sxs, sgx, NWARP * E, p.gx.row(n, h, t0), p.gx.sl, nt, tid);
        __syncthreads();   // softmax(x) may sit in the staging buffer the next prefetch overwrites
      }
    }
  }

  // dL/dW_0, and optionally the rebuilt W_0
  store_tile<E, C, R, NRG>(p.gWy.mat(n, h), rg, cg, Gy);
  store_tile<E, C, R, NRG>(p.gWq.mat(n, h), rg, cg, Gq);
  store_tile<E, C, R, NRG>(p.gWk.mat(n, h), rg, cg, Gk);
  const bool restore = (p.flags & 4u) != 0;
  if (restore) {   // W_0, or the initial shift W_0 - base in the extended form
    store_tile_diff<E, C, R, NRG>(gWy, has_base ? p.bWy.mat(n, h) : nullptr, rg, cg, Wy);
    store_tile_diff<E, C, R, NRG>(gWq, has_base ? p.bWq.mat(n, h) : nullptr, rg, cg, Wq);
    store_tile_diff<E, C, R, NRG>(gWk, has_base ? p.bWk.mat(n, h) : nullptr, rg, cg, Wk);
  }
  __syncthreads();
  {
    float* ggwb = p.gwb.mat(n, h);
    const float* bb = has_base ? p.bwb.mat(n, h) : nullptr;
    if constexpr (WBREG) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = (wrow + u) * 4 + jb;
        ggwb[i] = gbr[u];
        if (restore) gwb[i] = wbr[u] - (bb ? bb[i] : 0.f);
      }
    } else {
      for (int i = tid; i < 4 * E; i += P) {
        ggwb[i] = gbT[(i % 4) * E + i / 4];
        if (restore) gwb[i] = wbT[(i % 4) * E + i / 4] - (bb ? bb[i] : 0.f);
      }
    }
  }
  if constexpr (EXT) {
    if (p.flags & F_REDUCE) reduce_epilogue<E, P>(p, n, h, tid);
  }
}

// ---------------------------------------------------------------------------------------
// Backward with the state detached at every step.  The reinforcement-learning learner calls
// the layer one step at a time and detaches the state it carries
// (reinforcement_learning/torchbeast/layer.py:412-421 under the loop of
// reinforcement_learning/torchbeast_procgen/model.py:1180-1197), so only
// out_t = x_t.W_y(t-1) carries gradient:
//   gx_t = W_y(t-1) g_t  (then through the input softmax) ,  G_y += x_t^T g_t ,
// and W_q, W_k, w_b receive none.  W_y(t-1) is replayed FORWARD in time from base + shift
// with the saved k, beta_y, d_y (W_y += k^T (b_y d_y)), going back to base where done is set.
// No step waits on another step's reductions: the gx partials are parked per warp and
// combined once per chunk, so the kernel has no barrier inside the time loop.
// ---------------------------------------------------------------------------------------
struct SrwmBwdDetParams {
  int N, H, L;
  unsigned flags;                 // F_INPUT_SOFTMAX, F_SHIFT_IN, F_DONE
  unsigned long long* dbg;   // status word of the debug build (null otherwise)
  SeqView x, k, beta, yd, gout, gx;
  StateView bWy, sWy, gWy;        // initial W_y = bWy (+ sWy); gWy receives sum_t x_t^T g_t
  const unsigned char* done;
  long long done_sn, done_sl;
};

template <typename TIO, int E, int P, int T>
struct SrwmBwdDetSmem {
  static constexpr int NWARP = P / 32;
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int IN_BYTES = 2 * T * ROW_IO + 2 * T * ROW_F + T * 16;   // x, gout | k, yd | beta
  static constexpr int GX_BYTES = T * NWARP * ROW_F;
  static constexpr int XF_BYTES = sizeof(TIO) != 4 ? T * ROW_F : 0;
  static constexpr int DONE_BYTES = ((T + 15) / 16) * 16;
  static constexpr int TOTAL = 2 * IN_BYTES + GX_BYTES + XF_BYTES + DONE_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB>
__global__ void __launch_bounds__(P, MINB) srwm_bwd_det_kernel(const SrwmBwdDetParams p) {
  using TL = Tiling<E, P, R>;
  using SM = SrwmBwdDetSmem<TIO, E, P, T>;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2, NWARP = TL::NWARP;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int warp = tid / 32, lane = tid % 32;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const bool smx = (p.flags & F_INPUT_SOFTMAX) != 0;
  const bool has_done = (p.flags & F_DONE) != 0;

  extern __shared__ __align__(16) unsigned char smem[];
  float* sgx = reinterpret_cast<float*>(smem + 2 * SM::IN_BYTES);           // [T][NWARP][E]
  float* xf32 = reinterpret_cast<float*>(smem + 2 * SM::IN_BYTES + SM::GX_BYTES);
  unsigned char* sdone = smem + 2 * SM::IN_BYTES + SM::GX_BYTES + SM::XF_BYTES;

  u64 W[R2][C], G[R2][C];
  const float* gB = p.bWy.mat(n, h);
  load_tile_sum<E, C, R, NRG>(gB, (p.flags & F_SHIFT_IN) ? p.sWy.mat(n, h) : nullptr, rg, cg, W);
#pragma unroll
  for (int i2 = 0; i2 < R2; ++i2)
#pragma unroll
    for (int j = 0; j < C; ++j) G[i2][j] = 0ull;

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 4, t0, nt, L, T)) return;
    unsigned char* ib = in_buf(c & 1);
    stage_rows<SM::ROW_IO, P>(ib, p.x.row(n, h, t0), p.x.sl, nt, tid);
    stage_rows<SM::ROW_IO, P>(ib + T * SM::ROW_IO, p.gout.row(n, h, t0), p.gout.sl, nt, tid);
    unsigned char* fb = ib + 2 * T * SM::ROW_IO;
    stage_rows<SM::ROW_F, P>(fb, p.k.row(n, h, t0), p.k.sl, nt, tid);
    stage_rows<SM::ROW_F, P>(fb + T * SM::ROW_F, p.yd.row(n, h, t0), p.yd.sl, nt, tid);
    stage_rows<16, P>(fb + 2 * T * SM::ROW_F, p.beta.row(n, h, t0), p.beta.sl, nt, tid);
  };
  stage_chunk(0);
  cp_async_commit();
  int dn_next = 0;
  if (has_done && tid < min(T, L)) dn_next = p.done[(long long)n * p.done_sn + (long long)tid * p.done_sl];

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 4, t0, nt, L, T)) break;
    if (c + 1 < nchunks) stage_chunk(c + 1);
    cp_async_commit();
    if (has_done) {
      if (tid < T) sdone[tid] = (unsigned char)dn_next;
      if (tid < min(T, L - t0 - T))
        dn_next = p.done[(long long)n * p.done_sn + (long long)(t0 + T + tid) * p.done_sl];
    }
    cp_async_wait<1>();
    __syncthreads();   // chunk c staged; sgx, xf32 and sdone of the previous chunk no longer read

    unsigned char* ib = in_buf(c & 1);
    const TIO* sx = reinterpret_cast<const TIO*>(ib);
    const TIO* sg = reinterpret_cast<const TIO*>(ib + T * SM::ROW_IO);
    const float* sk = reinterpret_cast<const float*>(ib + 2 * T * SM::ROW_IO);
    const float* syd = sk + T * E;
    const float* sbeta = syd + T * E;
    const float* sxs = reinterpret_cast<const float*>(ib);
    if constexpr (sizeof(TIO) == 4) {
      if (smx) {
        softmax_rows<TIO, E, P, T>(sx, reinterpret_cast<float*>(ib), nt, tid);
        __syncthreads();
      }
    } else {
      if (smx) softmax_rows<TIO, E, P, T>(sx, xf32, nt, tid);
      else convert_rows<TIO, E, P>(sx, xf32, nt, tid);
      __syncthreads();
      sxs = xf32;
    }

    const unsigned dmask = has_done ? __ballot_sync(0xffffffffu, lane < nt && sdone[lane] != 0) : 0u;
#pragma unroll 1
    for (int t = 0; t < nt; ++t) {
      if ((dmask >> t) & 1u) load_tile<E, C, R, NRG>(gB, rg, cg, W);
      float xr[R], kr[R], g[C], dz[C];
      ld_rows<R, NRG>(sxs + t * E, rg, xr);
      ld_rows<R, NRG>(sk + t * E, rg, kr);
      ld_vec<C>(sg + t * E + cg * C, g);
      ld_vec<C>(syd + t * E + cg * C, dz);
      const float by = sbeta[t * 4];
      u64 gx2[R2], x2[R2], k2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        gx2[i2] = 0ull;
        x2[i2] = pack2(xr[2 * i2], xr[2 * i2 + 1]);
        k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
      }
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 g2 = dup2(g[j]);
        const u64 in2 = dup2(by * dz[j]);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          gx2[i2] = fma2<PK>(W[i2][j], g2, gx2[i2]);      // with W_y(t-1)
          G[i2][j] = fma2<PK>(x2[i2], g2, G[i2][j]);
          W[i2][j] = fma2<PK>(k2[i2], in2, W[i2][j]);     // the step's update
        }
      }
      float gxr[R];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(gx2[i2], gxr[2 * i2], gxr[2 * i2 + 1]);
#pragma unroll
      for (int i = 0; i < R; ++i) gxr[i] = allreduce_cols<NRG>(gxr[i]);
      if (lane < NRG) st_rows<R, NRG>(sgx + (t * NWARP + warp) * E, rg, gxr);
    }

    __syncthreads();
    for (int idx = tid; idx < nt * (E / 4); idx += P) {
      const int e4 = idx % (E / 4), t = idx / (E / 4);
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < NWARP; ++w) {
        float v[4];
        ld_vec<4>(sgx + (t * NWARP + w) * E + e4 * 4, v);
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] += v[u];
      }
      if (smx) st_vec<4>(sgx + (t * NWARP) * E + e4 * 4, acc);
      else st_vec<4>(reinterpret_cast<TIO*>(p.gx.row(n, h, t0 + t)) + e4 * 4, acc);
    }
    if (smx) {
      __syncthreads();
      softmax_bwd_rows<TIO, E, P, T>(sxs, sgx, NWARP * E, p.gx.row(n, h, t0), p.gx.sl, nt, tid);
      __syncthreads();   // softmax(x) may sit in the staging buffer the next prefetch overwrites
    }
  }
  store_tile<E, C, R, NRG>(p.gWy.mat(n, h), rg, cg, G);
}

}  // namespace srwm
