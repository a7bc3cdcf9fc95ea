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
// The three E x E blocks W_y, W_q, W_k share one register tiling (common.cuh); the small
// E x 4 block w_b lives transposed in shared memory and is handled by one column group
// per column (column j by group j*NCG/4).  One block-wide barrier per time step, placed
// where the softmax needs all of q~ / k~ (forward) or where the row sums of the backward
// have to cross warps.
#pragma once
#include "common.cuh"

namespace srwm {

struct SrwmFwdParams {
  int N, H, L;
  unsigned flags;
  SeqView x, out, q, k, beta, yd, qd, kd, bd;
  StateView Wy, Wq, Wk, wb;
};

struct SrwmBwdParams {
  int N, H, L;
  unsigned flags;
  SeqView x, q, k, beta, yd, qd, kd, bd, gout, gx;
  StateView Wy, Wq, Wk, wb, gWy, gWq, gWk, gwb;
};

template <int E, int C, int R, int NRG>
__device__ __forceinline__ void load_tile(const float* g, int rg, int cg, u64 (&W)[R / 2][C]) {
#pragma unroll
  for (int i2 = 0; i2 < R / 2; ++i2) {
    float a[C], b[C];
    ld_vec<C>(g + (rg * R + 2 * i2) * E + cg * C, a);
    ld_vec<C>(g + (rg * R + 2 * i2 + 1) * E + cg * C, b);
#pragma unroll
    for (int j = 0; j < C; ++j) W[i2][j] = pack2(a[j], b[j]);
  }
}
template <int E, int C, int R, int NRG>
__device__ __forceinline__ void store_tile(float* g, int rg, int cg, const u64 (&W)[R / 2][C]) {
#pragma unroll
  for (int i2 = 0; i2 < R / 2; ++i2) {
    float a[C], b[C];
#pragma unroll
    for (int j = 0; j < C; ++j) unpack2(W[i2][j], a[j], b[j]);
    st_vec<C>(g + (rg * R + 2 * i2) * E + cg * C, a);
    st_vec<C>(g + (rg * R + 2 * i2 + 1) * E + cg * C, b);
  }
}

// ---------------------------------------------------------------------------------------
// Forward
// ---------------------------------------------------------------------------------------
template <typename TIO, int E, int T>
struct SrwmFwdSmem {
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int IN_BYTES = T * ROW_IO;                       // x of one buffer
  static constexpr int OUT_BYTES = T * ROW_IO + 5 * T * ROW_F + 2 * T * 16;  // y | q k yd qd kd | beta bd
  static constexpr int XCHG_BYTES = 2 * 2 * ROW_F + 2 * 16;         // q~,k~ (x2 parity) + beta (x2)
  static constexpr int WB_BYTES = 4 * ROW_F;                        // w_b transposed [4][E]
  static constexpr int TOTAL = 2 * IN_BYTES + OUT_BYTES + XCHG_BYTES + WB_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB>
__global__ void __launch_bounds__(P, MINB) srwm_fwd_kernel(const SrwmFwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = SrwmFwdSmem<TIO, E, T>;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const bool save = !(p.flags & 1u);
  // w_b column handled by this thread's column group (-1: none)
  const int jb = (cg % TL::BETA_CG_STEP == 0) ? cg / TL::BETA_CG_STEP : -1;

  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* s_o = smem + 2 * SM::IN_BYTES;
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

  u64 Wy[R2][C], Wq[R2][C], Wk[R2][C];
  float* gWy = p.Wy.mat(n, h);
  float* gWq = p.Wq.mat(n, h);
  float* gWk = p.Wk.mat(n, h);
  float* gwb = p.wb.mat(n, h);
  load_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
  load_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
  load_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
  for (int i = tid; i < 4 * E; i += P) wbT[(i % 4) * E + i / 4] = gwb[i];   // [E][4] -> [4][E]

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return reinterpret_cast<TIO*>(smem + b * SM::IN_BYTES); };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    stage_rows<SM::ROW_IO, P>(in_buf(c & 1), p.x.row(n, h, t0), p.x.sl, nt, tid);
  };
  stage_chunk(0);
  cp_async_commit();

  int par = 0;
  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (c + 1 < nchunks) stage_chunk(c + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();   // chunk c (and, first time, w_b) visible; output stage free again
    const TIO* sx = in_buf(c & 1);

    for (int t = 0; t < nt; ++t, par ^= 1) {
      // ---- pass 1: [y, q~, k~, b~] = x.W ------------------------------------------------
      float xr[R];
      ld_vec<R>(sx + t * E + rg * R, xr);
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
        ld_vec<R>(wbT + jb * E + rg * R, wr);
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
      ld_vec<R>(xq_cur + rg * R, qr);
      ld_vec<R>(xq_cur + E + rg * R, kr);
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
        st_vec<R>(sq + t * E + rg * R, qr);
        st_vec<R>(sk + t * E + rg * R, kr);
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
        ld_vec<R>(wbT + jb * E + rg * R, wr);
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
        st_vec<R>(wbT + jb * E + rg * R, wr);   // only this thread ever touches these entries
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

  store_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
  store_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
  store_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
  __syncthreads();
  for (int i = tid; i < 4 * E; i += P) gwb[i] = wbT[(i % 4) * E + i / 4];
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
template <typename TIO, int E, int P, int T>
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
  static constexpr int TOTAL = 2 * IN_BYTES + GX_BYTES + XROW_BYTES + XSC_BYTES + WB_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB>
__global__ void __launch_bounds__(P, MINB) srwm_bwd_kernel(const SrwmBwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = SrwmBwdSmem<TIO, E, P, T>;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2, NWARP = TL::NWARP;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int warp = tid / 32, lane = tid % 32;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int jb = (cg % TL::BETA_CG_STEP == 0) ? cg / TL::BETA_CG_STEP : -1;

  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* s_o = smem + 2 * SM::IN_BYTES;
  float* sgx = reinterpret_cast<float*>(s_o);                               // [T][NWARP][E]
  float* xrow = reinterpret_cast<float*>(s_o + SM::GX_BYTES);               // [2][NWARP][2][E]
  float* xsc = reinterpret_cast<float*>(s_o + SM::GX_BYTES + SM::XROW_BYTES);  // [2][NWARP][8]
  float* wbT = xsc + 2 * NWARP * 8;                                         // [4][E]
  float* gbT = wbT + 4 * E;                                                 // [4][E]

  u64 Wy[R2][C], Wq[R2][C], Wk[R2][C], Gy[R2][C], Gq[R2][C], Gk[R2][C];
  float* gWy = p.Wy.mat(n, h);
  float* gWq = p.Wq.mat(n, h);
  float* gWk = p.Wk.mat(n, h);
  float* gwb = p.wb.mat(n, h);
  load_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
  load_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
  load_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
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
    for (int i = tid; i < 4 * E; i += P) {
      wbT[(i % 4) * E + i / 4] = gwb[i];
      gbT[(i % 4) * E + i / 4] = gin ? ggwb[i] : 0.f;
    }
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
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
  stage_chunk(nchunks - 1);
  cp_async_commit();

  int par = 0;
  for (int c = nchunks - 1; c >= 0; --c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (c > 0) stage_chunk(c - 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const unsigned char* ib = in_buf(c & 1);
    const TIO* sx = reinterpret_cast<const TIO*>(ib);
    const TIO* sg = reinterpret_cast<const TIO*>(ib + T * SM::ROW_IO);
    const float* sq = reinterpret_cast<const float*>(ib + 2 * T * SM::ROW_IO);
    const float* sk = sq + T * E;
    const float* syd = sk + T * E;
    const float* sqd = syd + T * E;
    const float* skd = sqd + T * E;
    const float* sbeta = skd + T * E;
    const float* sbd = sbeta + T * 4;

    for (int t = nt - 1; t >= 0; --t, par ^= 1) {
      // ================= phase 1 =================
      float kr[R], qr[R];
      ld_vec<R>(sk + t * E + rg * R, kr);
      ld_vec<R>(sq + t * E + rg * R, qr);
      float beta[4], bdv[4];
      ld_vec<4>(sbeta + t * 4, beta);
      ld_vec<4>(sbd + t * 4, bdv);
      float dyc[C], dqc[C], dkc[C];
      ld_vec<C>(syd + t * E + cg * C, dyc);
      ld_vec<C>(sqd + t * E + cg * C, dqc);
      ld_vec<C>(skd + t * E + cg * C, dkc);

      u64 k2[R2], gkr2[R2], u2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
        gkr2[i2] = 0ull;
        u2[i2] = 0ull;
      }
      // undo the update, r = k.G (column partial), gk partial = G ins (row partial)
      u64 ary[C], arq[C], ark[C];
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 iy = dup2(beta[0] * dyc[j]);
        const u64 iq = dup2(beta[1] * dqc[j]);
        const u64 ik = dup2(beta[2] * dkc[j]);
        ary[j] = 0ull; arq[j] = 0ull; ark[j] = 0ull;
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          const u64 nk = neg2(k2[i2]);
          Wy[i2][j] = fma2<PK>(nk, iy, Wy[i2][j]);
          Wq[i2][j] = fma2<PK>(nk, iq, Wq[i2][j]);
          Wk[i2][j] = fma2<PK>(nk, ik, Wk[i2][j]);
          ary[j] = fma2<PK>(k2[i2], Gy[i2][j], ary[j]);
          arq[j] = fma2<PK>(k2[i2], Gq[i2][j], arq[j]);
          ark[j] = fma2<PK>(k2[i2], Gk[i2][j], ark[j]);
          gkr2[i2] = fma2<PK>(Gy[i2][j], iy, gkr2[i2]);
          gkr2[i2] = fma2<PK>(Gq[i2][j], iq, gkr2[i2]);
          gkr2[i2] = fma2<PK>(Gk[i2][j], ik, gkr2[i2]);
        }
      }
      float gkr[R], ur[R];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(gkr2[i2], gkr[2 * i2], gkr[2 * i2 + 1]);
      // w_b column of this column group
      float rb = 0.f, insb = 0.f;
      float wr[R], gr[R];
      if (jb >= 0) {
        insb = beta[3] * bdv[jb];
        ld_vec<R>(wbT + jb * E + rg * R, wr);
        ld_vec<R>(gbT + jb * E + rg * R, gr);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          wr[i] = fmaf(-kr[i], insb, wr[i]);
          rb = fmaf(kr[i], gr[i], rb);
          gkr[i] = fmaf(gr[i], insb, gkr[i]);
        }
      }
      // complete r over the row groups; gd = b r; scalar partials r.d
      float gdy[C], gdq[C], gdk[C];
      float sb0 = 0.f, sb1 = 0.f, sb2 = 0.f, sb3 = 0.f;
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const float ry = allreduce_rows<NRG>(hsum2(ary[j]));
        const float rq = allreduce_rows<NRG>(hsum2(arq[j]));
        const float rk = allreduce_rows<NRG>(hsum2(ark[j]));
        gdy[j] = beta[0] * ry;
        gdq[j] = beta[1] * rq;
        gdk[j] = beta[2] * rk;
        sb0 = fmaf(ry, dyc[j], sb0);
        sb1 = fmaf(rq, dqc[j], sb1);
        sb2 = fmaf(rk, dkc[j], sb2);
      }
      rb = allreduce_rows<NRG>(rb);
      float gdb = 0.f;
      if (jb >= 0) {
        gdb = beta[3] * rb;
        sb3 = rb * bdv[jb];
      }
      if (rg != 0) { sb0 = 0.f; sb1 = 0.f; sb2 = 0.f; sb3 = 0.f; }   // one lane per column group counts
      // G += (q-k)^T gd ; u = W(t-1) gd (row partial)
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 gy2 = dup2(gdy[j]);
        const u64 gq2 = dup2(gdq[j]);
        const u64 gk2 = dup2(gdk[j]);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          const u64 d2 = pack2(qr[2 * i2] - kr[2 * i2], qr[2 * i2 + 1] - kr[2 * i2 + 1]);
          Gy[i2][j] = fma2<PK>(d2, gy2, Gy[i2][j]);
          Gq[i2][j] = fma2<PK>(d2, gq2, Gq[i2][j]);
          Gk[i2][j] = fma2<PK>(d2, gk2, Gk[i2][j]);
          u2[i2] = fma2<PK>(Wy[i2][j], gy2, u2[i2]);
          u2[i2] = fma2<PK>(Wq[i2][j], gq2, u2[i2]);
          u2[i2] = fma2<PK>(Wk[i2][j], gk2, u2[i2]);
        }
      }
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(u2[i2], ur[2 * i2], ur[2 * i2 + 1]);
      if (jb >= 0) {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          gr[i] = fmaf(qr[i] - kr[i], gdb, gr[i]);
          ur[i] = fmaf(wr[i], gdb, ur[i]);
        }
      }
      // row partials: gq = u, gk = G ins - u ; their dot products with q, k
      float dotq = 0.f, dotk = 0.f;
#pragma unroll
      for (int i = 0; i < R; ++i) {
        gkr[i] -= ur[i];
        dotq = fmaf(qr[i], ur[i], dotq);
        dotk = fmaf(kr[i], gkr[i], dotk);
      }
#pragma unroll
      for (int i = 0; i < R; ++i) {
        ur[i] = allreduce_cols<NRG>(ur[i]);
        gkr[i] = allreduce_cols<NRG>(gkr[i]);
      }
      sb0 = allreduce_warp(sb0);
      sb1 = allreduce_warp(sb1);
      sb2 = allreduce_warp(sb2);
      sb3 = allreduce_warp(sb3);
      dotq = allreduce_warp(dotq);
      dotk = allreduce_warp(dotk);
      float* xr_cur = xrow + (par * NWARP + warp) * 2 * E;
      float* xs_cur = xsc + (par * NWARP + warp) * 8;
      if (lane < NRG) {
        st_vec<R>(xr_cur + rg * R, ur);
        st_vec<R>(xr_cur + E + rg * R, gkr);
      }
      if (lane == 0) {
        float sc[8] = {sb0, sb1, sb2, sb3, dotq, dotk, 0.f, 0.f};
        st_vec<8>(xs_cur, sc);
      }
      __syncthreads();

      // ================= phase 2 =================
      float gqc[C], gkc[C], sc[8];
#pragma unroll
      for (int j = 0; j < C; ++j) { gqc[j] = 0.f; gkc[j] = 0.f; }
#pragma unroll
      for (int i = 0; i < 8; ++i) sc[i] = 0.f;
#pragma unroll
      for (int w = 0; w < NWARP; ++w) {
        float a[C], b[C], s[8];
        ld_vec<C>(xrow + (par * NWARP + w) * 2 * E + cg * C, a);
        ld_vec<C>(xrow + (par * NWARP + w) * 2 * E + E + cg * C, b);
        ld_vec<8>(xsc + (par * NWARP + w) * 8, s);
#pragma unroll
        for (int j = 0; j < C; ++j) { gqc[j] += a[j]; gkc[j] += b[j]; }
#pragma unroll
        for (int i = 0; i < 6; ++i) sc[i] += s[i];
      }
      float qc[C], kc[C], gc[C];
      ld_vec<C>(sq + t * E + cg * C, qc);
      ld_vec<C>(sk + t * E + cg * C, kc);
      ld_vec<C>(sg + t * E + cg * C, gc);
      float xr[R];
      ld_vec<R>(sx + t * E + rg * R, xr);
      u64 gx2[R2], x2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        gx2[i2] = 0ull;
        x2[i2] = pack2(xr[2 * i2], xr[2 * i2 + 1]);
      }
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 py = dup2(gc[j]);
        const u64 pq = dup2(qc[j] * (gqc[j] - sc[4]));
        const u64 pk = dup2(kc[j] * (gkc[j] - sc[5]));
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          gx2[i2] = fma2<PK>(Wy[i2][j], py, gx2[i2]);
          gx2[i2] = fma2<PK>(Wq[i2][j], pq, gx2[i2]);
          gx2[i2] = fma2<PK>(Wk[i2][j], pk, gx2[i2]);
          Gy[i2][j] = fma2<PK>(x2[i2], py, Gy[i2][j]);
          Gq[i2][j] = fma2<PK>(x2[i2], pq, Gq[i2][j]);
          Gk[i2][j] = fma2<PK>(x2[i2], pk, Gk[i2][j]);
        }
      }
      float gxr[R];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(gx2[i2], gxr[2 * i2], gxr[2 * i2 + 1]);
      if (jb >= 0) {
        const float b = beta[jb];
        const float pb = sc[jb] * b * (1.f - b);
#pragma unroll
        for (int i = 0; i < R; ++i) {
          gxr[i] = fmaf(wr[i], pb, gxr[i]);
          gr[i] = fmaf(xr[i], pb, gr[i]);
        }
        st_vec<R>(wbT + jb * E + rg * R, wr);
        st_vec<R>(gbT + jb * E + rg * R, gr);
      }
#pragma unroll
      for (int i = 0; i < R; ++i) gxr[i] = allreduce_cols<NRG>(gxr[i]);
      if (lane < NRG) st_vec<R>(sgx + (t * NWARP + warp) * E + rg * R, gxr);
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
      st_vec<4>(reinterpret_cast<TIO*>(p.gx.row(n, h, t0 + t)) + e4 * 4, acc);
    }
  }

  // dL/dW_0, and optionally the rebuilt W_0
  store_tile<E, C, R, NRG>(p.gWy.mat(n, h), rg, cg, Gy);
  store_tile<E, C, R, NRG>(p.gWq.mat(n, h), rg, cg, Gq);
  store_tile<E, C, R, NRG>(p.gWk.mat(n, h), rg, cg, Gk);
  const bool restore = (p.flags & 4u) != 0;
  if (restore) {
    store_tile<E, C, R, NRG>(gWy, rg, cg, Wy);
    store_tile<E, C, R, NRG>(gWq, rg, cg, Wq);
    store_tile<E, C, R, NRG>(gWk, rg, cg, Wk);
  }
  __syncthreads();
  {
    float* ggwb = p.gwb.mat(n, h);
    for (int i = tid; i < 4 * E; i += P) {
      ggwb[i] = gbT[(i % 4) * E + i / 4];
      if (restore) gwb[i] = wbT[(i % 4) * E + i / 4];
    }
  }
}

}  // namespace srwm
