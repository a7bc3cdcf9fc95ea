// SRWM reverse-time backward, second formulation, for the tile shapes in which every lane owns
// one row pair of one w_b column and the row sums leave the warp through a reduce-scatter
// (head sizes 32 and 64 in their default tilings).  Same arithmetic and same data layout as
// srwm_bwd_kernel (srwm.cuh; the arithmetic of self_ref_v0.cu:694-1187), restructured for a
// shorter per-step instruction stream and a shorter dependent chain:
//
//   * the step's dependent chain is  G -> r = k.G -> (column sums) -> gd -> u = W(t-1).gd ->
//     (row sums) -> barrier -> gq~, gk~ -> G += x^T pre.  The passes that are NOT on it -- undoing the
//     update, the row partial of G.ins, G += (q-k)^T gd -- are issued next to the shuffle trees of the
//     chain, so their FMAs fill the shuffle latency instead of preceding it;
//   * k, q-k and x are packed once per step and stay in registers (no second and third read of
//     the staged rows); the dot products q.gq and k.gk are packed FMAs on those registers;
//   * the per-lane pieces of the w_b column (two rows of one column per lane) take their k, q-k, x
//     values with one 8-byte shared-memory load each instead of register selects, and their
//     contributions to the row sums travel through a small per-warp scratch row instead of predicated
//     accumulations into a dynamically chosen register;
//   * the scalar partials r.d are formed before the column sums are completed (the reduction is
//     linear), so the saved d rows are read once;
//   * minus-gk is carried instead of gk (one packed add instead of negate-and-subtract per row);
//   * the W_y block's share of the last pass (gx += W_y g, G_y += x^T g) needs only the upstream
//     gradient, so it runs before the step's barrier, where it fills the waits of the reductions.
// Measured on B200 (592 sequences x 512 steps, bf16 streams): 1.81 ms against 1.84 ms for
// srwm_bwd_kernel; with G += (q-k)^T gd folded into the u pass instead of issued behind it 1.97 ms;
// with the gx row sums parked one step late (their shuffles moved to the next step's start) 2.18 ms
// (the carried registers spill).
#pragma once
#include "srwm.cuh"

namespace srwm {

template <typename TIO, int E, int P, int T>
struct SrwmBwd2Smem {
  static constexpr int NWARP = P / 32;
  static constexpr int CPW = 4 / NWARP;                          // w_b columns per warp
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  // x, gout (io) | q, k, yd, qd, kd (f32) | beta, bd ([T][4] f32)
  static constexpr int IN_BYTES = 2 * T * ROW_IO + 5 * T * ROW_F + 2 * T * 16;
  static constexpr int GX_BYTES = T * NWARP * ROW_F;             // per-warp partial gx
  static constexpr int XROW_BYTES = 2 * NWARP * 2 * ROW_F;       // [2 parity][NWARP][u, -gk][E]
  static constexpr int XSC_BYTES = 2 * 8 * NWARP * 4;            // [2][8 scalars][NWARP]
  static constexpr int WSB_BYTES = NWARP * CPW * 3 * ROW_F;      // [NWARP][CPW][u, -gk, gx][E] w_b pieces
  static constexpr int XF_BYTES = sizeof(TIO) != 4 ? T * ROW_F : 0;   // x (or softmax(x)) in fp32
  static constexpr int TOTAL = 2 * IN_BYTES + GX_BYTES + XROW_BYTES + XSC_BYTES + WSB_BYTES + XF_BYTES;
};

// S consecutive local rows starting at local row i0 (inside one quad when S <= 4, whole quads otherwise)
template <int S, int R, int NRG>
__device__ __forceinline__ void ld_rows_piece(const float* base, int rg, int i0, float (&v)[S]) {
  static_assert(R % 4 == 0, "quad row mapping");
  if constexpr (S <= 4) {
    ld_vec<S>(base + (i0 / 4) * (4 * NRG) + rg * 4 + (i0 % 4), v);
  } else {
    static_assert(S % 4 == 0, "pieces longer than a quad are whole quads");
#pragma unroll
    for (int q = 0; q < S / 4; ++q) {
      float t[4];
      ld_vec<4>(base + (i0 / 4 + q) * (4 * NRG) + rg * 4, t);
#pragma unroll
      for (int i = 0; i < 4; ++i) v[4 * q + i] = t[i];
    }
  }
}

// OPT (tuning bits): 1 = re-read the saved d rows for the undo pass instead of keeping them in
// registers; 2 = G += (q-k)^T gd inside the u pass (one broadcast pair per column, no overlap with the
// row sums); 4 = the W_y block's part of the last pass before the barrier; 8 = gx row sums parked one
// step late
template <typename TIO, int E, int P, int R, int T, int MINB, int OPT = 0>
__global__ void __launch_bounds__(P, MINB) srwm_bwd2_kernel(const SrwmBwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = SrwmBwd2Smem<TIO, E, P, T>;
  constexpr bool PK = true;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2, NWARP = TL::NWARP, CGW = TL::CGW;
  constexpr int CPW = 4 / NWARP;
  static_assert(R % 4 == 0, "row quads");
  static_assert(NWARP <= 4 && CGW == CPW * R2, "every lane owns one row pair of one w_b column");
  static_assert(CGW >= 2 && R % CGW == 0 && 8 % NRG == 0, "row sums leave the warp through a reduce-scatter");
  constexpr int S_ROW = (2 * R) / CGW;   // [u | -gk] values per lane after the scatter
  constexpr int S_GX = R / CGW;
  constexpr int S_SC = 8 / NRG;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int warp = tid / 32, lane = tid % 32;
  const int cgl = lane / NRG;
  const int n = blockIdx.x / p.H, h = blockIdx.x % p.H;
  const int wi2 = cgl % R2;                                   // row pair of this lane in its w_b column
  const int wrow = row_of<R, NRG>(rg, 2 * wi2);               // its first row (the second is wrow + 1)
  const int jl = cgl / R2;                                    // column slot within the warp
  const int jb = warp * CPW + jl;                             // w_b column of this lane
  float wbr[2] = {0.f, 0.f}, gbr[2] = {0.f, 0.f};

  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* s_o = smem + 2 * SM::IN_BYTES;
  float* sgx = reinterpret_cast<float*>(s_o);                                  // [T][NWARP][E]
  float* xrow = reinterpret_cast<float*>(s_o + SM::GX_BYTES);                  // [2][NWARP][2][E]
  float* xsc = reinterpret_cast<float*>(s_o + SM::GX_BYTES + SM::XROW_BYTES);  // [2][8][NWARP]
  float* wsb = xsc + 2 * 8 * NWARP + warp * CPW * 3 * E;                       // this warp's [CPW][3][E]
  float* xf32 = xsc + 2 * 8 * NWARP + NWARP * CPW * 3 * E;                     // [T][E] (16-bit streams)

  const bool smx = (p.flags & F_INPUT_SOFTMAX) != 0;
  const bool has_base = (p.flags & F_BASE) != 0;

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
  const bool gin = (p.flags & F_STATE_GRAD_IN) != 0;
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
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = (wrow + u) * 4 + jb;
      wbr[u] = gwb[i] + (bb ? bb[i] : 0.f);
      gbr[u] = gin ? ggwb[i] : 0.f;
    }
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 8, t0, nt, L, T)) return;
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
  if (nchunks > 0) stage_chunk(nchunks - 1);
  cp_async_commit();

  const u64 neg1 = pack2(-1.f, -1.f), one2 = pack2(1.f, 1.f);
  int par = 0;
  for (int c = nchunks - 1; c >= 0; --c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 8, t0, nt, L, T)) break;
    if (c > 0) stage_chunk(c - 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    unsigned char* ib = in_buf(c & 1);
    const TIO* sx = reinterpret_cast<const TIO*>(ib);
    const float* sxs = reinterpret_cast<const float*>(ib);   // x as fp32 rows (softmax(x) when the kernel applies it)
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
    const TIO* sg = reinterpret_cast<const TIO*>(ib + T * SM::ROW_IO);
    const float* sq = reinterpret_cast<const float*>(ib + 2 * T * SM::ROW_IO);
    const float* sk = sq + T * E;
    const float* syd = sk + T * E;
    const float* sbeta = syd + 3 * T * E;
    const float* sbd = sbeta + T * 4;

    // (OPT & 8) the gx row sums of a step are reduced and parked at the start of the NEXT step, where
    // their shuffles overlap that step's first pass instead of ending the loop body
    u64 gxc[R2];
    int tprev = -1;
    auto park_gx = [&](const u64 (&g2)[R2], int tt) {
      float gxr[R];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) unpack2(g2[i2], gxr[2 * i2], gxr[2 * i2 + 1]);
      reduce_scatter<R, CGW, NRG>(gxr, lane);
      float piece[S_GX];
#pragma unroll
      for (int i = 0; i < S_GX; ++i) piece[i] = gxr[i];
#pragma unroll
      for (int s = 0; s < CPW; ++s) {
        float wp[S_GX];
        ld_rows_piece<S_GX, R, NRG>(wsb + (s * 3 + 2) * E, rg, cgl * S_GX, wp);
#pragma unroll
        for (int i = 0; i < S_GX; ++i) piece[i] += wp[i];
      }
      st_rows_piece<S_GX, R, NRG>(sgx + (tt * NWARP + warp) * E, rg, cgl * S_GX, piece);
    };
#pragma unroll 1
    for (int t = nt - 1; t >= 0; --t, par ^= 1) {
      // ================= phase 1 =================
      float beta[4];
      ld_vec<4>(sbeta + t * 4, beta);
      u64 k2[R2], d2[R2];
      {
        float kr[R], qr[R];
        ld_rows<R, NRG>(sk + t * E, rg, kr);
        ld_rows<R, NRG>(sq + t * E, rg, qr);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
          d2[i2] = fma2<PK>(k2[i2], neg1, pack2(qr[2 * i2], qr[2 * i2 + 1]));   // q - k
        }
      }
      // this lane's two rows of its w_b column
      const float2 kp = *reinterpret_cast<const float2*>(sk + t * E + wrow);
      const float2 qp = *reinterpret_cast<const float2*>(sq + t * E + wrow);
      const float bdj = sbd[t * 4 + jb];
      float dz[3][C];
#pragma unroll
      for (int z = 0; z < 3; ++z) ld_vec<C>(syd + z * T * E + t * E + cg * C, dz[z]);   // y_diff, q_diff, k_diff rows are adjacent

      if constexpr ((OPT & 8) != 0) {
        if (tprev >= 0) park_gx(gxc, tprev);
      }
      // ---- r = k.G: column partials, and the scalar partials r.d (linear, so taken before the sum)
      float rcol[3][C];
      float sc8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      auto rpass = [&](const u64 (&G)[R2][C], const float (&dzz)[C], float (&rz)[C], float& scz) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          u64 ar = 0ull;
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) ar = fma2<PK>(k2[i2], G[i2][j], ar);
          rz[j] = hsum2(ar);
          scz = fmaf(rz[j], dzz[j], scz);
        }
      };
      rpass(Gy, dz[0], rcol[0], sc8[0]);
      rpass(Gq, dz[1], rcol[1], sc8[1]);
      rpass(Gk, dz[2], rcol[2], sc8[2]);
      float rb = fmaf(kp.y, gbr[1], kp.x * gbr[0]);
      sc8[3] = rb * bdj;
      // complete the column sums over the row groups (w_b: over all rows of the column)
#pragma unroll
      for (int z = 0; z < 3; ++z)
#pragma unroll
        for (int j = 0; j < C; ++j) rcol[z][j] = allreduce_rows<NRG>(rcol[z][j]);
#pragma unroll
      for (int off = 1; off < NRG * R2; off <<= 1) rb += __shfl_xor_sync(0xffffffffu, rb, off);

      // ---- undo the update (W(t-1)), and the row partial of -G.ins: independent of the sums above
      u64 s2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) s2[i2] = 0ull;
      auto undo = [&](u64 (&W)[R2][C], const u64 (&G)[R2][C], const float (&dzz)[C], float bz) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 nins = dup2(-bz * dzz[j]);
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) {
            W[i2][j] = fma2<PK>(k2[i2], nins, W[i2][j]);
            s2[i2] = fma2<PK>(G[i2][j], nins, s2[i2]);
          }
        }
      };
      if constexpr (OPT & 1) {
#pragma unroll
        for (int z = 0; z < 3; ++z) {
          float dzz[C];
          ld_vec<C>(syd + z * T * E + t * E + cg * C, dzz);
          if (z == 0) undo(Wy, Gy, dzz, beta[0]);
          else if (z == 1) undo(Wq, Gq, dzz, beta[1]);
          else undo(Wk, Gk, dzz, beta[2]);
        }
      } else {
        undo(Wy, Gy, dz[0], beta[0]);
        undo(Wq, Gq, dz[1], beta[1]);
        undo(Wk, Gk, dz[2], beta[2]);
      }
      const float ninsb = -beta[3] * bdj;
      wbr[0] = fmaf(kp.x, ninsb, wbr[0]);
      wbr[1] = fmaf(kp.y, ninsb, wbr[1]);
      float sb0 = gbr[0] * ninsb, sb1 = gbr[1] * ninsb;   // -G_b.ins_b on this lane's two rows

      // ---- gd = b r ; u = W(t-1).gd (row partial)
      const float gdb = beta[3] * rb;
#pragma unroll
      for (int z = 0; z < 3; ++z)
#pragma unroll
        for (int j = 0; j < C; ++j) rcol[z][j] *= beta[z];
      u64 u2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) u2[i2] = 0ull;
      auto upass = [&](const u64 (&W)[R2][C], u64 (&G)[R2][C], const float (&gd)[C]) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 g2 = dup2(gd[j]);
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) {
            u2[i2] = fma2<PK>(W[i2][j], g2, u2[i2]);
            if constexpr (OPT & 2) G[i2][j] = fma2<PK>(d2[i2], g2, G[i2][j]);
          }
        }
      };
      upass(Wy, Gy, rcol[0]);
      upass(Wq, Gq, rcol[1]);
      upass(Wk, Gk, rcol[2]);
      const float ub0 = wbr[0] * gdb, ub1 = wbr[1] * gdb;
      sb0 += ub0;
      sb1 += ub1;
      // row partials: gq = u ; -gk = u - G.ins ; dot products q.gq and k.(-gk) on the packed rows
      u64 aq = 0ull, ak = 0ull;
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        s2[i2] = fma2<PK>(u2[i2], one2, s2[i2]);
        aq = fma2<PK>(d2[i2], u2[i2], aq);
        aq = fma2<PK>(k2[i2], u2[i2], aq);
        ak = fma2<PK>(k2[i2], s2[i2], ak);
      }
      sc8[4] = fmaf(qp.y, ub1, fmaf(qp.x, ub0, hsum2(aq)));
      sc8[5] = fmaf(kp.y, sb1, fmaf(kp.x, sb0, hsum2(ak)));
      // the w_b pieces of the two row vectors go through the warp's scratch rows
      *reinterpret_cast<float2*>(wsb + (jl * 3 + 0) * E + wrow) = make_float2(ub0, ub1);
      *reinterpret_cast<float2*>(wsb + (jl * 3 + 1) * E + wrow) = make_float2(sb0, sb1);
      __syncwarp();
      float* xr_cur = xrow + (par * NWARP + warp) * 2 * E;
      float* xs_cur = xsc + par * 8 * NWARP;
      {
        float v[2 * R];
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          unpack2(u2[i2], v[2 * i2], v[2 * i2 + 1]);
          unpack2(s2[i2], v[R + 2 * i2], v[R + 2 * i2 + 1]);
        }
        reduce_scatter<2 * R, CGW, NRG>(v, lane);
        // lanes of the lower half of the column groups hold pieces of u, the upper half of -gk
        const int which = cgl >= CGW / 2 ? 1 : 0;
        const int i0 = (cgl % (CGW / 2)) * S_ROW;
        float piece[S_ROW];
#pragma unroll
        for (int i = 0; i < S_ROW; ++i) piece[i] = v[i];
#pragma unroll
        for (int s = 0; s < CPW; ++s) {
          float wp[S_ROW];
          ld_rows_piece<S_ROW, R, NRG>(wsb + (s * 3 + which) * E, rg, i0, wp);
#pragma unroll
          for (int i = 0; i < S_ROW; ++i) piece[i] += wp[i];
        }
        st_rows_piece<S_ROW, R, NRG>(xr_cur + which * E, rg, i0, piece);
        reduce_scatter<8, NRG, 1>(sc8, lane);
#pragma unroll
        for (int i = 0; i < S_SC; ++i) {
          const float sp = allreduce_cols<NRG>(sc8[i]);
          if (cgl == 0) xs_cur[(rg * S_SC + i) * NWARP + warp] = sp;
        }
      }
      // ---- G += (q-k)^T gd: off the chain, fills the latency of the reductions above
      auto gpass = [&](u64 (&G)[R2][C], const float (&gd)[C]) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 g2 = dup2(gd[j]);
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) G[i2][j] = fma2<PK>(d2[i2], g2, G[i2][j]);
        }
      };
      if constexpr (!(OPT & 2)) {
        gpass(Gy, rcol[0]);
        gpass(Gq, rcol[1]);
        gpass(Gk, rcol[2]);
      }
      gbr[0] = fmaf(qp.x - kp.x, gdb, gbr[0]);
      gbr[1] = fmaf(qp.y - kp.y, gdb, gbr[1]);
      // x rows, and (OPT & 4) the W_y block's share of gx and of G += x^T pre: its coefficient is the
      // upstream gradient, known before the barrier, so these FMAs can fill phase 1's waits
      u64 gx2[R2], x2[R2];
      float pre[3][C];
      auto load_x = [&]() {
        float xr[R];
        ld_rows<R, NRG>(sxs + t * E, rg, xr);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          gx2[i2] = 0ull;
          x2[i2] = pack2(xr[2 * i2], xr[2 * i2 + 1]);
        }
        ld_vec<C>(sg + t * E + cg * C, pre[0]);
      };
      auto blk3 = [&](const u64 (&W)[R2][C], u64 (&G)[R2][C], const float (&pz)[C]) {
#pragma unroll
        for (int j = 0; j < C; ++j) {
          const u64 pd = dup2(pz[j]);
#pragma unroll
          for (int i2 = 0; i2 < R2; ++i2) {
            G[i2][j] = fma2<PK>(x2[i2], pd, G[i2][j]);
            gx2[i2] = fma2<PK>(W[i2][j], pd, gx2[i2]);
          }
        }
      };
      if constexpr ((OPT & 4) != 0) {
        load_x();
        blk3(Wy, Gy, pre[0]);
      }
      __syncthreads();

      // ================= phase 2 =================
      // The 2C values gq~ / gk~ of this column group are needed by all its NRG lanes.  Each lane
      // finishes a share of them (sum of the per-warp partials, softmax backward) and the
      // lanes exchange the results with shuffles.
      constexpr int VPLN = (2 * C + NRG - 1) / NRG;   // values finished per lane
      float mine[VPLN];
#pragma unroll
      for (int u = 0; u < VPLN; ++u) {
        const int v = rg + u * NRG;                   // 0..C-1: gq~ of column v ; C..2C-1: gk~ of column v-C
        const int which = (v >= C) ? 1 : 0;
        const int col = cg * C + (which ? v - C : v);
        float acc = 0.f;
        if (v < 2 * C) {
          float dw[NWARP];
          ld_vec<NWARP>(xs_cur + (4 + which) * NWARP, dw);
          float dot = 0.f;
#pragma unroll
          for (int w = 0; w < NWARP; ++w) {
            acc += xrow[(par * NWARP + w) * 2 * E + which * E + col];
            dot += dw[w];
          }
          const float sm_val = (which ? sk : sq)[t * E + col];
          acc = sm_val * (acc - dot);                 // q (gq - q.gq) ;  for k this is MINUS k (gk - k.gk)
          acc = which ? -acc : acc;
        }
        mine[u] = acc;
      }
#pragma unroll
      for (int j = 0; j < C; ++j) {
        pre[1][j] = __shfl_sync(0xffffffffu, mine[j / NRG], (lane & ~(NRG - 1)) + (j % NRG));
        pre[2][j] = __shfl_sync(0xffffffffu, mine[(C + j) / NRG], (lane & ~(NRG - 1)) + ((C + j) % NRG));
      }
      float pb;
      {
        float sw[NWARP];
        ld_vec<NWARP>(xs_cur + jb * NWARP, sw);
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) s += sw[w];
        const float b = sbeta[t * 4 + jb];
        pb = s * b * (1.f - b);
      }
      const float2 xp = *reinterpret_cast<const float2*>(sxs + t * E + wrow);
      if constexpr ((OPT & 4) == 0) {
        load_x();
        blk3(Wy, Gy, pre[0]);
      }
      blk3(Wq, Gq, pre[1]);
      blk3(Wk, Gk, pre[2]);
      *reinterpret_cast<float2*>(wsb + (jl * 3 + 2) * E + wrow) = make_float2(wbr[0] * pb, wbr[1] * pb);
      gbr[0] = fmaf(xp.x, pb, gbr[0]);
      gbr[1] = fmaf(xp.y, pb, gbr[1]);
      __syncwarp();
      if constexpr ((OPT & 8) != 0) {
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) gxc[i2] = gx2[i2];
        tprev = t;
      } else {
        park_gx(gx2, t);
      }
    }
    if constexpr ((OPT & 8) != 0) {
      if (tprev >= 0) park_gx(gxc, tprev);
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
      if (smx) st_vec<4>(sgx + (t * NWARP) * E + e4 * 4, acc);   // finished below, through the softmax
      else st_vec<4>(reinterpret_cast<TIO*>(p.gx.row(n, h, t0 + t)) + e4 * 4, acc);
    }
    if (smx) {
      __syncthreads();
      softmax_bwd_rows<TIO, E, P, T>(sxs, sgx, NWARP * E, p.gx.row(n, h, t0), p.gx.sl, nt, tid);
      __syncthreads();   // softmax(x) may sit in the staging buffer the next prefetch overwrites
    }
  }

  // dL/dW_0, and optionally the rebuilt W_0
  store_tile<E, C, R, NRG>(p.gWy.mat(n, h), rg, cg, Gy);
  store_tile<E, C, R, NRG>(p.gWq.mat(n, h), rg, cg, Gq);
  store_tile<E, C, R, NRG>(p.gWk.mat(n, h), rg, cg, Gk);
  const bool restore = (p.flags & F_RESTORE) != 0;
  if (restore) {   // W_0, or the initial shift W_0 - base in the extended form
    store_tile_diff<E, C, R, NRG>(gWy, has_base ? p.bWy.mat(n, h) : nullptr, rg, cg, Wy);
    store_tile_diff<E, C, R, NRG>(gWq, has_base ? p.bWq.mat(n, h) : nullptr, rg, cg, Wq);
    store_tile_diff<E, C, R, NRG>(gWk, has_base ? p.bWk.mat(n, h) : nullptr, rg, cg, Wk);
  }
  {
    float* ggwb = p.gwb.mat(n, h);
    const float* bb = has_base ? p.bwb.mat(n, h) : nullptr;
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = (wrow + u) * 4 + jb;
      ggwb[i] = gbr[u];
      if (restore) gwb[i] = wbr[u] - (bb ? bb[i] : 0.f);
    }
  }
  if (p.flags & F_REDUCE) reduce_epilogue<E, P>(p, n, h, tid);
}

}  // namespace srwm
