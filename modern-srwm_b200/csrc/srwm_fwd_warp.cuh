// SRWM forward with ONE WARP per sequence, for head sizes up to 32 (the sizes the reference's own
// experiments use: d_head 16 in the few-shot scripts, 32 in the larger models and the agents).
//
// At these sizes a step has few FMAs (3 blocks x E x E x 3 passes) and the cost of the other
// forward kernels is their fixed per-step overhead: three warps that each load the operand vectors,
// a two-warp named barrier and a block-wide barrier per step.  Here E lanes hold all of
// [W_y | W_q | W_k | w_b] of one sequence: lane c holds column c (all E rows) of each of the three E x E
// blocks and row c of w_b; a warp serves 32 / E sequences side by side (one at E = 32, two at 16, four
// at 8), every instruction working for all of them, so
//   * an operand vector (x, q-k, k) is loaded once per step and feeds the three blocks,
//   * q~ / k~ land one per lane: the softmax is a reduction over the E lanes of the sequence
//     (redux.sync max with the group's member mask, shuffle-tree sum),
//   * q, k, q-k reach the other lanes through the output staging rows and a __syncwarp -- the kernel
//     has no barrier at all inside the time loop,
//   * row c of w_b lives in the lane that also holds k[c], so its rank-1 update is thread-local; its
//     four column sums are one small reduce-scatter.
// Semantics, saved tensors and the layer-level form (input softmax, base + shift state, episode
// resets) are those of the other forward kernels (srwm.cuh).
#pragma once
#include "srwm.cuh"

namespace srwm {

template <typename TIO, int E, int T, bool EXT>
struct SrwmFwdWarpSmem {
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int IN_BYTES = ((T * ROW_IO + 15) / 16) * 16;
  static constexpr int XF_BYTES = sizeof(TIO) == 4 ? 0 : T * ROW_F;   // x (or softmax(x)) in fp32
  static constexpr int OUT_BYTES = T * ROW_IO + 5 * T * ROW_F + 2 * T * 16;   // y | q k yd qd kd | beta bd
  static constexpr int DQ_BYTES = 2 * ROW_F;                          // q - k, double buffered
  static constexpr int DONE_BYTES = EXT ? ((T + 15) / 16) * 16 : 0;
  static constexpr int TOTAL = 2 * IN_BYTES + XF_BYTES + OUT_BYTES + DQ_BYTES + DONE_BYTES;
};

// sum of v[0..4) over the E lanes of a sequence (E a power of two >= 8), returned in every one of them
// (a reduce-scatter over the two low lane bits, log2(E) - 2 butterfly stages, four broadcasts)
template <int E>
__device__ __forceinline__ void allreduce4_group(float (&v)[4], int lane) {
  reduce_scatter<4, 4, 1>(v, lane);          // lane l holds the partial of value l % 4
  float s = v[0];
#pragma unroll
  for (int off = 4; off < E; off <<= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  const int g0 = lane & ~(E - 1);
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = __shfl_sync(0xffffffffu, s, g0 + j);
}

// max over the lanes named by `mask` (the E lanes of the caller's sequence)
__device__ __forceinline__ float group_max(float v, unsigned mask) {
  float r;
  asm volatile("redux.sync.max.f32 %0, %1, %2;" : "=f"(r) : "f"(v), "r"(mask));
  return r;
}

template <typename TIO, int E, int T, int MINB, bool EXT = false, bool RST = false>
__global__ void __launch_bounds__(32, MINB) srwm_fwd_warp_kernel(const SrwmFwdParams p) {
  static_assert(E == 8 || E == 16 || E == 32, "one warp per sequence: head sizes up to 32");
  using SM = SrwmFwdWarpSmem<TIO, E, T, EXT>;
  constexpr int P = E;                 // threads that serve one sequence
  constexpr int SPW = 32 / E;          // sequences per warp
  constexpr int RL = E;                // rows per lane: whole columns
  constexpr int RL2 = RL / 2;
  constexpr int NA = RL2 >= 4 ? 2 : 1;  // accumulator chains per block and pass
  static_assert(T <= E, "reset flags of a chunk travel in the ballot bits of the sequence's lanes");
  const int lane = threadIdx.x;
  const int c = lane % E, sub = lane / E;
  constexpr int r0 = 0;
  const unsigned gmask = E == 32 ? 0xffffffffu : (((1u << (E % 32)) - 1u) << (sub * E));
  // sequences beyond the grid (last warp of an odd grid) redo the last one and store nothing
  const long long nseq = (long long)p.N * p.H;
  const long long seq_raw = (long long)blockIdx.x * SPW + sub;
  const bool active = seq_raw < nseq;
  const long long seq = active ? seq_raw : nseq - 1;
  const int n = (int)(seq / p.H), h = (int)(seq % p.H);
  const bool save = !(p.flags & F_NO_SAVE) && active;
  constexpr bool owner = true;         // every lane holds row c of w_b and stores column c's results

  extern __shared__ __align__(16) unsigned char smem_all[];
  unsigned char* smem = smem_all + sub * SM::TOTAL;   // this sequence's staging area
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
  float* sdq = sbd + T * 4;     // [2][E]  q - k of the current step
  unsigned char* sdone = reinterpret_cast<unsigned char*>(sdq + 2 * E);   // [T] (EXT)

  const bool smx = EXT && (p.flags & F_INPUT_SOFTMAX);
  const bool has_base = EXT && (p.flags & F_BASE);
  const bool has_done = EXT && RST && (p.flags & F_DONE);

  u64 Wy[RL2], Wq[RL2], Wk[RL2];
  float wb[4];
  float* gWy = p.Wy.mat(n, h);
  float* gWq = p.Wq.mat(n, h);
  float* gWk = p.Wk.mat(n, h);
  float* gwb = p.wb.mat(n, h);
  // W = ga (+ gb): column c, rows r0 .. r0 + RL
  auto load_col = [&](const float* ga, const float* gb, u64 (&W)[RL2]) {
#pragma unroll
    for (int i2 = 0; i2 < RL2; ++i2) {
      float a = ga[(r0 + 2 * i2) * E + c], b = ga[(r0 + 2 * i2 + 1) * E + c];
      if (EXT && gb) { a += gb[(r0 + 2 * i2) * E + c]; b += gb[(r0 + 2 * i2 + 1) * E + c]; }
      W[i2] = pack2(a, b);
    }
  };
  auto load_wb = [&](const float* ga, const float* gb) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (owner) {
      v = *reinterpret_cast<const float4*>(ga + c * 4);
      if (EXT && gb) {
        const float4 w = *reinterpret_cast<const float4*>(gb + c * 4);
        v.x += w.x; v.y += w.y; v.z += w.z; v.w += w.w;
      }
    }
    wb[0] = v.x; wb[1] = v.y; wb[2] = v.z; wb[3] = v.w;
  };
  if (has_base) {
    const bool sh = (p.flags & F_SHIFT_IN) != 0;
    load_col(p.bWy.mat(n, h), sh ? p.sWy.mat(n, h) : nullptr, Wy);
    load_col(p.bWq.mat(n, h), sh ? p.sWq.mat(n, h) : nullptr, Wq);
    load_col(p.bWk.mat(n, h), sh ? p.sWk.mat(n, h) : nullptr, Wk);
    load_wb(p.bwb.mat(n, h), sh ? p.swb.mat(n, h) : nullptr);
  } else {
    load_col(gWy, nullptr, Wy);
    load_col(gWq, nullptr, Wq);
    load_col(gWk, nullptr, Wk);
    load_wb(gwb, nullptr);
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return reinterpret_cast<TIO*>(smem + b * SM::IN_BYTES); };
  auto stage_chunk = [&](int ch) {
    const int t0 = ch * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 9, t0, nt, L, T)) return;
    stage_rows<SM::ROW_IO, P>(in_buf(ch & 1), p.x.row(n, h, t0), p.x.sl, nt, c);
  };
  stage_chunk(0);
  cp_async_commit();
  int dn_next = 0;
  if (has_done && c < min(T, L)) dn_next = p.done[(long long)n * p.done_sn + (long long)c * p.done_sl];
  const u64 zero2 = 0ull;
  int par = 0;

  for (int ch = 0; ch < nchunks; ++ch) {
    const int t0 = ch * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 9, t0, nt, L, T)) break;
    if (ch + 1 < nchunks) stage_chunk(ch + 1);
    cp_async_commit();
    if (has_done) {
      if (c < T) sdone[c] = (unsigned char)dn_next;
      if (c < min(T, L - t0 - T))
        dn_next = p.done[(long long)n * p.done_sn + (long long)(t0 + T + c) * p.done_sl];
    }
    cp_async_wait<1>();
    __syncwarp();   // chunk ch staged; the output stage of the previous chunk has been flushed
    const float* sxf;
    if constexpr (sizeof(TIO) == 4) {
      float* xs = reinterpret_cast<float*>(in_buf(ch & 1));
      if (smx) {
        softmax_rows<TIO, E, P, T>(xs, xs, nt, c);
        __syncwarp();
      }
      sxf = xs;
    } else {
      if (smx) softmax_rows<TIO, E, P, T>(in_buf(ch & 1), xf32, nt, c);
      else convert_rows<TIO, E, P>(in_buf(ch & 1), xf32, nt, c);
      __syncwarp();
      sxf = xf32;
    }
    // reset flags of the chunk: bit t of the sequence's own lanes' ballot
    const unsigned dmask = has_done ? ((__ballot_sync(0xffffffffu, c < nt && sdone[c] != 0) & gmask) >> (sub * E)) : 0u;

#pragma unroll 1
    for (int t = 0; t < nt; ++t, par ^= 1) {
      if constexpr (EXT && RST) {
        if ((dmask >> t) & 1u) {   // episode boundary: the shift goes back to zero
          load_col(p.bWy.mat(n, h), nullptr, Wy);
          load_col(p.bWq.mat(n, h), nullptr, Wq);
          load_col(p.bWk.mat(n, h), nullptr, Wk);
          load_wb(p.bwb.mat(n, h), nullptr);
        }
      }
      float* dq = sdq + par * E;
      // ---- pass 1: [y, q~, k~] = x.W on column c (rows of this part), b~ from row c of w_b --------
      float y, qv, kv;
      {
        u64 ay[NA], aq[NA], ak[NA];
#pragma unroll
        for (int a = 0; a < NA; ++a) { ay[a] = zero2; aq[a] = zero2; ak[a] = zero2; }
        float xr[RL];
        ld_vec<RL>(sxf + t * E + r0, xr);
#pragma unroll
        for (int i2 = 0; i2 < RL2; ++i2) {
          const u64 x2 = pack2(xr[2 * i2], xr[2 * i2 + 1]);
          ay[i2 % NA] = fma2<true>(x2, Wy[i2], ay[i2 % NA]);
          aq[i2 % NA] = fma2<true>(x2, Wq[i2], aq[i2 % NA]);
          ak[i2 % NA] = fma2<true>(x2, Wk[i2], ak[i2 % NA]);
        }
        y = hsum2(ay[0]); qv = hsum2(aq[0]); kv = hsum2(ak[0]);
        if constexpr (NA == 2) { y += hsum2(ay[1]); qv += hsum2(aq[1]); kv += hsum2(ak[1]); }
      }
      float beta[4];
      {
        const float xc = owner ? sxf[t * E + c] : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) beta[j] = xc * wb[j];
        allreduce4_group<E>(beta, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) beta[j] = fast_sigmoid(beta[j]);
      }
      // ---- softmax over the E columns of the sequence ----------------------------------------------
      {
        const float mq = group_max(qv, gmask), mk = group_max(kv, gmask);
        qv = __expf(qv - mq);
        kv = __expf(kv - mk);
        float sq_ = qv, sk_ = kv;
#pragma unroll
        for (int off = 1; off < E; off <<= 1) {
          sq_ += __shfl_xor_sync(0xffffffffu, sq_, off);
          sk_ += __shfl_xor_sync(0xffffffffu, sk_, off);
        }
        qv *= __fdividef(1.f, sq_);
        kv *= __fdividef(1.f, sk_);
      }
      if (owner) {
        from_f32(sy[t * E + c], y);
        sq[t * E + c] = qv;
        sk[t * E + c] = kv;
        dq[c] = qv - kv;
        if (c < 4) sbeta[t * 4 + c] = c == 0 ? beta[0] : (c == 1 ? beta[1] : (c == 2 ? beta[2] : beta[3]));
      }
      __syncwarp();
      // ---- pass 2: d_Z = (q - k).W_Z ---------------------------------------------------------------
      float dy, dqv, dkv;
      {
        u64 ay[NA], aq[NA], ak[NA];
#pragma unroll
        for (int a = 0; a < NA; ++a) { ay[a] = zero2; aq[a] = zero2; ak[a] = zero2; }
        float dr[RL];
        ld_vec<RL>(dq + r0, dr);
#pragma unroll
        for (int i2 = 0; i2 < RL2; ++i2) {
          const u64 d2 = pack2(dr[2 * i2], dr[2 * i2 + 1]);
          ay[i2 % NA] = fma2<true>(d2, Wy[i2], ay[i2 % NA]);
          aq[i2 % NA] = fma2<true>(d2, Wq[i2], aq[i2 % NA]);
          ak[i2 % NA] = fma2<true>(d2, Wk[i2], ak[i2 % NA]);
        }
        dy = hsum2(ay[0]); dqv = hsum2(aq[0]); dkv = hsum2(ak[0]);
        if constexpr (NA == 2) { dy += hsum2(ay[1]); dqv += hsum2(aq[1]); dkv += hsum2(ak[1]); }
      }
      float db[4];
      {
        const float dc = owner ? qv - kv : 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) db[j] = dc * wb[j];
        allreduce4_group<E>(db, lane);
      }
      if (save && owner) {
        syd[t * E + c] = dy;
        sqd[t * E + c] = dqv;
        skd[t * E + c] = dkv;
        if (c < 4) sbd[t * 4 + c] = c == 0 ? db[0] : (c == 1 ? db[1] : (c == 2 ? db[2] : db[3]));
      }
      // ---- rank-1 update: W_Z[r][c] += k[r] (beta_Z d_Z[c]); row c of w_b += k[c] (beta_b d_b) ------
      {
        const u64 iy = dup2(beta[0] * dy), iq = dup2(beta[1] * dqv), ik = dup2(beta[2] * dkv);
        float kr[RL];
        ld_vec<RL>(sk + t * E + r0, kr);
#pragma unroll
        for (int i2 = 0; i2 < RL2; ++i2) {
          const u64 k2 = pack2(kr[2 * i2], kr[2 * i2 + 1]);
          Wy[i2] = fma2<true>(k2, iy, Wy[i2]);
          Wq[i2] = fma2<true>(k2, iq, Wq[i2]);
          Wk[i2] = fma2<true>(k2, ik, Wk[i2]);
        }
        if (owner) {
          const float kb = kv * beta[3];
#pragma unroll
          for (int j = 0; j < 4; ++j) wb[j] = fmaf(kb, db[j], wb[j]);
        }
      }
    }

    __syncwarp();
    if (active) flush_rows<SM::ROW_IO, P>(p.out.row(n, h, t0), p.out.sl, sy, nt, c);
    if (save) {
      flush_rows<SM::ROW_F, P>(p.q.row(n, h, t0), p.q.sl, sq, nt, c);
      flush_rows<SM::ROW_F, P>(p.k.row(n, h, t0), p.k.sl, sk, nt, c);
      flush_rows<SM::ROW_F, P>(p.yd.row(n, h, t0), p.yd.sl, syd, nt, c);
      flush_rows<SM::ROW_F, P>(p.qd.row(n, h, t0), p.qd.sl, sqd, nt, c);
      flush_rows<SM::ROW_F, P>(p.kd.row(n, h, t0), p.kd.sl, skd, nt, c);
      flush_rows<16, P>(p.beta.row(n, h, t0), p.beta.sl, sbeta, nt, c);
      flush_rows<16, P>(p.bd.row(n, h, t0), p.bd.sl, sbd, nt, c);
    }
  }

  // final state (or, with the slow weights given separately, the final shift W_L - base)
  auto store_col = [&](float* g, const float* gbase, const u64 (&W)[RL2]) {
#pragma unroll
    for (int i2 = 0; i2 < RL2; ++i2) {
      float a, b;
      unpack2(W[i2], a, b);
      if (EXT && gbase) { a -= gbase[(r0 + 2 * i2) * E + c]; b -= gbase[(r0 + 2 * i2 + 1) * E + c]; }
      g[(r0 + 2 * i2) * E + c] = a;
      g[(r0 + 2 * i2 + 1) * E + c] = b;
    }
  };
  if (!active) return;
  store_col(gWy, has_base ? p.bWy.mat(n, h) : nullptr, Wy);
  store_col(gWq, has_base ? p.bWq.mat(n, h) : nullptr, Wq);
  store_col(gWk, has_base ? p.bWk.mat(n, h) : nullptr, Wk);
  {
    float4 v = make_float4(wb[0], wb[1], wb[2], wb[3]);
    if (has_base) {
      const float4 w = *reinterpret_cast<const float4*>(p.bwb.mat(n, h) + c * 4);
      v.x -= w.x; v.y -= w.y; v.z -= w.z; v.w -= w.w;
    }
    *reinterpret_cast<float4*>(gwb + c * 4) = v;
  }
}

}  // namespace srwm
