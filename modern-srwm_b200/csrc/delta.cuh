// Delta-rule fast-weight recurrence, forward and single-pass backward, for sm_100a.
//
// Semantics follow the reference's ground-truth loop
// (supervised_learning/fast_weight/__init__.py:186-191) and what its kernels save / leave
// behind (supervised_learning/fast_weight/fast_weight_cuda.cu:101-169, :391):
//   v_old = k.W ; ins = beta*(v - v_old) ; W += k^T ins ; out = q.W   (post-update W)
// The state W[E][M] (M == E) of one (batch, head) sequence is a register tile spread over
// the P threads of one CTA (see common.cuh); there is no block-wide barrier inside the
// time loop of either kernel -- only warp shuffles.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace srwm {

// The packed (layer-level) form, selected by F_PACKED: instead of four prepared tensors the
// kernels read the raw rows [q | k | v | b] (3E+1 values) that the layers' slow net produces
// (supervised_learning/layer.py:74-77, reinforcement_learning/torchbeast/layer.py:144-147) and
// apply the layers' preparation themselves, per staged chunk:
//   q = a(q) / (sum a(q) + eps),  k likewise,  a(x) = elu(x) + 1 ;  beta = sigmoid(b)
// (layer.py:79, 86-90 with eps = 0; torchbeast/layer.py:30-33 with eps = 1e-5).  The backward
// returns the gradient of the raw rows in the same packed layout.  Rows only need element
// alignment: they are staged as the 16-byte blocks that cover them.
constexpr unsigned F_PACKED = 8u, F_ZERO_INIT = 16u;

struct DeltaFwdParams {
  int N, H, L;
  unsigned flags;
  unsigned long long* dbg;   // status word of the debug build (null otherwise)
  int seq0;   // first sequence of this launch (a call may be split into launches of different configurations)
  SeqView Q, K, V, beta, out, v_old, v_ins;   // Q doubles as the packed rows
  StateView W;
  float eps;
};

struct DeltaBwdParams {
  int N, H, L;
  unsigned flags;
  unsigned long long* dbg;   // status word of the debug build (null otherwise)
  int seq0;   // first sequence of this launch
  SeqView Q, K, V, beta, v_old, v_ins, gout, gQ, gK, gV, gbeta;   // Q / gQ double as the packed rows
  StateView W, gW0;
  float eps;
};

__device__ __forceinline__ float elu_p1(float x) { return x > 0.f ? x + 1.f : __expf(x); }

// Stage nt packed rows of RSB bytes each: every row as the 16-byte blocks covering it
// (row r lands at dst + r*PITCH, its first byte at offset (address & 15) inside).
template <int RSB, int PITCH, int P>
__device__ __forceinline__ void stage_packed_rows(unsigned char* dst, const char* row0, long long row_stride_bytes,
                                                  int nt, int tid) {
  constexpr int NB = PITCH / 16;
  for (int idx = tid; idx < nt * NB; idx += P) {
    const int r = idx / NB, blk = idx % NB;
    const char* a = row0 + r * row_stride_bytes;
    const int off = (int)(reinterpret_cast<uintptr_t>(a) & 15);
    if (blk * 16 < off + RSB) cp_async16(dst + r * PITCH + blk * 16, a - off + blk * 16);
  }
}

// The layers' preparation of a staged chunk of packed rows: dense fp32 q, k (normalised), v and
// beta rows; optionally the normalisers (sum + eps) for the backward.  A row is handled by E/4
// adjacent lanes (4 values of each of q, k, v per lane).
template <typename TIO, int E, int P, int T, int PITCH>
__device__ __forceinline__ void prepare_packed_rows(const unsigned char* raw, const char* row0,
                                                    long long row_stride_bytes, float eps, float* dq, float* dk,
                                                    float* dv, float* db, float* dsq, float* dsk, int nt, int tid) {
  constexpr int LPR = E / 4, NG = P / LPR, K = (T + NG - 1) / NG;
  const int grp = tid / LPR, l = tid % LPR;
#pragma unroll
  for (int kk = 0; kk < K; ++kk) {
    const int t = grp + kk * NG;
    const int tc = min(t, nt - 1);
    const int off = (int)(reinterpret_cast<uintptr_t>(row0 + tc * row_stride_bytes) & 15);
    const TIO* r = reinterpret_cast<const TIO*>(raw + tc * PITCH + off);
    float q[4], k[4], v[4], sq = 0.f, sk = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      q[i] = elu_p1(to_f32(r[l * 4 + i]));
      k[i] = elu_p1(to_f32(r[E + l * 4 + i]));
      v[i] = to_f32(r[2 * E + l * 4 + i]);
      sq += q[i];
      sk += k[i];
    }
#pragma unroll
    for (int o = 1; o < LPR; o <<= 1) {
      sq += __shfl_xor_sync(0xffffffffu, sq, o);
      sk += __shfl_xor_sync(0xffffffffu, sk, o);
    }
    sq += eps;
    sk += eps;
    const float iq = __fdividef(1.f, sq), ik = __fdividef(1.f, sk);
#pragma unroll
    for (int i = 0; i < 4; ++i) { q[i] *= iq; k[i] *= ik; }
    if (t < nt) {
      st_vec<4>(dq + t * E + l * 4, q);
      st_vec<4>(dk + t * E + l * 4, k);
      st_vec<4>(dv + t * E + l * 4, v);
      if (l == 0) {
        db[t] = fast_sigmoid(to_f32(r[3 * E]));
        if (dsq) { dsq[t] = sq; dsk[t] = sk; }
      }
    }
  }
}

template <typename TIO, int E, int T, bool PACKED = false>
struct DeltaFwdSmem {
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int BETA_BYTES = ((T * 4 + 15) / 16) * 16;
  static constexpr int RSB = (3 * E + 1) * (int)sizeof(TIO);     // bytes of a packed row
  static constexpr int PK_PITCH = ((RSB + 30) / 16) * 16;        // the 16-byte blocks that can cover it
  static constexpr int IN_BYTES = PACKED ? T * PK_PITCH : 3 * T * ROW_IO + BETA_BYTES;   // one staging buffer
  static constexpr int DENSE_BYTES = PACKED ? 3 * T * ROW_F + BETA_BYTES : 0;   // prepared q,k,v,beta (fp32)
  static constexpr int OUT_BYTES = T * ROW_IO + 2 * T * ROW_F;   // out, v_old, v_ins
  static constexpr int TOTAL = 2 * IN_BYTES + DENSE_BYTES + OUT_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB, bool PACKED = false>
__global__ void __launch_bounds__(P, MINB) delta_fwd_kernel(const DeltaFwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = DeltaFwdSmem<TIO, E, T, PACKED>;
  using TS = typename std::conditional<PACKED, float, TIO>::type;   // element type the step loop reads
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int seq = blockIdx.x + p.seq0;
  const int n = seq / p.H, h = seq % p.H;
  const bool save = !(p.flags & 1u);

  extern __shared__ __align__(16) unsigned char smem[];
  float* dense = reinterpret_cast<float*>(smem + 2 * SM::IN_BYTES);   // PACKED: q | k | v | beta
  unsigned char* s_out = smem + 2 * SM::IN_BYTES + SM::DENSE_BYTES;
  TIO* so = reinterpret_cast<TIO*>(s_out);
  float* svold = reinterpret_cast<float*>(s_out + T * SM::ROW_IO);
  float* svins = svold + T * E;

  // state tile
  u64 W[R2][C];
  float* Wg = p.W.mat(n, h);
  const bool zero_init = PACKED && (p.flags & F_ZERO_INIT);
#pragma unroll
  for (int i2 = 0; i2 < R2; ++i2) {
    float a[C], b[C];
    if (zero_init) {
#pragma unroll
      for (int j = 0; j < C; ++j) { a[j] = 0.f; b[j] = 0.f; }
    } else {
      ld_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
      ld_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
    }
#pragma unroll
    for (int j = 0; j < C; ++j) W[i2][j] = pack2(a[j], b[j]);
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 5, t0, nt, L, T)) return;
    unsigned char* ib = in_buf(c & 1);
    if constexpr (PACKED) {
      stage_packed_rows<SM::RSB, SM::PK_PITCH, P>(ib, p.Q.row(n, h, t0), p.Q.sl, nt, tid);
    } else {
      stage_rows<SM::ROW_IO, P>(ib, p.Q.row(n, h, t0), p.Q.sl, nt, tid);
      stage_rows<SM::ROW_IO, P>(ib + T * SM::ROW_IO, p.K.row(n, h, t0), p.K.sl, nt, tid);
      stage_rows<SM::ROW_IO, P>(ib + 2 * T * SM::ROW_IO, p.V.row(n, h, t0), p.V.sl, nt, tid);
    }
  };
  auto beta_ld = [&](int c, int i) -> float {   // i-th step of chunk c (plain load: rows are 1 element)
    return to_f32(*reinterpret_cast<const TIO*>(p.beta.row(n, h, c * T + i)));
  };
  auto beta_buf = [&](int b) { return reinterpret_cast<float*>(in_buf(b) + 3 * T * SM::ROW_IO); };

  stage_chunk(0);
  cp_async_commit();
  if constexpr (!PACKED)
    for (int i = tid; i < min(T, L); i += P) beta_buf(0)[i] = beta_ld(0, i);

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 5, t0, nt, L, T)) break;
    const bool has_next = (c + 1 < nchunks);
    const int nt_next = has_next ? min(T, L - (t0 + T)) : 0;
    float bnext[(T + P - 1) / P];
    if (has_next) {
      stage_chunk(c + 1);
      if constexpr (!PACKED) {
#pragma unroll
        for (int u = 0; u < (T + P - 1) / P; ++u) {
          const int i = tid + u * P;
          bnext[u] = (i < nt_next) ? beta_ld(c + 1, i) : 0.f;
        }
      }
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const unsigned char* ib = in_buf(c & 1);
    const TS *sq, *sk, *sv;
    const float* sb;
    if constexpr (PACKED) {
      float* dq = dense;
      prepare_packed_rows<TIO, E, P, T, SM::PK_PITCH>(ib, p.Q.row(n, h, t0), p.Q.sl, p.eps, dq, dq + T * E,
                                                      dq + 2 * T * E, dq + 3 * T * E, nullptr, nullptr, nt, tid);
      __syncthreads();
      sq = dq; sk = dq + T * E; sv = dq + 2 * T * E; sb = dq + 3 * T * E;
    } else {
      sq = reinterpret_cast<const TS*>(ib);
      sk = reinterpret_cast<const TS*>(ib + T * SM::ROW_IO);
      sv = reinterpret_cast<const TS*>(ib + 2 * T * SM::ROW_IO);
      sb = beta_buf(c & 1);
    }

    #pragma unroll 1

    for (int t = 0; t < nt; ++t) {
      float kr[R], qr[R], vc[C];
      ld_rows<R, NRG>(sk + t * E, rg, kr);
      ld_rows<R, NRG>(sq + t * E, rg, qr);
      ld_vec<C>(sv + t * E + cg * C, vc);
      const float bt = sb[t];

      u64 av[C], ao[C];
#pragma unroll
      for (int j = 0; j < C; ++j) { av[j] = 0ull; ao[j] = 0ull; }
      float qk = 0.f;
      u64 k2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
        const u64 q2 = pack2(qr[2 * i2], qr[2 * i2 + 1]);
        qk = fmaf(kr[2 * i2], qr[2 * i2], qk);
        qk = fmaf(kr[2 * i2 + 1], qr[2 * i2 + 1], qk);
#pragma unroll
        for (int j = 0; j < C; ++j) {
          av[j] = fma2<PK>(k2[i2], W[i2][j], av[j]);
          ao[j] = fma2<PK>(q2, W[i2][j], ao[j]);
        }
      }
      float vold[C], o[C], ins[C];
      qk = allreduce_rows<NRG>(qk);
#pragma unroll
      for (int j = 0; j < C; ++j) {
        vold[j] = allreduce_rows<NRG>(hsum2(av[j]));
        o[j] = allreduce_rows<NRG>(hsum2(ao[j]));
        ins[j] = bt * (vc[j] - vold[j]);
        o[j] = fmaf(qk, ins[j], o[j]);   // q.(W + k^T ins) = q.W + (q.k) ins
      }
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 i2v = dup2(ins[j]);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) W[i2][j] = fma2<PK>(k2[i2], i2v, W[i2][j]);
      }
      if (rg == 0) {
        st_vec<C>(so + t * E + cg * C, o);
        if (save) {
          st_vec<C>(svold + t * E + cg * C, vold);
          st_vec<C>(svins + t * E + cg * C, ins);
        }
      }
    }

    if constexpr (!PACKED) {
      if (has_next) {
#pragma unroll
        for (int u = 0; u < (T + P - 1) / P; ++u) {
          const int i = tid + u * P;
          if (i < nt_next) beta_buf((c + 1) & 1)[i] = bnext[u];
        }
      }
    }
    __syncthreads();
    flush_rows<SM::ROW_IO, P>(p.out.row(n, h, t0), p.out.sl, so, nt, tid);
    if (save) {
      flush_rows<SM::ROW_F, P>(p.v_old.row(n, h, t0), p.v_old.sl, svold, nt, tid);
      flush_rows<SM::ROW_F, P>(p.v_ins.row(n, h, t0), p.v_ins.sl, svins, nt, tid);
    }
  }

  // final state back in place
#pragma unroll
  for (int i2 = 0; i2 < R2; ++i2) {
    float a[C], b[C];
#pragma unroll
    for (int j = 0; j < C; ++j) unpack2(W[i2][j], a[j], b[j]);
    st_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    st_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
  }
}

// ---------------------------------------------------------------------------------------
// Forward, column layout (E = 32 or 64): P = 32 or 64 threads per sequence, thread (cq, rp) holds
// CPL adjacent columns x E/NRP rows of W as row pairs; the warps of a sequence own disjoint
// columns and never talk to each other.  Both products reduce over rows, so with whole
// columns per lane (NRP = 1) nothing in a step crosses lanes at all: k and q are read from the
// staged rows as 16-byte shared-memory broadcasts, v / out / v_old / v_insert are per column.
//   pass A:  v_old[c] = sum_r k[r] W[r][c]          ins[c] = beta (v[c] - v_old[c])
//   pass B:  W[r][c] += k[r] ins[c]  and, with the updated value, out[c] += q[r] W[r][c]
// NRP = 2 splits the rows of a column group over two lanes (half the broadcast loads, one
// shuffle stage per column sum).  16-bit streams are converted to fp32 rows once per chunk.
// No barrier exists in this kernel beyond the hand-over of a staged chunk.
// ---------------------------------------------------------------------------------------
template <typename TIO, int E, int T, bool PACKED = false>
struct DeltaFwdColSmem {
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int BETA_BYTES = ((T * 4 + 15) / 16) * 16;
  static constexpr int RSB = (3 * E + 1) * (int)sizeof(TIO);
  static constexpr int PK_PITCH = ((RSB + 30) / 16) * 16;
  static constexpr int IN_BYTES = PACKED ? T * PK_PITCH : 3 * T * ROW_IO + BETA_BYTES;
  // k, q as fp32 rows (16-bit streams), or the prepared q, k, v, beta of the packed form
  static constexpr int CONV_BYTES = PACKED ? 3 * T * ROW_F + BETA_BYTES : (sizeof(TIO) == 4 ? 0 : 2 * T * ROW_F);
  static constexpr int OUT_BYTES = T * ROW_IO + 2 * T * ROW_F;
  static constexpr int TOTAL = 2 * IN_BYTES + CONV_BYTES + OUT_BYTES;
};

template <typename TIO, int E, int P, int T, bool PK, int MINB, int NRP, bool PACKED = false, int UNR = 1>
__global__ void __launch_bounds__(P, MINB) delta_fwd_col_kernel(const DeltaFwdParams p) {
  using SM = DeltaFwdColSmem<TIO, E, T, PACKED>;
  using TS = typename std::conditional<PACKED, float, TIO>::type;   // element type of the staged v rows
  constexpr int CPL = (E * NRP) / P, RL = E / NRP, RL2 = RL / 2;
  constexpr int NA = (CPL == 1 && RL >= 16) ? 4 : 2;   // accumulator chains per column
  static_assert(NRP == 1 || NRP == 2, "row parts per column group");
  static_assert(P % 32 == 0 && CPL >= 1 && CPL * P == E * NRP && RL % 4 == 0, "bad column-layout shape");
  const int lane = threadIdx.x;   // thread index within the sequence's P threads
  constexpr int LPP = 32 / NRP;   // lanes per row part within a warp
  const int rp = (lane % 32) / LPP, c0 = ((lane / 32) * LPP + lane % LPP) * CPL;
  const int seq = blockIdx.x + p.seq0;
  const int n = seq / p.H, h = seq % p.H;
  const bool save = !(p.flags & 1u);

  extern __shared__ __align__(16) unsigned char smem[];
  float* conv = reinterpret_cast<float*>(smem + 2 * SM::IN_BYTES);   // [2][T][E] k, q (16-bit streams)
  unsigned char* s_out = smem + 2 * SM::IN_BYTES + SM::CONV_BYTES;
  TIO* so = reinterpret_cast<TIO*>(s_out);
  float* svold = reinterpret_cast<float*>(s_out + T * SM::ROW_IO);
  float* svins = svold + T * E;

  // local row r of row part rp is global row ((r/4)*NRP + rp)*4 + r%4 (row quads interleaved over
  // the row parts: the lanes of a column group read an operand vector as adjacent 16-byte pieces)
  auto grow = [&](int r) { return ((r / 4) * NRP + rp) * 4 + (r % 4); };
  u64 W[RL2][CPL];
  float* Wg = p.W.mat(n, h);
  const bool zero_init = PACKED && (p.flags & F_ZERO_INIT);
#pragma unroll
  for (int e2 = 0; e2 < RL2; ++e2) {
    float a[CPL], b[CPL];
    if (zero_init) {
#pragma unroll
      for (int c = 0; c < CPL; ++c) { a[c] = 0.f; b[c] = 0.f; }
    } else {
      ld_vec<CPL>(Wg + grow(2 * e2) * E + c0, a);
      ld_vec<CPL>(Wg + grow(2 * e2 + 1) * E + c0, b);
    }
#pragma unroll
    for (int c = 0; c < CPL; ++c) W[e2][c] = pack2(a[c], b[c]);
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 6, t0, nt, L, T)) return;
    unsigned char* ib = in_buf(c & 1);
    if constexpr (PACKED) {
      stage_packed_rows<SM::RSB, SM::PK_PITCH, P>(ib, p.Q.row(n, h, t0), p.Q.sl, nt, lane);
    } else {
      stage_rows<SM::ROW_IO, P>(ib, p.Q.row(n, h, t0), p.Q.sl, nt, lane);
      stage_rows<SM::ROW_IO, P>(ib + T * SM::ROW_IO, p.K.row(n, h, t0), p.K.sl, nt, lane);
      stage_rows<SM::ROW_IO, P>(ib + 2 * T * SM::ROW_IO, p.V.row(n, h, t0), p.V.sl, nt, lane);
    }
  };
  auto beta_buf = [&](int b) { return reinterpret_cast<float*>(in_buf(b) + 3 * T * SM::ROW_IO); };
  static_assert(T <= 32, "one thread per step loads beta");

  stage_chunk(0);
  cp_async_commit();
  if constexpr (!PACKED)
    if (lane < min(T, L)) beta_buf(0)[lane] = to_f32(*reinterpret_cast<const TIO*>(p.beta.row(n, h, lane)));

  for (int c = 0; c < nchunks; ++c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 6, t0, nt, L, T)) break;
    const bool has_next = (c + 1 < nchunks);
    const int nt_next = has_next ? min(T, L - (t0 + T)) : 0;
    float bnext = 0.f;
    if (has_next) {
      stage_chunk(c + 1);
      if constexpr (!PACKED)
        if (lane < nt_next) bnext = to_f32(*reinterpret_cast<const TIO*>(p.beta.row(n, h, t0 + T + lane)));
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();   // chunk c staged; the output stage of the previous chunk has been flushed

    const unsigned char* ib = in_buf(c & 1);
    const float *sq, *sk, *sb;
    const TS* sv;
    if constexpr (PACKED) {
      prepare_packed_rows<TIO, E, P, T, SM::PK_PITCH>(ib, p.Q.row(n, h, t0), p.Q.sl, p.eps, conv, conv + T * E,
                                                      conv + 2 * T * E, conv + 3 * T * E, nullptr, nullptr, nt, lane);
      __syncthreads();
      sq = conv;
      sk = conv + T * E;
      sv = conv + 2 * T * E;
      sb = conv + 3 * T * E;
    } else {
      if constexpr (sizeof(TIO) == 4) {
        sq = reinterpret_cast<const float*>(ib);
        sk = reinterpret_cast<const float*>(ib + T * SM::ROW_IO);
      } else {
        convert_rows<TIO, E, P>(reinterpret_cast<const TIO*>(ib), conv, nt, lane);
        convert_rows<TIO, E, P>(reinterpret_cast<const TIO*>(ib + T * SM::ROW_IO), conv + T * E, nt, lane);
        __syncthreads();
        sq = conv;
        sk = conv + T * E;
      }
      sv = reinterpret_cast<const TS*>(ib + 2 * T * SM::ROW_IO);
      sb = beta_buf(c & 1);
    }

#pragma unroll UNR
    for (int t = 0; t < nt; ++t) {
      const float4* k4 = reinterpret_cast<const float4*>(sk + t * E);
      const float4* q4 = reinterpret_cast<const float4*>(sq + t * E);
      // ---- pass A: v_old = k.W on this lane's columns ------------------------------------
      // (NA independent accumulator chains per column: with one column per lane two chains of
      // RL/4 dependent FMAs would leave the lane waiting on its own results)
      u64 acc[NA][CPL];
#pragma unroll
      for (int a = 0; a < NA; ++a)
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) acc[a][cc] = 0ull;
#pragma unroll
      for (int e4 = 0; e4 < RL / 4; ++e4) {
        const float4 kv = k4[e4 * NRP + rp];
        const u64 k0 = pack2(kv.x, kv.y), k1 = pack2(kv.z, kv.w);
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) {
          acc[(2 * e4) % NA][cc] = fma2<PK>(k0, W[2 * e4][cc], acc[(2 * e4) % NA][cc]);
          acc[(2 * e4 + 1) % NA][cc] = fma2<PK>(k1, W[2 * e4 + 1][cc], acc[(2 * e4 + 1) % NA][cc]);
        }
      }
      float vc[CPL], vold[CPL], ins[CPL];
      ld_vec<CPL>(sv + t * E + c0, vc);
      const float bt = sb[t];
      u64 ins2[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) {
        float part = hsum2(acc[0][cc]) + hsum2(acc[1][cc]);
        if constexpr (NA == 4) part += hsum2(acc[2][cc]) + hsum2(acc[3][cc]);
        vold[cc] = allreduce_parts<NRP>(part);
        ins[cc] = bt * (vc[cc] - vold[cc]);
        ins2[cc] = dup2(ins[cc]);
#pragma unroll
        for (int a = 0; a < NA; ++a) acc[a][cc] = 0ull;
      }
      // ---- pass B: W += k^T ins, out = q.W (updated) --------------------------------------
#pragma unroll
      for (int e4 = 0; e4 < RL / 4; ++e4) {
        const float4 kv = k4[e4 * NRP + rp];
        const float4 qv = q4[e4 * NRP + rp];
        const u64 k0 = pack2(kv.x, kv.y), k1 = pack2(kv.z, kv.w);
        const u64 q0 = pack2(qv.x, qv.y), q1 = pack2(qv.z, qv.w);
#pragma unroll
        for (int cc = 0; cc < CPL; ++cc) {
          W[2 * e4][cc] = fma2<PK>(k0, ins2[cc], W[2 * e4][cc]);
          W[2 * e4 + 1][cc] = fma2<PK>(k1, ins2[cc], W[2 * e4 + 1][cc]);
          acc[(2 * e4) % NA][cc] = fma2<PK>(q0, W[2 * e4][cc], acc[(2 * e4) % NA][cc]);
          acc[(2 * e4 + 1) % NA][cc] = fma2<PK>(q1, W[2 * e4 + 1][cc], acc[(2 * e4 + 1) % NA][cc]);
        }
      }
      float o[CPL];
#pragma unroll
      for (int cc = 0; cc < CPL; ++cc) {
        float part = hsum2(acc[0][cc]) + hsum2(acc[1][cc]);
        if constexpr (NA == 4) part += hsum2(acc[2][cc]) + hsum2(acc[3][cc]);
        o[cc] = allreduce_parts<NRP>(part);
      }
      if (rp == 0) {
        st_vec<CPL>(so + t * E + c0, o);
        if (save) {
          st_vec<CPL>(svold + t * E + c0, vold);
          st_vec<CPL>(svins + t * E + c0, ins);
        }
      }
    }

    if constexpr (!PACKED)
      if (has_next && lane < nt_next) beta_buf((c + 1) & 1)[lane] = bnext;
    __syncthreads();
    flush_rows<SM::ROW_IO, P>(p.out.row(n, h, t0), p.out.sl, so, nt, lane);
    if (save) {
      flush_rows<SM::ROW_F, P>(p.v_old.row(n, h, t0), p.v_old.sl, svold, nt, lane);
      flush_rows<SM::ROW_F, P>(p.v_ins.row(n, h, t0), p.v_ins.sl, svins, nt, lane);
    }
  }

#pragma unroll
  for (int e2 = 0; e2 < RL2; ++e2) {
    float a[CPL], b[CPL];
#pragma unroll
    for (int cc = 0; cc < CPL; ++cc) unpack2(W[e2][cc], a[cc], b[cc]);
    st_vec<CPL>(Wg + grow(2 * e2) * E + c0, a);
    st_vec<CPL>(Wg + grow(2 * e2 + 1) * E + c0, b);
  }
}

// ---------------------------------------------------------------------------------------
// Backward.  With G = dL/dW_t carried backwards in time and g = dL/dout_t:
//   G += q^T g ; gq = W_t g ; r = k.G ; gv = beta r ; gbeta = r.(v - v_old)
//   gk = G ins + W_{t-1} (-beta r) ; W_{t-1} = W_t - k^T ins ; G += k^T (-beta r)
// (same arithmetic as fast_weight_cuda.cu:489-552 and :336-389, in one pass).
// Column results (gv) are complete after the row-group shuffle; row results (gq, gk) and
// gbeta are reduced across the column groups of a warp with shuffles, parked per warp in
// shared memory and summed across warps when the chunk is written out -- they are outputs
// only, so nothing on the recurrence's critical path waits for a barrier.
// ---------------------------------------------------------------------------------------
template <typename TIO, int E, int P, int T, bool PACKED = false>
struct DeltaBwdSmem {
  static constexpr int NWARP = P / 32;
  static constexpr int ROW_IO = E * (int)sizeof(TIO);
  static constexpr int ROW_F = E * 4;
  static constexpr int BETA_BYTES = ((T * 4 + 15) / 16) * 16;
  static constexpr int RSB = (3 * E + 1) * (int)sizeof(TIO);
  static constexpr int PK_PITCH = ((RSB + 30) / 16) * 16;
  // q,k,v (io, or the packed rows) | gout (io) | v_old, v_ins (f32) | beta
  static constexpr int QKV_BYTES = PACKED ? T * PK_PITCH : 3 * T * ROW_IO;
  static constexpr int IN_BYTES = QKV_BYTES + T * ROW_IO + 2 * T * ROW_F + (PACKED ? 0 : BETA_BYTES);
  static constexpr int DENSE_BYTES = PACKED ? 3 * T * ROW_F + 3 * BETA_BYTES : 0;   // q,k,v | beta, sum_q, sum_k
  static constexpr int GV_BYTES = T * ROW_IO;
  static constexpr int PART_BYTES = T * NWARP * 2 * ROW_F;       // per-warp partial gq, gk
  static constexpr int GB_BYTES = ((T * NWARP * 4 + 15) / 16) * 16;
  static constexpr int TOTAL = 2 * IN_BYTES + GV_BYTES + PART_BYTES + GB_BYTES + DENSE_BYTES;
};

template <typename TIO, int E, int P, int R, int T, bool PK, int MINB, bool PACKED = false>
__global__ void __launch_bounds__(P, MINB) delta_bwd_kernel(const DeltaBwdParams p) {
  using TL = Tiling<E, P, R>;
  using SM = DeltaBwdSmem<TIO, E, P, T, PACKED>;
  using TS = typename std::conditional<PACKED, float, TIO>::type;
  constexpr int NRG = TL::NRG, C = TL::C, R2 = R / 2, NWARP = TL::NWARP, CGW = TL::CGW;
  // row sums leave the warp through a reduce-scatter when the tile shape allows it
  constexpr bool SCATTER = (CGW >= 2) && ((2 * R) % CGW == 0) && ((2 * R) / CGW <= 4 || ((2 * R) / CGW) % 4 == 0);
  constexpr int S_ROW = SCATTER ? (2 * R) / CGW : R;
  const int tid = threadIdx.x;
  const int rg = tid % NRG, cg = tid / NRG;
  const int warp = tid / 32, lane = tid % 32;
  const int cgl = lane / NRG;
  const int seq = blockIdx.x + p.seq0;
  const int n = seq / p.H, h = seq % p.H;

  extern __shared__ __align__(16) unsigned char smem[];
  unsigned char* s_o = smem + 2 * SM::IN_BYTES;
  TIO* sgv = reinterpret_cast<TIO*>(s_o);
  float* spart = reinterpret_cast<float*>(s_o + SM::GV_BYTES);          // [T][NWARP][2][E]
  float* sgb = reinterpret_cast<float*>(s_o + SM::GV_BYTES + SM::PART_BYTES);  // [T][NWARP]
  float* dense = reinterpret_cast<float*>(s_o + SM::GV_BYTES + SM::PART_BYTES + SM::GB_BYTES);   // PACKED

  u64 W[R2][C], G[R2][C];
  float* Wg = p.W.mat(n, h);
#pragma unroll
  for (int i2 = 0; i2 < R2; ++i2) {
    float a[C], b[C];
    ld_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    ld_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
#pragma unroll
    for (int j = 0; j < C; ++j) { W[i2][j] = pack2(a[j], b[j]); G[i2][j] = 0ull; }
  }

  const int L = p.L;
  const int nchunks = (L + T - 1) / T;
  auto in_buf = [&](int b) { return smem + b * SM::IN_BYTES; };
  auto stage_chunk = [&](int c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 7, t0, nt, L, T)) return;
    unsigned char* ib = in_buf(c & 1);
    if constexpr (PACKED) {
      stage_packed_rows<SM::RSB, SM::PK_PITCH, P>(ib, p.Q.row(n, h, t0), p.Q.sl, nt, tid);
    } else {
      stage_rows<SM::ROW_IO, P>(ib, p.Q.row(n, h, t0), p.Q.sl, nt, tid);
      stage_rows<SM::ROW_IO, P>(ib + T * SM::ROW_IO, p.K.row(n, h, t0), p.K.sl, nt, tid);
      stage_rows<SM::ROW_IO, P>(ib + 2 * T * SM::ROW_IO, p.V.row(n, h, t0), p.V.sl, nt, tid);
    }
    stage_rows<SM::ROW_IO, P>(ib + SM::QKV_BYTES, p.gout.row(n, h, t0), p.gout.sl, nt, tid);
    unsigned char* fb = ib + SM::QKV_BYTES + T * SM::ROW_IO;
    stage_rows<SM::ROW_F, P>(fb, p.v_old.row(n, h, t0), p.v_old.sl, nt, tid);
    stage_rows<SM::ROW_F, P>(fb + T * SM::ROW_F, p.v_ins.row(n, h, t0), p.v_ins.sl, nt, tid);
  };
  auto beta_ld = [&](int c, int i) -> float {
    return to_f32(*reinterpret_cast<const TIO*>(p.beta.row(n, h, c * T + i)));
  };
  auto beta_buf = [&](int b) {
    return reinterpret_cast<float*>(in_buf(b) + SM::QKV_BYTES + T * SM::ROW_IO + 2 * T * SM::ROW_F);
  };

  if (nchunks > 0) {   // (an empty sequence has nothing to stage: W_0 = W_L, dL/dW_0 = 0)
    const int c0 = nchunks - 1;
    stage_chunk(c0);
    cp_async_commit();
    const int nt0 = L - c0 * T;
    if constexpr (!PACKED)
      for (int i = tid; i < nt0; i += P) beta_buf(c0 & 1)[i] = beta_ld(c0, i);
  }

  for (int c = nchunks - 1; c >= 0; --c) {
    const int t0 = c * T, nt = min(T, L - t0);
    if (SRWM_BAD_ROWS(p.dbg, 7, t0, nt, L, T)) break;
    const bool has_next = (c > 0);
    float bnext[(T + P - 1) / P];
    if (has_next) {
      stage_chunk(c - 1);   // full chunk of T steps
      if constexpr (!PACKED) {
#pragma unroll
        for (int u = 0; u < (T + P - 1) / P; ++u) {
          const int i = tid + u * P;
          bnext[u] = (i < T) ? beta_ld(c - 1, i) : 0.f;
        }
      }
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const unsigned char* ib = in_buf(c & 1);
    const TS *sq, *sk, *sv;
    const float* sb;
    float* dsq = dense + 3 * T * E + SM::BETA_BYTES / 4;   // PACKED: sum a(q) + eps, sum a(k) + eps per row
    float* dsk = dsq + SM::BETA_BYTES / 4;
    if constexpr (PACKED) {
      float* dq = dense;
      prepare_packed_rows<TIO, E, P, T, SM::PK_PITCH>(ib, p.Q.row(n, h, t0), p.Q.sl, p.eps, dq, dq + T * E,
                                                      dq + 2 * T * E, dq + 3 * T * E, dsq, dsk, nt, tid);
      __syncthreads();
      sq = dq; sk = dq + T * E; sv = dq + 2 * T * E; sb = dq + 3 * T * E;
    } else {
      sq = reinterpret_cast<const TS*>(ib);
      sk = reinterpret_cast<const TS*>(ib + T * SM::ROW_IO);
      sv = reinterpret_cast<const TS*>(ib + 2 * T * SM::ROW_IO);
      sb = beta_buf(c & 1);
    }
    const TIO* sg = reinterpret_cast<const TIO*>(ib + SM::QKV_BYTES);
    const float* svo = reinterpret_cast<const float*>(ib + SM::QKV_BYTES + T * SM::ROW_IO);
    const float* svi = svo + T * E;

    #pragma unroll 1

    for (int t = nt - 1; t >= 0; --t) {
      float kr[R], qr[R], gc[C], insc[C], vc[C], voc[C];
      ld_rows<R, NRG>(sk + t * E, rg, kr);
      ld_rows<R, NRG>(sq + t * E, rg, qr);
      ld_vec<C>(sg + t * E + cg * C, gc);
      ld_vec<C>(svi + t * E + cg * C, insc);
      ld_vec<C>(sv + t * E + cg * C, vc);
      ld_vec<C>(svo + t * E + cg * C, voc);
      const float bt = sb[t];

      u64 k2[R2], gq2[R2], gk2[R2];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        k2[i2] = pack2(kr[2 * i2], kr[2 * i2 + 1]);
        gq2[i2] = 0ull;
        gk2[i2] = 0ull;
      }
      // G += q^T g ; gq partial = W_t g ; r partial = k.G
      u64 ar[C];
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 g2 = dup2(gc[j]);
        ar[j] = 0ull;
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          const u64 q2 = pack2(qr[2 * i2], qr[2 * i2 + 1]);
          G[i2][j] = fma2<PK>(q2, g2, G[i2][j]);
          gq2[i2] = fma2<PK>(W[i2][j], g2, gq2[i2]);
          ar[j] = fma2<PK>(k2[i2], G[i2][j], ar[j]);
        }
      }
      float gv[C], gb = 0.f;
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const float r = allreduce_rows<NRG>(hsum2(ar[j]));
        gv[j] = bt * r;
        gb = fmaf(r, vc[j] - voc[j], gb);
      }
      // gk partial = G ins + W_{t-1} (-gv) ; revert W ; G += k^T (-gv)
#pragma unroll
      for (int j = 0; j < C; ++j) {
        const u64 ins2 = dup2(insc[j]);
        const u64 ngv2 = dup2(-gv[j]);
#pragma unroll
        for (int i2 = 0; i2 < R2; ++i2) {
          gk2[i2] = fma2<PK>(G[i2][j], ins2, gk2[i2]);
          W[i2][j] = fma2<PK>(neg2(k2[i2]), ins2, W[i2][j]);
          gk2[i2] = fma2<PK>(W[i2][j], ngv2, gk2[i2]);
          G[i2][j] = fma2<PK>(k2[i2], ngv2, G[i2][j]);
        }
      }
      if (rg == 0) st_vec<C>(sgv + t * E + cg * C, gv);
      // row results: reduce across this warp's column groups, park per warp
      float gqr[R], gkr[R];
#pragma unroll
      for (int i2 = 0; i2 < R2; ++i2) {
        unpack2(gq2[i2], gqr[2 * i2], gqr[2 * i2 + 1]);
        unpack2(gk2[i2], gkr[2 * i2], gkr[2 * i2 + 1]);
      }
      gb = allreduce_cols<NRG>(rg == 0 ? gb : 0.f);
      float* part = spart + ((t * NWARP + warp) * 2) * E;
      if constexpr (SCATTER) {
        float v[2 * R];
#pragma unroll
        for (int i = 0; i < R; ++i) { v[i] = gqr[i]; v[R + i] = gkr[i]; }
        reduce_scatter<2 * R, CGW, NRG>(v, lane);
        const int which = cgl >= CGW / 2 ? 1 : 0;   // lower half of the column groups: gq pieces, upper: gk
        st_rows_piece<S_ROW, R, NRG>(part + which * E, rg, (cgl % (CGW / 2)) * S_ROW, v);
      } else {
#pragma unroll
        for (int i = 0; i < R; ++i) {
          gqr[i] = allreduce_cols<NRG>(gqr[i]);
          gkr[i] = allreduce_cols<NRG>(gkr[i]);
        }
        if (lane < NRG) {   // column group 0 of the warp: lane == rg
          st_rows<R, NRG>(part, rg, gqr);
          st_rows<R, NRG>(part + E, rg, gkr);
        }
      }
      if (lane == 0) sgb[t * NWARP + warp] = gb;
    }

    if constexpr (!PACKED) {
      if (has_next) {
#pragma unroll
        for (int u = 0; u < (T + P - 1) / P; ++u) {
          const int i = tid + u * P;
          if (i < T) beta_buf((c - 1) & 1)[i] = bnext[u];
        }
      }
    }
    __syncthreads();
    if constexpr (!PACKED) flush_rows<SM::ROW_IO, P>(p.gV.row(n, h, t0), p.gV.sl, sgv, nt, tid);
    // combine the per-warp partial rows and write gq, gk (4 values per thread-iteration)
    for (int idx = tid; idx < nt * 2 * (E / 4); idx += P) {
      const int e4 = idx % (E / 4);
      const int which = (idx / (E / 4)) % 2;
      const int t = idx / (2 * (E / 4));
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < NWARP; ++w) {
        float v[4];
        ld_vec<4>(spart + ((t * NWARP + w) * 2 + which) * E + e4 * 4, v);
#pragma unroll
        for (int u = 0; u < 4; ++u) acc[u] += v[u];
      }
      if constexpr (PACKED) {
        st_vec<4>(spart + ((t * NWARP) * 2 + which) * E + e4 * 4, acc);   // finished below
      } else {
        const SeqView& dstv = which ? p.gK : p.gQ;
        st_vec<4>(reinterpret_cast<TIO*>(dstv.row(n, h, t0 + t)) + e4 * 4, acc);
      }
    }
    if constexpr (PACKED) {
      // back through the layers' preparation, into the packed gradient row [gq | gk | gv | gb]:
      //   q = a / S  =>  ga = (gq - gq.q) / S ;  a = elu(x) + 1  =>  gx = ga * (x > 0 ? 1 : a), x > 0 <=> a > 1
      __syncthreads();
      constexpr int LPR = E / 4, NG = P / LPR, K = (T + NG - 1) / NG;
      const int grp = tid / LPR, l = tid % LPR;
#pragma unroll
      for (int kk = 0; kk < K; ++kk) {
        const int t = grp + kk * NG;
        const int tc = min(t, nt - 1);
        float gq[4], gk[4], q[4], k[4], gv[4];
        ld_vec<4>(spart + ((tc * NWARP) * 2) * E + l * 4, gq);
        ld_vec<4>(spart + ((tc * NWARP) * 2 + 1) * E + l * 4, gk);
        ld_vec<4>(sq + tc * E + l * 4, q);
        ld_vec<4>(sk + tc * E + l * 4, k);
        ld_vec<4>(sgv + tc * E + l * 4, gv);
        float dq_ = 0.f, dk_ = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          dq_ = fmaf(gq[i], q[i], dq_);
          dk_ = fmaf(gk[i], k[i], dk_);
        }
#pragma unroll
        for (int o = 1; o < LPR; o <<= 1) {
          dq_ += __shfl_xor_sync(0xffffffffu, dq_, o);
          dk_ += __shfl_xor_sync(0xffffffffu, dk_, o);
        }
        const float Sq = dsq[tc], Sk = dsk[tc];
        const float iq = __fdividef(1.f, Sq), ik = __fdividef(1.f, Sk);
        if (t < nt) {
          TIO* g = reinterpret_cast<TIO*>(p.gQ.row(n, h, t0 + t));
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float aq = q[i] * Sq, ak = k[i] * Sk;
            from_f32(g[l * 4 + i], (gq[i] - dq_) * iq * (aq > 1.f ? 1.f : aq));
            from_f32(g[E + l * 4 + i], (gk[i] - dk_) * ik * (ak > 1.f ? 1.f : ak));
            from_f32(g[2 * E + l * 4 + i], gv[i]);
          }
          if (l == 0) {
            float sgbv = 0.f;
#pragma unroll
            for (int w = 0; w < NWARP; ++w) sgbv += sgb[t * NWARP + w];
            const float b = sb[t];
            from_f32(g[3 * E], sgbv * b * (1.f - b));
          }
        }
      }
    } else {
      for (int t = tid; t < nt; t += P) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < NWARP; ++w) s += sgb[t * NWARP + w];
        from_f32(*reinterpret_cast<TIO*>(p.gbeta.row(n, h, t0 + t)), s);
      }
    }
  }

  // W now holds W_0: restore it in place (as the reference does); G is dL/dW_0.
#pragma unroll
  for (int i2 = 0; i2 < R2; ++i2) {
    float a[C], b[C];
#pragma unroll
    for (int j = 0; j < C; ++j) unpack2(W[i2][j], a[j], b[j]);
    st_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
    st_vec<C>(Wg + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
  }
  if (p.gW0.base != nullptr) {
    float* Gg = p.gW0.mat(n, h);
#pragma unroll
    for (int i2 = 0; i2 < R2; ++i2) {
      float a[C], b[C];
#pragma unroll
      for (int j = 0; j < C; ++j) unpack2(G[i2][j], a[j], b[j]);
      st_vec<C>(Gg + (row_of<R, NRG>(rg, 2 * i2)) * E + cg * C, a);
      st_vec<C>(Gg + (row_of<R, NRG>(rg, 2 * i2 + 1)) * E + cg * C, b);
    }
  }
}

}  // namespace srwm
