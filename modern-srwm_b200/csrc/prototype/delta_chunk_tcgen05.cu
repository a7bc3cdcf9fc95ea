// PROTOTYPE (not part of libsrwm_b200.so, not on any product path): the chunkwise (UT-transform)
// form of the delta-rule forward on the Blackwell tensor cores -- tcgen05.mma kind::tf32 with the
// accumulators in tensor memory -- as a standalone program with its own CPU check.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O2 -std=c++17 -o delta_chunk_tcgen05 delta_chunk_tcgen05.cu
//   ./delta_chunk_tcgen05 [sequences] [steps]        (inputs are bfloat16, as in the sweep configuration)
//
// Per chunk of C = 64 steps and one sequence (one CTA of 128 threads, d = 64), with K, Q, V the
// chunk's rows, b its gates and W the state at the start of the chunk
// (recurrence: supervised_learning/fast_weight/__init__.py:186-191):
//   [P ; O1]  = [K ; Q] W                  (128 x 64 x 64 MMA tiles, accumulator D1; W = W_hi + W_lo)
//   [S1; S2]  = [K ; Q] K^T                (D2)
//   U         = (I + tril(b S1, -1))^-1 b (V - P)      fp32 forward substitution, one feature column per thread
//   [VO; O2]  = [tril(S1,-1) ; tril(S2)] U (D3; U = U_hi + U_lo)    v_old = P + VO, out = O1 + O2, v_insert = U
//   W^T      += U^T K                      (DW; the state is kept transposed in tensor memory so that the
//                                           thread that reads row g of it writes row g of the next B operand)
// All operands are K-major in the canonical no-swizzle shared-memory layout (8-row x 16-byte core
// matrices).  The MMA truncates fp32 operands to tf32, so W and U are given as two tf32 terms
// (round-to-nearest high part + remainder).  The chunk's rows arrive through cp.async one chunk
// ahead.  Every wait on the MMA completion barrier is bounded and gives up with a status code.
//
// Status: v_insert and the final state agree with the fp64 recurrence to 1e-6 / 1e-5 of their scale;
// out and v_old to 4e-4 (the triangular factors S1, S2 still enter the third product as single tf32
// terms).  It takes about twice the time of the shipped sequential kernel (3.4 ms against 1.8 ms for
// 1184 sequences x 2048 steps); the per-phase cycle counts it prints show where: the 64-thread
// substitution and the scattered operand conversion.  Kept as the starting point of that row.
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <cmath>
#include <cstring>
#include <cuda_runtime.h>
#include <cuda_bf16.h>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {   // K-major, no swizzle, LBO 128, SBO 2048
  return (uint64_t)((saddr & 0x3FFFF) >> 4) | ((uint64_t)(128 >> 4) << 16) | ((uint64_t)(2048 >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ int canon(int r, int k) { return (r / 8) * 2048 + (k / 4) * 128 + (r % 8) * 16 + (k % 4) * 4; }

__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float (&v)[64]) {
  uint32_t* r = reinterpret_cast<uint32_t*>(v);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    uint32_t* q = r + 32 * h;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
                 : "=r"(q[0]), "=r"(q[1]), "=r"(q[2]), "=r"(q[3]), "=r"(q[4]), "=r"(q[5]), "=r"(q[6]), "=r"(q[7]), "=r"(q[8]), "=r"(q[9]), "=r"(q[10]), "=r"(q[11]), "=r"(q[12]), "=r"(q[13]), "=r"(q[14]), "=r"(q[15]), "=r"(q[16]), "=r"(q[17]), "=r"(q[18]), "=r"(q[19]), "=r"(q[20]), "=r"(q[21]), "=r"(q[22]), "=r"(q[23]), "=r"(q[24]), "=r"(q[25]), "=r"(q[26]), "=r"(q[27]), "=r"(q[28]), "=r"(q[29]), "=r"(q[30]), "=r"(q[31])
                 : "r"(taddr + 32 * h));
  }
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_st64(uint32_t taddr, const float (&v)[64]) {
  const uint32_t* r = reinterpret_cast<const uint32_t*>(v);
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const uint32_t* q = r + 32 * h;
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%32], {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31};"
                 :: "r"(q[0]), "r"(q[1]), "r"(q[2]), "r"(q[3]), "r"(q[4]), "r"(q[5]), "r"(q[6]), "r"(q[7]), "r"(q[8]), "r"(q[9]), "r"(q[10]), "r"(q[11]), "r"(q[12]), "r"(q[13]), "r"(q[14]), "r"(q[15]), "r"(q[16]), "r"(q[17]), "r"(q[18]), "r"(q[19]), "r"(q[20]), "r"(q[21]), "r"(q[22]), "r"(q[23]), "r"(q[24]), "r"(q[25]), "r"(q[26]), "r"(q[27]), "r"(q[28]), "r"(q[29]), "r"(q[30]), "r"(q[31]),
                    "r"(taddr + 32 * h) : "memory");
  }
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void mma_tile(uint32_t d_tmem, uint32_t a_saddr, uint32_t b_saddr, bool accumulate_first) {
  const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((64u >> 3) << 17) | ((128u >> 4) << 24);
#pragma unroll
  for (int k8 = 0; k8 < 8; ++k8) {
    const uint64_t da = make_desc(a_saddr + k8 * 256), db = make_desc(b_saddr + k8 * 256);
    const uint32_t acc = (k8 > 0 || accumulate_first) ? 1u : 0u;
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(da), "l"(db), "r"(idesc), "r"(acc) : "memory");
  }
}
__device__ __forceinline__ bool wait_bar(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < 4000000; ++it) {
    uint32_t done;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

constexpr int C = 64, E = 64, PADW = 65;
constexpr int OFF_KQ = 0, OFF_KT = 32768, OFF_WT = 49152, OFF_WL = 65536, OFF_L = 81920, OFF_UT = 114688, OFF_UL = 131072,
              OFF_A = 147456;
constexpr int OFF_R = OFF_A + C * PADW * 4, OFF_ST = OFF_R + C * PADW * 4 + 128;   // staging: K, Q, V rows (bf16)
constexpr int ST_BYTES = 3 * C * E * 2, SMEM_TOTAL = OFF_ST + ST_BYTES;
__device__ __forceinline__ float tf32_hi(float x) { uint32_t r; asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x)); return __uint_as_float(r); }
__device__ __forceinline__ void cp16(void* d, const void* g) { asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(d)), "l"(g) : "memory"); }

__global__ void __launch_bounds__(128, 1)
k_chunk(const __nv_bfloat16* Q, const __nv_bfloat16* K, const __nv_bfloat16* V, const float* B, float* W, float* out,
        float* vold, float* vins, int L, int* status) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ __align__(8) uint64_t mbar;
  __shared__ uint32_t tmem_base_s;
  const int tid = threadIdx.x, warp = tid / 32;
  const int n = blockIdx.x;
  const __nv_bfloat16* Qn = Q + (size_t)n * L * E; const __nv_bfloat16* Kn = K + (size_t)n * L * E;
  const __nv_bfloat16* Vn = V + (size_t)n * L * E;
  __nv_bfloat16* stK = reinterpret_cast<__nv_bfloat16*>(smem + OFF_ST);
  __nv_bfloat16* stQ = stK + C * E;
  __nv_bfloat16* stV = stQ + C * E;
  auto stage = [&](int c) {   // 64 rows x 128 B per tensor, contiguous in global: 512 x 16 B each
    const int t0 = c * C;
    for (int i = tid; i < 512; i += 128) {
      cp16(reinterpret_cast<char*>(stK) + i * 16, reinterpret_cast<const char*>(Kn + (size_t)t0 * E) + i * 16);
      cp16(reinterpret_cast<char*>(stQ) + i * 16, reinterpret_cast<const char*>(Qn + (size_t)t0 * E) + i * 16);
      cp16(reinterpret_cast<char*>(stV) + i * 16, reinterpret_cast<const char*>(Vn + (size_t)t0 * E) + i * 16);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  const float* Bn = B + (size_t)n * L; float* Wn = W + (size_t)n * E * E;
  float* outn = out + (size_t)n * L * E; float* voldn = vold + (size_t)n * L * E; float* vinsn = vins + (size_t)n * L * E;
  float* sA = reinterpret_cast<float*>(smem + OFF_A);
  float* sR = reinterpret_cast<float*>(smem + OFF_R);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&mbar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(256));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tm = tmem_base_s;
  const uint32_t trow = tm + ((uint32_t)(warp * 32) << 16);     // this warp's lanes
  const uint32_t D1 = 0, D2 = 64, D3 = 128, DW = 192;
  const uint32_t bar = smem_u32(&mbar);
  const uint32_t sbase = smem_u32(smem);
  uint32_t phase = 0;
  bool alive = true;
  long long tacc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  long long tl = clock64();
#define TICK(i) { long long tn = clock64(); tacc[i] += tn - tl; tl = tn; }
  // W^T into TMEM (row g = column g of W) and into the B operand buffer
  if (tid < 64) {
    float wrow[64];
#pragma unroll
    for (int k = 0; k < 64; ++k) wrow[k] = Wn[k * E + tid];
    tmem_st64(trow + DW, wrow);
#pragma unroll
    for (int k4 = 0; k4 < 16; ++k4) {
      float h[4], l[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { h[i] = tf32_hi(wrow[4 * k4 + i]); l[i] = wrow[4 * k4 + i] - h[i]; }
      *reinterpret_cast<float4*>(smem + OFF_WT + canon(tid, 4 * k4)) = make_float4(h[0], h[1], h[2], h[3]);
      *reinterpret_cast<float4*>(smem + OFF_WL + canon(tid, 4 * k4)) = make_float4(l[0], l[1], l[2], l[3]);
    }
  }
  const int nchunks = L / C;
  stage(0);
  for (int c = 0; c < nchunks && alive; ++c) {
    const int t0 = c * C;
    // (1) operands from the chunk's rows
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    TICK(0)
    for (int i = tid; i < C * E; i += 128) {
      const int t = i / E, f = i % E;
      const float kv = __bfloat162float(stK[i]), qv = __bfloat162float(stQ[i]);
      *reinterpret_cast<float*>(smem + OFF_KQ + canon(t, f)) = kv;
      *reinterpret_cast<float*>(smem + OFF_KQ + canon(64 + t, f)) = qv;
      *reinterpret_cast<float*>(smem + OFF_KT + canon(f, t)) = kv;
    }
    float vrow[64];          // this thread's V row (token rows only)
    if (tid < 64) {
#pragma unroll
      for (int cc = 0; cc < 64; ++cc) vrow[cc] = __bfloat162float(stV[tid * E + cc]);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    TICK(1)
    // (2) [P;O1] = [K;Q] W ,  [S1;S2] = [K;Q] K^T
    if (tid == 0) {
      mma_tile(tm + D1, sbase + OFF_KQ, sbase + OFF_WT, false);
      mma_tile(tm + D1, sbase + OFF_KQ, sbase + OFF_WL, true);
      mma_tile(tm + D2, sbase + OFF_KQ, sbase + OFF_KQ, false);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
    if (c + 1 < nchunks) stage(c + 1);   // staging buffer was fully consumed before the barrier above
    if (!wait_bar(bar, phase)) { alive = false; if (tid == 0) status[0] = 1 + c; }
    alive = __syncthreads_and(alive ? 1 : 0) != 0;
    phase ^= 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    TICK(2)
    float keep[64];   // P (token rows) or O1 (query rows)
    if (alive) {
      float s[64];
      tmem_ld64(trow + D1, keep);
      tmem_ld64(trow + D2, s);
      if (tid < 64) {
        const int t = tid;
        const float bt = Bn[t0 + t];
#pragma unroll
        for (int cc = 0; cc < 64; ++cc) sR[t * PADW + cc] = bt * (vrow[cc] - keep[cc]);
#pragma unroll
        for (int ss = 0; ss < 64; ++ss) sA[t * PADW + ss] = ss < t ? bt * s[ss] : 0.f;
#pragma unroll
        for (int s4 = 0; s4 < 16; ++s4)
          *reinterpret_cast<float4*>(smem + OFF_L + canon(t, 4 * s4)) =
              make_float4(4 * s4 < t ? s[4 * s4] : 0.f, 4 * s4 + 1 < t ? s[4 * s4 + 1] : 0.f, 4 * s4 + 2 < t ? s[4 * s4 + 2] : 0.f,
                          4 * s4 + 3 < t ? s[4 * s4 + 3] : 0.f);
      } else {
        const int t = tid - 64;
#pragma unroll
        for (int s4 = 0; s4 < 16; ++s4)
          *reinterpret_cast<float4*>(smem + OFF_L + canon(64 + t, 4 * s4)) =
              make_float4(4 * s4 <= t ? s[4 * s4] : 0.f, 4 * s4 + 1 <= t ? s[4 * s4 + 1] : 0.f, 4 * s4 + 2 <= t ? s[4 * s4 + 2] : 0.f,
                          4 * s4 + 3 <= t ? s[4 * s4 + 3] : 0.f);
      }
    }
    __syncthreads();
    TICK(3)
    // (4) forward substitution, one feature column per thread
    if (alive && tid < 64) {
      const int cc = tid;
      float u[64];
#pragma unroll
      for (int t = 0; t < 64; ++t) {
        float a8[8] = {sR[t * PADW + cc], 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ss = 0; ss < t; ++ss) a8[ss % 8] = fmaf(-sA[t * PADW + ss], u[ss], a8[ss % 8]);
        u[t] = ((a8[0] + a8[1]) + (a8[2] + a8[3])) + ((a8[4] + a8[5]) + (a8[6] + a8[7]));
      }
#pragma unroll
      for (int t = 0; t < 64; ++t) vinsn[(size_t)(t0 + t) * E + cc] = u[t];
#pragma unroll
      for (int t4 = 0; t4 < 16; ++t4) {
        float h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { h[i] = tf32_hi(u[4 * t4 + i]); l[i] = u[4 * t4 + i] - h[i]; }
        *reinterpret_cast<float4*>(smem + OFF_UT + canon(cc, 4 * t4)) = make_float4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<float4*>(smem + OFF_UL + canon(cc, 4 * t4)) = make_float4(l[0], l[1], l[2], l[3]);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    TICK(4)
    // (5) [VO;O2] = [L1;L2] U ,  W^T += U^T K
    if (tid == 0 && alive) {
      mma_tile(tm + D3, sbase + OFF_L, sbase + OFF_UT, false);
      mma_tile(tm + D3, sbase + OFF_L, sbase + OFF_UL, true);
      mma_tile(tm + DW, sbase + OFF_UT, sbase + OFF_KT, true);
      mma_tile(tm + DW, sbase + OFF_UL, sbase + OFF_KT, true);
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
    }
    if (alive && !wait_bar(bar, phase)) { alive = false; if (tid == 0) status[0] = 1000 + c; }
    alive = __syncthreads_and(alive ? 1 : 0) != 0;
    phase ^= 1;
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    TICK(5)
    if (alive) {
      float d3[64];
      tmem_ld64(trow + D3, d3);
      if (tid < 64) {
        const int t = tid;
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4)
          *reinterpret_cast<float4*>(voldn + (size_t)(t0 + t) * E + 4 * c4) =
              make_float4(keep[4 * c4] + d3[4 * c4], keep[4 * c4 + 1] + d3[4 * c4 + 1], keep[4 * c4 + 2] + d3[4 * c4 + 2], keep[4 * c4 + 3] + d3[4 * c4 + 3]);
        float wrow[64];
        tmem_ld64(trow + DW, wrow);
#pragma unroll
        for (int k4 = 0; k4 < 16; ++k4) {
          float h[4], l[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) { h[i] = tf32_hi(wrow[4 * k4 + i]); l[i] = wrow[4 * k4 + i] - h[i]; }
          *reinterpret_cast<float4*>(smem + OFF_WT + canon(tid, 4 * k4)) = make_float4(h[0], h[1], h[2], h[3]);
          *reinterpret_cast<float4*>(smem + OFF_WL + canon(tid, 4 * k4)) = make_float4(l[0], l[1], l[2], l[3]);
        }
        if (c == nchunks - 1) {
#pragma unroll
          for (int k = 0; k < 64; ++k) Wn[k * E + tid] = wrow[k];
        }
      } else {
        const int t = tid - 64;
#pragma unroll
        for (int c4 = 0; c4 < 16; ++c4)
          *reinterpret_cast<float4*>(outn + (size_t)(t0 + t) * E + 4 * c4) =
              make_float4(keep[4 * c4] + d3[4 * c4], keep[4 * c4 + 1] + d3[4 * c4 + 1], keep[4 * c4 + 2] + d3[4 * c4 + 2], keep[4 * c4 + 3] + d3[4 * c4 + 3]);
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    TICK(6)
  }
  if (tid == 0 && n == 0) for (int i = 0; i < 8; ++i) reinterpret_cast<long long*>(status + 2)[i] = tacc[i];
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tm), "r"(256));
}

int main(int argc, char** argv) {
  const int N = argc > 1 ? atoi(argv[1]) : 4, L = argc > 2 ? atoi(argv[2]) : 256;
  const size_t nl = (size_t)N * L * E;
  std::vector<float> Q(nl), K(nl), V(nl), B((size_t)N * L), W((size_t)N * E * E), out(nl), vold(nl), vins(nl);
  srand(3);
  auto rnd = []() { return (rand() % 20001 - 10000) / 10000.f; };
  for (size_t i = 0; i < (size_t)N * L; ++i) {   // q,k = softmax(normal-ish), beta = sigmoid
    double sq = 0, sk = 0; float q[64], k[64];
    for (int f = 0; f < E; ++f) { q[f] = expf(1.7f * rnd()); k[f] = expf(1.7f * rnd()); sq += q[f]; sk += k[f]; }
    for (int f = 0; f < E; ++f) { Q[i * E + f] = (float)(q[f] / sq); K[i * E + f] = (float)(k[f] / sk); V[i * E + f] = 1.5f * rnd(); }
    B[i] = 1.f / (1.f + expf(-2.f * rnd()));
  }
  auto bf = [](float x) { uint32_t u; memcpy(&u, &x, 4); u = (u + 0x7FFF + ((u >> 16) & 1)) & 0xFFFF0000u; float y; memcpy(&y, &u, 4); return y; };
  { for (auto& x : Q) x = bf(x); for (auto& x : K) x = bf(x); for (auto& x : V) x = bf(x); for (auto& x : B) x = bf(x); }
  for (auto& w : W) w = 0.1f * rnd();
  // reference (double)
  std::vector<double> Wd(W.begin(), W.end());
  std::vector<float> r_out(nl), r_vold(nl), r_vins(nl);
  for (int n = 0; n < N; ++n) for (int t = 0; t < L; ++t) {
    double* Wn = Wd.data() + (size_t)n * E * E; const size_t o = ((size_t)n * L + t) * E;
    double vo[64], ins[64];
    for (int c = 0; c < E; ++c) { double s = 0; for (int r = 0; r < E; ++r) s += (double)K[o + r] * Wn[r * E + c]; vo[c] = s; ins[c] = (double)B[(size_t)n * L + t] * (V[o + c] - s); }
    for (int r = 0; r < E; ++r) for (int c = 0; c < E; ++c) Wn[r * E + c] += (double)K[o + r] * ins[c];
    for (int c = 0; c < E; ++c) { double s = 0; for (int r = 0; r < E; ++r) s += (double)Q[o + r] * Wn[r * E + c]; r_out[o + c] = (float)s; r_vold[o + c] = (float)vo[c]; r_vins[o + c] = (float)ins[c]; }
  }
  float *dB, *dW, *dO, *dVo, *dVi; int* dS; __nv_bfloat16 *dQ, *dK, *dV;
  cudaMalloc(&dQ, nl * 2); cudaMalloc(&dK, nl * 2); cudaMalloc(&dV, nl * 2); cudaMalloc(&dB, (size_t)N * L * 4); cudaMalloc(&dW, W.size() * 4);
  std::vector<__nv_bfloat16> hQ(nl), hK(nl), hV(nl);
  for (size_t i = 0; i < nl; ++i) { hQ[i] = __float2bfloat16(Q[i]); hK[i] = __float2bfloat16(K[i]); hV[i] = __float2bfloat16(V[i]); }
  cudaMalloc(&dO, nl * 4); cudaMalloc(&dVo, nl * 4); cudaMalloc(&dVi, nl * 4); cudaMalloc(&dS, 128);
  cudaMemcpy(dQ, hQ.data(), nl * 2, cudaMemcpyHostToDevice); cudaMemcpy(dK, hK.data(), nl * 2, cudaMemcpyHostToDevice);
  cudaMemcpy(dV, hV.data(), nl * 2, cudaMemcpyHostToDevice); cudaMemcpy(dB, B.data(), (size_t)N * L * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dW, W.data(), W.size() * 4, cudaMemcpyHostToDevice); cudaMemset(dS, 0, 128);
  cudaMemset(dO, 0, nl * 4); cudaMemset(dVo, 0, nl * 4); cudaMemset(dVi, 0, nl * 4);
  cudaFuncSetAttribute(k_chunk, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL + 1024);
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaEventRecord(e0);
  k_chunk<<<N, 128, SMEM_TOTAL + 1024>>>(dQ, dK, dV, dB, dW, dO, dVo, dVi, L, dS);
  cudaEventRecord(e1);
  cudaError_t e = cudaDeviceSynchronize();
  printf("kernel: %s\n", cudaGetErrorString(e));
  if (e != cudaSuccess) return 0;
  float ms; cudaEventElapsedTime(&ms, e0, e1);
  int st; cudaMemcpy(&st, dS, 4, cudaMemcpyDeviceToHost);
  long long ta[8]; cudaMemcpy(ta, reinterpret_cast<char*>(dS) + 8, 64, cudaMemcpyDeviceToHost);
  printf("cycles per chunk (thread 0): wait-stage %lld convert %lld mma1-wait %lld ld+build %lld solve %lld mma2-wait %lld epilogue %lld\n", ta[0] / (L / 64), ta[1] / (L / 64), ta[2] / (L / 64), ta[3] / (L / 64), ta[4] / (L / 64), ta[5] / (L / 64), ta[6] / (L / 64));
  cudaMemcpy(out.data(), dO, nl * 4, cudaMemcpyDeviceToHost); cudaMemcpy(vold.data(), dVo, nl * 4, cudaMemcpyDeviceToHost);
  cudaMemcpy(vins.data(), dVi, nl * 4, cudaMemcpyDeviceToHost); cudaMemcpy(W.data(), dW, W.size() * 4, cudaMemcpyDeviceToHost);
  auto relmax = [](const std::vector<float>& a, const std::vector<float>& b) { double me = 0, mr = 0; for (size_t i = 0; i < a.size(); ++i) { me = fmax(me, fabs((double)a[i] - b[i])); mr = fmax(mr, fabs((double)b[i])); } return me / mr; };
  std::vector<float> r_W(Wd.begin(), Wd.end());
  printf("status %d  time %.3f ms  rel err: out %.3g  v_old %.3g  v_ins %.3g  W_L %.3g\n", st, ms, relmax(out, r_out), relmax(vold, r_vold), relmax(vins, r_vins), relmax(W, r_W));
  return 0;
}
