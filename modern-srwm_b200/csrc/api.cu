// C ABI of libsrwm_b200.so (see include/srwm_b200.h): argument validation, conversion of
// element strides to the kernels' byte strides, dispatch to the compiled configuration.
// All validation happens before the first CUDA call.
#include "srwm_b200.h"

#include "configs.h"
#include "launch.h"

#ifdef SRWM_DEBUG_CHECKS
// Status word of the debug build's row checks (common.cuh::bad_rows), one per device.
__device__ unsigned long long g_debug_status = 0ull;
#endif

namespace {

thread_local int g_last_cuda_error = 0;

// Device address of the status word (debug build), null in the ordinary build.
inline unsigned long long* debug_word() {
#ifdef SRWM_DEBUG_CHECKS
  unsigned long long* ptr = nullptr;
  if (cudaGetSymbolAddress((void**)&ptr, g_debug_status) != cudaSuccess) {
    (void)cudaGetLastError();
    return nullptr;
  }
  return ptr;
#else
  return nullptr;
#endif
}

inline int esize(int dtype) { return dtype == SRWM_B200_BF16 ? 2 : 4; }

inline bool head_dim_ok(int E) { return E == 8 || E == 16 || E == 32 || E == 64; }

// Every row of a streamed tensor must start on a 16-byte boundary.
inline bool seq_aligned(const srwm_b200_seq& t, int es) {
  return ((uintptr_t)t.data % 16 == 0) && ((t.stride_n * es) % 16 == 0) && ((t.stride_h * es) % 16 == 0) &&
         ((t.stride_l * es) % 16 == 0);
}
inline bool state_aligned(const srwm_b200_state& t) {
  return ((uintptr_t)t.data % 16 == 0) && ((t.stride_n * 4) % 16 == 0) && ((t.stride_h * 4) % 16 == 0);
}
inline srwm::SeqView view(const srwm_b200_seq& t, int es) {
  srwm::SeqView v;
  v.base = reinterpret_cast<char*>(t.data);
  v.sn = t.stride_n * es;
  v.sh = t.stride_h * es;
  v.sl = t.stride_l * es;
  return v;
}
inline srwm::StateView view(const srwm_b200_state& t) {
  srwm::StateView v;
  v.base = t.data;
  v.sn = t.stride_n;
  v.sh = t.stride_h;
  return v;
}

inline int check_dims(int N, int H, int L, long long* grid) {
  if (N < 0 || H < 0 || L < 0) return SRWM_B200_ERR_SHAPE;
  const long long g = (long long)N * H;
  if (g > 0x7fffffffLL) return SRWM_B200_ERR_SHAPE;
  *grid = g;
  return 0;
}

// Extension block of the layer-level calls: all four base_* or none; shift and done need a
// base.  Sets the kernels' flag bits.
inline int check_ext(const srwm_b200_srwm_ext* x, bool forward, unsigned* flags) {
  *flags = 0;
  if (!x) return 0;
  const int nb = (x->base_W_y.data != nullptr) + (x->base_W_q.data != nullptr) + (x->base_W_k.data != nullptr) +
                 (x->base_w_b.data != nullptr);
  const int ns = (x->shift_W_y.data != nullptr) + (x->shift_W_q.data != nullptr) + (x->shift_W_k.data != nullptr) +
                 (x->shift_w_b.data != nullptr);
  if (nb != 0 && nb != 4) return SRWM_B200_ERR_NULL;
  if (ns != 0 && ns != 4) return SRWM_B200_ERR_NULL;
  if (nb == 0) return (ns != 0 || x->done != nullptr) ? SRWM_B200_ERR_NULL : 0;
  if (!state_aligned(x->base_W_y) || !state_aligned(x->base_W_q) || !state_aligned(x->base_W_k) ||
      !state_aligned(x->base_w_b))
    return SRWM_B200_ERR_ALIGN;
  *flags |= srwm::F_BASE;
  if (forward && ns == 4) {
    if (!state_aligned(x->shift_W_y) || !state_aligned(x->shift_W_q) || !state_aligned(x->shift_W_k) ||
        !state_aligned(x->shift_w_b))
      return SRWM_B200_ERR_ALIGN;
    *flags |= srwm::F_SHIFT_IN;
  }
  if (forward && x->done) *flags |= srwm::F_DONE;
  // a reverse-time backward cannot cross an in-kernel reset (the pre-reset state is gone)
  if (!forward && x->done) return SRWM_B200_ERR_UNSUPPORTED;
  return 0;
}

inline int finish(int rc, int cuda_err) {
  if (rc == -7) {
    g_last_cuda_error = cuda_err;
    return SRWM_B200_ERR_CUDA;
  }
  if (rc == -6) return SRWM_B200_ERR_VARIANT;
  if (rc == -3) return SRWM_B200_ERR_HEAD_DIM;
  return rc;
}

}  // namespace

extern "C" {

int srwm_b200_abi_version(void) { return SRWM_B200_ABI_VERSION; }

int srwm_b200_head_dim_supported(int32_t E) { return head_dim_ok(E) ? 1 : 0; }

int srwm_b200_last_cuda_error(void) { return g_last_cuda_error; }

const char* srwm_b200_strerror(int code) {
  switch (code) {
    case SRWM_B200_OK: return "ok";
    case SRWM_B200_ERR_NULL: return "a required pointer is NULL";
    case SRWM_B200_ERR_SHAPE: return "invalid shape (negative size or N*H too large)";
    case SRWM_B200_ERR_HEAD_DIM: return "head dimension not supported (E must be 8, 16, 32 or 64; delta rule needs M == E)";
    case SRWM_B200_ERR_DTYPE: return "unknown io_dtype";
    case SRWM_B200_ERR_ALIGN: return "a tensor row does not start on a 16-byte boundary";
    case SRWM_B200_ERR_VARIANT: return "kernel variant not compiled in";
    case SRWM_B200_ERR_CUDA: return "CUDA runtime error (see srwm_b200_last_cuda_error)";
    case SRWM_B200_ERR_TOO_LARGE: return "size exceeds the fixed capacity of this entry point";
    case SRWM_B200_ERR_UNSUPPORTED: return "this combination of arguments is not supported by the entry point";
    default: return "unknown error code";
  }
}

int srwm_b200_describe_for_grid(int32_t op, int32_t E, int32_t io_dtype, int32_t variant, int64_t grid,
                                int32_t num_sms, int32_t out[5]) {
  if (!out) return SRWM_B200_ERR_NULL;
  if (io_dtype != SRWM_B200_F32 && io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid < 0 || grid > 0x7fffffffLL) return SRWM_B200_ERR_SHAPE;
  srwm::KernelInfo info = {0, 0, 0, 0, 0};
  int ce = 0, rc;
  const bool bf = io_dtype == SRWM_B200_BF16;
  const int g = (int)grid, sms = num_sms > 0 ? num_sms : srwm::DEFAULT_SMS;
  switch (op) {
    case srwm::OP_SRWM_FWD: {
      srwm::SrwmFwdParams p = {};
      rc = bf ? srwm::dispatch_srwm_fwd_bf16(E, variant, p, g, 0, &info, 1, &ce, sms)
              : srwm::dispatch_srwm_fwd_f32(E, variant, p, g, 0, &info, 1, &ce, sms);
      break;
    }
    case srwm::OP_SRWM_BWD: {
      srwm::SrwmBwdParams p = {};
      rc = bf ? srwm::dispatch_srwm_bwd_bf16(E, variant, p, g, 0, &info, 1, &ce, sms)
              : srwm::dispatch_srwm_bwd_f32(E, variant, p, g, 0, &info, 1, &ce, sms);
      break;
    }
    case srwm::OP_SRWM_BWD_DET: {
      srwm::SrwmBwdDetParams p = {};
      rc = bf ? srwm::dispatch_srwm_bwd_det_bf16(E, variant, p, g, 0, &info, 1, &ce, sms)
              : srwm::dispatch_srwm_bwd_det_f32(E, variant, p, g, 0, &info, 1, &ce, sms);
      break;
    }
    case srwm::OP_DELTA_FWD: {
      srwm::DeltaFwdParams p = {};
      rc = bf ? srwm::dispatch_delta_fwd_bf16(E, variant, p, g, 0, &info, 1, &ce, sms)
              : srwm::dispatch_delta_fwd_f32(E, variant, p, g, 0, &info, 1, &ce, sms);
      break;
    }
    case srwm::OP_DELTA_BWD: {
      srwm::DeltaBwdParams p = {};
      rc = bf ? srwm::dispatch_delta_bwd_bf16(E, variant, p, g, 0, &info, 1, &ce, sms)
              : srwm::dispatch_delta_bwd_f32(E, variant, p, g, 0, &info, 1, &ce, sms);
      break;
    }
    default:
      return SRWM_B200_ERR_SHAPE;
  }
  if (rc != 0) return finish(rc, ce);
  out[0] = info.P; out[1] = info.R; out[2] = info.T; out[3] = info.smem; out[4] = info.id;
  return 0;
}

int srwm_b200_describe(int32_t op, int32_t E, int32_t io_dtype, int32_t variant, int32_t out[4]) {
  if (!out) return SRWM_B200_ERR_NULL;
  int32_t o5[5];
  // a grid large enough to fill any GPU: the configuration of full waves
  const int rc = srwm_b200_describe_for_grid(op, E, io_dtype, variant, 1 << 20, 0, o5);
  if (rc != 0) return rc;
  out[0] = o5[0]; out[1] = o5[1]; out[2] = o5[2]; out[3] = o5[3];
  return 0;
}

int srwm_b200_num_variants(int32_t op, int32_t E) {
  int n = 0;
  int32_t tmp[4];
  while (n < 64 && srwm_b200_describe(op, E, SRWM_B200_F32, n, tmp) == 0) ++n;
  return n;
}

// ---------------------------------------------------------------------------------------
int srwm_b200_srwm_forward(const srwm_b200_srwm_fwd_args* a, void* stream) {
  return srwm_b200_srwm_layer_forward(a, nullptr, stream);
}

int srwm_b200_srwm_backward(const srwm_b200_srwm_bwd_args* a, void* stream) {
  return srwm_b200_srwm_layer_backward(a, nullptr, stream);
}

int srwm_b200_srwm_layer_forward(const srwm_b200_srwm_fwd_args* a, const srwm_b200_srwm_ext* x, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E)) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0 || a->L == 0) return 0;
  const bool save = !(a->flags & SRWM_B200_FLAG_NO_SAVE);
  if (!a->x.data || !a->out.data || !a->W_y.data || !a->W_q.data || !a->W_k.data || !a->w_b.data)
    return SRWM_B200_ERR_NULL;
  if (save && (!a->q.data || !a->k.data || !a->beta.data || !a->y_diff.data || !a->q_diff.data ||
               !a->k_diff.data || !a->beta_diff.data))
    return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = seq_aligned(a->x, es) && seq_aligned(a->out, es) && state_aligned(a->W_y) && state_aligned(a->W_q) &&
            state_aligned(a->W_k) && state_aligned(a->w_b);
  if (save)
    ok = ok && seq_aligned(a->q, 4) && seq_aligned(a->k, 4) && seq_aligned(a->beta, 4) && seq_aligned(a->y_diff, 4) &&
         seq_aligned(a->q_diff, 4) && seq_aligned(a->k_diff, 4) && seq_aligned(a->beta_diff, 4);
  if (!ok) return SRWM_B200_ERR_ALIGN;
  unsigned ext_flags = 0;
  if (int rc = check_ext(x, /*forward=*/true, &ext_flags)) return rc;

  srwm::SrwmFwdParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L;
  p.flags = (a->flags & (SRWM_B200_FLAG_NO_SAVE | SRWM_B200_FLAG_INPUT_SOFTMAX)) | ext_flags;
  if (ext_flags & srwm::F_BASE) {
    p.bWy = view(x->base_W_y); p.bWq = view(x->base_W_q); p.bWk = view(x->base_W_k); p.bwb = view(x->base_w_b);
    p.sWy = view(x->shift_W_y); p.sWq = view(x->shift_W_q); p.sWk = view(x->shift_W_k); p.swb = view(x->shift_w_b);
    p.done = x->done; p.done_sn = x->done_stride_n; p.done_sl = x->done_stride_l;
  }
  p.x = view(a->x, es); p.out = view(a->out, es);
  p.q = view(a->q, 4); p.k = view(a->k, 4); p.beta = view(a->beta, 4);
  p.yd = view(a->y_diff, 4); p.qd = view(a->q_diff, 4); p.kd = view(a->k_diff, 4); p.bd = view(a->beta_diff, 4);
  p.Wy = view(a->W_y); p.Wq = view(a->W_q); p.Wk = view(a->W_k); p.wb = view(a->w_b);
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_srwm_fwd_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_srwm_fwd_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}

namespace {
// group size of the fused batch reduction, and the scratch it needs: [H][ng+1] counters (padded to 256
// bytes), then [H][ng] partial states when there is more than one group
constexpr int REDUCE_GROUP = 32;
inline int reduce_groups(int N) { return N <= 2 * REDUCE_GROUP ? 1 : (N + REDUCE_GROUP - 1) / REDUCE_GROUP; }
inline int reduce_group_size(int N) { return N <= 2 * REDUCE_GROUP ? (N > 0 ? N : 1) : REDUCE_GROUP; }
inline size_t reduce_counter_bytes(int N, int H) {
  return (((size_t)H * (reduce_groups(N) + 1) * 4) + 255) / 256 * 256;
}
inline size_t reduce_scratch_bytes(int N, int H, int E) {
  const int ng = reduce_groups(N);
  return reduce_counter_bytes(N, H) + (ng > 1 ? (size_t)H * ng * (3 * E * E + 4 * E) * 4 : 0);
}
int layer_backward_impl(const srwm_b200_srwm_bwd_args* a, const srwm_b200_srwm_ext* x,
                        const srwm_b200_srwm_reduce* red, void* scratch, void* stream);
}  // namespace

size_t srwm_b200_srwm_reduce_scratch_bytes(int32_t N, int32_t H, int32_t E) {
  if (N < 0 || H < 0 || !head_dim_ok(E)) return 0;
  return reduce_scratch_bytes(N, H, E);
}

int srwm_b200_srwm_layer_backward(const srwm_b200_srwm_bwd_args* a, const srwm_b200_srwm_ext* x, void* stream) {
  return layer_backward_impl(a, x, nullptr, nullptr, stream);
}

int srwm_b200_srwm_layer_backward_reduced(const srwm_b200_srwm_bwd_args* a, const srwm_b200_srwm_ext* x,
                                          const srwm_b200_srwm_reduce* red, void* stream) {
  if (!red) return SRWM_B200_ERR_NULL;
  if (a && a->N > 0 && a->H > 0 && head_dim_ok(a->E)) {
    if (!red->scratch) return SRWM_B200_ERR_NULL;
    if ((uintptr_t)red->scratch % 256) return SRWM_B200_ERR_ALIGN;
    if (red->scratch_bytes < 0 || (size_t)red->scratch_bytes < reduce_scratch_bytes(a->N, a->H, a->E))
      return SRWM_B200_ERR_TOO_LARGE;
  }
  return layer_backward_impl(a, x, red, red->scratch, stream);
}

// ---------------------------------------------------------------------------------------
// The same call for hosts that cannot allocate device memory.  Its working memory is this
// array, which is part of the library image: every GPU that loads the library sets the
// SRWM_B200_STATIC_SCRATCH_BYTES aside until the process exits, whether or not the entry point
// is ever called.  In host code the array's name is only a handle for the runtime, not a
// device address, so the address is looked up with cudaGetSymbolAddress -- once per device,
// with that device current -- and that pointer is what the kernel receives.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_static_reduce_scratch[SRWM_B200_STATIC_SCRATCH_BYTES];

namespace {
// Device address of the array on the current device; looked up on the first call per device and
// remembered (the look-up allocates nothing, but it is a runtime call that should not fall inside
// a stream capture, which is why the first call on a device should be made outside one).
void* static_scratch_address(int* cuda_err) {
  static void* cache[64] = {nullptr};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { *cuda_err = (int)e; return nullptr; }
  if (dev < 0 || dev >= 64) { *cuda_err = (int)cudaErrorInvalidDevice; return nullptr; }
  void* ptr = __atomic_load_n(&cache[dev], __ATOMIC_ACQUIRE);
  if (ptr) return ptr;
  e = cudaGetSymbolAddress((void**)&ptr, g_static_reduce_scratch);
  if (e != cudaSuccess || !ptr) {
    *cuda_err = (int)(e != cudaSuccess ? e : cudaErrorInvalidSymbol);
    (void)cudaGetLastError();
    return nullptr;
  }
  __atomic_store_n(&cache[dev], ptr, __ATOMIC_RELEASE);
  return ptr;
}
}  // namespace

int srwm_b200_srwm_layer_backward_reduced_static(const srwm_b200_srwm_bwd_args* a, const srwm_b200_srwm_ext* x,
                                                 const srwm_b200_srwm_reduce* red, void* stream) {
  if (!a || !red) return SRWM_B200_ERR_NULL;
  void* ptr = nullptr;
  if (a->N > 0 && a->H > 0 && head_dim_ok(a->E)) {
    // sizes first: a call that does not fit is refused before anything touches the device
    if (reduce_scratch_bytes(a->N, a->H, a->E) > (size_t)SRWM_B200_STATIC_SCRATCH_BYTES) return SRWM_B200_ERR_TOO_LARGE;
    int ce = 0;
    ptr = static_scratch_address(&ce);
    if (!ptr) {
      g_last_cuda_error = ce;
      return SRWM_B200_ERR_CUDA;
    }
  }
  // red->scratch / scratch_bytes are not looked at.  The shared routine clears the counters at the head
  // of the array on the caller's stream (cudaMemsetAsync) before the kernel runs: whatever the
  // previous call left in the array is either cleared (counters) or overwritten before it is read
  // (group partials).
  return layer_backward_impl(a, x, red, ptr, stream);
}

namespace {
int layer_backward_impl(const srwm_b200_srwm_bwd_args* a, const srwm_b200_srwm_ext* x,
                        const srwm_b200_srwm_reduce* red, void* scratch, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E)) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0) return 0;
  if (!a->W_y.data || !a->W_q.data || !a->W_k.data || !a->w_b.data || !a->grad_W_y.data || !a->grad_W_q.data ||
      !a->grad_W_k.data || !a->grad_w_b.data)
    return SRWM_B200_ERR_NULL;
  if (a->L > 0 && (!a->x.data || !a->q.data || !a->k.data || !a->beta.data || !a->y_diff.data || !a->q_diff.data ||
                   !a->k_diff.data || !a->beta_diff.data || !a->grad_out.data || !a->grad_x.data))
    return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = state_aligned(a->W_y) && state_aligned(a->W_q) && state_aligned(a->W_k) && state_aligned(a->w_b) &&
            state_aligned(a->grad_W_y) && state_aligned(a->grad_W_q) && state_aligned(a->grad_W_k) &&
            state_aligned(a->grad_w_b);
  if (a->L > 0)
    ok = ok && seq_aligned(a->x, es) && seq_aligned(a->grad_out, es) && seq_aligned(a->grad_x, es) &&
         seq_aligned(a->q, 4) && seq_aligned(a->k, 4) && seq_aligned(a->beta, 4) && seq_aligned(a->y_diff, 4) &&
         seq_aligned(a->q_diff, 4) && seq_aligned(a->k_diff, 4) && seq_aligned(a->beta_diff, 4);
  if (!ok) return SRWM_B200_ERR_ALIGN;
  unsigned ext_flags = 0;
  if (int rc = check_ext(x, /*forward=*/false, &ext_flags)) return rc;

  srwm::SrwmBwdParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L;
  p.flags = (a->flags & (SRWM_B200_FLAG_STATE_GRAD_IN | SRWM_B200_FLAG_RESTORE_STATE | SRWM_B200_FLAG_INPUT_SOFTMAX)) |
            ext_flags;
  if (ext_flags & srwm::F_BASE) {
    p.bWy = view(x->base_W_y); p.bWq = view(x->base_W_q); p.bWk = view(x->base_W_k); p.bwb = view(x->base_w_b);
  }
  p.x = view(a->x, es); p.gout = view(a->grad_out, es); p.gx = view(a->grad_x, es);
  p.q = view(a->q, 4); p.k = view(a->k, 4); p.beta = view(a->beta, 4);
  p.yd = view(a->y_diff, 4); p.qd = view(a->q_diff, 4); p.kd = view(a->k_diff, 4); p.bd = view(a->beta_diff, 4);
  p.Wy = view(a->W_y); p.Wq = view(a->W_q); p.Wk = view(a->W_k); p.wb = view(a->w_b);
  p.gWy = view(a->grad_W_y); p.gWq = view(a->grad_W_q); p.gWk = view(a->grad_W_k); p.gwb = view(a->grad_w_b);
  if (red) {
    if (!red->grad_base_W_y.data || !red->grad_base_W_q.data || !red->grad_base_W_k.data || !red->grad_base_w_b.data)
      return SRWM_B200_ERR_NULL;
    if (!state_aligned(red->grad_base_W_y) || !state_aligned(red->grad_base_W_q) ||
        !state_aligned(red->grad_base_W_k) || !state_aligned(red->grad_base_w_b))
      return SRWM_B200_ERR_ALIGN;
    p.flags |= srwm::F_REDUCE;
    p.red.oWy = view(red->grad_base_W_y); p.red.oWq = view(red->grad_base_W_q);
    p.red.oWk = view(red->grad_base_W_k); p.red.owb = view(red->grad_base_w_b);
    p.red.gs = reduce_group_size(a->N);
    p.red.ng = reduce_groups(a->N);
    p.red.accumulate = red->accumulate != 0;
    p.red.cnt = reinterpret_cast<unsigned*>(scratch);
    p.red.part = reinterpret_cast<float*>(reinterpret_cast<char*>(scratch) + reduce_counter_bytes(a->N, a->H));
    // the counters start at zero (the kernel leaves them at zero too; clearing them here keeps a call
    // independent of what an aborted earlier call may have left behind)
    const cudaError_t e = cudaMemsetAsync(scratch, 0, reduce_counter_bytes(a->N, a->H), (cudaStream_t)stream);
    if (e != cudaSuccess) {
      g_last_cuda_error = (int)e;
      return SRWM_B200_ERR_CUDA;
    }
  }
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_srwm_bwd_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_srwm_bwd_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}
}  // namespace

int srwm_b200_srwm_backward_detached(const srwm_b200_srwm_bwd_detached_args* a, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E)) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0) return 0;
  if (!a->base_W_y.data || !a->grad_W_y.data) return SRWM_B200_ERR_NULL;
  if (a->L > 0 && (!a->x.data || !a->k.data || !a->beta.data || !a->y_diff.data || !a->grad_out.data || !a->grad_x.data))
    return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = state_aligned(a->base_W_y) && state_aligned(a->grad_W_y) &&
            (a->shift_W_y.data == nullptr || state_aligned(a->shift_W_y));
  if (a->L > 0)
    ok = ok && seq_aligned(a->x, es) && seq_aligned(a->grad_out, es) && seq_aligned(a->grad_x, es) &&
         seq_aligned(a->k, 4) && seq_aligned(a->beta, 4) && seq_aligned(a->y_diff, 4);
  if (!ok) return SRWM_B200_ERR_ALIGN;

  srwm::SrwmBwdDetParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L;
  p.flags = (a->flags & SRWM_B200_FLAG_INPUT_SOFTMAX) | (a->shift_W_y.data ? srwm::F_SHIFT_IN : 0u) |
            (a->done ? srwm::F_DONE : 0u);
  p.x = view(a->x, es); p.gout = view(a->grad_out, es); p.gx = view(a->grad_x, es);
  p.k = view(a->k, 4); p.beta = view(a->beta, 4); p.yd = view(a->y_diff, 4);
  p.bWy = view(a->base_W_y); p.sWy = view(a->shift_W_y); p.gWy = view(a->grad_W_y);
  p.done = a->done; p.done_sn = a->done_stride_n; p.done_sl = a->done_stride_l;
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_srwm_bwd_det_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_srwm_bwd_det_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}

int srwm_b200_delta_forward(const srwm_b200_delta_fwd_args* a, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E) || a->M != a->E) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0 || a->L == 0) return 0;
  const bool save = !(a->flags & SRWM_B200_FLAG_NO_SAVE);
  if (!a->Q.data || !a->K.data || !a->V.data || !a->beta.data || !a->W.data || !a->out.data) return SRWM_B200_ERR_NULL;
  if (save && (!a->v_old.data || !a->v_insert.data)) return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = seq_aligned(a->Q, es) && seq_aligned(a->K, es) && seq_aligned(a->V, es) && seq_aligned(a->out, es) &&
            state_aligned(a->W) && ((uintptr_t)a->beta.data % es == 0);
  if (save) ok = ok && seq_aligned(a->v_old, 4) && seq_aligned(a->v_insert, 4);
  if (!ok) return SRWM_B200_ERR_ALIGN;

  srwm::DeltaFwdParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L; p.flags = a->flags & SRWM_B200_FLAG_NO_SAVE;
  p.Q = view(a->Q, es); p.K = view(a->K, es); p.V = view(a->V, es); p.beta = view(a->beta, es);
  p.out = view(a->out, es); p.v_old = view(a->v_old, 4); p.v_ins = view(a->v_insert, 4);
  p.W = view(a->W);
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_delta_fwd_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_delta_fwd_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}

int srwm_b200_delta_backward(const srwm_b200_delta_bwd_args* a, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E) || a->M != a->E) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0) return 0;
  if (!a->W.data) return SRWM_B200_ERR_NULL;
  if (a->L > 0 && (!a->Q.data || !a->K.data || !a->V.data || !a->beta.data || !a->v_old.data || !a->v_insert.data ||
                   !a->grad_out.data || !a->grad_Q.data || !a->grad_K.data || !a->grad_V.data || !a->grad_beta.data))
    return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = state_aligned(a->W) && (a->grad_W0.data == nullptr || state_aligned(a->grad_W0));
  if (a->L > 0)
    ok = ok && seq_aligned(a->Q, es) && seq_aligned(a->K, es) && seq_aligned(a->V, es) && seq_aligned(a->grad_out, es) &&
         seq_aligned(a->grad_Q, es) && seq_aligned(a->grad_K, es) && seq_aligned(a->grad_V, es) &&
         seq_aligned(a->v_old, 4) && seq_aligned(a->v_insert, 4) && ((uintptr_t)a->beta.data % es == 0) &&
         ((uintptr_t)a->grad_beta.data % es == 0);
  if (!ok) return SRWM_B200_ERR_ALIGN;

  srwm::DeltaBwdParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L; p.flags = 0;
  p.Q = view(a->Q, es); p.K = view(a->K, es); p.V = view(a->V, es); p.beta = view(a->beta, es);
  p.v_old = view(a->v_old, 4); p.v_ins = view(a->v_insert, 4); p.gout = view(a->grad_out, es);
  p.gQ = view(a->grad_Q, es); p.gK = view(a->grad_K, es); p.gV = view(a->grad_V, es); p.gbeta = view(a->grad_beta, es);
  p.W = view(a->W); p.gW0 = view(a->grad_W0);
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_delta_bwd_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_delta_bwd_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}

int srwm_b200_delta_packed_forward(const srwm_b200_delta_packed_fwd_args* a, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E)) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0 || a->L == 0) return 0;
  const bool save = !(a->flags & SRWM_B200_FLAG_NO_SAVE);
  if (!a->qkvb.data || !a->W.data || !a->out.data) return SRWM_B200_ERR_NULL;
  if (save && (!a->v_old.data || !a->v_insert.data)) return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = ((uintptr_t)a->qkvb.data % es == 0) && seq_aligned(a->out, es) && state_aligned(a->W);
  if (save) ok = ok && seq_aligned(a->v_old, 4) && seq_aligned(a->v_insert, 4);
  if (!ok) return SRWM_B200_ERR_ALIGN;

  srwm::DeltaFwdParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L;
  p.flags = (a->flags & SRWM_B200_FLAG_NO_SAVE) | srwm::F_PACKED |
            ((a->flags & SRWM_B200_FLAG_ZERO_INIT) ? srwm::F_ZERO_INIT : 0u);
  p.eps = a->norm_eps;
  p.Q = view(a->qkvb, es);
  p.out = view(a->out, es); p.v_old = view(a->v_old, 4); p.v_ins = view(a->v_insert, 4);
  p.W = view(a->W);
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_delta_fwd_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_delta_fwd_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}

int srwm_b200_delta_packed_backward(const srwm_b200_delta_packed_bwd_args* a, void* stream) {
  if (!a) return SRWM_B200_ERR_NULL;
  long long grid;
  if (int rc = check_dims(a->N, a->H, a->L, &grid)) return rc;
  if (!head_dim_ok(a->E)) return SRWM_B200_ERR_HEAD_DIM;
  if (a->io_dtype != SRWM_B200_F32 && a->io_dtype != SRWM_B200_BF16) return SRWM_B200_ERR_DTYPE;
  if (grid == 0) return 0;
  if (!a->W.data) return SRWM_B200_ERR_NULL;
  if (a->L > 0 && (!a->qkvb.data || !a->v_old.data || !a->v_insert.data || !a->grad_out.data || !a->grad_qkvb.data))
    return SRWM_B200_ERR_NULL;
  const int es = esize(a->io_dtype);
  bool ok = state_aligned(a->W) && (a->grad_W0.data == nullptr || state_aligned(a->grad_W0));
  if (a->L > 0)
    ok = ok && ((uintptr_t)a->qkvb.data % es == 0) && ((uintptr_t)a->grad_qkvb.data % es == 0) &&
         seq_aligned(a->grad_out, es) && seq_aligned(a->v_old, 4) && seq_aligned(a->v_insert, 4);
  if (!ok) return SRWM_B200_ERR_ALIGN;

  srwm::DeltaBwdParams p = {};
  p.dbg = debug_word();
  p.N = a->N; p.H = a->H; p.L = a->L;
  p.flags = srwm::F_PACKED;
  p.eps = a->norm_eps;
  p.Q = view(a->qkvb, es); p.gQ = view(a->grad_qkvb, es);
  p.v_old = view(a->v_old, 4); p.v_ins = view(a->v_insert, 4); p.gout = view(a->grad_out, es);
  p.W = view(a->W); p.gW0 = view(a->grad_W0);
  int ce = 0;
  const int rc = a->io_dtype == SRWM_B200_BF16
                     ? srwm::dispatch_delta_bwd_bf16(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0)
                     : srwm::dispatch_delta_bwd_f32(a->E, a->variant, p, (int)grid, (cudaStream_t)stream, nullptr, 0, &ce, 0);
  return finish(rc, ce);
}

#ifdef SRWM_DEBUG_CHECKS
namespace {
__global__ void debug_selftest_kernel(unsigned long long* dbg) {
  // a chunk that starts before the sequence: must be recorded and reported as bad, touching nothing
  (void)SRWM_BAD_ROWS(dbg, 255, -16, 16, 0, 16);
}
}  // namespace
#endif

int srwm_b200_debug_status(uint64_t* status) {
  if (!status) return SRWM_B200_ERR_NULL;
  *status = 0;
#ifdef SRWM_DEBUG_CHECKS
  unsigned long long w = 0ull, zero = 0ull;
  cudaError_t e = cudaMemcpyFromSymbol(&w, g_debug_status, sizeof(w));   // waits for the kernels in flight
  if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_debug_status, &zero, sizeof(zero));
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return SRWM_B200_ERR_CUDA;
  }
  *status = w;
  return 0;
#else
  return 1;
#endif
}

int srwm_b200_debug_selftest(void* stream) {
#ifdef SRWM_DEBUG_CHECKS
  unsigned long long* w = debug_word();
  if (!w) return SRWM_B200_ERR_CUDA;
  debug_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(w);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return SRWM_B200_ERR_CUDA;
  }
  return 0;
#else
  (void)stream;
  return 1;
#endif
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Batch reduction: dst[i] (+)= sum_n src[n*stride_n + i].  A block of 1024 threads covers 128
// outputs (32 lanes x float4) and splits the batch over its 32 warps (four independent loads
// in flight per thread); the 32 partial sums are combined through shared memory in a fixed
// order, so the result does not depend on timing.  Reads are 16-byte and coalesced.
// ---------------------------------------------------------------------------------------
namespace {
constexpr int RB_SLICES = 32;
__device__ __forceinline__ void add4(float4& a, const float4& v) { a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w; }

__global__ void __launch_bounds__(32 * RB_SLICES) reduce_batch_kernel(const float* __restrict__ src, long long stride_n,
                                                                      int N, long long count, float* __restrict__ dst,
                                                                      int accumulate) {
  __shared__ float4 part[RB_SLICES][32];
  const int lane = threadIdx.x % 32, slice = threadIdx.x / 32;
  const long long i = ((long long)blockIdx.x * 32 + lane) * 4;
  const bool full = i + 4 <= count;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (full) {
    const float* s0 = src + i;
    int n = slice;
    for (; n + 3 * RB_SLICES < N; n += 4 * RB_SLICES) {
      const float4 v0 = *reinterpret_cast<const float4*>(s0 + (long long)n * stride_n);
      const float4 v1 = *reinterpret_cast<const float4*>(s0 + (long long)(n + RB_SLICES) * stride_n);
      const float4 v2 = *reinterpret_cast<const float4*>(s0 + (long long)(n + 2 * RB_SLICES) * stride_n);
      const float4 v3 = *reinterpret_cast<const float4*>(s0 + (long long)(n + 3 * RB_SLICES) * stride_n);
      add4(acc, v0); add4(acc, v1); add4(acc, v2); add4(acc, v3);
    }
    for (; n < N; n += RB_SLICES) add4(acc, *reinterpret_cast<const float4*>(s0 + (long long)n * stride_n));
  }
  part[slice][lane] = acc;
  __syncthreads();
  if (slice != 0 || i >= count) return;
  if (full) {
    float4 t = accumulate ? *reinterpret_cast<const float4*>(dst + i) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int s8 = 0; s8 < RB_SLICES; ++s8) add4(t, part[s8][lane]);
    *reinterpret_cast<float4*>(dst + i) = t;
  } else {   // ragged end: fewer than four outputs left
    for (long long j = i; j < count; ++j) {
      float t = accumulate ? dst[j] : 0.f;
      for (int n = 0; n < N; ++n) t += src[(long long)n * stride_n + j];
      dst[j] = t;
    }
  }
}
}  // namespace

extern "C" int srwm_b200_reduce_batch(const float* src, int64_t stride_n, int32_t N, int64_t count, float* dst,
                                      int32_t accumulate, void* stream) {
  if (N < 0 || count < 0) return SRWM_B200_ERR_SHAPE;
  if (count == 0) return 0;
  if (!dst || (N > 0 && !src)) return SRWM_B200_ERR_NULL;
  if ((uintptr_t)src % 16 || (uintptr_t)dst % 16 || (stride_n * 4) % 16) return SRWM_B200_ERR_ALIGN;
  const long long blocks = (count + 127) / 128;
  if (blocks > 0x7fffffffLL) return SRWM_B200_ERR_SHAPE;
  reduce_batch_kernel<<<(unsigned)blocks, 32 * RB_SLICES, 0, (cudaStream_t)stream>>>(src, stride_n, N, count, dst, accumulate);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda_error = (int)e;
    return SRWM_B200_ERR_CUDA;
  }
  return 0;
}
