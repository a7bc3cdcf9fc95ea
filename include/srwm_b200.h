/*
 * srwm_b200.h -- C ABI of libsrwm_b200.so: the self-referential weight matrix (SRWM) and
 * delta-rule fast-weight recurrences as hand-written sm_100a kernels.
 *
 * The four compute entry points replace, one for one, the four pybind functions of the
 * reference's CUDA extensions (file:line cited at each declaration).  Everything is plain
 * C: device pointers, sizes, element strides, a CUDA stream handle passed as void*.
 * No buffer is owned by the library and no state is kept between calls (the calls are
 * re-entrant; concurrent calls from several host threads are fine as long as each uses
 * its own buffers).  Nothing is allocated on the device by these calls; the one call that
 * needs working memory beyond its inputs and outputs takes it from the caller.
 *
 * Conventions
 *   - Sequence tensors are 4-D views [N, H, L, X] (batch, head, time, feature) whose
 *     innermost dimension is contiguous; the other three strides are given in ELEMENTS.
 *     Each row (X elements) must start on a 16-byte boundary: base pointer and
 *     stride*sizeof(element) are multiples of 16.  (A misaligned view returns
 *     SRWM_B200_ERR_ALIGN; the Python layer then makes one contiguous copy.)
 *   - State tensors are [N, H, E, X] fp32 with a dense inner [E][X] block; strides over
 *     N and H in elements.  "matvec" is row-vector times matrix: out[m] = sum_e v[e]*W[e][m].
 *   - io_dtype selects the element type of the streamed activations (x / out / q,k,v,beta
 *     of the delta rule / their gradients).  State, saved activations and state gradients
 *     are always fp32.
 *   - Return value: 0 on success, a negative SRWM_B200_ERR_* otherwise.  Arguments are
 *     validated before any CUDA call, so invalid calls are rejected on machines without
 *     a GPU as well.  N*H*L == 0 is a successful no-op.
 *   - Supported head dimensions: E in {8, 16, 32, 64} (delta rule: M == E).
 *   - Device: the kernels are launched on the calling thread's CURRENT CUDA device, which must be
 *     the device that owns every pointer of the call and the stream (call cudaSetDevice first;
 *     the Python layer does).  The library never changes the current device.
 */
#ifndef SRWM_B200_H_
#define SRWM_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SRWM_B200_ABI_VERSION 2

/* io_dtype */
#define SRWM_B200_F32  0
#define SRWM_B200_BF16 1

/* error codes */
#define SRWM_B200_OK              0
#define SRWM_B200_ERR_NULL       -1  /* a required pointer is NULL                       */
#define SRWM_B200_ERR_SHAPE      -2  /* negative size, or N*H exceeds the grid limit      */
#define SRWM_B200_ERR_HEAD_DIM   -3  /* E (or M != E) not supported                       */
#define SRWM_B200_ERR_DTYPE      -4  /* io_dtype unknown                                  */
#define SRWM_B200_ERR_ALIGN      -5  /* a row does not start on a 16-byte boundary        */
#define SRWM_B200_ERR_VARIANT    -6  /* tuning variant id not compiled in                 */
#define SRWM_B200_ERR_CUDA       -7  /* CUDA runtime error; see srwm_b200_last_cuda_error */
#define SRWM_B200_ERR_TOO_LARGE  -8  /* size beyond a fixed capacity / scratch too small     */
#define SRWM_B200_ERR_UNSUPPORTED -9 /* combination of arguments the entry point cannot serve
                                        (e.g. `done` given to the reverse-time layer backward) */

/* flags */
#define SRWM_B200_FLAG_NO_SAVE        1u /* forward: do not write the saved-for-backward
                                            tensors (inference; their pointers may be NULL) */
#define SRWM_B200_FLAG_STATE_GRAD_IN  2u /* SRWM backward: grad_W_* hold dL/dW_L on entry and
                                            are accumulated through time (stateful variant);
                                            without it they are treated as zero on entry     */
#define SRWM_B200_FLAG_RESTORE_STATE  4u /* SRWM backward: also write the rebuilt initial
                                            state W_0 back into W_* (the reference leaves W_L) */
#define SRWM_B200_FLAG_INPUT_SOFTMAX  8u /* SRWM forward/backward: x holds RAW activations and the
                                            kernels apply softmax over the head dimension (the
                                            callers' F.softmax, supervised_learning/layer.py:162-163,
                                            reinforcement_learning/torchbeast/layer.py:383);
                                            grad_x is then the gradient of the raw values      */

typedef struct srwm_b200_seq {      /* [N,H,L,X] view, innermost contiguous */
  void*   data;
  int64_t stride_n, stride_h, stride_l;   /* elements */
} srwm_b200_seq;

typedef struct srwm_b200_state {    /* [N,H,E,X] fp32, inner [E][X] dense */
  float*  data;
  int64_t stride_n, stride_h;             /* elements */
} srwm_b200_state;

/* ------------------------------------------------------------------------------------
 * SRWM forward.  Replaces
 *   void self_ref_forward(x, W_y, W_q, W_k, w_b, q, k, beta, y_diff, q_diff, k_diff,
 *                         beta_diff, output)
 *   supervised_learning/self_ref_v0/self_ref_v0.cu:436-530 (kernel :24-432), bound at
 *   :1344-1349; identical copy in reinforcement_learning/torchbeast/self_ref_v0/.
 * Per step t:  [y,q~,k~,b~] = x_t.W ; q=softmax(q~), k=softmax(k~), beta=sigmoid(b~);
 *   d_Z = (q-k).W_Z ; W_Z += k^T (beta_Z d_Z)   for Z in {y,q,k,b}; out_t = y (pre-update).
 * The final state is written back IN PLACE into W_y, W_q, W_k, w_b (callers rely on it).
 * Outputs are plain stores: no zero-filling by the caller is needed.
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_srwm_fwd_args {
  int32_t N, H, L, E;
  int32_t io_dtype;
  uint32_t flags;
  int32_t variant;                  /* 0 = the library chooses the kernel configuration (by head size and by
                                       how N*H sequences fill the GPU); ids >= 1 name one compiled
                                       configuration and are always honoured (srwm_b200_num_variants) */
  int32_t reserved;
  srwm_b200_seq   x;                /* in  [N,H,L,E] io_dtype */
  srwm_b200_state W_y, W_q, W_k;    /* in/out [N,H,E,E] */
  srwm_b200_state w_b;              /* in/out [N,H,E,4] */
  srwm_b200_seq   out;              /* out [N,H,L,E] io_dtype */
  srwm_b200_seq   q, k;             /* saved [N,H,L,E] fp32 (softmax outputs) */
  srwm_b200_seq   beta;             /* saved [N,H,L,4] fp32 (post-sigmoid) */
  srwm_b200_seq   y_diff, q_diff, k_diff;  /* saved [N,H,L,E] fp32: (q-k).W_Z */
  srwm_b200_seq   beta_diff;        /* saved [N,H,L,4] fp32 */
} srwm_b200_srwm_fwd_args;

int srwm_b200_srwm_forward(const srwm_b200_srwm_fwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * SRWM backward.  Replaces
 *   void self_ref_backward(x, q, k, beta, y_diff, q_diff, k_diff, beta_diff, grad_out,
 *                          Wy, Wq, Wk, wb, grad_x, grad_Wy, grad_Wq, grad_Wk, grad_wb)
 *   supervised_learning/self_ref_v0/self_ref_v0.cu:1238-1341 (kernel :534-1234), bound at
 *   :1350-1355.
 * Reverse-time pass that rebuilds W_{t-1} from W_t by undoing the rank-1 update; W_* must
 * hold the FINAL state left by the forward.  grad_W_* receive dL/dW_0 (plain stores).
 * Unlike the reference the whole sequence is one launch, so L is not limited by a
 * shared-memory time chunk.
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_srwm_bwd_args {
  int32_t N, H, L, E;
  int32_t io_dtype;
  uint32_t flags;
  int32_t variant;
  int32_t reserved;
  srwm_b200_seq   x;                /* in  [N,H,L,E] io_dtype */
  srwm_b200_seq   q, k;             /* in  saved fp32 */
  srwm_b200_seq   beta;             /* in  saved fp32 [N,H,L,4] */
  srwm_b200_seq   y_diff, q_diff, k_diff;
  srwm_b200_seq   beta_diff;
  srwm_b200_seq   grad_out;         /* in  [N,H,L,E] io_dtype */
  srwm_b200_state W_y, W_q, W_k, w_b;             /* in (W_L); out W_0 with RESTORE_STATE */
  srwm_b200_seq   grad_x;           /* out [N,H,L,E] io_dtype */
  srwm_b200_state grad_W_y, grad_W_q, grad_W_k, grad_w_b;   /* (in)/out fp32 */
} srwm_b200_srwm_bwd_args;

int srwm_b200_srwm_backward(const srwm_b200_srwm_bwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * Layer-level SRWM calls: what the callers do around the kernel, taken into it.  No
 * reference function corresponds one to one; each piece cites the caller code it absorbs.
 *
 * With an extension block whose base_* are set, the state is  W = base + shift:
 *   - base_*   the un-repeated slow weights [1,H,E,.] (stride_n = 0) -- the callers'
 *              `self.W_y.repeat(bsz,1,1,1)` (supervised_learning/layer.py:169-177,
 *              reinforcement_learning/torchbeast/layer.py:392-395) is never materialised;
 *   - shift_*  optional initial shift [N,H,E,.] (the carried `state`; NULL data = zero);
 *   - forward: W_y, W_q, W_k, w_b of the main block are OUTPUTS only and receive the final
 *              shift  W_L - base  (the callers' subtraction, layer.py:200-204 / :412-415);
 *   - backward: W_* hold that final shift on entry (W_L = base + W_*); with RESTORE_STATE they
 *              receive W_0 - base.  grad_W_* are dL/dW_0 per sample, as in the plain call:
 *              dL/dshift = grad_W_*, dL/dbase = their sum over the batch
 *              (srwm_b200_reduce_batch) minus the sum of the incoming dL/dshift_out;
 *   - done     optional bytes [N,L] (forward): done[n,t] != 0 sets the shift of sample n to
 *              zero before step t -- the per-step `nd * state` of the learner's unroll
 *              (reinforcement_learning/torchbeast_procgen/model.py:1180-1194), which lets T
 *              one-step calls become one call of length T.  The reverse-time backward cannot
 *              cross such a reset (the pre-reset state is gone): srwm_b200_srwm_layer_backward
 *              returns SRWM_B200_ERR_UNSUPPORTED when `done` is set; use the detached backward.
 * With L == 0 the forward is a no-op that leaves W_* untouched (the caller carries the shift
 * through: shift_in, or zero).
 * ext == NULL (or all base_* NULL) makes these identical to the plain calls above.
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_srwm_ext {
  srwm_b200_state base_W_y, base_W_q, base_W_k;    /* [1 or N, H, E, E] */
  srwm_b200_state base_w_b;                        /* [1 or N, H, E, 4] */
  srwm_b200_state shift_W_y, shift_W_q, shift_W_k, shift_w_b;   /* optional, forward only */
  const uint8_t*  done;                            /* optional, forward only */
  int64_t done_stride_n, done_stride_l;            /* bytes */
} srwm_b200_srwm_ext;

int srwm_b200_srwm_layer_forward(const srwm_b200_srwm_fwd_args* args, const srwm_b200_srwm_ext* ext,
                                 void* cuda_stream);
int srwm_b200_srwm_layer_backward(const srwm_b200_srwm_bwd_args* args, const srwm_b200_srwm_ext* ext,
                                  void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * Layer-level SRWM backward with the batch reduction fused into it.  The gradient of the
 * un-repeated slow weights is the sum over the batch of the per-sample dL/dW_0 -- the backward of
 * the callers' `W.repeat(bsz, 1, 1, 1)` (supervised_learning/layer.py:174-177, no reference
 * function corresponds one to one).  grad_W_* of the main block still receive the per-sample
 * gradients (dL/dshift); in addition grad_base_* receive their batch sums, formed inside the
 * backward kernel: the CTAs of one head are grouped by consecutive samples, the CTA of a group
 * that finishes last adds the group's gradients in sample order, the group of a head that
 * finishes last adds the group sums in group order (atomic counters tell which; no CTA waits for
 * another).  Every addition has a fixed order: the result is deterministic.
 * `scratch` is device memory of srwm_b200_srwm_reduce_scratch_bytes(N, H, E) bytes, 256-byte
 * aligned, used only during the call (calls that overlap on the GPU need separate scratch).
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_srwm_reduce {
  srwm_b200_state grad_base_W_y, grad_base_W_q, grad_base_W_k;   /* out [1,H,E,E] fp32 (stride_n unused) */
  srwm_b200_state grad_base_w_b;                                 /* out [1,H,E,4] */
  int32_t accumulate;               /* != 0: add to what grad_base_* hold instead of overwriting */
  int32_t reserved;
  void*   scratch;
  int64_t scratch_bytes;
} srwm_b200_srwm_reduce;

size_t srwm_b200_srwm_reduce_scratch_bytes(int32_t N, int32_t H, int32_t E);   /* 0 for invalid sizes */
int srwm_b200_srwm_layer_backward_reduced(const srwm_b200_srwm_bwd_args* args, const srwm_b200_srwm_ext* ext,
                                          const srwm_b200_srwm_reduce* red, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * srwm_b200_srwm_layer_backward_reduced for hosts that cannot allocate device memory.
 * (No counterpart in the reference: its extensions take every buffer from PyTorch.)
 *
 * Who this is for: a host that was handed its buffers and has no allocator of its own to ask for
 * a scratch block -- a C plug-in inside a process whose device memory belongs entirely to another
 * runtime's pool, or a fixed-budget deployment that sizes all device memory at start-up -- and a
 * latency-critical loop such as the agents' inference thread running beside the learner on one
 * GPU, where a cudaMalloc in the call path would stall the other thread's work because it
 * synchronises the device.
 *
 * Same arguments, same kernel and same results as the call above; `scratch` and `scratch_bytes`
 * of the reduce block are ignored.  The working memory is a fixed array inside the library image
 * of SRWM_B200_STATIC_SCRATCH_BYTES bytes (each GPU that loads the library holds it until the
 * process exits).  The call makes no cudaMalloc / cudaFree and calls no allocating routine.
 *   - Limit: srwm_b200_srwm_reduce_scratch_bytes(N, H, E) must not exceed the array; otherwise
 *     SRWM_B200_ERR_TOO_LARGE is returned and nothing runs.  Any N <= 64 fits (counters only);
 *     beyond that the need is about H * ceil(N/32) * (3E*E + 4E) * 4 bytes, e.g. N=128, H=16
 *     fits for every supported E, N=1024, H=16, E=64 does not.
 *   - First call on a device: it looks up the array's device address (cudaGetSymbolAddress, with
 *     that device current) and keeps it.  Make that first call outside any stream capture.
 *   - All calls share the one array per device and it keeps what the last call left in it (the
 *     call clears the part that has to start at zero).  Calls that overlap on the GPU -- two
 *     streams, or two host threads without ordering between their streams -- race on it and give
 *     wrong sums; order them, or use the caller-scratch variant for one of them.
 * ---------------------------------------------------------------------------------- */
#define SRWM_B200_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int srwm_b200_srwm_layer_backward_reduced_static(const srwm_b200_srwm_bwd_args* args,
                                                 const srwm_b200_srwm_ext* ext,
                                                 const srwm_b200_srwm_reduce* red, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * SRWM backward with the state DETACHED at every step: the gradient the reference's
 * reinforcement-learning learner computes, which calls the layer one step at a time and
 * detaches the state it carries (reinforcement_learning/torchbeast/layer.py:412-421 under
 * torchbeast_procgen/model.py:1180-1197).  Only out_t = x_t.W_y(t-1) carries gradient:
 *   grad_x_t = W_y(t-1) grad_out_t  (through the input softmax with INPUT_SOFTMAX),
 *   grad_W_y = sum_t x_t^T grad_out_t  per sample;   W_q, W_k, w_b receive none.
 * W_y(t-1) is replayed forward in time from base_W_y (+ shift_W_y) with the saved k, beta,
 * y_diff of the forward, returning to base where done is set.
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_srwm_bwd_detached_args {
  int32_t N, H, L, E;
  int32_t io_dtype;
  uint32_t flags;                   /* INPUT_SOFTMAX */
  int32_t variant;
  int32_t reserved;
  srwm_b200_seq   x;                /* in  [N,H,L,E] io_dtype */
  srwm_b200_seq   k;                /* in  saved fp32 */
  srwm_b200_seq   beta;             /* in  saved fp32 [N,H,L,4] */
  srwm_b200_seq   y_diff;           /* in  saved fp32 */
  srwm_b200_seq   grad_out;         /* in  [N,H,L,E] io_dtype */
  srwm_b200_state base_W_y;         /* in  W_y before the first step, or the slow weights */
  srwm_b200_state shift_W_y;        /* in  optional initial shift (NULL data = none) */
  const uint8_t*  done;             /* in  optional [N,L] */
  int64_t done_stride_n, done_stride_l;
  srwm_b200_seq   grad_x;           /* out [N,H,L,E] io_dtype */
  srwm_b200_state grad_W_y;         /* out [N,H,E,E] fp32 */
} srwm_b200_srwm_bwd_detached_args;

int srwm_b200_srwm_backward_detached(const srwm_b200_srwm_bwd_detached_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * Delta-rule forward.  Replaces
 *   void fast_weight_forward(Q, K, V, beta, v_old, v_insert, kv, out)
 *   supervised_learning/fast_weight/fast_weight_cuda.cu:182-240 (kernel :17-178), bound at
 *   :667-672; identical copy in reinforcement_learning/torchbeast/fast_weight/.
 * Per step:  v_old = k.W ; ins = beta (v - v_old) ; W += k^T ins ; out = q.W (post-update).
 * Q and K are used as given (already normalised by the caller), beta is post-sigmoid.
 * The final W is written back in place.
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_delta_fwd_args {
  int32_t N, H, L, E, M;
  int32_t io_dtype;
  uint32_t flags;
  int32_t variant;
  srwm_b200_seq   Q, K;             /* in [N,H,L,E] io_dtype */
  srwm_b200_seq   V;                /* in [N,H,L,M] io_dtype */
  srwm_b200_seq   beta;             /* in [N,H,L,1] io_dtype (any stride; no alignment rule) */
  srwm_b200_state W;                /* in/out [N,H,E,M] */
  srwm_b200_seq   out;              /* out [N,H,L,M] io_dtype */
  srwm_b200_seq   v_old, v_insert;  /* saved [N,H,L,M] fp32 */
} srwm_b200_delta_fwd_args;

int srwm_b200_delta_forward(const srwm_b200_delta_fwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * Delta-rule backward.  Replaces
 *   void fast_weight_backward(Q, K, V, beta, v_old, v_insert, grad_out, fw_mem,
 *                             grad_q, grad_k, grad_v, grad_betas)
 *   supervised_learning/fast_weight/fast_weight_cuda.cu:564-664 (kernels :244-393 and
 *   :397-560), bound at :673-678.
 * One reverse-time pass (the reference uses two and a [N,H,L,M] temporary).  W holds W_L
 * on entry and the rebuilt W_0 on exit, as in the reference (:391).  grad_W0 is optional
 * (NULL data = not wanted; the reference's autograd function returns None for it).
 * ---------------------------------------------------------------------------------- */
typedef struct srwm_b200_delta_bwd_args {
  int32_t N, H, L, E, M;
  int32_t io_dtype;
  uint32_t flags;
  int32_t variant;
  srwm_b200_seq   Q, K, V, beta;    /* in, io_dtype */
  srwm_b200_seq   v_old, v_insert;  /* in, saved fp32 */
  srwm_b200_seq   grad_out;         /* in [N,H,L,M] io_dtype */
  srwm_b200_state W;                /* in W_L / out W_0 */
  srwm_b200_seq   grad_Q, grad_K;   /* out [N,H,L,E] io_dtype */
  srwm_b200_seq   grad_V;           /* out [N,H,L,M] io_dtype */
  srwm_b200_seq   grad_beta;        /* out [N,H,L,1] io_dtype (any stride) */
  srwm_b200_state grad_W0;          /* optional out [N,H,E,M] fp32 */
} srwm_b200_delta_bwd_args;

int srwm_b200_delta_backward(const srwm_b200_delta_bwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * Layer-level delta-rule calls: the kernels read the RAW rows the layers' slow net produces,
 *   qkvb[n,h,t,:] = [ q (E) | k (E) | v (E) | b (1) ]
 * (supervised_learning/layer.py:74-77, reinforcement_learning/torchbeast/layer.py:144-147:
 * `qkvb.view(slen, bsz, num_head, 3*dim_head+1)` split four ways) and do the layers'
 * preparation themselves:
 *   q = a(q) / (sum a(q) + norm_eps), k likewise, a(x) = elu(x) + 1;  beta = sigmoid(b)
 * (layer.py:79,86-90: norm_eps = 0;  torchbeast/layer.py:30-33,156-157: norm_eps = 1e-5).
 * The backward returns the gradient of the raw rows in the same packed layout.  No reference
 * function corresponds one to one.  Packed rows need only ELEMENT alignment (any strides);
 * they are staged as the 16-byte blocks that cover them, so the buffers they live in must be
 * allocated with 16-byte granularity (every cudaMalloc-family allocation is).
 * ZERO_INIT (forward): W_0 = 0 and W is not read -- the layers' `torch.zeros` fast weights
 * (layer.py:92-94) need not be filled; W still receives W_L for the backward.
 * ---------------------------------------------------------------------------------- */
#define SRWM_B200_FLAG_ZERO_INIT 16u

typedef struct srwm_b200_delta_packed_fwd_args {
  int32_t N, H, L, E;
  int32_t io_dtype;
  uint32_t flags;                   /* NO_SAVE, ZERO_INIT */
  int32_t variant;
  float   norm_eps;
  srwm_b200_seq   qkvb;             /* in  [N,H,L,3E+1] io_dtype, element-aligned rows */
  srwm_b200_state W;                /* in/out [N,H,E,E] */
  srwm_b200_seq   out;              /* out [N,H,L,E] io_dtype */
  srwm_b200_seq   v_old, v_insert;  /* saved [N,H,L,E] fp32 */
} srwm_b200_delta_packed_fwd_args;

int srwm_b200_delta_packed_forward(const srwm_b200_delta_packed_fwd_args* args, void* cuda_stream);

typedef struct srwm_b200_delta_packed_bwd_args {
  int32_t N, H, L, E;
  int32_t io_dtype;
  uint32_t flags;
  int32_t variant;
  float   norm_eps;
  srwm_b200_seq   qkvb;             /* in  raw rows, as given to the forward */
  srwm_b200_seq   v_old, v_insert;  /* in  saved fp32 */
  srwm_b200_seq   grad_out;         /* in  [N,H,L,E] io_dtype */
  srwm_b200_state W;                /* in W_L / out W_0 */
  srwm_b200_seq   grad_qkvb;        /* out [N,H,L,3E+1] io_dtype, element-aligned rows */
  srwm_b200_state grad_W0;          /* optional out [N,H,E,E] fp32 */
} srwm_b200_delta_packed_bwd_args;

int srwm_b200_delta_packed_backward(const srwm_b200_delta_packed_bwd_args* args, void* cuda_stream);

/* ------------------------------------------------------------------------------------
 * Batch reduction of per-sample state gradients into the slow-weight gradient:
 *   dst[i] (+)= sum_n src[n*stride_n + i],  i < count   (fp32, deterministic order).
 * This is the backward of the callers' `W.repeat(bsz, 1, 1, 1)`
 * (supervised_learning/layer.py:174-177); dst may point into a flat all-reduce bucket.
 * accumulate != 0 adds to dst instead of overwriting it.
 * ---------------------------------------------------------------------------------- */
int srwm_b200_reduce_batch(const float* src, int64_t stride_n, int32_t N, int64_t count,
                           float* dst, int32_t accumulate, void* cuda_stream);

/* ---- queries (no CUDA call is made by these) ---- */
int         srwm_b200_abi_version(void);
int         srwm_b200_head_dim_supported(int32_t E);           /* 1 / 0 */
int         srwm_b200_num_variants(int32_t op, int32_t E);     /* valid variant values are 0 .. this-1.
                                                                  op: 0 srwm_fwd 1 srwm_bwd
                                                                  2 delta_fwd 3 delta_bwd
                                                                  4 srwm_bwd_detached */
const char* srwm_b200_strerror(int code);
int         srwm_b200_last_cuda_error(void);   /* cudaError_t of the last failed call of the
                                                  calling thread, 0 if none */
/* Describes the kernel configuration a call would use (threads per sequence, rows per
 * thread, time-chunk length, dynamic shared memory bytes): writes "P R T smem" into out.
 * With variant 0 this is the configuration of a grid that fills the GPU. */
int         srwm_b200_describe(int32_t op, int32_t E, int32_t io_dtype, int32_t variant,
                               int32_t out[4]);
/* The same for a given number of sequences (grid = N*H) on a GPU with num_sms multiprocessors
 * (<= 0: 148): writes "P R T smem id" into out, id being the configuration that variant 0 resolves
 * to.  (A delta-rule backward call whose last wave would be partial runs its whole waves on one
 * configuration and the remainder on another; the one of the whole waves is reported.) */
int         srwm_b200_describe_for_grid(int32_t op, int32_t E, int32_t io_dtype, int32_t variant,
                                        int64_t grid, int32_t num_sms, int32_t out[5]);

/* ---- debug build (csrc/build.py --debug -> libsrwm_b200_debug.so; no reference counterpart) ----
 * In the debug build every chunk of rows a kernel stages or writes is checked against the sequence
 * length before an address is formed; the first violation is recorded in a per-device status word and
 * the access is skipped (nothing traps, the context stays usable).
 * srwm_b200_debug_status: waits for the device, returns the word through *status and clears it.
 *   0 = no violation; otherwise bit 63 | site id (8 bits) << 48 | CTA index (24) << 24 | first row (24).
 *   Return value 0 in the debug build, 1 ("checks not compiled in", *status = 0) in the ordinary one.
 * srwm_b200_debug_selftest: launches a one-warp kernel that runs the check on a chunk starting before
 *   the sequence (site id 255) without touching memory, so that the reporting path can be tested. */
int         srwm_b200_debug_status(uint64_t* status);
int         srwm_b200_debug_selftest(void* cuda_stream);

#ifdef __cplusplus
}
#endif
#endif  /* SRWM_B200_H_ */
