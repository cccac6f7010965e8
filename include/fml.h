/*
 * fml.h -- C ABI of libflutter_ml_b200.so, the B200 (sm_100a) compute backend
 * for the flutter_ml autograd framework.
 *
 * The library replaces the reference's native stub (cuda_lib/kernel.cu, bound
 * from Dart by lib/cuda/cudacaller.dart:6-19).  The two legacy symbols keep
 * their signatures; everything else is a handle-based surface the Dart tape
 * (lib/autogradEngine/tensor.dart) calls once per op instead of running the
 * scalar loops itself.
 *
 * Conventions
 *   - All matrices are row-major float32 in device memory; `ld*` are row
 *     strides in elements.  Device pointers are plain `float*` obtained from
 *     fml_alloc (or any other CUDA allocation on the same device).
 *   - Every function returns 0 on success or a negative fml_status;
 *     fml_last_error() gives the message.  Nothing throws, aborts or traps.
 *   - Calls are asynchronous on the context's stream; fml_download_* and
 *     fml_sync wait.  A context is driven by one host thread at a time; one thread may drive
 *     several contexts, on the same or on different GPUs (every entry point makes its
 *     context's device current first).
 *   - There is no CPU fallback: without a CUDA device fml_init fails.
 */
#ifndef FML_H_
#define FML_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct fml_ctx fml_ctx;

typedef enum {
  FML_OK = 0,
  FML_ERR_INVALID = -1,   /* bad argument / shape / alignment                */
  FML_ERR_CUDA = -2,      /* a CUDA runtime or driver call failed            */
  FML_ERR_NO_DEVICE = -3, /* no usable CUDA device                           */
  FML_ERR_TIMEOUT = -4,   /* a bounded device-side wait expired              */
  FML_ERR_NCCL = -5,      /* NCCL missing or a collective failed             */
  FML_ERR_OOM = -6        /* allocation failed or a size limit was exceeded  */
} fml_status;

/* Product precision of the dense contractions. */
typedef enum {
  FML_PREC_TF32 = 0,   /* tcgen05 kind::tf32, fp32 accumulate (rel. error ~5e-4) */
  FML_PREC_3XTF32 = 1, /* hi/lo split, three tf32 products (rel. error ~1e-6)     */
  FML_PREC_FP32 = 2    /* CUDA-core fp32 FMA path (small or unaligned shapes)     */
} fml_precision;

/* Epilogue activation, applied to alpha*A.B + bias.  Mirrors the reference's
 * reluMatrix / sigmoidMatrix / tanhMatrix (lib/autogradEngine/tensor.dart:1013,
 * 1123, 1178); GELU (exact, erf form) is an extension. */
typedef enum { FML_ACT_NONE = 0, FML_ACT_RELU = 1, FML_ACT_SIGMOID = 2, FML_ACT_TANH = 3, FML_ACT_GELU = 4 } fml_act;

typedef struct {
  int32_t device;           /* CUDA ordinal                                          */
  int32_t precision;        /* fml_precision used when a call passes -1              */
  int64_t workspace_bytes;  /* scratch arena for 3xTF32 splits etc.; 0 = grow on use */
} fml_config;

/* ---- lifetime, errors, device query ------------------------------------- */
int32_t fml_init(const fml_config* cfg, fml_ctx** out);
int32_t fml_shutdown(fml_ctx* ctx);
/* ctx may be NULL: returns the last error of a call that had no context. */
const char* fml_last_error(fml_ctx* ctx);
/* Replaces cuda_lib/device_query.cu:5-26. */
int32_t fml_device_count(int32_t* count);
int32_t fml_device_name(int32_t device, char* buf, int32_t buf_len);
int32_t fml_sm_count(fml_ctx* ctx, int32_t* count);
/* The persistent tensor-core products launched after this call occupy at most (SM count - sms) SMs.  A gradient
 * exchange that runs on a side stream beside them needs SMs of its own: a persistent kernel that fills the machine
 * (one CTA per SM, all of its shared memory) would otherwise hold the collective back until it retires, and nothing
 * would overlap.  Set it before the products that run under an exchange and back to 0 afterwards. */
int32_t fml_set_sm_reserve(fml_ctx* ctx, int32_t sms);
/* Use an existing cudaStream_t (as void*) instead of the context's own. */
int32_t fml_set_stream(fml_ctx* ctx, void* cuda_stream);
int32_t fml_sync(fml_ctx* ctx);
/* What kernels could not do, read back once (reading synchronises, then clears):
 *   - a bounded device-side wait that expired instead of hanging: returns FML_ERR_TIMEOUT, *code = the role that gave up;
 *   - a token id or class label outside its range (201 embedding forward, 202 embedding backward, 203 cross-entropy
 *     label): returns FML_ERR_INVALID, *code = which.  The kernel skipped the access, so memory is intact.
 * 0 / FML_OK means neither happened. */
int32_t fml_device_status(fml_ctx* ctx, int32_t* code);
/* Failure-path self test: one CTA waits (with the bounded wait all pipeline roles use) on a barrier that nothing
 * signals; after limit_us microseconds it records code 99 and returns.  fml_device_status then reports
 * FML_ERR_TIMEOUT once and the context stays usable.  Nothing faults, traps or hangs. */
int32_t fml_selftest_wait_timeout(fml_ctx* ctx, int32_t limit_us);
/* Host-only self test (no device needed) of the bookkeeping behind one-time kernel set-up: function attributes such
 * as the shared-memory opt-in belong to one device, so the library keeps one "done" flag per (call site, device).
 * Each call passes through such a guard around a counter for `device` and returns the counter in *runs: it must read
 * 1 however often the same ordinal is passed, and every new ordinal (0..63) must run the body once more.  Ordinals
 * outside that range have no slot and run the body every time. */
int32_t fml_selftest_per_device_once(int32_t device, int32_t* runs);

/* ---- memory ---------------------------------------------------------------
 * Dart lists are float64 (lib/cuda/cudacaller.dart:38-43 narrows element by
 * element); the f64 variants convert once, in C. */
int32_t fml_alloc(fml_ctx* ctx, int64_t n_floats, float** out);
/* Free and total bytes of the context's device (cudaMemGetInfo) and the current size of the context's scratch
 * arena; any pointer may be NULL.  A caller can hold the figures from before and after a call against each other
 * to see whether the call took device memory. */
int32_t fml_mem_info(fml_ctx* ctx, int64_t* free_bytes, int64_t* total_bytes, int64_t* arena_bytes);
int32_t fml_free(fml_ctx* ctx, float* p);
int32_t fml_zero(fml_ctx* ctx, float* p, int64_t n_floats);
int32_t fml_fill(fml_ctx* ctx, float* p, int64_t n_floats, float value);
int32_t fml_upload_f32(fml_ctx* ctx, float* dst, const float* host, int64_t n);
int32_t fml_upload_f64(fml_ctx* ctx, float* dst, const double* host, int64_t n);
int32_t fml_upload_i32(fml_ctx* ctx, int32_t* dst, const int32_t* host, int64_t n);
int32_t fml_download_f32(fml_ctx* ctx, float* host, const float* src, int64_t n);
int32_t fml_download_f64(fml_ctx* ctx, double* host, const float* src, int64_t n);
int32_t fml_copy(fml_ctx* ctx, float* dst, const float* src, int64_t n);

/* Page-locked host memory for staging (the reference stages through pageable
 * calloc buffers, lib/cuda/cudacaller.dart:32-34). */
int32_t fml_host_alloc(fml_ctx* ctx, int64_t bytes, void** out);
int32_t fml_host_free(fml_ctx* ctx, void* p);
/* Gather `rows` rows of `row_elems` elements from a host array into a staging buffer (normally page-locked, from
 * fml_host_alloc) on several host threads, narrowing on the way: src_kind 0 float32, 1 float64 (Dart's doubles,
 * lib/cuda/cudacaller.dart:38-43 narrows them one element at a time on one thread) -> float32; 2 int32, 3 int64 ->
 * int32.  Row r comes from source row index[r], or first_row + r when index is NULL.  threads <= 0 picks a count from
 * the size (at least 1 MiB per thread, at most 16).  Synchronous: dst is complete on return. */
int32_t fml_stage_rows(fml_ctx* ctx, void* dst, const void* src, int32_t src_kind, int64_t row_elems,
                       const int64_t* index, int64_t first_row, int64_t rows, int32_t threads);
/* The same gather on background threads only: returns at once, so the caller can go on enqueueing the current
 * step's kernels while the next batch is staged.  dst, src and index must stay valid, and dst unread, until
 * fml_stage_wait has returned; several background gathers may be outstanding, fml_stage_wait joins them all. */
int32_t fml_stage_rows_async(fml_ctx* ctx, void* dst, const void* src, int32_t src_kind, int64_t row_elems,
                             const int64_t* index, int64_t first_row, int64_t rows, int32_t threads);
int32_t fml_stage_wait(fml_ctx* ctx);

/* Copy lanes: four extra streams (lanes 0..3) for host<->device copies and gradient exchanges that overlap the kernels
 * on the context's stream (the reference copies synchronously before and after every product,
 * cuda_lib/kernel.cu:23-24,44).  Ordering between the main stream (lane -1) and the lanes is
 * expressed with the numbered events of the pool below: record on one, wait on another. */
int32_t fml_lane_h2d(fml_ctx* ctx, int32_t lane, float* dst, const float* host, int64_t n);
int32_t fml_lane_d2h(fml_ctx* ctx, int32_t lane, float* host, const float* src, int64_t n);
int32_t fml_lane_sync(fml_ctx* ctx, int32_t lane);
int32_t fml_event_record_on(fml_ctx* ctx, int32_t slot, int32_t lane);
int32_t fml_wait_event(fml_ctx* ctx, int32_t lane, int32_t slot);
/* The HOST waits until the event last recorded in `slot` has happened (e.g. before it rewrites a staging buffer
 * that a copy on a lane was reading), without draining anything enqueued after it. */
int32_t fml_event_sync(fml_ctx* ctx, int32_t slot);

/* ---- CUDA graphs --------------------------------------------------------------
 * Launch-bound sequences (the 64-row MLP step of lib/nets/snet.dart:74-85 is ~15 small kernels) can be
 * recorded once and replayed with one launch.  Everything the library enqueues on the context's stream
 * between begin and end, including fml_alloc/fml_free pairs, becomes part of the graph; buffers that must
 * outlive the recording have to be allocated before it starts, every buffer allocated inside has to be freed
 * inside, and anything that would grow the scratch arena must have run once before (run the sequence
 * eagerly first).  Host reads (fml_download_*, fml_sync) are not allowed while recording. */
int32_t fml_graph_begin(fml_ctx* ctx);
int32_t fml_graph_end(fml_ctx* ctx, int32_t* graph_id);
int32_t fml_graph_launch(fml_ctx* ctx, int32_t graph_id);
int32_t fml_graph_destroy(fml_ctx* ctx, int32_t graph_id);

/* ---- timing (CUDA events on the context's stream) ------------------------- */
int32_t fml_timer_start(fml_ctx* ctx);
int32_t fml_timer_stop_ms(fml_ctx* ctx, float* ms); /* waits for the stop event */
/* A small pool of numbered events (0..63) for timing individual launches. */
int32_t fml_event_record(fml_ctx* ctx, int32_t slot);
int32_t fml_event_elapsed_ms(fml_ctx* ctx, int32_t slot_start, int32_t slot_stop, float* ms);

/* ---- dense contraction ------------------------------------------------------
 * C[M x N] = act(alpha * op(A)[M x K] . op(B)[K x N] + bias) (+ C if beta == 1)
 * Replaces matMul forward (tensor.dart:867-899, no transposes), the two backward
 * products dA += dC.B^T (tensor.dart:918-924: transB = 1) and dB += A^T.dC
 * (tensor.dart:935-941: transA = 1) without materialising the transposes the
 * reference builds (:877-884, :908-915, :927-934), the bias add
 * addMatrixAndVector (tensor.dart:679-709) and the activation.
 *   transA = 0: A stored [M x K];  1: stored [K x M].   same for B with [K x N] / [N x K].
 *   preact, if non-NULL, receives alpha*A.B + bias before the activation (ldc).
 *   batch1/batch2 > 1 run independent problems at the given element strides
 *   (attention heads inside sequences: QK^T and P.V of
 *   lib/layertypes/singleHeadAttentionLayer.dart:77-86).
 *   precision = -1 uses the context default.
 * The tensor-core path needs 16-byte aligned pointers and lda/ldb/strides that
 * are multiples of 4; anything else runs on the FP32 CUDA-core kernel. */
typedef struct {
  int32_t M, N, K;
  int32_t transA, transB;
  int64_t lda, ldb, ldc;
  const float* A;
  const float* B;
  float* C;
  const float* bias; /* length N, or NULL */
  float* preact;     /* [M x N] at ldc, or NULL */
  int32_t act;       /* fml_act */
  float alpha;
  float beta;        /* 0 or 1 */
  int32_t batch1, batch2;          /* >= 1 */
  int64_t sA1, sA2, sB1, sB2, sC1, sC2; /* element strides per batch level */
  int32_t precision; /* fml_precision or -1 */
  /* Gradient epilogue: if dact_saved != NULL the result is multiplied elementwise by act'(dact_saved)
   * before it is stored: the dLoss/dAct multiply of the layer BELOW, fused into the product that
   * computes the gradient of its output (dX = dZ.W^T of tensor.dart:918-924 followed by
   * tensor.dart:1030 / :552 / :598).  dact_saved is [M x N] at ldc with C's batch strides; it holds the
   * pre-activation for RELU/GELU and the activation output for SIGMOID/TANH, as in fml_act_bwd. */
  const float* dact_saved;
  int32_t dact; /* fml_act of the layer below */
  /* Row epilogue for attention scores (N <= 512, N a multiple of 32; no bias/act/preact/beta):
   *   rowop = 1: C = row softmax of alpha * (A.B), columns j > row masked when rowop_causal != 0
   *              (matMul + scaleMatrix + softmaxMatrix of singleHeadAttentionLayer.dart:77-81 in one kernel);
   *   rowop = 2: C = alpha * P * ((A.B) - rowsum((A.B) * P)) with P = rowop_aux laid out like C
   *              (the softmax backward of softmax.dart:98-112 applied to the product dP = dO.V^T).
   * The whole row of a 128-row block stays in tensor memory, so the scores never make a round trip. */
  int32_t rowop;
  int32_t rowop_causal;
  const float* rowop_aux;
} fml_gemm_desc;

int32_t fml_gemm(fml_ctx* ctx, const fml_gemm_desc* d);
/* Which kernel the last fml_gemm used: 1 = tcgen05 tensor-core, 2 = CUDA-core. */
int32_t fml_gemm_last_path(fml_ctx* ctx, int32_t* path);
/* How the last tensor-core fml_gemm was tiled (all zero after a CUDA-core launch): ctas_per_tile = 1 (128-row tiles,
 * one CTA each) or 2 (256 x 256 tiles over a pair of CTAs, cta_group::2), tile_cols = 64 / 128 / 256, k_splits =
 * CTAs (or pairs) sharing one output tile along K, k_chunks = accumulation chunks per tile.  Any pointer may be
 * NULL.  Lets a test prove which variant of the kernel produced the result it compares. */
int32_t fml_gemm_last_tile(fml_ctx* ctx, int32_t* ctas_per_tile, int32_t* tile_cols, int32_t* k_splits, int32_t* k_chunks);

/* ---- legacy symbols (cuda_lib/kernel.cu:6-11 and :57-58) --------------------
 * Host pointers, row-major, A m x k, B k x n, C m x n; same argument order as
 * the reference.  Backed by a cached context on device 0 and the kernels above
 * instead of per-call cudaMalloc + cublasCreate + cublasSgemm.  multiplyMatrices
 * stays void; failures are readable through fml_last_error(NULL). */
void multiplyMatrices(float* h_a, float* h_b, float* h_c, int32_t m, int32_t k, int32_t n);
/* Largest square size (steps of 100) whose round trip stays under 1000 ms. */
int32_t benchtest(void);

/* ---- elementwise -------------------------------------------------------------
 * y = act(x)                                    (tensor.dart:1013-1038, 1123-1151, 1178-1209)
 * dx (+)= dy * act'(saved); saved = x for RELU/GELU (tensor.dart:1030), y for
 * SIGMOID/TANH (tensor.dart:552, 598).  accumulate != 0 adds into dx as the
 * reference's closures do.  If dbias != NULL (cols > 0) it also receives
 * (accumulated) column sums of the produced gradient: addMatrixAndVector
 * backward, tensor.dart:698-704. */
int32_t fml_act_fwd(fml_ctx* ctx, int32_t act, const float* x, float* y, int64_t n);
int32_t fml_act_bwd(fml_ctx* ctx, int32_t act, const float* saved, const float* dy, float* dx,
                    int64_t rows, int64_t cols, int32_t accumulate, float* dbias);
/* y = a + b (addMatrix tensor.dart:651-677); y may alias a. */
int32_t fml_add(fml_ctx* ctx, const float* a, const float* b, float* y, int64_t n);
/* y += s * x  (gradient fan-in, scaleMatrix tensor.dart:1075-1101) */
int32_t fml_axpy(fml_ctx* ctx, float s, const float* x, float* y, int64_t n);
/* y = a * b (elementWiseMultiply tensor.dart:478-497) */
int32_t fml_mul(fml_ctx* ctx, const float* a, const float* b, float* y, int64_t n);
/* Y = X + 1.b^T and db (+)= column sums of dY (tensor.dart:679-709). */
int32_t fml_add_bias(fml_ctx* ctx, const float* x, const float* b, float* y, int64_t rows, int64_t cols);
int32_t fml_col_sum(fml_ctx* ctx, const float* dy, float* db, int64_t rows, int64_t cols, int32_t accumulate);
/* out[cols x rows] = in[rows x cols]^T (transpose tensor.dart:1211-1236) */
int32_t fml_transpose(fml_ctx* ctx, const float* in, float* out, int64_t rows, int64_t cols);

/* ---- row kernels --------------------------------------------------------------
 * Row softmax of scale*x (softmaxMatrix lib/activationFunctions/softmax.dart:68-96
 * with scaleMatrix lib/layertypes/singleHeadAttentionLayer.dart:80 folded in).
 * causal_period > 0 masks column j > (row mod causal_period) (extension).
 * Backward: dx = scale * y * (dy - sum(dy*y)) (softmax.dart:98-112). */
int32_t fml_softmax_rows_fwd(fml_ctx* ctx, const float* x, float* y, int64_t rows, int32_t cols,
                             float scale, int32_t causal_period);
int32_t fml_softmax_rows_bwd(fml_ctx* ctx, const float* y, const float* dy, float* dx, int64_t rows,
                             int32_t cols, float scale, int32_t accumulate);
/* y = gamma * xhat + beta over rows of (x [+ residual]); saves xhat and
 * rstd = 1/sqrt(var+eps) (layerNorm lib/transformer/layerNormalization.dart:137-169;
 * the residual add is addMatrix of transformerEncodingLayer.dart:63,68 fused in).
 * Backward (:174-200): dx, and dgamma/dbeta accumulated. */
int32_t fml_layernorm_fwd(fml_ctx* ctx, const float* x, const float* residual, const float* gamma,
                          const float* beta, float* y, float* xhat, float* rstd, int64_t rows,
                          int32_t cols, float eps);
int32_t fml_layernorm_bwd(fml_ctx* ctx, const float* dy, const float* gamma, const float* xhat,
                          const float* rstd, float* dx, float* dgamma, float* dbeta, int64_t rows,
                          int32_t cols, int32_t accumulate_dx);
/* Softmax cross-entropy (extension): loss_sum += sum_r -log softmax(z_r)[label_r] * inv_count,
 * dz = (softmax(z) - onehot) * inv_count written in place of z when dz == z.  A label outside
 * [0, cols) contributes no loss and no one-hot term and is reported by fml_device_status. */
int32_t fml_softmax_xent(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz,
                         float* loss_sum, int64_t rows, int32_t cols, float inv_count);
/* fml_softmax_xent that also ADDS the column sums of dz into dbias: the bias gradient of the layer that produced
 * the logits (addMatrixAndVector backward, tensor.dart:698-704) without a second pass over the gradient. */
int32_t fml_softmax_xent_dbias(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz,
                               float* loss_sum, int64_t rows, int32_t cols, float inv_count, float* dbias);
/* Same computation and results as fml_softmax_xent, for callers that must not allocate.
 * (No counterpart in the reference: it has neither this loss nor device memory management.)
 * fml_softmax_xent may grow the context's scratch arena with cudaMalloc; this entry point never
 * calls cudaMalloc, cudaFree or any allocating routine.  Its per-row scratch is a fixed array
 * inside the library (FML_XENT_STATIC_MAX_ROWS floats = 256 KiB, held by every GPU that loads
 * the library until the process exits).  Use it from hosts whose own allocator owns all device
 * memory, or that cannot tolerate the device-wide synchronisation an allocation implies.
 *   - rows > FML_XENT_STATIC_MAX_ROWS is refused with FML_ERR_OOM; split the batch.
 *   - The first call on each device resolves the array's device address; make that call
 *     before starting any stream capture.
 *   - All calls share the one array and it keeps the previous call's contents (nothing in it
 *     needs clearing: each call overwrites the slots it reads).  Calls that overlap on the GPU,
 *     from different streams or contexts of the same device, race on it: serialise them. */
#define FML_XENT_STATIC_MAX_ROWS 65536
int32_t fml_softmax_xent_static(fml_ctx* ctx, const float* z, const int32_t* labels, float* dz,
                                float* loss_sum, int64_t rows, int32_t cols, float inv_count);
/* mseMatrix (tensor.dart:982-1011): loss_sum += mean((p-t)^2); dp = 2(p-t)/n * upstream. */
int32_t fml_mse(fml_ctx* ctx, const float* p, const float* t, float* dp, float* loss_sum, int64_t n,
                float upstream);

/* ---- embedding / positional --------------------------------------------------
 * out[i] = table[ids[i]] (+ pe[i mod period]) (embeddingLayer.dart:47-56,
 * positionalEncodingLayer.dart:55-65); backward scatter-adds (:58-65).  table and dtable have
 * `vocab` rows.  An id outside [0, vocab) (the reference would raise a RangeError at :53) is
 * never used as an address: its row gets no table contribution, and fml_device_status reports
 * FML_ERR_INVALID afterwards. */
int32_t fml_embedding_fwd(fml_ctx* ctx, const float* table, const int32_t* ids, const float* pe,
                          float* out, int64_t n, int32_t dim, int32_t pe_period, int32_t vocab);
int32_t fml_embedding_bwd(fml_ctx* ctx, const float* dout, const int32_t* ids, float* dtable,
                          int64_t n, int32_t dim, int32_t vocab);
/* The reference's table: angle = pos / 10000^(2i/dModel), sin for even i, cos for odd i
 * (positionalEncodingLayer.dart:39-48). */
int32_t fml_positional_table(fml_ctx* ctx, float* pe, int32_t max_len, int32_t d_model);

/* ---- optimizers ---------------------------------------------------------------
 * SGD.step lib/optimizers/sgd.dart:24-42; Adam.step lib/optimizers/adam.dart:44-77
 * (t = step count after the increment at :46).  grad_scale multiplies g first
 * (1 for the reference behaviour).  Hyper-parameters are doubles, as in Dart: 1 - beta and
 * 1 - beta^t are formed in double before narrowing (1 - 0.999f would be off by 1e-5). */
int32_t fml_sgd_step(fml_ctx* ctx, float* w, const float* g, int64_t n, double lr, double grad_scale);
int32_t fml_adam_step(fml_ctx* ctx, float* w, const float* g, float* m, float* v, int64_t n,
                      double lr, double beta1, double beta2, double eps, int32_t t, double grad_scale);
/* The same update enqueued on copy lane `lane` (-1: the main stream), for a slice of the parameters whose gradient
 * exchange has just been enqueued on that lane: the update of finished layers then runs under the backward pass of
 * the others.  zero_grad != 0 also clears g as it is read (Optimizer.zeroGrad, optimizers.dart:62-66, in the same
 * pass).  Order it against the main stream with the event calls. */
int32_t fml_adam_step_on(fml_ctx* ctx, int32_t lane, float* w, float* g, float* m, float* v, int64_t n,
                         double lr, double beta1, double beta2, double eps, int32_t t, double grad_scale, int32_t zero_grad);

/* The other optimizers of lib/optimizers, one kernel (state buffers start at zero; unused ones may be NULL):
 *   FML_OPT_MOMENTUM sgdmomentum.dart:56-57 (h1 = momentum; s1 = velocity)
 *   FML_OPT_NAG      nag.dart:58-60         (h1 = momentum; s1 = velocity)
 *   FML_OPT_RMSPROP  rmsprop.dart:57-58     (h1 = beta, h2 = epsilon; s1 = mean square)
 *   FML_OPT_ADAGRAD  adagrad.dart:54-55     (h2 = epsilon; s1 = squared-gradient sum)
 *   FML_OPT_ADAMW    adamw.dart:82-89       (h1 = beta1, h2 = beta2, h3 = epsilon, h4 = weight decay; s1 = m, s2 = v)
 *   FML_OPT_AMSGRAD  amsgrad.dart:80-86     (h1 = beta1, h2 = beta2, h3 = epsilon; s1 = m, s2 = v, s3 = max v) */
typedef enum { FML_OPT_MOMENTUM = 1, FML_OPT_NAG = 2, FML_OPT_RMSPROP = 3, FML_OPT_ADAGRAD = 4, FML_OPT_ADAMW = 6,
               FML_OPT_AMSGRAD = 7 } fml_optimizer;
int32_t fml_optimizer_step(fml_ctx* ctx, int32_t kind, float* w, const float* g, float* s1, float* s2, float* s3,
                           int64_t n, double lr, double h1, double h2, double h3, double h4, int32_t t);

/* The other activations of lib/activationFunctions, with their parameter: FML_ACT2_LEAKY_RELU (alpha, leakyRelu.dart:35-48),
 * FML_ACT2_ELU (alpha, elu.dart:27-41), FML_ACT2_SWISH (silu.dart:29-49), FML_ACT2_MISH (mish.dart:29-31).
 * Backward takes the INPUT x and adds into dx when accumulate != 0. */
typedef enum { FML_ACT2_LEAKY_RELU = 5, FML_ACT2_ELU = 6, FML_ACT2_SWISH = 7, FML_ACT2_MISH = 8 } fml_act2;
int32_t fml_act2_fwd(fml_ctx* ctx, int32_t kind, float alpha, const float* x, float* y, int64_t n);
int32_t fml_act2_bwd(fml_ctx* ctx, int32_t kind, float alpha, const float* x, const float* dy, float* dx, int64_t n,
                     int32_t accumulate);

/* ---- tape executor ---------------------------------------------------------------
 * One call runs a whole list of autograd nodes on the device: the replacement for
 * walking Node.opName / Node.extraParams (lib/autogradEngine/tensor.dart:5-19) and
 * calling one closure per node (Tensor.backward, tensor.dart:43-75).  The caller lists
 * the nodes in creation (topological) order, as tensor.dart:54-66 produces them; every
 * tensor is a device buffer of rows x cols floats (vectors: rows = 1, scalars: 1 x 1).
 *
 *   FML_TAPE_FORWARD   computes out of every op, first to last.
 *   FML_TAPE_BACKWARD  sets gout of the LAST op to 1 (tensor.dart:70) and runs the
 *                      gradient rule of every op last to first.  Gradients ACCUMULATE
 *                      into gin[] (+=) exactly as the reference's closures do, so the
 *                      caller zeroes gradient buffers first (Tensor.zeroGrad,
 *                      tensor.dart:77-91).  A NULL gin[i] means "no gradient wanted".
 *   FML_TAPE_BACKWARD_NOSEED  the same without touching the last gout.
 *
 * kind follows the reference's opName strings (fml_tape_kind maps a string to its kind):
 *   matMul              out[r x c] = in0[r x inner] . in1[inner x c]          tensor.dart:867-947
 *   matVecMul           out[c] = in0[c x inner] . in1[inner]                   tensor.dart:949-980
 *   addMatrixAndVector  out = in0 + 1.in1^T                                    tensor.dart:679-709
 *   add_matrix, add_vector, add_3d               out = in0 + in1               tensor.dart:651-677, 395-414
 *   multiply_matrix, multiply_vector             out = in0 * in1 (elementwise) tensor.dart:478-497, 835-865
 *   relu_*, sigmoid_*, tanh_* (vector and matrix forms), gelu (extension)      tensor.dart:521-605, 1013-1209
 *   leaky_relu, elu(_matrix), swish, mish        s = alpha                     lib/activationFunctions
 *   scale_matrix        out = s * in0                                          tensor.dart:1075-1101
 *   transpose           out[r x c] = in0[c x r]^T                              tensor.dart:1211-1236
 *   concat_matrix_col, concat_vector   out = [parts[0] | parts[1] | ...], n_parts buffers of
 *                       part_cols[i] columns each (gparts[i] may be NULL)      tensor.dart:739-763, 437-455
 *   softmax_matrix, softmax            rows; iparam = causal period (0 = none; extension)  softmax.dart:68-115
 *   layer_norm(_vector) in0 = x, in1 = gamma, in2 = beta, s = epsilon; aux0 [r x c] and aux1 [r]
 *                       are caller-provided buffers for x-hat and 1/sigma      layerNormalization.dart:137-202
 *   embedding_lookup    in0 = table [inner x c], ids = r row indices           embeddingLayer.dart:47-67
 *   mse_matrix, mse_vector   in0 = prediction, in1 = target, inner = their element count, out 1 x 1
 *                                                                              tensor.dart:499-519, 982-1011
 *   sum_matrix, sum_vector   out 1 x 1 = sum of the inner elements of in0      tensor.dart:561-579, 1153-1176
 *   softmax_xent (extension) in0 = logits [inner x iparam], ids = labels, s = 1/count, out 1 x 1; aux0
 *                       [inner x iparam] keeps the gradient between the sweeps
 *   conv2d              out[r x c] = in0 (image) cross-correlated with in1 (kernel, inner x iparam taps),
 *                       s = padding on every side (0 'valid', (inner - 1) / 2 'same')  tensor.dart:765-833
 *   addScalarToMatrix   out = in0 + in1[0] (in1 is 1 x 1)                      tensor.dart:711-737
 *   attention (extension)  out[r x c] = softmax(s * Q.K^T [+ causal mask]) . V for r / inner sequences of inner positions
 *                       and c / 64 heads in one fused kernel (fml_attention_fwd): in0, in1, in2 = Q, K, V, each [r x c]
 *                       with head h in columns 64 h .. 64 h + 63; s = scale, iparam != 0 = causal; aux0 and aux1 are
 *                       caller-provided buffers of r * c / 64 floats (row statistics, backward scratch)
 *   dense (extension)   out = act(in0[r x inner] . in1[inner x c] + in2), iparam = fml_act, aux0 = pre-activation
 *                       buffer for GELU: matMul + addMatrixAndVector + activation of
 *                       DenseLayerMatrix.forward (denseLayer.dart:116-125) as one launch; its backward rule
 *                       leaves dLoss/dZ in gout */
typedef enum {
  FML_OP_MATMUL = 1, FML_OP_MATVECMUL = 2, FML_OP_ADD_MATRIX_AND_VECTOR = 3, FML_OP_ADD = 4, FML_OP_MULTIPLY = 5,
  FML_OP_RELU = 6, FML_OP_SIGMOID = 7, FML_OP_TANH = 8, FML_OP_GELU = 9, FML_OP_LEAKY_RELU = 10, FML_OP_ELU = 11,
  FML_OP_SWISH = 12, FML_OP_MISH = 13, FML_OP_SCALE_MATRIX = 14, FML_OP_TRANSPOSE = 15, FML_OP_CONCAT = 16,
  FML_OP_SOFTMAX_MATRIX = 17, FML_OP_LAYER_NORM = 18, FML_OP_EMBEDDING_LOOKUP = 19, FML_OP_MSE = 20, FML_OP_SUM = 21,
  FML_OP_SOFTMAX_XENT = 22, FML_OP_DENSE = 23, FML_OP_CONV2D = 24, FML_OP_ADD_SCALAR_TO_MATRIX = 25, FML_OP_ATTENTION = 26
} fml_op_kind;
typedef enum { FML_TAPE_FORWARD = 0, FML_TAPE_BACKWARD = 1, FML_TAPE_BACKWARD_NOSEED = 2 } fml_tape_direction;

typedef struct fml_op {
  int32_t kind;            /* fml_op_kind */
  int32_t rows, cols;      /* shape of out */
  int32_t inner;           /* contraction length / table rows, see above */
  float* in[3];            /* input values */
  float* gin[3];           /* their gradient buffers, same shapes, or NULL */
  float* out;              /* output value */
  float* gout;             /* its gradient buffer (read by the backward rule) */
  float* aux[2];           /* op-private saved tensors, caller-allocated (see the list above) */
  const int32_t* ids;      /* embedding_lookup row indices / softmax_xent labels (device) */
  float* const* parts;     /* concat: host array of n_parts device pointers */
  float* const* gparts;    /* concat: their gradient buffers (entries may be NULL), or NULL */
  const int32_t* part_cols;/* concat: host array of n_parts column counts */
  int32_t n_parts;
  float s;                 /* extraParams: 's' (tensor.dart:1098), alpha, epsilon, 1/count */
  int32_t iparam;          /* causal period / activation code */
  int32_t precision;       /* contraction precision, -1 = context default */
} fml_op;

int32_t fml_tape_run(fml_ctx* ctx, const fml_op* ops, int32_t n_ops, int32_t direction);
/* opName string -> fml_op_kind, 0 if the executor does not know the name. */
int32_t fml_tape_kind(const char* op_name);

/* ---- fused attention ---------------------------------------------------------------
 * softmax(scale * Q.K^T [+ causal mask]) . V for every (sequence, head) in one kernel, the scores kept on chip:
 * transpose + matMul + scaleMatrix + softmaxMatrix + matMul of SingleHeadAttention.forward
 * (lib/layertypes/singleHeadAttentionLayer.dart:77-86) and the head concat of
 * lib/transformer/multiHeadAttentionLayer.dart:80.  q, k, v are row-major [n_seq * seq_len, >= heads * 64]
 * matrices with row stride ld_qkv (they may be column slices of one fused projection); head h occupies columns
 * 64 h .. 64 h + 63.  out has the same form with stride ld_out.  d_head must be 64 and seq_len a multiple of 128.
 * lse (optional, [n_seq][heads][seq_len]) receives log2 of every row's softmax denominator in the scaled domain
 * (max + log2 sum), which a backward pass needs to rebuild the probabilities. */
typedef struct fml_attention_desc {
  int32_t n_seq, seq_len, heads, d_head;
  const float* q; const float* k; const float* v;
  int64_t ld_qkv;
  float* out;
  int64_t ld_out;
  float* lse;
  float scale;
  int32_t causal;
} fml_attention_desc;
int32_t fml_attention_fwd(fml_ctx* ctx, const fml_attention_desc* d);
/* Backward of fml_attention_fwd (d as in the forward call, with the out and lse it produced).  dout is the gradient of
 * out (row stride ld_dout); dq, dk, dv have the layout of q, k, v with row stride ld_dqkv and are overwritten, or
 * added to when accumulate != 0.  scratch: n_seq * heads * seq_len floats.  Two kernels rebuild the probabilities
 * from lse on chip - one per query block for dQ, one per key block (scores transposed) for dK and dV - so no
 * score-sized tensor is written to or read from global memory in either pass. */
int32_t fml_attention_bwd(fml_ctx* ctx, const fml_attention_desc* d, const float* dout, int64_t ld_dout, float* dq,
                          float* dk, float* dv, int64_t ld_dqkv, int32_t accumulate, float* scratch);

/* ---- convolution -----------------------------------------------------------------
 * conv2d (tensor.dart:765-833) for every kernel of a Conv2DLayer (lib/layertypes/conv2d.dart:60-75) and every image
 * of a batch in one launch: in [n_img][H][W], w [n_k][kh][kw], bias [n_k] or NULL (addScalarToMatrix,
 * tensor.dart:711-737), out [n_img][n_k][OH][OW] with OH = H + 2 pad - kh + 1.  pad = 0 is 'valid', (kh - 1) / 2
 * is 'same'.  Backward ADDS into din / dw / dbias (NULL skips one), padded positions contribute nothing. */
int32_t fml_conv2d_fwd(fml_ctx* ctx, const float* in, const float* w, const float* bias, float* out, int32_t n_img,
                       int32_t H, int32_t W, int32_t n_k, int32_t kh, int32_t kw, int32_t pad);
int32_t fml_conv2d_bwd(fml_ctx* ctx, const float* in, const float* w, const float* dout, float* din, float* dw,
                       float* dbias, int32_t n_img, int32_t H, int32_t W, int32_t n_k, int32_t kh, int32_t kw, int32_t pad);

/* ---- checkpoints -----------------------------------------------------------------
 * (No counterpart in the reference, which has no serialisation.)  One file holds named fp32 device buffers -
 * parameter arena, optimizer state - plus a caller-defined step counter; every entry carries a CRC-32.  Load
 * looks entries up by name, checks sizes and checksums BEFORE it overwrites anything, and may restore a subset.
 * Both calls stage through pinned memory on a copy lane and return when the file / the buffers are complete.
 * Save orders itself behind everything queued on the context's MAIN stream; work still running on the copy lanes
 * (an overlapped gradient exchange, an upload) must be joined by the caller first (fml_lane_sync or an event).  The
 * file is written under <path>.tmp, flushed to stable storage, renamed, and the directory entry flushed: after a
 * crash the name holds the old complete file or the new complete file; a failed save removes its temporary. */
int32_t fml_checkpoint_save(fml_ctx* ctx, const char* path, int64_t step, int32_t n, const char* const* names,
                            const float* const* bufs, const int64_t* sizes);
int32_t fml_checkpoint_load(fml_ctx* ctx, const char* path, int64_t* step, int32_t n, const char* const* names,
                            float* const* bufs, const int64_t* sizes);

/* ---- LSTM ---------------------------------------------------------------------
 * One layer over a batch of sequences (LSTMLayer.forward lib/layertypes/lstmLayer.dart:112-150).
 * W: 4 gate matrices [H x (H+I)] in order f,i,c~,o (:64) with columns [h_{t-1} | x_t] (:119),
 * stored as one [4H x (H+I)] matrix; b [4H]; x [T][B][I] (time-major); h0 = c0 = 0.
 * The forward keeps gates [T][B][4H], cells [T+1][B][H] and hidden states [T+1][B][H] for BPTT.
 * Backward takes dh_last [B][H] and produces dW, db (accumulated) and optionally dx. */
typedef struct {
  int32_t T, B, I, H;
  const float* W;
  const float* b;
  const float* x;
  float* gates;  /* [T][B][H][4] activated gates f,i,c~,o per unit */
  float* cells;  /* [T+1][B][H], slot 0 zeroed by the call */
  float* hs;     /* [T+1][B][H], slot 0 zeroed by the call */
  float* xproj;  /* scratch [T*B][4H]                      */
} fml_lstm_desc;
int32_t fml_lstm_fwd(fml_ctx* ctx, const fml_lstm_desc* d);
int32_t fml_lstm_bwd(fml_ctx* ctx, const fml_lstm_desc* d, const float* dh_last, float* dW, float* db,
                     float* dx, float* scratch /* [T*B][4H] + 2*[B][H] floats */);

/* One LSTM cell update on pre-activations the caller has formed: the pointwise part of the reference's tiered recurrent
 * layers (MultiTierLSTMLayer._lstmStep lib/layertypes/multilstm.dart:160-178, DualLSTMLayer lib/layertypes/duallstm.dart),
 * whose tiers combine different inputs at different clocks.  pre and gates are [B][4H] in gate blocks f | i | c~ | o
 * (column g*H + u: the reference's four weight matrices stacked), c_prev, c, h are [B][H].
 * Backward: dh and dc are the gradients arriving at h and c from later steps (either may be NULL = zero); writes the
 * gradient of the pre-activations and writes, or adds to (accumulate_dc_prev != 0), the gradient of c_prev. */
int32_t fml_lstm_cell_fwd(fml_ctx* ctx, const float* pre, const float* c_prev, float* gates, float* c, float* h, int64_t B, int64_t H);
int32_t fml_lstm_cell_bwd(fml_ctx* ctx, const float* gates, const float* c_prev, const float* c, const float* dh, const float* dc,
                          float* dpre, float* dc_prev, int32_t accumulate_dc_prev, int64_t B, int64_t H);

/* ---- data parallel (one process per GPU) -------------------------------------
 * The reference has no multi-device code.  Rank 0 creates an id, the host
 * distributes the 128 bytes by any means, every rank joins, and gradients are
 * summed in place with NCCL over NVLink. */
int32_t fml_dp_unique_id(uint8_t out[128]);
/* Creates the communicator without blocking inside NCCL: the call polls its progress and, if the other ranks have
 * not all joined within the limit (fml_dp_set_timeout, default 120 s), aborts it and returns FML_ERR_TIMEOUT; the
 * context stays usable and fml_dp_init may be called again with a fresh id.  The same limit bounds the host side of
 * every fml_dp_allreduce_sum* call (a rank that left between steps), which also reports NCCL's asynchronous errors. */
int32_t fml_dp_init(fml_ctx* ctx, const uint8_t id[128], int32_t rank, int32_t world);
int32_t fml_dp_set_timeout(fml_ctx* ctx, int32_t timeout_ms);
/* Upper limit on the CTAs (SMs) a collective of this context's communicator occupies; call before fml_dp_init.
 * Together with fml_set_sm_reserve it partitions the SMs between an exchange and the products that run beside it. */
int32_t fml_dp_set_max_ctas(fml_ctx* ctx, int32_t ctas);
int32_t fml_dp_allreduce_sum(fml_ctx* ctx, float* buf, int64_t n);
/* The same on copy lane `lane` (or -1: the main stream), to overlap the exchange of finished gradient
 * slices with the rest of the backward pass; order it against the main stream with the event calls. */
int32_t fml_dp_allreduce_sum_on(fml_ctx* ctx, int32_t lane, float* buf, int64_t n);
int32_t fml_dp_shutdown(fml_ctx* ctx);

#ifdef __cplusplus
}
#endif
#endif /* FML_H_ */
