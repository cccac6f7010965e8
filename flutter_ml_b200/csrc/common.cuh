// Shared declarations of the library's translation units.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <atomic>
#include <map>
#include <mutex>
#include <string>
#include <tuple>
#include <unordered_set>
#include <vector>

#include "fml.h"

struct fml_ctx {
  int device = 0;
  int sm_count = 0;
  int precision = FML_PREC_TF32;
  cudaStream_t stream = nullptr;
  bool own_stream = true;
  std::string last_error;
  int* d_status = nullptr;  // device word written by kernels whose bounded waits expire
  // scratch arena (3xTF32 operand splits)
  char* ws = nullptr;
  size_t ws_bytes = 0;
  std::unordered_set<void*> allocs;
  cudaEvent_t ev0 = nullptr, ev1 = nullptr;
  cudaEvent_t ev_pool[64] = {};
  cudaStream_t lanes[4] = {nullptr, nullptr, nullptr, nullptr};  // side streams (copies, exchange), created on first use
  std::vector<cudaGraphExec_t> graphs;         // instantiated graphs, index = graph id
  bool capturing = false;
  int sm_reserve = 0;  // SMs the persistent tensor-core kernels leave free (fml_set_sm_reserve)
  int last_gemm_path = 0;
  int last_gemm_tile[4] = {0, 0, 0, 0};  // of the last tensor-core launch: CTAs per tile (1 or 2), tile columns, K splits, K chunks
  // tensor-map cache: key -> encoded CUtensorMap
  std::map<std::tuple<const void*, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, int>, CUtensorMap> tmaps;
  // NCCL (loaded lazily with dlopen)
  void* nccl_comm = nullptr;
  int dp_rank = 0, dp_world = 1;
  int dp_max_ctas = 0;         // upper limit on the CTAs of a collective (0: NCCL's choice)
  int dp_timeout_ms = 120000;  // host-side limit for communicator creation and for enqueueing a collective
};

void fml_set_global_error(const std::string& msg);
int32_t fml_fail(fml_ctx* ctx, int32_t code, const std::string& msg);
int32_t fml_ensure_workspace(fml_ctx* ctx, size_t bytes);
// stream of copy lane `lane` (created on first use); lane < 0 is the context's main stream
extern "C" int32_t fml_any_stream(fml_ctx* ctx, int32_t lane, cudaStream_t* out);
// like fml_ensure_workspace, but fails instead of reallocating when work already queued on the stream uses the arena
int32_t fml_ensure_workspace_keep(fml_ctx* ctx, size_t bytes);

#define FML_CUDA(ctx, call)                                                              \
  do {                                                                                   \
    cudaError_t e__ = (call);                                                            \
    if (e__ != cudaSuccess)                                                              \
      return fml_fail((ctx), FML_ERR_CUDA, std::string(#call) + ": " + cudaGetErrorString(e__)); \
  } while (0)

// One host thread may drive contexts on several GPUs (the reference's host is a single isolate), so every entry
// point makes its context's device current before it touches the runtime.  cudaGetDevice is a thread-local read.
#define FML_ENTER(ctx)                                                        \
  do {                                                                        \
    if (ctx) {                                                                \
      int cur__ = -1;                                                         \
      if (cudaGetDevice(&cur__) != cudaSuccess || cur__ != (ctx)->device)     \
        FML_CUDA((ctx), cudaSetDevice((ctx)->device));                        \
    }                                                                         \
  } while (0)

// Runs `...` once per (call site, device of ctx).  Function attributes such as the dynamic shared memory opt-in
// belong to ONE device, so a process-wide flag would leave every later device without them.  Two threads may both
// run the body the first time; the bodies used here are idempotent.
#define FML_MAX_DEVICES 64
#define FML_ONCE_PER_DEVICE(ctx, ...)                                                        \
  do {                                                                                       \
    static std::atomic<bool> done__[FML_MAX_DEVICES];                                        \
    const int dev__ = (ctx)->device;                                                         \
    const bool slot__ = dev__ >= 0 && dev__ < FML_MAX_DEVICES;                               \
    if (!slot__ || !done__[dev__].load(std::memory_order_acquire)) {                         \
      __VA_ARGS__;                                                                           \
      if (slot__) done__[dev__].store(true, std::memory_order_release);                      \
    }                                                                                        \
  } while (0)

#define FML_REQUIRE(ctx, cond, msg) \
  do {                              \
    if (!(cond)) return fml_fail((ctx), FML_ERR_INVALID, (msg)); \
  } while (0)

#define FML_LAUNCH_CHECK(ctx, what)                                                     \
  do {                                                                                  \
    cudaError_t e__ = cudaGetLastError();                                               \
    if (e__ != cudaSuccess)                                                             \
      return fml_fail((ctx), FML_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e__)); \
  } while (0)

// Second word of the context's status block: set (first writer wins) by a kernel that met a token id or a class label
// outside its range.  The kernel skips the access, so a bad index is a reported error, never an illegal address.
#define FML_STATUS_BAD_INDEX_WORD 1
enum { FML_BAD_INDEX_EMBEDDING_FWD = 201, FML_BAD_INDEX_EMBEDDING_BWD = 202, FML_BAD_INDEX_LABEL = 203 };
__device__ __forceinline__ void fml_flag_bad_index(int* status, int code) {
  if (status) atomicCAS(status + FML_STATUS_BAD_INDEX_WORD, 0, code);
}

// LSTM gate epilogue of the tensor-core GEMM: the product's columns are gate-interleaved
// (column 4*r + q = gate q of hidden unit r, q in f,i,c~,o); `addend` [M x N] is added to the product
// (the input projection of this timestep), then the thread that owns a row applies the gate
// nonlinearities and the cell update for 8 hidden units per 32-column block.
struct fml_lstm_epilogue {
  const float* addend;  // [M][N] pre-activation part computed ahead of time (ld = N)
  const float* c_prev;  // [M][N/4]
  float* c_out;         // [M][N/4]
  float* h_out;         // [M][N/4]
  float* gates;         // [M][N] activated gates, interleaved like the columns
  int fast_math;        // TF32 mode: hardware exponential and reciprocal in the gate functions (error ~1e-6, far inside
                        // the 1e-3 bound of that mode; the epilogue warps are latency-bound and these are 40 calls per thread)
};

// internal entry points between translation units
int32_t fml_gemm_tc(fml_ctx* ctx, const fml_gemm_desc* d, int precision, const fml_lstm_epilogue* lstm = nullptr);
int32_t fml_gemm_simt(fml_ctx* ctx, const fml_gemm_desc* d);
bool fml_gemm_tc_eligible(const fml_gemm_desc* d);

__device__ __forceinline__ float fml_sigmoid(float x) { return 1.f / (1.f + expf(-x)); }
// the reference's tanh: (e^{2x}-1)/(e^{2x}+1), exactly 1 when e^{2x} overflows (tensor.dart:582-586)
__device__ __forceinline__ float fml_tanh_ref(float x) {
  const float e2x = expf(2.f * x);
  return isinf(e2x) ? 1.f : (e2x - 1.f) / (e2x + 1.f);
}

// 2^x on the special-function unit, results below 2^-126 flushed to zero (exp2f adds a rescaling sequence for them)
__device__ __forceinline__ float fml_exp2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float fml_sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float fml_tanh_fast(float x) {
  const float e2x = __expf(2.f * x);          // same algebra and the same overflow rule as fml_tanh_ref
  return e2x > 3.0e38f ? 1.f : __fdividef(e2x - 1.f, e2x + 1.f);
}

// Standard normal CDF and e^{-x^2/2} from ONE exponential: erfc(z) = t (a1 + t (a2 + t (a3 + t (a4 + t a5)))) e^{-z^2},
// t = 1/(1 + p z), z = |x|/sqrt(2) (Abramowitz & Stegun 7.1.26, |error| <= 1.5e-7 on erf, i.e. 7.5e-8 on the CDF:
// one float ulp at 0.5..1).  erff costs about three times as many instructions and a divergent branch; with it the
// GELU' + bias-gradient pass ran at 0.76-0.81 of the copy bandwidth, with this form at 1.0.
__device__ __forceinline__ float fml_norm_cdf(float x, float* e_out) {
  const float e = __expf(-0.5f * x * x);
  const float t = __fdividef(1.f, fmaf(0.3275911f * 0.70710678118654752440f, fabsf(x), 1.f));
  float p = fmaf(1.061405429f, t, -1.453152027f);
  p = fmaf(p, t, 1.421413741f);
  p = fmaf(p, t, -0.284496736f);
  p = fmaf(p, t, 0.254829592f);
  const float q = 0.5f * p * t * e;  // 0.5 * erfc(|x| / sqrt 2)
  *e_out = e;
  return x >= 0.f ? 1.f - q : q;
}
__device__ __forceinline__ float fml_gelu(float x) {
  float e;
  return x * fml_norm_cdf(x, &e);
}
__device__ __forceinline__ float fml_gelu_grad(float x) {  // Phi(x) + x phi(x)
  float e;
  const float cdf = fml_norm_cdf(x, &e);
  return fmaf(x * 0.39894228040143267794f, e, cdf);
}

// The transcendental activations live in ONE out-of-line function: inlined into the GEMM epilogue they
// were expanded 32 times per code path and the kernel outgrew the instruction cache (a 4096 x 4096 x 64
// product spent 60 of its 76 us fetching epilogue code).
static __device__ __noinline__ float fml_act_apply_slow(int act, float v) {
  switch (act) {
    case FML_ACT_SIGMOID: return 1.f / (1.f + expf(-v));
    case FML_ACT_TANH: {
      // same algebra as the reference: (e^{2x}-1)/(e^{2x}+1), 1 when e^{2x} overflows
      float e2x = expf(2.f * v);
      return isinf(e2x) ? 1.f : (e2x - 1.f) / (e2x + 1.f);
    }
    case FML_ACT_GELU: return fml_gelu(v);
    default: return v;
  }
}
__device__ __forceinline__ float fml_act_apply(int act, float v) {
  if (act == FML_ACT_NONE) return v;
  if (act == FML_ACT_RELU) return v > 0.f ? v : 0.f;
  return fml_act_apply_slow(act, v);
}
// derivative from the saved tensor: x for RELU/GELU, y for SIGMOID/TANH
static __device__ __noinline__ float fml_act_grad_gelu(float s) { return fml_gelu_grad(s); }
// compact form for the GEMM epilogue (the erf code stays out of line)
__device__ __forceinline__ float fml_act_grad_small(int act, float s) {
  if (act == FML_ACT_RELU) return s > 0.f ? 1.f : 0.f;
  if (act == FML_ACT_SIGMOID) return s * (1.f - s);
  if (act == FML_ACT_TANH) return 1.f - s * s;
  if (act == FML_ACT_GELU) return fml_act_grad_gelu(s);
  return 1.f;
}
__device__ __forceinline__ float fml_act_grad(int act, float s) {
  switch (act) {
    case FML_ACT_RELU: return s > 0.f ? 1.f : 0.f;
    case FML_ACT_SIGMOID: return s * (1.f - s);
    case FML_ACT_TANH: return 1.f - s * s;
    case FML_ACT_GELU: return fml_gelu_grad(s);
    default: return 1.f;
  }
}
