// Context, memory, timing, dispatch of fml_gemm and the two legacy symbols.
#include <algorithm>
#include <chrono>
#include <cstring>
#include <mutex>
#include <thread>
#include <vector>

#include "common.cuh"

static std::string g_last_error;
static std::mutex g_mu;

void fml_set_global_error(const std::string& msg) {
  std::lock_guard<std::mutex> lk(g_mu);
  g_last_error = msg;
}
int32_t fml_fail(fml_ctx* ctx, int32_t code, const std::string& msg) {
  if (ctx) ctx->last_error = msg;
  fml_set_global_error(msg);
  return code;
}

int32_t fml_ensure_workspace(fml_ctx* ctx, size_t bytes) {
  if (bytes <= ctx->ws_bytes) return FML_OK;
  if (ctx->capturing)
    return fml_fail(ctx, FML_ERR_INVALID, "the scratch arena would have to grow while a graph is being recorded; run the sequence once eagerly first");
  // Stream-ordered: the old arena is released after everything already queued on the stream has used it, and the
  // new one comes from the pool, so growing the arena in the middle of a step does not synchronise the device.
  if (ctx->ws) {
    FML_CUDA(ctx, cudaFreeAsync(ctx->ws, ctx->stream));
    ctx->ws = nullptr;
    ctx->ws_bytes = 0;
  }
  size_t want = std::max(bytes, (size_t)(64u << 20));
  cudaError_t e = cudaMallocAsync(reinterpret_cast<void**>(&ctx->ws), want, ctx->stream);
  if (e != cudaSuccess) return fml_fail(ctx, FML_ERR_OOM, std::string("workspace cudaMalloc: ") + cudaGetErrorString(e));
  ctx->ws_bytes = want;
  return FML_OK;
}

int32_t fml_ensure_workspace_keep(fml_ctx* ctx, size_t bytes) {
  // fml_ensure_workspace synchronises the stream before it frees the old arena, so queued readers
  // of the old arena have finished; the contents are not preserved, which callers of this variant
  // avoid by sizing the arena up front.
  if (bytes <= ctx->ws_bytes) return FML_OK;
  return fml_fail(ctx, FML_ERR_OOM, "scratch arena too small for a request that must not move it");
}

__global__ void f64_to_f32_kernel(const double* __restrict__ in, float* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = (float)in[i];
}
__global__ void f32_to_f64_kernel(const float* __restrict__ in, double* __restrict__ out, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = (double)in[i];
}

extern "C" {

int32_t fml_device_count(int32_t* count) {
  int n = 0;
  cudaError_t e = cudaGetDeviceCount(&n);
  if (e != cudaSuccess) {
    *count = 0;
    return fml_fail(nullptr, FML_ERR_NO_DEVICE, std::string("cudaGetDeviceCount: ") + cudaGetErrorString(e));
  }
  *count = n;
  return FML_OK;
}

int32_t fml_device_name(int32_t device, char* buf, int32_t buf_len) {
  cudaDeviceProp prop;
  cudaError_t e = cudaGetDeviceProperties(&prop, device);
  if (e != cudaSuccess) return fml_fail(nullptr, FML_ERR_NO_DEVICE, std::string("cudaGetDeviceProperties: ") + cudaGetErrorString(e));
  snprintf(buf, buf_len, "%s", prop.name);
  return FML_OK;
}

// Everything fml_init acquires after the context object exists; on any failure the caller releases what was
// acquired so far and deletes the context (nothing is left behind by a failed fml_init).
static int32_t init_resources(fml_ctx* ctx, const fml_config* cfg) {
  FML_CUDA(ctx, cudaSetDevice(ctx->device));
  FML_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
  {
    cudaMemPool_t pool;
    FML_CUDA(ctx, cudaDeviceGetDefaultMemPool(&pool, ctx->device));
    uint64_t keep = UINT64_MAX;
    FML_CUDA(ctx, cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep));
  }
  FML_CUDA(ctx, cudaMalloc(&ctx->d_status, 256));
  FML_CUDA(ctx, cudaMemset(ctx->d_status, 0, 256));
  FML_CUDA(ctx, cudaEventCreate(&ctx->ev0));
  FML_CUDA(ctx, cudaEventCreate(&ctx->ev1));
  if (cfg && cfg->workspace_bytes > 0) {
    int32_t rc = fml_ensure_workspace(ctx, (size_t)cfg->workspace_bytes);
    if (rc) return rc;
  }
  return FML_OK;
}
static void release_resources(fml_ctx* ctx) {
  if (ctx->ws) cudaFree(ctx->ws);
  if (ctx->d_status) cudaFree(ctx->d_status);
  if (ctx->ev0) cudaEventDestroy(ctx->ev0);
  if (ctx->ev1) cudaEventDestroy(ctx->ev1);
  if (ctx->stream && ctx->own_stream) cudaStreamDestroy(ctx->stream);
  ctx->ws = nullptr; ctx->d_status = nullptr; ctx->ev0 = ctx->ev1 = nullptr; ctx->stream = nullptr;
}

int32_t fml_init(const fml_config* cfg, fml_ctx** out) {
  if (!out) return fml_fail(nullptr, FML_ERR_INVALID, "fml_init: out is NULL");
  *out = nullptr;
  int n = 0;
  if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0)
    return fml_fail(nullptr, FML_ERR_NO_DEVICE, "fml_init: no CUDA device is visible; this library has no CPU path");
  const int dev = cfg ? cfg->device : 0;
  if (dev < 0 || dev >= n) return fml_fail(nullptr, FML_ERR_INVALID, "fml_init: device ordinal out of range");
  cudaDeviceProp prop;
  if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return fml_fail(nullptr, FML_ERR_CUDA, "cudaGetDeviceProperties failed");
  if (prop.major != 10)
    return fml_fail(nullptr, FML_ERR_NO_DEVICE, std::string("fml_init: kernels are built for sm_100a only; device is ") + prop.name);
  fml_ctx* ctx = new fml_ctx();
  ctx->device = dev;
  ctx->sm_count = prop.multiProcessorCount;
  ctx->precision = cfg ? cfg->precision : FML_PREC_TF32;
  const int32_t rc = init_resources(ctx, cfg);
  if (rc != FML_OK) {  // the message stays readable through fml_last_error(NULL)
    release_resources(ctx);
    delete ctx;
    return rc;
  }
  *out = ctx;
  return FML_OK;
}

int32_t fml_shutdown(fml_ctx* ctx) {
  if (!ctx) return FML_OK;
  cudaSetDevice(ctx->device);
  cudaStreamSynchronize(ctx->stream);
  fml_dp_shutdown(ctx);
  for (void* p : ctx->allocs) cudaFreeAsync(p, ctx->stream);
  cudaStreamSynchronize(ctx->stream);
  if (ctx->ws) cudaFree(ctx->ws);
  cudaFree(ctx->d_status);
  cudaEventDestroy(ctx->ev0);
  cudaEventDestroy(ctx->ev1);
  for (cudaEvent_t e : ctx->ev_pool)
    if (e) cudaEventDestroy(e);
  for (cudaGraphExec_t ge : ctx->graphs)
    if (ge) cudaGraphExecDestroy(ge);
  for (cudaStream_t l : ctx->lanes)
    if (l) { cudaStreamSynchronize(l); cudaStreamDestroy(l); }
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  delete ctx;
  return FML_OK;
}

const char* fml_last_error(fml_ctx* ctx) {
  if (ctx) return ctx->last_error.c_str();
  static thread_local std::string copy;
  std::lock_guard<std::mutex> lk(g_mu);
  copy = g_last_error;
  return copy.c_str();
}

int32_t fml_sm_count(fml_ctx* ctx, int32_t* count) {
  FML_ENTER(ctx);
  *count = ctx->sm_count;
  return FML_OK;
}

int32_t fml_set_sm_reserve(fml_ctx* ctx, int32_t sms) {
  FML_REQUIRE(ctx, ctx && sms >= 0 && sms < ctx->sm_count - 1, "fml_set_sm_reserve: must leave at least two SMs for the kernels");
  ctx->sm_reserve = sms;
  return FML_OK;
}

int32_t fml_set_stream(fml_ctx* ctx, void* s) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  if (ctx->own_stream) cudaStreamDestroy(ctx->stream);
  ctx->stream = reinterpret_cast<cudaStream_t>(s);
  ctx->own_stream = false;
  return FML_OK;
}

int32_t fml_sync(fml_ctx* ctx) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return FML_OK;
}

int32_t fml_device_status(fml_ctx* ctx, int32_t* code) {
  FML_ENTER(ctx);
  int v[2] = {0, 0};  // word 0: expired waits; word 1: indices out of range
  FML_CUDA(ctx, cudaMemcpyAsync(v, ctx->d_status, sizeof v, cudaMemcpyDeviceToHost, ctx->stream));
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  *code = v[0] ? v[0] : v[1];
  if (v[0] != 0) {
    cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
    return fml_fail(ctx, FML_ERR_TIMEOUT, "a device-side bounded wait expired (role code " + std::to_string(v[0]) + ")");
  }
  if (v[1] != 0) {
    cudaMemsetAsync(ctx->d_status + FML_STATUS_BAD_INDEX_WORD, 0, sizeof(int), ctx->stream);
    return fml_fail(ctx, FML_ERR_INVALID,
                    std::string(v[1] == FML_BAD_INDEX_LABEL ? "a class label was outside [0, cols)" : "a token id was outside [0, vocab)") +
                        "; the access was skipped (code " + std::to_string(v[1]) + ")");
  }
  return FML_OK;
}

int32_t fml_mem_info(fml_ctx* ctx, int64_t* free_bytes, int64_t* total_bytes, int64_t* arena_bytes) {
  FML_ENTER(ctx);
  size_t f = 0, t = 0;
  FML_CUDA(ctx, cudaMemGetInfo(&f, &t));
  if (free_bytes) *free_bytes = (int64_t)f;
  if (total_bytes) *total_bytes = (int64_t)t;
  if (arena_bytes) *arena_bytes = (int64_t)ctx->ws_bytes;
  return FML_OK;
}

int32_t fml_alloc(fml_ctx* ctx, int64_t n, float** out) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, n >= 0 && out, "fml_alloc: bad arguments");
  void* p = nullptr;
  // stream-ordered pool: a block freed on the context's stream is reused by later calls on the
  // same stream without a device synchronisation (training loops allocate per op)
  cudaError_t e = cudaMallocAsync(&p, (size_t)std::max<int64_t>(n, 1) * sizeof(float), ctx->stream);
  if (e != cudaSuccess) return fml_fail(ctx, FML_ERR_OOM, std::string("fml_alloc: ") + cudaGetErrorString(e));
  ctx->allocs.insert(p);
  *out = reinterpret_cast<float*>(p);
  return FML_OK;
}

int32_t fml_free(fml_ctx* ctx, float* p) {
  FML_ENTER(ctx);
  if (!p) return FML_OK;
  auto it = ctx->allocs.find(p);
  FML_REQUIRE(ctx, it != ctx->allocs.end(), "fml_free: pointer was not allocated by this context");
  ctx->allocs.erase(it);
  // The pool keeps the range mapped (release threshold = max), so cached tensor maps that
  // point into it stay valid for the next owner of the same address.
  FML_CUDA(ctx, cudaFreeAsync(p, ctx->stream));
  return FML_OK;
}

int32_t fml_zero(fml_ctx* ctx, float* p, int64_t n) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaMemsetAsync(p, 0, (size_t)n * sizeof(float), ctx->stream));
  return FML_OK;
}

int32_t fml_upload_f32(fml_ctx* ctx, float* dst, const float* host, int64_t n) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaMemcpyAsync(dst, host, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
  return FML_OK;
}
int32_t fml_upload_i32(fml_ctx* ctx, int32_t* dst, const int32_t* host, int64_t n) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaMemcpyAsync(dst, host, (size_t)n * 4, cudaMemcpyHostToDevice, ctx->stream));
  return FML_OK;
}
int32_t fml_upload_f64(fml_ctx* ctx, float* dst, const double* host, int64_t n) {
  FML_ENTER(ctx);
  // stage the doubles in the scratch arena and narrow on the device
  int32_t rc = fml_ensure_workspace(ctx, (size_t)n * 8);
  if (rc) return rc;
  FML_CUDA(ctx, cudaMemcpyAsync(ctx->ws, host, (size_t)n * 8, cudaMemcpyHostToDevice, ctx->stream));
  f64_to_f32_kernel<<<(int)std::min<int64_t>((n + 255) / 256, 4096), 256, 0, ctx->stream>>>(
      reinterpret_cast<const double*>(ctx->ws), dst, n);
  FML_LAUNCH_CHECK(ctx, "f64_to_f32_kernel");
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return FML_OK;
}
int32_t fml_download_f32(fml_ctx* ctx, float* host, const float* src, int64_t n) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaMemcpyAsync(host, src, (size_t)n * 4, cudaMemcpyDeviceToHost, ctx->stream));
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return FML_OK;
}
int32_t fml_download_f64(fml_ctx* ctx, double* host, const float* src, int64_t n) {
  FML_ENTER(ctx);
  int32_t rc = fml_ensure_workspace(ctx, (size_t)n * 8);
  if (rc) return rc;
  f32_to_f64_kernel<<<(int)std::min<int64_t>((n + 255) / 256, 4096), 256, 0, ctx->stream>>>(
      src, reinterpret_cast<double*>(ctx->ws), n);
  FML_LAUNCH_CHECK(ctx, "f32_to_f64_kernel");
  FML_CUDA(ctx, cudaMemcpyAsync(host, ctx->ws, (size_t)n * 8, cudaMemcpyDeviceToHost, ctx->stream));
  FML_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
  return FML_OK;
}
int32_t fml_copy(fml_ctx* ctx, float* dst, const float* src, int64_t n) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaMemcpyAsync(dst, src, (size_t)n * 4, cudaMemcpyDeviceToDevice, ctx->stream));
  return FML_OK;
}

int32_t fml_timer_start(fml_ctx* ctx) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
  return FML_OK;
}
int32_t fml_timer_stop_ms(fml_ctx* ctx, float* ms) {
  FML_ENTER(ctx);
  FML_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
  FML_CUDA(ctx, cudaEventSynchronize(ctx->ev1));
  FML_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev0, ctx->ev1));
  return FML_OK;
}

int32_t fml_event_record(fml_ctx* ctx, int32_t slot) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, slot >= 0 && slot < 64, "fml_event_record: slot out of range");
  if (!ctx->ev_pool[slot]) FML_CUDA(ctx, cudaEventCreate(&ctx->ev_pool[slot]));
  FML_CUDA(ctx, cudaEventRecord(ctx->ev_pool[slot], ctx->stream));
  return FML_OK;
}
int32_t fml_event_elapsed_ms(fml_ctx* ctx, int32_t a, int32_t b, float* ms) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, a >= 0 && a < 64 && b >= 0 && b < 64 && ctx->ev_pool[a] && ctx->ev_pool[b],
              "fml_event_elapsed_ms: slot not recorded");
  FML_CUDA(ctx, cudaEventSynchronize(ctx->ev_pool[b]));
  FML_CUDA(ctx, cudaEventElapsedTime(ms, ctx->ev_pool[a], ctx->ev_pool[b]));
  return FML_OK;
}

static int32_t lane_stream(fml_ctx* ctx, int32_t lane, cudaStream_t* out) {
  FML_REQUIRE(ctx, lane >= 0 && lane < 4, "copy lane must be 0 .. 3");
  if (!ctx->lanes[lane]) FML_CUDA(ctx, cudaStreamCreateWithFlags(&ctx->lanes[lane], cudaStreamNonBlocking));
  *out = ctx->lanes[lane];
  return FML_OK;
}
int32_t fml_any_stream(fml_ctx* ctx, int32_t lane, cudaStream_t* out) {
  FML_ENTER(ctx);
  if (lane < 0) { *out = ctx->stream; return FML_OK; }
  return lane_stream(ctx, lane, out);
}
static int32_t any_stream(fml_ctx* ctx, int32_t lane, cudaStream_t* out) { return fml_any_stream(ctx, lane, out); }
int32_t fml_event_record_on(fml_ctx* ctx, int32_t slot, int32_t lane) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, slot >= 0 && slot < 64, "fml_event_record_on: slot out of range");
  cudaStream_t s;
  int32_t rc = any_stream(ctx, lane, &s);
  if (rc) return rc;
  if (!ctx->ev_pool[slot]) FML_CUDA(ctx, cudaEventCreate(&ctx->ev_pool[slot]));
  FML_CUDA(ctx, cudaEventRecord(ctx->ev_pool[slot], s));
  return FML_OK;
}
int32_t fml_wait_event(fml_ctx* ctx, int32_t lane, int32_t slot) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, slot >= 0 && slot < 64 && ctx->ev_pool[slot], "fml_wait_event: slot not recorded");
  cudaStream_t s;
  int32_t rc = any_stream(ctx, lane, &s);
  if (rc) return rc;
  FML_CUDA(ctx, cudaStreamWaitEvent(s, ctx->ev_pool[slot], 0));
  return FML_OK;
}
int32_t fml_event_sync(fml_ctx* ctx, int32_t slot) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, slot >= 0 && slot < 64 && ctx->ev_pool[slot], "fml_event_sync: slot not recorded");
  FML_CUDA(ctx, cudaEventSynchronize(ctx->ev_pool[slot]));
  return FML_OK;
}
int32_t fml_lane_h2d(fml_ctx* ctx, int32_t lane, float* dst, const float* host, int64_t n) {
  FML_ENTER(ctx);
  cudaStream_t s;
  int32_t rc = lane_stream(ctx, lane, &s);
  if (rc) return rc;
  FML_CUDA(ctx, cudaMemcpyAsync(dst, host, (size_t)n * 4, cudaMemcpyHostToDevice, s));
  return FML_OK;
}
int32_t fml_lane_d2h(fml_ctx* ctx, int32_t lane, float* host, const float* src, int64_t n) {
  FML_ENTER(ctx);
  cudaStream_t s;
  int32_t rc = lane_stream(ctx, lane, &s);
  if (rc) return rc;
  FML_CUDA(ctx, cudaMemcpyAsync(host, src, (size_t)n * 4, cudaMemcpyDeviceToHost, s));
  return FML_OK;
}
int32_t fml_lane_sync(fml_ctx* ctx, int32_t lane) {
  FML_ENTER(ctx);
  cudaStream_t s;
  int32_t rc = lane_stream(ctx, lane, &s);
  if (rc) return rc;
  FML_CUDA(ctx, cudaStreamSynchronize(s));
  return FML_OK;
}

int32_t fml_graph_begin(fml_ctx* ctx) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, !ctx->capturing, "fml_graph_begin: a recording is already in progress");
  FML_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
  ctx->capturing = true;
  return FML_OK;
}
int32_t fml_graph_end(fml_ctx* ctx, int32_t* graph_id) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, ctx->capturing && graph_id, "fml_graph_end: no recording in progress");
  ctx->capturing = false;
  cudaGraph_t g = nullptr;
  FML_CUDA(ctx, cudaStreamEndCapture(ctx->stream, &g));
  cudaGraphExec_t ge = nullptr;
  cudaError_t e = cudaGraphInstantiate(&ge, g, 0);
  cudaGraphDestroy(g);
  if (e != cudaSuccess) return fml_fail(ctx, FML_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e));
  ctx->graphs.push_back(ge);
  *graph_id = (int32_t)ctx->graphs.size() - 1;
  return FML_OK;
}
int32_t fml_graph_launch(fml_ctx* ctx, int32_t id) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, id >= 0 && id < (int32_t)ctx->graphs.size() && ctx->graphs[id], "fml_graph_launch: unknown graph");
  FML_CUDA(ctx, cudaGraphLaunch(ctx->graphs[id], ctx->stream));
  return FML_OK;
}
int32_t fml_graph_destroy(fml_ctx* ctx, int32_t id) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, id >= 0 && id < (int32_t)ctx->graphs.size() && ctx->graphs[id], "fml_graph_destroy: unknown graph");
  FML_CUDA(ctx, cudaGraphExecDestroy(ctx->graphs[id]));
  ctx->graphs[id] = nullptr;
  return FML_OK;
}

int32_t fml_host_alloc(fml_ctx* ctx, int64_t bytes, void** out) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, bytes > 0 && out, "fml_host_alloc: bad arguments");
  cudaError_t e = cudaHostAlloc(out, (size_t)bytes, cudaHostAllocDefault);
  if (e != cudaSuccess) return fml_fail(ctx, FML_ERR_OOM, std::string("fml_host_alloc: ") + cudaGetErrorString(e));
  return FML_OK;
}
int32_t fml_host_free(fml_ctx* ctx, void* p) {
  FML_ENTER(ctx);
  if (p) FML_CUDA(ctx, cudaFreeHost(p));
  return FML_OK;
}

// Rows of a host array -> a (page-locked) staging buffer, on several host threads.  One thread moves about
// 10 GB/s, a quarter of what the PCIe link takes, so a single-threaded gather would be the bottleneck of a feeder.
extern "C++" {
namespace {
template <typename S, typename D>
void stage_rows_range(D* dst, const S* src, int64_t row_elems, const int64_t* index, int64_t first, int64_t r0, int64_t r1) {
  for (int64_t r = r0; r < r1; r++) {
    const S* s = src + (index ? index[r] : first + r) * row_elems;
    D* d = dst + r * row_elems;
    if (sizeof(S) == sizeof(D)) {
      memcpy(d, s, (size_t)row_elems * sizeof(D));
    } else {
      for (int64_t i = 0; i < row_elems; i++) d[i] = (D)s[i];
    }
  }
}
}  // namespace
}  // extern "C++"

extern "C++" {
namespace {
// Workers of a background gather (fml_stage_rows_async); joined by fml_stage_wait or by the next gather.
std::mutex g_stage_mu;
std::vector<std::thread> g_stage_pool;

void stage_join_locked() {
  for (auto& th : g_stage_pool)
    if (th.joinable()) th.join();
  g_stage_pool.clear();
}

void stage_run(void* dst, const void* src, int32_t src_kind, int64_t row_elems, const int64_t* index, int64_t first_row,
               int64_t r0, int64_t r1) {
  switch (src_kind) {
    case 0: stage_rows_range((float*)dst, (const float*)src, row_elems, index, first_row, r0, r1); break;
    case 1: stage_rows_range((float*)dst, (const double*)src, row_elems, index, first_row, r0, r1); break;
    case 2: stage_rows_range((int32_t*)dst, (const int32_t*)src, row_elems, index, first_row, r0, r1); break;
    default: stage_rows_range((int32_t*)dst, (const int64_t*)src, row_elems, index, first_row, r0, r1); break;
  }
}

int stage_thread_count(int32_t threads, int64_t rows, int64_t row_elems) {
  const int64_t bytes = rows * row_elems * 4;
  int nt = threads > 0 ? threads : (int)std::min<int64_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
  return (int)std::max<int64_t>(1, std::min<int64_t>(nt, std::min<int64_t>(rows, bytes / (1 << 20) + 1)));  // >= 1 MiB each
}
}  // namespace
}  // extern "C++"

static int32_t stage_rows_impl(fml_ctx* ctx, void* dst, const void* src, int32_t src_kind, int64_t row_elems,
                               const int64_t* index, int64_t first_row, int64_t rows, int32_t threads, bool background) {
  FML_REQUIRE(ctx, dst && src && row_elems > 0 && rows >= 0, "fml_stage_rows: bad arguments");
  FML_REQUIRE(ctx, src_kind >= 0 && src_kind <= 3, "fml_stage_rows: src_kind is 0 f32, 1 f64, 2 i32, 3 i64");
  std::lock_guard<std::mutex> lock(g_stage_mu);
  // background gathers accumulate in g_stage_pool until fml_stage_wait joins them; a foreground one leaves them alone
  if (rows == 0) return FML_OK;
  const int nt = stage_thread_count(threads, rows, row_elems);
  if (nt == 1) {   // under 1 MiB: the copy is cheaper than starting a thread, in either form
    stage_run(dst, src, src_kind, row_elems, index, first_row, 0, rows);
    return FML_OK;
  }
  const int64_t per = (rows + nt - 1) / nt;
  std::vector<std::thread> local;
  std::vector<std::thread>& pool = background ? g_stage_pool : local;
  int64_t done_to = background ? 0 : std::min(rows, per);   // the caller's own share in the foreground form
  const int64_t first_spawned = done_to;
  try {
    for (int64_t r0 = first_spawned; r0 < rows; r0 += per) {
      pool.emplace_back(stage_run, dst, src, src_kind, row_elems, index, first_row, r0, std::min(rows, r0 + per));
      done_to = std::min(rows, r0 + per);
    }
  } catch (...) {   // thread creation failed: the rest is done here, on the calling thread
    stage_run(dst, src, src_kind, row_elems, index, first_row, done_to, rows);
  }
  if (!background) {
    stage_run(dst, src, src_kind, row_elems, index, first_row, 0, first_spawned);
    for (auto& th : local) th.join();
  }
  return FML_OK;
}

int32_t fml_stage_rows(fml_ctx* ctx, void* dst, const void* src, int32_t src_kind, int64_t row_elems,
                       const int64_t* index, int64_t first_row, int64_t rows, int32_t threads) {
  return stage_rows_impl(ctx, dst, src, src_kind, row_elems, index, first_row, rows, threads, false);
}
int32_t fml_stage_rows_async(fml_ctx* ctx, void* dst, const void* src, int32_t src_kind, int64_t row_elems,
                             const int64_t* index, int64_t first_row, int64_t rows, int32_t threads) {
  return stage_rows_impl(ctx, dst, src, src_kind, row_elems, index, first_row, rows, threads, true);
}
int32_t fml_stage_wait(fml_ctx* ctx) {
  (void)ctx;
  std::lock_guard<std::mutex> lock(g_stage_mu);
  stage_join_locked();
  return FML_OK;
}

int32_t fml_gemm(fml_ctx* ctx, const fml_gemm_desc* d) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, d && d->A && d->B && d->C, "fml_gemm: NULL operand");
  FML_REQUIRE(ctx, d->M > 0 && d->N > 0 && d->K > 0, "fml_gemm: M, N, K must be positive");
  FML_REQUIRE(ctx, d->beta == 0.f || d->beta == 1.f, "fml_gemm: beta must be 0 or 1");
  FML_REQUIRE(ctx, d->lda >= (d->transA ? d->M : d->K), "fml_gemm: lda smaller than a row of A");
  FML_REQUIRE(ctx, d->ldb >= (d->transB ? d->K : d->N), "fml_gemm: ldb smaller than a row of B");
  FML_REQUIRE(ctx, d->ldc >= d->N, "fml_gemm: ldc smaller than N");
  FML_REQUIRE(ctx, d->act >= FML_ACT_NONE && d->act <= FML_ACT_GELU, "fml_gemm: unknown activation");
  FML_REQUIRE(ctx, !d->dact_saved || (d->dact >= FML_ACT_NONE && d->dact <= FML_ACT_GELU), "fml_gemm: unknown dact");
  FML_REQUIRE(ctx, !d->dact_saved || d->beta == 0.f, "fml_gemm: the gradient epilogue cannot accumulate (beta must be 0)");
  if (d->rowop) {
    FML_REQUIRE(ctx, d->rowop == 1 || d->rowop == 2, "fml_gemm: unknown rowop");
    FML_REQUIRE(ctx, d->N <= 512 && (d->N & 31) == 0, "fml_gemm: the row epilogue needs N <= 512 and N % 32 == 0");
    FML_REQUIRE(ctx, !d->bias && !d->preact && d->act == FML_ACT_NONE && d->beta == 0.f && !d->dact_saved,
                "fml_gemm: the row epilogue excludes bias, activation, pre-activation output, beta and dact");
    FML_REQUIRE(ctx, d->rowop != 2 || d->rowop_aux, "fml_gemm: rowop 2 needs rowop_aux (the softmax output)");
    FML_REQUIRE(ctx, (d->precision < 0 ? ctx->precision : d->precision) != FML_PREC_FP32 && fml_gemm_tc_eligible(d) &&
                         (reinterpret_cast<uintptr_t>(d->C) & 15) == 0 && (d->ldc & 3) == 0 &&
                         (!d->rowop_aux || (reinterpret_cast<uintptr_t>(d->rowop_aux) & 15) == 0),
                "fml_gemm: the row epilogue exists on the tensor-core path only (aligned operands, not FML_PREC_FP32)");
  }
  int prec = d->precision < 0 ? ctx->precision : d->precision;
  FML_REQUIRE(ctx, prec >= FML_PREC_TF32 && prec <= FML_PREC_FP32, "fml_gemm: unknown precision");
  if (prec != FML_PREC_FP32 && fml_gemm_tc_eligible(d)) return fml_gemm_tc(ctx, d, prec);
  return fml_gemm_simt(ctx, d);
}

int32_t fml_gemm_last_path(fml_ctx* ctx, int32_t* path) {
  *path = ctx->last_gemm_path;
  return FML_OK;
}

int32_t fml_selftest_per_device_once(int32_t device, int32_t* runs) {
  // host only: the same guard the kernels' one-time, per-device set-up uses, around a counter
  static std::atomic<int> count[FML_MAX_DEVICES + 1];
  if (!runs) return fml_fail(nullptr, FML_ERR_INVALID, "fml_selftest_per_device_once: runs is NULL");
  fml_ctx probe;
  probe.device = device;
  const int slot = device >= 0 && device < FML_MAX_DEVICES ? device : FML_MAX_DEVICES;
  FML_ONCE_PER_DEVICE(&probe, { count[slot]++; });
  *runs = count[slot].load();
  return FML_OK;
}

int32_t fml_gemm_last_tile(fml_ctx* ctx, int32_t* ctas_per_tile, int32_t* tile_cols, int32_t* k_splits, int32_t* k_chunks) {
  FML_REQUIRE(ctx, ctx != nullptr, "fml_gemm_last_tile: ctx is NULL");
  if (ctas_per_tile) *ctas_per_tile = ctx->last_gemm_tile[0];
  if (tile_cols) *tile_cols = ctx->last_gemm_tile[1];
  if (k_splits) *k_splits = ctx->last_gemm_tile[2];
  if (k_chunks) *k_chunks = ctx->last_gemm_tile[3];
  return FML_OK;
}

// ------------------------------------------------------------------- legacy symbols
static fml_ctx* g_legacy = nullptr;
static float *g_la = nullptr, *g_lb = nullptr, *g_lc = nullptr;
static int64_t g_lcap[3] = {0, 0, 0};

static int32_t legacy_ctx() {
  if (g_legacy) return FML_OK;
  fml_config cfg = {0, FML_PREC_TF32, 0};
  return fml_init(&cfg, &g_legacy);
}
static int32_t legacy_buf(float** p, int64_t* cap, int64_t n) {
  if (n <= *cap) return FML_OK;
  if (*p) fml_free(g_legacy, *p);
  *p = nullptr;
  *cap = 0;
  int32_t rc = fml_alloc(g_legacy, n, p);
  if (rc == FML_OK) *cap = n;
  return rc;
}

void multiplyMatrices(float* h_a, float* h_b, float* h_c, int32_t m, int32_t k, int32_t n) {
  // this symbol has no status return: fml_last_error(NULL) afterwards is empty exactly when the call succeeded,
  // whatever an earlier call on some other context left there
  fml_set_global_error("");
  if (legacy_ctx()) return;
  if (!h_a || !h_b || !h_c || m <= 0 || k <= 0 || n <= 0) {
    fml_fail(g_legacy, FML_ERR_INVALID, "multiplyMatrices: bad arguments");
    return;
  }
  // device buffers are cached between calls; rows are padded to a multiple of 4 floats so the
  // tensor-core path always applies
  const int64_t ldk = (k + 3) & ~3, ldn = (n + 3) & ~3;
  if (legacy_buf(&g_la, &g_lcap[0], (int64_t)m * ldk) || legacy_buf(&g_lb, &g_lcap[1], (int64_t)k * ldn) ||
      legacy_buf(&g_lc, &g_lcap[2], (int64_t)m * ldn))
    return;
  cudaStream_t st = g_legacy->stream;
  if (cudaMemcpy2DAsync(g_la, ldk * 4, h_a, (size_t)k * 4, (size_t)k * 4, m, cudaMemcpyHostToDevice, st) != cudaSuccess ||
      cudaMemcpy2DAsync(g_lb, ldn * 4, h_b, (size_t)n * 4, (size_t)n * 4, k, cudaMemcpyHostToDevice, st) != cudaSuccess) {
    fml_fail(g_legacy, FML_ERR_CUDA, "multiplyMatrices: host to device copy failed");
    return;
  }
  fml_gemm_desc d = {};
  d.M = m; d.N = n; d.K = k;
  d.lda = ldk; d.ldb = ldn; d.ldc = ldn;
  d.A = g_la; d.B = g_lb; d.C = g_lc;
  d.alpha = 1.f; d.batch1 = d.batch2 = 1; d.precision = -1;
  if (fml_gemm(g_legacy, &d)) return;
  if (cudaMemcpy2DAsync(h_c, (size_t)n * 4, g_lc, ldn * 4, (size_t)n * 4, m, cudaMemcpyDeviceToHost, st) != cudaSuccess ||
      cudaStreamSynchronize(st) != cudaSuccess)
    fml_fail(g_legacy, FML_ERR_CUDA, "multiplyMatrices: device to host copy failed");
}

int32_t benchtest(void) {
  // Same search as the reference (cuda_lib/kernel.cu:57-99): grow the square size by 100 until one
  // round trip exceeds 1000 ms; host buffers are zero-filled here (the reference leaves them
  // uninitialised, :69-71).  Capped so the host buffers stay below 3 x 1.6 GB.
  int last_ok = 0;
  for (int size = 100; size <= 20000; size += 100) {
    std::vector<float> a((size_t)size * size, 0.f), b((size_t)size * size, 0.f), c((size_t)size * size, 0.f);
    auto t0 = std::chrono::steady_clock::now();
    multiplyMatrices(a.data(), b.data(), c.data(), size, size, size);
    auto ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    if (ms > 1000.0) break;
    last_ok = size;
  }
  return last_ok;
}

}  // extern "C"
