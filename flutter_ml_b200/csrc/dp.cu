// Data-parallel gradient exchange: one process per GPU, NCCL over NVLink.  NCCL is resolved at
// run time with dlopen so the library itself has no link-time dependency on it (the process may
// already have loaded a copy, e.g. the one bundled with PyTorch; dlopen then returns that one).
// <nccl.h> supplies types and constants only.
//
// Failure detection on the host: the communicator is created NON-BLOCKING, so neither its creation
// nor a collective can park the calling thread inside NCCL.  Every call polls
// ncclCommGetAsyncError against a deadline; when the deadline passes (a peer that never joined,
// a peer that died between steps) the communicator is aborted and the call returns
// FML_ERR_TIMEOUT, after which fml_dp_init may be called again with a new id.
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

#include <chrono>
#include <thread>

#include "common.cuh"

namespace {

typedef ncclResult_t (*GetUniqueIdFn)(ncclUniqueId*);
typedef ncclResult_t (*CommInitRankConfigFn)(ncclComm_t*, int, ncclUniqueId, int, ncclConfig_t*);
typedef ncclResult_t (*AllReduceFn)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
typedef ncclResult_t (*CommFn)(ncclComm_t);
typedef ncclResult_t (*AsyncErrorFn)(ncclComm_t, ncclResult_t*);
typedef const char* (*GetErrorStringFn)(ncclResult_t);

struct NcclApi {
  void* handle = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankConfigFn comm_init_rank_config = nullptr;
  AllReduceFn all_reduce = nullptr;
  CommFn comm_destroy = nullptr;
  CommFn comm_abort = nullptr;
  CommFn comm_finalize = nullptr;
  AsyncErrorFn async_error = nullptr;
  GetErrorStringFn error_string = nullptr;
};

NcclApi* nccl() {
  static NcclApi api;
  static std::once_flag once;
  std::call_once(once, [] {
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (api.handle) {
      api.get_unique_id = (GetUniqueIdFn)dlsym(api.handle, "ncclGetUniqueId");
      api.comm_init_rank_config = (CommInitRankConfigFn)dlsym(api.handle, "ncclCommInitRankConfig");
      api.all_reduce = (AllReduceFn)dlsym(api.handle, "ncclAllReduce");
      api.comm_destroy = (CommFn)dlsym(api.handle, "ncclCommDestroy");
      api.comm_abort = (CommFn)dlsym(api.handle, "ncclCommAbort");
      api.comm_finalize = (CommFn)dlsym(api.handle, "ncclCommFinalize");
      api.async_error = (AsyncErrorFn)dlsym(api.handle, "ncclCommGetAsyncError");
      api.error_string = (GetErrorStringFn)dlsym(api.handle, "ncclGetErrorString");
    }
  });
  if (!api.handle || !api.get_unique_id || !api.comm_init_rank_config || !api.all_reduce || !api.comm_destroy ||
      !api.comm_abort || !api.async_error)
    return nullptr;
  return &api;
}

int32_t nccl_fail(fml_ctx* ctx, const char* what, int code) {
  NcclApi* a = nccl();
  std::string msg = std::string(what) + " failed";
  if (a && a->error_string) msg += std::string(": ") + a->error_string((ncclResult_t)code);
  return fml_fail(ctx, FML_ERR_NCCL, msg);
}

void abort_comm(fml_ctx* ctx) {
  NcclApi* a = nccl();
  if (a && ctx->nccl_comm) a->comm_abort((ncclComm_t)ctx->nccl_comm);
  ctx->nccl_comm = nullptr;
  ctx->dp_world = 1;
  ctx->dp_rank = 0;
}

// Waits until the communicator has left ncclInProgress (the last non-blocking call is complete on the host side:
// the communicator exists, or the collective is enqueued on its stream).  Past the deadline, or on an asynchronous
// error, the communicator is aborted.
int32_t settle(fml_ctx* ctx, const char* what) {
  NcclApi* a = nccl();
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(ctx->dp_timeout_ms);
  int spins = 0;
  for (;;) {
    ncclResult_t state = ncclSuccess;
    ncclResult_t rc = a->async_error((ncclComm_t)ctx->nccl_comm, &state);
    if (rc != ncclSuccess) { abort_comm(ctx); return nccl_fail(ctx, "ncclCommGetAsyncError", rc); }
    if (state == ncclSuccess) return FML_OK;
    if (state != ncclInProgress) { abort_comm(ctx); return nccl_fail(ctx, what, state); }
    if (std::chrono::steady_clock::now() > deadline) {
      abort_comm(ctx);
      return fml_fail(ctx, FML_ERR_TIMEOUT, std::string(what) + ": no progress within " + std::to_string(ctx->dp_timeout_ms) +
                                                " ms (a peer did not arrive); the communicator was aborted");
    }
    if (++spins < 2000) std::this_thread::yield();
    else std::this_thread::sleep_for(std::chrono::microseconds(200));
  }
}

}  // namespace

extern "C" {

int32_t fml_dp_unique_id(uint8_t out[128]) {
  NcclApi* a = nccl();
  if (!a) return fml_fail(nullptr, FML_ERR_NCCL, "libnccl.so.2 could not be loaded");
  static_assert(sizeof(ncclUniqueId) == 128, "the id travels as 128 bytes");
  ncclUniqueId id;
  ncclResult_t rc = a->get_unique_id(&id);
  if (rc) return nccl_fail(nullptr, "ncclGetUniqueId", rc);
  memcpy(out, id.internal, 128);
  return FML_OK;
}

int32_t fml_dp_set_timeout(fml_ctx* ctx, int32_t timeout_ms) {
  FML_REQUIRE(ctx, ctx && timeout_ms > 0, "fml_dp_set_timeout: the limit must be positive");
  ctx->dp_timeout_ms = timeout_ms;
  return FML_OK;
}

int32_t fml_dp_set_max_ctas(fml_ctx* ctx, int32_t ctas) {
  FML_REQUIRE(ctx, ctx && ctas >= 0 && ctas <= 64, "fml_dp_set_max_ctas: 0 (NCCL's choice) .. 64");
  FML_REQUIRE(ctx, !ctx->nccl_comm, "fml_dp_set_max_ctas: call it before fml_dp_init");
  ctx->dp_max_ctas = ctas;
  return FML_OK;
}

int32_t fml_dp_init(fml_ctx* ctx, const uint8_t id_bytes[128], int32_t rank, int32_t world) {
  FML_ENTER(ctx);
  FML_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world, "fml_dp_init: bad rank/world");
  FML_REQUIRE(ctx, !ctx->nccl_comm, "fml_dp_init: a communicator already exists (fml_dp_shutdown first)");
  ctx->dp_rank = rank;
  ctx->dp_world = world;
  if (world == 1) return FML_OK;  // nothing to exchange
  NcclApi* a = nccl();
  if (!a) return fml_fail(ctx, FML_ERR_NCCL, "libnccl.so.2 could not be loaded");
  ncclUniqueId id;
  memcpy(id.internal, id_bytes, 128);
  ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
  cfg.blocking = 0;
  if (ctx->dp_max_ctas > 0) {
    // Keep the collective to the SMs set aside for it, and do not group its CTAs into clusters: a cluster needs all of
    // its SMs free inside ONE GPC at the same moment, which a persistent product spread over the machine never leaves.
    cfg.maxCTAs = ctx->dp_max_ctas;
    cfg.cgaClusterSize = 0;
  }
  ncclComm_t comm = nullptr;
  ncclResult_t rc = a->comm_init_rank_config(&comm, world, id, rank, &cfg);
  ctx->nccl_comm = comm;
  if (rc != ncclSuccess && rc != ncclInProgress) {
    if (comm) abort_comm(ctx);
    ctx->dp_world = 1; ctx->dp_rank = 0;
    return nccl_fail(ctx, "ncclCommInitRankConfig", rc);
  }
  return settle(ctx, "fml_dp_init (ncclCommInitRankConfig)");
}

int32_t fml_dp_allreduce_sum_on(fml_ctx* ctx, int32_t lane, float* buf, int64_t n) {
  FML_ENTER(ctx);
  if (ctx->dp_world == 1) return FML_OK;
  FML_REQUIRE(ctx, ctx->nccl_comm, "fml_dp_allreduce_sum: fml_dp_init has not been called");
  cudaStream_t s;
  int32_t rc0 = fml_any_stream(ctx, lane, &s);
  if (rc0) return rc0;
  NcclApi* a = nccl();
  ncclResult_t rc = a->all_reduce(buf, buf, (size_t)n, ncclFloat32, ncclSum, (ncclComm_t)ctx->nccl_comm, s);
  if (rc != ncclSuccess && rc != ncclInProgress) { abort_comm(ctx); return nccl_fail(ctx, "ncclAllReduce", rc); }
  // the collective is ordered on `s` only once the communicator reports it enqueued
  return settle(ctx, "fml_dp_allreduce_sum (ncclAllReduce)");
}

int32_t fml_dp_allreduce_sum(fml_ctx* ctx, float* buf, int64_t n) {
  FML_ENTER(ctx);
  return fml_dp_allreduce_sum_on(ctx, -1, buf, n);
}

int32_t fml_dp_shutdown(fml_ctx* ctx) {
  FML_ENTER(ctx);
  if (ctx->nccl_comm) {
    NcclApi* a = nccl();
    if (a) {
      // a non-blocking communicator is finalised first (flushes what was issued), polled until that has happened
      // (settle aborts it instead when the limit passes), then destroyed
      bool alive = true;
      if (a->comm_finalize) {
        ncclResult_t rc = a->comm_finalize((ncclComm_t)ctx->nccl_comm);
        if (rc == ncclSuccess || rc == ncclInProgress) alive = settle(ctx, "fml_dp_shutdown (ncclCommFinalize)") == FML_OK;
      }
      if (alive && ctx->nccl_comm) a->comm_destroy((ncclComm_t)ctx->nccl_comm);
    }
    ctx->nccl_comm = nullptr;
  }
  ctx->dp_world = 1;
  ctx->dp_rank = 0;
  return FML_OK;
}

}  // extern "C"
