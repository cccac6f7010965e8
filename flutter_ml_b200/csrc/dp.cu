// Data-parallel gradient exchange: one process per GPU, NCCL over NVLink.  NCCL is resolved at
// run time with dlopen so the library itself has no link-time dependency on it (the process may
// already have loaded a copy, e.g. the one bundled with PyTorch; dlopen then returns that one).
#include <dlfcn.h>
#include <string.h>

#include "common.cuh"

namespace {

struct NcclUniqueId { char internal[128]; };
typedef int (*GetUniqueIdFn)(NcclUniqueId*);
typedef int (*CommInitRankFn)(void**, int, NcclUniqueId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*CommDestroyFn)(void*);
typedef const char* (*GetErrorStringFn)(int);

struct NcclApi {
  void* handle = nullptr;
  GetUniqueIdFn get_unique_id = nullptr;
  CommInitRankFn comm_init_rank = nullptr;
  AllReduceFn all_reduce = nullptr;
  CommDestroyFn comm_destroy = nullptr;
  GetErrorStringFn error_string = nullptr;
};

NcclApi* nccl() {
  static NcclApi api;
  static bool tried = false;
  if (!tried) {
    tried = true;
    for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
      api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
      if (api.handle) break;
    }
    if (api.handle) {
      api.get_unique_id = (GetUniqueIdFn)dlsym(api.handle, "ncclGetUniqueId");
      api.comm_init_rank = (CommInitRankFn)dlsym(api.handle, "ncclCommInitRank");
      api.all_reduce = (AllReduceFn)dlsym(api.handle, "ncclAllReduce");
      api.comm_destroy = (CommDestroyFn)dlsym(api.handle, "ncclCommDestroy");
      api.error_string = (GetErrorStringFn)dlsym(api.handle, "ncclGetErrorString");
    }
  }
  if (!api.handle || !api.get_unique_id || !api.comm_init_rank || !api.all_reduce || !api.comm_destroy) return nullptr;
  return &api;
}

int32_t nccl_fail(fml_ctx* ctx, const char* what, int code) {
  NcclApi* a = nccl();
  std::string msg = std::string(what) + " failed";
  if (a && a->error_string) msg += std::string(": ") + a->error_string(code);
  return fml_fail(ctx, FML_ERR_NCCL, msg);
}

}  // namespace

extern "C" {

int32_t fml_dp_unique_id(uint8_t out[128]) {
  NcclApi* a = nccl();
  if (!a) return fml_fail(nullptr, FML_ERR_NCCL, "libnccl.so.2 could not be loaded");
  NcclUniqueId id;
  int rc = a->get_unique_id(&id);
  if (rc) return nccl_fail(nullptr, "ncclGetUniqueId", rc);
  memcpy(out, id.internal, 128);
  return FML_OK;
}

int32_t fml_dp_init(fml_ctx* ctx, const uint8_t id_bytes[128], int32_t rank, int32_t world) {
  FML_REQUIRE(ctx, world >= 1 && rank >= 0 && rank < world, "fml_dp_init: bad rank/world");
  ctx->dp_rank = rank;
  ctx->dp_world = world;
  if (world == 1) return FML_OK;  // nothing to exchange
  NcclApi* a = nccl();
  if (!a) return fml_fail(ctx, FML_ERR_NCCL, "libnccl.so.2 could not be loaded");
  FML_CUDA(ctx, cudaSetDevice(ctx->device));
  NcclUniqueId id;
  memcpy(id.internal, id_bytes, 128);
  int rc = a->comm_init_rank(&ctx->nccl_comm, world, id, rank);
  if (rc) return nccl_fail(ctx, "ncclCommInitRank", rc);
  return FML_OK;
}

int32_t fml_dp_allreduce_sum_on(fml_ctx* ctx, int32_t lane, float* buf, int64_t n) {
  if (ctx->dp_world == 1) return FML_OK;
  FML_REQUIRE(ctx, ctx->nccl_comm, "fml_dp_allreduce_sum: fml_dp_init has not been called");
  cudaStream_t s;
  int32_t rc0 = fml_any_stream(ctx, lane, &s);
  if (rc0) return rc0;
  NcclApi* a = nccl();
  int rc = a->all_reduce(buf, buf, (size_t)n, /*ncclFloat32*/ 7, /*ncclSum*/ 0, ctx->nccl_comm, s);
  if (rc) return nccl_fail(ctx, "ncclAllReduce", rc);
  return FML_OK;
}

int32_t fml_dp_allreduce_sum(fml_ctx* ctx, float* buf, int64_t n) { return fml_dp_allreduce_sum_on(ctx, -1, buf, n); }

int32_t fml_dp_shutdown(fml_ctx* ctx) {
  if (ctx->nccl_comm) {
    NcclApi* a = nccl();
    if (a) a->comm_destroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
  }
  ctx->dp_world = 1;
  ctx->dp_rank = 0;
  return FML_OK;
}

}  // extern "C"
