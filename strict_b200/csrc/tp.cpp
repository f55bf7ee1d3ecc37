// Tensor-parallel plumbing: NCCL over NVLink, bound at run time with dlopen so the library
// loads (and the single-GPU path runs) on machines without NCCL, and so that it shares the
// NCCL already loaded by the host process when there is one.
#include <dlfcn.h>

#include <cstring>

#include "common.cuh"

namespace {
typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
enum { NCCL_INT8 = 0, NCCL_FLOAT32 = 7, NCCL_SUM = 0 };
struct Nccl {
  void* lib = nullptr;
  int (*GetUniqueId)(nccl_uid*) = nullptr;
  int (*CommInitRank)(nccl_comm*, int, nccl_uid, int) = nullptr;
  int (*AllReduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t) = nullptr;
  int (*AllGather)(const void*, void*, size_t, int, nccl_comm, cudaStream_t) = nullptr;
  int (*CommDestroy)(nccl_comm) = nullptr;
  const char* (*GetErrorString)(int) = nullptr;
};
Nccl g_nccl;

int load_nccl() {
  if (g_nccl.lib) return STRICTB200_OK;
  void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
  if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
  if (!h) return sb_fail(STRICTB200_ERR_NCCL, std::string("cannot load libnccl.so.2: ") + dlerror());
#define SYM(field, name)                                                                       \
  *(void**)(&g_nccl.field) = dlsym(h, name);                                                   \
  if (!g_nccl.field) return sb_fail(STRICTB200_ERR_NCCL, std::string("libnccl lacks ") + name);
  SYM(GetUniqueId, "ncclGetUniqueId")
  SYM(CommInitRank, "ncclCommInitRank")
  SYM(AllReduce, "ncclAllReduce")
  SYM(AllGather, "ncclAllGather")
  SYM(CommDestroy, "ncclCommDestroy")
  SYM(GetErrorString, "ncclGetErrorString")
#undef SYM
  g_nccl.lib = h;
  return STRICTB200_OK;
}
int nccl_fail(const char* what, int rc) {
  return sb_fail(STRICTB200_ERR_NCCL, std::string(what) + ": " + (g_nccl.GetErrorString ? g_nccl.GetErrorString(rc) : "?"));
}
}  // namespace

struct TpState {
  nccl_comm comm = nullptr;
};

int sb_tp_allreduce_f32(strictb200_ctx* ctx, float* buf, int64_t count) {
  if (ctx->tp_world == 1) return STRICTB200_OK;
  int rc = g_nccl.AllReduce(buf, buf, (size_t)count, NCCL_FLOAT32, NCCL_SUM, ctx->tp->comm, ctx->stream);
  if (rc) return nccl_fail("ncclAllReduce", rc);
  return STRICTB200_OK;
}
int sb_tp_allgather(strictb200_ctx* ctx, const void* send, void* recv, int64_t bytes_per_rank) {
  if (ctx->tp_world == 1) {
    if (send != recv) SB_CUDA(cudaMemcpyAsync(recv, send, (size_t)bytes_per_rank, cudaMemcpyDeviceToDevice, ctx->stream));
    return STRICTB200_OK;
  }
  int rc = g_nccl.AllGather(send, recv, (size_t)bytes_per_rank, NCCL_INT8, ctx->tp->comm, ctx->stream);
  if (rc) return nccl_fail("ncclAllGather", rc);
  return STRICTB200_OK;
}
void sb_tp_destroy(strictb200_ctx* ctx) {
  if (ctx->tp) {
    if (ctx->tp->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(ctx->tp->comm);
    delete ctx->tp;
    ctx->tp = nullptr;
  }
}

extern "C" {
int strictb200_tp_unique_id(void* h_id128) {
  if (!h_id128) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null id buffer");
  SB_TRY(load_nccl());
  nccl_uid id;
  int rc = g_nccl.GetUniqueId(&id);
  if (rc) return nccl_fail("ncclGetUniqueId", rc);
  memcpy(h_id128, &id, 128);
  return STRICTB200_OK;
}
int strictb200_tp_init(strictb200_ctx* ctx, int world, int rank, const void* h_id128) {
  SB_ENTER(ctx);
  SB_REQUIRE(world == 1 || world == 2 || world == 4 || world == 8, "world must be 1, 2, 4 or 8");
  SB_REQUIRE(rank >= 0 && rank < world, "rank out of range");
  SB_REQUIRE(!ctx->tp, "tensor parallelism already initialised on this context");
  if (world == 1) return STRICTB200_OK;
  SB_REQUIRE(h_id128, "null id buffer");
  SB_TRY(load_nccl());
  nccl_uid id;
  memcpy(&id, h_id128, 128);
  TpState* tp = new TpState;
  int rc = g_nccl.CommInitRank(&tp->comm, world, id, rank);
  if (rc) {
    delete tp;
    return nccl_fail("ncclCommInitRank", rc);
  }
  ctx->tp = tp;
  ctx->tp_world = world;
  ctx->tp_rank = rank;
  return STRICTB200_OK;
}
int strictb200_tp_info(strictb200_ctx* ctx, int* world, int* rank) {
  if (!ctx) return sb_fail(STRICTB200_ERR_INVALID_ARG, "null context");
  if (world) *world = ctx->tp_world;
  if (rank) *rank = ctx->tp_rank;
  return STRICTB200_OK;
}
int strictb200_tp_allreduce_f32(strictb200_ctx* ctx, float* d_buf, int64_t count) {
  SB_ENTER(ctx);
  SB_REQUIRE(count >= 0, "negative count");
  if (!count) return STRICTB200_OK;
  SB_REQUIRE(d_buf, "null pointer");
  return sb_tp_allreduce_f32(ctx, d_buf, count);
}
}
