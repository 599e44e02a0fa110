// Data-parallel exchange behind the C ABI: one NCCL communicator per ctx and ONE all-reduce
// (sum) of the flat LoRA-gradient buffer per optimiser step.  The reference has no counterpart
// (one process, one device: src/train.rs:339-351 accumulates the batch's examples in turn); the
// sum over ranks takes the place of that accumulation, so every rank weights its targets with the
// GLOBAL 1/batch_tokens (src/train.rs:330) and runs the same clip + AdamW afterwards.
//
// libnccl is opened at first use (dlopen), not linked: a single-GPU host needs no NCCL at all,
// and a process that already holds an NCCL (torch's) shares that copy instead of loading a second.
#include "model.h"
#include <dlfcn.h>
#include <nccl.h>
#include <string.h>

namespace {

struct NcclApi {
  void* handle = nullptr;
  ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
  ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
  ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
  ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
  const char* (*GetErrorString)(ncclResult_t) = nullptr;
  bool ok = false;
};

NcclApi& nccl() {
  static NcclApi api;
  static bool tried = false;
  if (tried) return api;
  tried = true;
  for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
    api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
    if (api.handle) break;
  }
  if (!api.handle) return api;
  api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(api.handle, "ncclGetUniqueId");
  api.CommInitRank = (decltype(api.CommInitRank))dlsym(api.handle, "ncclCommInitRank");
  api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
  api.AllReduce = (decltype(api.AllReduce))dlsym(api.handle, "ncclAllReduce");
  api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
  api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllReduce && api.GetErrorString;
  return api;
}

rt_status nccl_fail(rt_ctx* c, ncclResult_t r, const char* where) {
  return c->fail(RT_ERR_NCCL, std::string(where) + ": " + nccl().GetErrorString(r));
}

}  // namespace

extern "C" {

rt_status rt_comm_unique_id(uint8_t* id_out, size_t id_bytes) {
  if (!id_out || id_bytes != RT_COMM_ID_BYTES) return RT_ERR_BAD_ARG;
  static_assert(RT_COMM_ID_BYTES == NCCL_UNIQUE_ID_BYTES, "id size");
  if (!nccl().ok) return RT_ERR_NCCL;
  ncclUniqueId id;
  if (nccl().GetUniqueId(&id) != ncclSuccess) return RT_ERR_NCCL;
  memcpy(id_out, id.internal, RT_COMM_ID_BYTES);
  return RT_OK;
}

rt_status rt_comm_init_rank(rt_ctx* c, int nranks, int rank, const uint8_t* id, size_t id_bytes) {
  if (!c || !id || id_bytes != RT_COMM_ID_BYTES) return RT_ERR_BAD_ARG;
  if (nranks < 1 || rank < 0 || rank >= nranks) return c->fail(RT_ERR_BAD_ARG, "rank outside the world");
  if (c->comm) return c->fail(RT_ERR_BAD_ARG, "the context already has a communicator");
  if (!nccl().ok) return c->fail(RT_ERR_NCCL, "libnccl.so.2 not found or incomplete");
  RT_CUDA(c, cudaSetDevice(c->device));
  ncclUniqueId uid;
  memcpy(uid.internal, id, RT_COMM_ID_BYTES);
  ncclComm_t comm = nullptr;
  ncclResult_t r = nccl().CommInitRank(&comm, nranks, uid, rank);
  if (r != ncclSuccess) return nccl_fail(c, r, "ncclCommInitRank");
  c->comm = comm;
  c->comm_ranks = nranks;
  c->comm_rank = rank;
  return RT_OK;
}

rt_status rt_comm_destroy(rt_ctx* c) {
  if (!c) return RT_ERR_BAD_ARG;
  if (!c->comm) return RT_OK;
  cudaSetDevice(c->device);
  cudaStreamSynchronize(c->stream);
  ncclResult_t r = nccl().CommDestroy((ncclComm_t)c->comm);
  c->comm = nullptr;
  c->comm_ranks = 1;
  c->comm_rank = 0;
  return r == ncclSuccess ? RT_OK : nccl_fail(c, r, "ncclCommDestroy");
}

int rt_comm_size(const rt_ctx* c) { return c ? c->comm_ranks : 0; }
int rt_comm_rank(const rt_ctx* c) { return c ? c->comm_rank : 0; }

rt_status rt_comm_allreduce_f32(rt_ctx* c, float* buf_dev, size_t n) {
  if (!c || (!buf_dev && n)) return RT_ERR_BAD_ARG;
  if (!c->comm || n == 0) return RT_OK;  // a world of one: the sum over ranks is the buffer itself
  RT_CUDA(c, cudaSetDevice(c->device));
  ncclResult_t r = nccl().AllReduce(buf_dev, buf_dev, n, ncclFloat, ncclSum, (ncclComm_t)c->comm, c->stream);
  if (r != ncclSuccess) return nccl_fail(c, r, "ncclAllReduce");
  RT_COUNT_LAUNCH(1);
  return RT_OK;
}

rt_status rt_model_allreduce_grads(rt_model* m) {
  if (!m) return RT_ERR_BAD_ARG;
  if (m->n_params == 0) return m->ctx->fail(RT_ERR_BAD_ARG, "no adapters attached");
  return rt_comm_allreduce_f32(m->ctx, m->G.as<float>(), m->n_params);
}

}  // extern "C"
