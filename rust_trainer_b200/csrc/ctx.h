// Per-GPU context and the opaque handle types behind the C ABI.
#pragma once
#include "qformat.cuh"
#include "rt_internal.h"
#include <map>
#include <string>
#include <tuple>
#include <vector>

struct rt_ctx {
  int device = 0;
  int num_sms = 0;
  cudaStream_t stream = nullptr;       // the stream in use (own_stream unless the host set one)
  cudaStream_t own_stream = nullptr;
  int* status_dev = nullptr;   // device word the kernels report bounded-wait failures into
  int* status_host = nullptr;  // pinned mirror
  std::string err;
  uint64_t launches = 0;       // kernels launched through this ctx
  bool profiling = false;
  std::vector<cudaEvent_t> prof_events;  // start/stop pairs of profiled matmul launches
  size_t prof_used = 0;
  double prof_flops = 0, prof_bytes = 0;
  // encoded TMA descriptors, keyed by (base, rows, cols, box, type): the same buffers recur every layer
  std::map<std::tuple<const void*, uint64_t, uint64_t, uint32_t, uint32_t, bool>, CUtensorMap> tmap_cache;
  struct ProfRec { int cls, M, rows, contract; };  // cls: 0 fwd, 1 bwd, 2 skinny LoRA helper, 3 token contraction
  std::vector<ProfRec> prof_recs;
  // data-parallel communicator (an ncclComm_t once rt_comm_init_rank has run; a world of one otherwise)
  void* comm = nullptr;
  int comm_ranks = 1, comm_rank = 0;
  // grow-only scratch buffers for the host-pointer entry points
  void* scratch[4] = {nullptr, nullptr, nullptr, nullptr};
  size_t scratch_bytes[4] = {0, 0, 0, 0};

  rt_status fail(rt_status code, const std::string& msg) {
    err = msg;
    return code;
  }
  rt_status cuda_fail(cudaError_t e, const char* where) {
    err = std::string(where) + ": " + cudaGetErrorString(e);
    return RT_ERR_CUDA;
  }
  void* get_scratch(int slot, size_t bytes);
  // Reads the device status word (after synchronising); maps non-zero to an error.
  rt_status check_device_status(const char* where);
};

#define RT_CUDA(ctx, call)                                        \
  do {                                                            \
    cudaError_t e__ = (call);                                     \
    if (e__ != cudaSuccess) return (ctx)->cuda_fail(e__, #call);  \
  } while (0)

namespace rt {
// Handles outlive their context when a host tears things down out of order (a garbage collector
// does).  Destroy functions ask before they touch the context.
bool ctx_alive(const rt_ctx* c);
}

struct rt_frozen {
  rt_ctx* ctx = nullptr;
  int device = 0;
  rt::QWeight w;
  bool borrowed = false;  // the weight bytes live in a buffer another object owns (a stacked group of linears)
};

#include "ops.h"
