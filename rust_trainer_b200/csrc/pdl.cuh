// Programmatic dependent launch: a kernel launched through pdl(...) may be scheduled while the
// kernel before it on the stream is still running; it must not touch global memory before
// pdl_wait(), which returns once that kernel has completed and its writes are visible.  What runs
// before the wait (barrier init, TMEM allocation, tensor-map prefetch, block scheduling itself)
// overlaps the predecessor's tail.  Rules kept by every kernel launched this way:
//   - every CTA executes pdl_wait() before its first global access and before any early return
//     (a grid counts as complete only when all of it has waited, so ordering stays transitive);
//   - pdl_launch_dependents() is called at entry: the next kernel may be scheduled as soon as
//     every CTA of this one has started.
// Inside stream capture these launches become programmatic edges of the graph.
// OFF by default: measured on the headline step (one graph replay of 1290 launches) it gained
// nothing (52.2 / 52.0 ms with, 51.8 / 51.7 ms without, alternating runs on one GPU): the heavy
// kernels fill every SM, so a successor's CTAs only start when a predecessor's CTA exits, and the
// graph's own kernel-to-kernel gaps are already short.  RT_B200_PDL=1 in the environment turns
// it on (the kernels carry the wait either way; without the launch attribute it returns at once).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>
#include <utility>

namespace rt {

__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// the usual entry sequence of a kernel that has no prologue worth overlapping
__device__ __forceinline__ void pdl_entry() {
  pdl_launch_dependents();
  pdl_wait();
}

inline bool pdl_enabled() {
  static int on = -1;
  if (on < 0) {
    const char* e = getenv("RT_B200_PDL");
    on = (e && atoi(e)) ? 1 : 0;
  }
  return on != 0;
}

template <typename... KArgs>
struct PdlLaunch {
  void (*kernel)(KArgs...);
  dim3 grid, block;
  size_t smem;
  cudaStream_t st;
  template <typename... A>
  cudaError_t operator()(A&&... a) const {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(std::forward<A>(a))...);
  }
};

// kernel<<<grid, block, smem, st>>>(args...)  becomes  pdl(kernel, grid, block, smem, st)(args...)
template <typename... KArgs>
inline PdlLaunch<KArgs...> pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st) {
  return PdlLaunch<KArgs...>{kernel, grid, block, smem, st};
}

}  // namespace rt
