// Kernel launch helper: every kernel of the library is launched through arcb_launch(), which adds the
// programmatic-stream-serialization attribute when programmatic dependent launch is enabled.
//
// Protocol inside the kernels (common.cuh): pdl_launch_dependents() at entry lets the NEXT kernel in
// the stream (or captured graph) be scheduled as soon as every block of this one is resident, so its
// launch latency and its prologue (barrier initialisation, tensor-memory allocation, descriptor
// prefetch) overlap this kernel's tail; pdl_wait() returns only when the PREVIOUS kernel has
// completed and its writes are visible, and every kernel calls it before its first access to global
// memory other than its own parameters.  Because a grid completes only after the blocks that did its
// work have passed their own wait, completion is transitive along the stream: passing the wait on
// kernel N-1 implies kernels N-2, N-3, ... have completed too.
#pragma once
#include <cuda_runtime.h>

#include <utility>

bool arcb_pdl_enabled();
void arcb_pdl_set(bool on);
// Launches made by this thread while suppressed carry no programmatic attribute (used around the
// event-record nodes of the decode graph: a programmatic edge must join two kernel nodes).
void arcb_pdl_suppress(bool on);
bool arcb_pdl_suppressed();

template <typename... KArgs, typename... Args>
inline cudaError_t arcb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                               Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  const bool pdl = arcb_pdl_enabled() && !arcb_pdl_suppressed();
  cfg.attrs = pdl ? attr : nullptr;
  cfg.numAttrs = pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
  if (e != cudaSuccess) cudaGetLastError();   // reported through the return value; do not leave it for the next API call
  return e;
}
