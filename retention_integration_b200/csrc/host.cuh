// Host-side helpers shared by every entry point of the C ABI: error strings,
// CUDA error checks, the per-device status word that kernels write when a
// bounded wait runs out, and TMA tensor-map encoding through the driver entry
// point (no link-time dependency on libcuda).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>

#include "../../include/pr_b200.h"

namespace pr {

inline char* err_buf() {
  static thread_local char buf[512] = {0};
  return buf;
}
inline int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(err_buf(), 512, fmt, ap);
  va_end(ap);
  return code;
}

#define PR_CUDA(expr)                                                                          \
  do {                                                                                         \
    cudaError_t e__ = (expr);                                                                  \
    if (e__ != cudaSuccess)                                                                    \
      return ::pr::fail(PR_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__), \
                        __FILE__, __LINE__);                                                   \
  } while (0)

#define PR_REQUIRE(cond, code, ...) \
  do {                              \
    if (!(cond)) return ::pr::fail(code, __VA_ARGS__); \
  } while (0)

// Per-device status word in mapped pinned host memory.  Kernels write a non-zero
// value only on failure, so the fast path costs nothing.
int status_word(int device, int** dev_ptr, volatile int** host_ptr);

// 2-D..4-D tiled tensor map with 128-byte swizzle (or none).  dims/strides are
// innermost first; strides[0] is implied (elem size) and strides[i] are bytes.
int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128);

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Dynamic shared memory of a kernel: the attribute is raised once per kernel and device (and again only when a
// later launch needs more), not on every launch.  The record is kept per kernel function, not per call site: a
// second site that set a smaller size for the same kernel would lower the limit under the first one's launches.
// `carveout`: also ask for the largest shared-memory partition.
int smem_attr(const void* kernel, size_t bytes, int device, bool carveout);
#define PR_SMEM_ATTR(kernel, bytes, device, carveout)                                                    \
  do {                                                                                                   \
    int rc_ = ::pr::smem_attr(reinterpret_cast<const void*>(kernel), (bytes), (device), (carveout));     \
    if (rc_) return rc_;                                                                                 \
  } while (0)

// 0 when the environment variable PR_PDL=0 asks for plain stream order (read once).
bool pdl_enabled();

// Kernel launch with programmatic stream serialisation allowed (see pdl_wait() in sm100.cuh): the
// kernel may start while its predecessor in the stream drains and blocks at its own
// griddepcontrol.wait.  Stream capture records the edge as a programmatic dependency.
template <typename... KArgs, typename... Args>
cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace pr
