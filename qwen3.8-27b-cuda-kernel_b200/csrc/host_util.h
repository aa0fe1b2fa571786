// Host-side helpers of the launchers: argument checks that produce a status + message instead of an
// exception (the C ABI cannot throw), the cached SM count, and one-time kernel attribute set-up.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/q38_kernels.h"

namespace q38 {

void set_error(const char* fmt, ...);  // defined in c_abi.cu
int num_sms();                         // SM count of the device current at first use (one device per process)
int max_optin_smem();

#define Q38_REQUIRE(cond, ...)            \
  do {                                    \
    if (!(cond)) {                        \
      ::q38::set_error(__VA_ARGS__);      \
      return Q38_ERR_INVALID;             \
    }                                     \
  } while (0)

#define Q38_CUDA_OK(expr)                                                                   \
  do {                                                                                      \
    const cudaError_t err__ = (expr);                                                       \
    if (err__ != cudaSuccess) {                                                             \
      ::q38::set_error("%s failed: %s", #expr, cudaGetErrorString(err__));                  \
      return Q38_ERR_CUDA;                                                                  \
    }                                                                                       \
  } while (0)

// Launch check that is legal during stream capture (reads the launch status only).
#define Q38_LAUNCH_OK(name)                                                                 \
  do {                                                                                      \
    const cudaError_t err__ = cudaPeekAtLastError();                                        \
    if (err__ != cudaSuccess) {                                                             \
      ::q38::set_error("launch of %s failed: %s", name, cudaGetErrorString(err__));         \
      (void)cudaGetLastError();                                                             \
      return Q38_ERR_CUDA;                                                                  \
    }                                                                                       \
  } while (0)

inline cudaStream_t as_stream(void* s) { return static_cast<cudaStream_t>(s); }

// Every kernel of the library is launched through this helper. With programmatic dependent launch allowed (the
// default, q38_set_dependent_launch) a kernel may be scheduled while its predecessor in the stream is still
// draining: its prologue (barrier set-up, TMEM allocation, prefetch of weights, which no kernel writes) overlaps
// the predecessor's tail, and griddepcontrol.wait inside the kernel holds back everything that touches data the
// predecessor produces. The attribute is recorded as a programmatic edge when the stream is being captured.
bool dependent_launch_allowed();  // defined in c_abi.cu
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = dependent_launch_allowed() ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

}  // namespace q38
