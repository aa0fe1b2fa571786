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

}  // namespace q38
