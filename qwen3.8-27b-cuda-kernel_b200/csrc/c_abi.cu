// Library-wide pieces of the C ABI: error reporting, device properties, layout helpers.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "host_util.h"

namespace q38 {

namespace {
thread_local char g_error[512] = "";
}

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}

namespace {
struct DeviceProps {
  int sms = 0;
  int smem_optin = 0;
  DeviceProps() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    cudaDeviceGetAttribute(&smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
  }
};
const DeviceProps& props() {
  static const DeviceProps p;
  return p;
}
}  // namespace

namespace {
bool g_dependent_launch = true;
}
bool dependent_launch_allowed() { return g_dependent_launch; }

int num_sms() { return props().sms > 0 ? props().sms : 1; }
int max_optin_smem() { return props().smem_optin; }

// per-translation-unit device error words
unsigned int qgemm_stream_error(bool clear);
unsigned int qgemm_dispatch_error(bool clear);
unsigned int qgemm_umma_error(bool clear);
unsigned int attention_error(bool clear);
unsigned int gdn_error(bool clear);
unsigned int misc_error(bool clear);

unsigned int* qgemm_stream_error_address();
unsigned int* qgemm_dispatch_error_address();
unsigned int* qgemm_umma_error_address();
unsigned int* attention_error_address();
unsigned int* gdn_error_address();
unsigned int* misc_error_address();

namespace {
constexpr int kErrorWords = 6;
struct ErrorWords {
  unsigned int* word[kErrorWords];
};

// Moves the first non-zero error word of the library into *dst and clears the words; *dst is left alone when no
// kernel reported anything, so a host that polls it sees the first failure until it clears the word itself.
__global__ void collect_errors_kernel(ErrorWords w, unsigned int* dst) {
  pdl_wait();
  pdl_launch_dependents();
  unsigned int first = 0;
  for (int i = 0; i < kErrorWords; ++i) {
    const unsigned int v = atomicExch(w.word[i], 0u);
    if (first == 0) first = v;
  }
  if (first != 0) {
    *dst = first;
    __threadfence_system();
  }
}

constexpr int kMaxErrorDevices = 64;
struct ErrorWordCache {
  std::once_flag once;
  ErrorWords words{};
  bool ok = false;
};
ErrorWordCache g_error_words[kMaxErrorDevices];
}  // namespace

}  // namespace q38

extern "C" const char* q38_last_error(void) { return q38::g_error; }

extern "C" int q38_device_error_collect(unsigned int* dst, void* stream) {
  using namespace q38;
  Q38_REQUIRE(dst != nullptr, "device_error_collect: null destination");
  int dev = 0;
  Q38_CUDA_OK(cudaGetDevice(&dev));
  Q38_REQUIRE(dev >= 0 && dev < kMaxErrorDevices, "device_error_collect: device index %d out of range", dev);
  ErrorWordCache& c = g_error_words[dev];
  std::call_once(c.once, [&c] {  // with this device current; the first call must come before any stream capture
    unsigned int* p[kErrorWords] = {qgemm_stream_error_address(), qgemm_dispatch_error_address(),
                                    qgemm_umma_error_address(),   attention_error_address(),
                                    gdn_error_address(),          misc_error_address()};
    c.ok = true;
    for (int i = 0; i < kErrorWords; ++i) {
      c.words.word[i] = p[i];
      c.ok = c.ok && p[i] != nullptr;
    }
  });
  Q38_REQUIRE(c.ok, "device_error_collect: the error words of the library could not be located");
  (void)launch_kernel(collect_errors_kernel, dim3(1), dim3(1), 0, as_stream(stream), c.words, dst);
  Q38_LAUNCH_OK("collect_errors_kernel");
  return Q38_OK;
}

extern "C" int q38_device_error_inject(unsigned int code) {
  using namespace q38;
  unsigned int* word = misc_error_address();
  Q38_REQUIRE(word != nullptr, "device_error_inject: error word not found");
  Q38_CUDA_OK(cudaMemcpy(word, &code, sizeof(code), cudaMemcpyHostToDevice));
  return Q38_OK;
}

extern "C" void q38_set_dependent_launch(int allowed) { q38::g_dependent_launch = allowed != 0; }

extern "C" unsigned int q38_device_error(int clear) {
  cudaDeviceSynchronize();
  unsigned int e = 0;
  e |= q38::qgemm_stream_error(clear != 0);
  e |= q38::qgemm_dispatch_error(clear != 0);
  e |= q38::qgemm_umma_error(clear != 0);
  e |= q38::attention_error(clear != 0);
  e |= q38::gdn_error(clear != 0);
  e |= q38::misc_error(clear != 0);
  return e;
}

extern "C" int q38_num_sms(void) { return q38::num_sms(); }

extern "C" size_t q38_kv_page_bytes(int dtype, int kv_heads) {
  return dtype == Q38_KV_INT8 ? 2 * size_t(kv_heads) * Q38_PAGE_TOKENS * (Q38_HEAD_DIM + 4 * 2)
                              : 2 * size_t(kv_heads) * Q38_PAGE_TOKENS * Q38_HEAD_DIM * 2;
}

// ---- device memory shared between the processes of one node (tensor-parallel all-reduce buffers) -------------------
extern "C" int q38_peer_alloc(size_t bytes, void** ptr) {
  Q38_REQUIRE(ptr && bytes > 0, "peer_alloc: null argument");
  void* p = nullptr;
  Q38_CUDA_OK(cudaMalloc(&p, bytes));
  const cudaError_t e = cudaMemset(p, 0, bytes);
  if (e != cudaSuccess) {
    (void)cudaFree(p);
    Q38_CUDA_OK(e);
  }
  *ptr = p;
  return Q38_OK;
}

extern "C" int q38_peer_free(void* ptr) {
  if (ptr) Q38_CUDA_OK(cudaFree(ptr));
  return Q38_OK;
}

extern "C" int q38_peer_export(void* ptr, unsigned char handle[64]) {
  Q38_REQUIRE(ptr && handle, "peer_export: null argument");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  cudaIpcMemHandle_t h;
  Q38_CUDA_OK(cudaIpcGetMemHandle(&h, ptr));
  memcpy(handle, &h, 64);
  return Q38_OK;
}

extern "C" int q38_peer_open(const unsigned char handle[64], void** ptr) {
  Q38_REQUIRE(ptr && handle, "peer_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  void* p = nullptr;
  Q38_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = p;
  return Q38_OK;
}

extern "C" int q38_peer_close(void* ptr) {
  if (ptr) Q38_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return Q38_OK;
}
