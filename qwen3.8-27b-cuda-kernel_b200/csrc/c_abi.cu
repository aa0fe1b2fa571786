// Library-wide pieces of the C ABI: error reporting, device properties, layout helpers.
#include <cstdarg>
#include <cstdio>
#include <cstring>

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

}  // namespace q38

extern "C" const char* q38_last_error(void) { return q38::g_error; }

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
