// GEMM dispatcher: argument validation, tile-configuration choice (tuning hook or M heuristic) and the
// BQ dequantisation dump. Replaces the host part of the reference's src/kernels/qgemm.cu:470-616.
#include <algorithm>
#include <mutex>

#include "bq_dequant.cuh"
#include "common.cuh"
#include "host_util.h"
#include "qgemm.h"

namespace q38 {
namespace {

struct ConfigInfo {
  const char* name;
  int tile_m;   // tokens per launch
  bool umma;
  int mblocks;  // tcgen05 kernel: token blocks of tile_m / mblocks rows inside one launch
  bool a_in_tmem;  // tcgen05 kernel: decoded weights reach the MMA through tensor memory
};
constexpr ConfigInfo kConfigs[] = {
    {"stream_m8", 8, false, 1, false},  {"stream_m16", 16, false, 1, false}, {"umma_t32", 32, true, 1, false},
    {"umma_t64", 64, true, 1, false},   {"umma_t128", 128, true, 1, false},  {"umma_t256", 256, true, 1, false},
    {"umma_t512", 512, true, 1, false}, {"umma_t256x2", 512, true, 2, false}, {"tmem_t32", 32, true, 1, true},
    {"tmem_t64", 64, true, 1, true},    {"tmem_t128", 128, true, 1, true},   {"tmem_t256", 256, true, 1, true},
    {"tmem_t256x2", 512, true, 2, true},
};
constexpr int kNumConfigs = int(sizeof(kConfigs) / sizeof(kConfigs[0]));

q38_gemm_tuning_lookup g_tuning = nullptr;

// Small batches stream the weights through mma.sync (tokens are the 8-wide operand); from 17 tokens on the
// tcgen05 kernel keeps the accumulators in TMEM and, in the tmem_* configurations, also hands the decoded weights
// to the MMA through TMEM (no shared-memory round trip of the bf16 tile: faster at every token count measured, so
// the umma_* configurations are only reachable by explicit choice or through a tuning table).
// Above 256 tokens two 256-token blocks share one launch (whole weight tiles per CTA).
int auto_config(int m, const q38_bq_weight& w, const q38_gemm_workspace* ws) {
  (void)ws;
  if (m <= 8) return 0;
  if (m <= 16) return 1;  // (with the Store epilogue tmem_t32 is level or ahead on the 40-tile matrices, with their Residual epilogue it is not)
  if (m <= 32) return 8;
  if (m <= 64) return 9;
  if (m <= 128) return 10;
  if (m <= 256) return 11;
  return 12;
}

// One lane decodes one slab exactly as the GEMM does and writes the 32 weights to W[n][k] (bf16).
template <int BITS>
__global__ void bq_dequant_kernel(const uint8_t* __restrict__ lo, const uint8_t* __restrict__ hi,
                                  const uint8_t* __restrict__ sc, int n, int k, __nv_bfloat16* __restrict__ out) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  using G = BqGeom<BITS>;
  const int lane = threadIdx.x & 31;
  const long long slab = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long slabs = (long long)(n / 64) * (k / 16);
  if (slab >= slabs) return;
  const int kb = int(slab % (k / 16));
  const long long nb = slab / (k / 16);
  const int g = lane >> 2, t = lane & 3;
  const uint4 lv = *reinterpret_cast<const uint4*>(lo + slab * 512 + lane * 16);
  const uint32_t lw[4] = {lv.x, lv.y, lv.z, lv.w};
  uint32_t hw[4] = {0, 0, 0, 0};
  for (int i = 0; i < G::kHiLaneWords; ++i)
    hw[i] = *reinterpret_cast<const uint32_t*>(hi + slab * G::kHiSlabBytes + lane * 4 * G::kHiLaneWords + 4 * i);
  uint32_t s2[8];
  expand_scales(*reinterpret_cast<const uint4*>(sc + (nb * (k / 64) + kb / 4) * 128 + 16 * g), s2);
  uint32_t w[16];
  decode_slab<BITS>(lw, hw, s2, w, DecodeConsts{0x000F000Fu, 0x43004300u, BITS == 6 ? 0x00300030u : 0x00100010u});
#pragma unroll
  for (int q = 0; q < 16; ++q) {
    const int j = q >> 1, h = q & 1;
    const long long row = nb * 64 + 8 * j + g;
    const int col = kb * 16 + 2 * t + 8 * h;
    *reinterpret_cast<uint32_t*>(out + row * k + col) = w[q];
  }
}

}  // namespace
}  // namespace q38

using namespace q38;

extern "C" int q38_qgemm_num_configs(void) { return kNumConfigs; }
extern "C" const char* q38_qgemm_config_name(int c) { return c >= 0 && c < kNumConfigs ? kConfigs[c].name : "?"; }
extern "C" int q38_qgemm_config_tile_m(int c) { return c >= 0 && c < kNumConfigs ? kConfigs[c].tile_m : 0; }
extern "C" void q38_set_qgemm_tuning(q38_gemm_tuning_lookup lookup) { g_tuning = lookup; }
extern "C" int q38_qgemm_auto_config(int bits, int n, int k, int m) {
  if (g_tuning) {
    const int t = g_tuning(bits, n, k, m);
    if (t >= 0 && t < kNumConfigs) return t;
  }
  q38_bq_weight w{};
  w.bits = bits;
  w.n = n;
  w.k = k;
  return auto_config(m, w, nullptr);
}

extern "C" int q38_qgemm(const q38_bf16* a, int m, const q38_bq_weight* w, const q38_gemm_epilogue* ep,
                         const q38_gemm_workspace* ws, void* stream, int config) {
  Q38_REQUIRE(a && w && ep, "qgemm: null argument");
  Q38_REQUIRE(m > 0, "qgemm: m must be positive, got %d", m);
  Q38_REQUIRE(w->bits == 4 || w->bits == 5 || w->bits == 6 || w->bits == 8, "qgemm: unsupported bit width %d", w->bits);
  Q38_REQUIRE(w->n > 0 && w->n % 128 == 0 && w->k > 0 && w->k % 64 == 0, "qgemm: BQ shape %d x %d", w->n, w->k);
  Q38_REQUIRE(w->lo && w->scales && (w->bits == 4 || w->hi), "qgemm: missing weight plane");
  Q38_REQUIRE(config >= -1 && config < kNumConfigs, "qgemm: config %d out of range", config);
  Q38_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0, "qgemm: A must be 16-byte aligned");
  if (ep->kind == Q38_EPI_RESIDUAL || ep->kind == Q38_EPI_ALLREDUCE_RESIDUAL) {
    Q38_REQUIRE(ep->residual && ep->xbf && ep->partials_out, "qgemm: Residual epilogue needs residual/xbf/partials");
    if (ep->kind == Q38_EPI_ALLREDUCE_RESIDUAL) {
      const q38_peer_allreduce* ar = ep->allreduce;
      Q38_REQUIRE(ar != nullptr, "qgemm: the all-reduce epilogue needs its peer description");
      Q38_REQUIRE(m <= Q38_ALLREDUCE_ROWS, "qgemm: the all-reduce epilogue serves up to %d tokens, got %d", Q38_ALLREDUCE_ROWS, m);
      Q38_REQUIRE(ar->world >= 1 && ar->world <= Q38_MAX_PEERS && ar->rank >= 0 && ar->rank < ar->world && ar->seq,
                  "qgemm: all-reduce world %d rank %d", ar->world, ar->rank);
      for (int r = 0; r < ar->world; ++r)
        Q38_REQUIRE(ar->recv[r] && ar->flags[r] && (reinterpret_cast<uintptr_t>(ar->recv[r]) & 15) == 0,
                    "qgemm: all-reduce buffers of rank %d", r);
    }
  } else {
    Q38_REQUIRE(ep->kind >= 0 && ep->kind <= 3 && ep->out && ep->ldo > 0, "qgemm: epilogue output");
  }
  if (ep->partials_in) Q38_REQUIRE(ep->hidden > 0 && ep->hidden % 128 == 0, "qgemm: hidden %d", ep->hidden);
  if (config < 0 && g_tuning) {
    const int t = g_tuning(w->bits, w->n, w->k, m);
    if (t >= 0 && t < kNumConfigs) config = t;
  }
  if (config < 0) config = auto_config(m, *w, ws);
  Q38_REQUIRE(ep->kind != Q38_EPI_ALLREDUCE_RESIDUAL || !kConfigs[config].umma,
              "qgemm: the all-reduce epilogue exists in the streaming kernel only (configurations stream_*)");
  const int tm = kConfigs[config].tile_m;
  const cudaStream_t s = as_stream(stream);
  const __nv_bfloat16* ap = reinterpret_cast<const __nv_bfloat16*>(a);
  for (int r0 = 0; r0 < m; r0 += tm) {
    const int rows = std::min(tm, m - r0);
    q38_gemm_epilogue e = *ep;
    if (e.kind == Q38_EPI_RESIDUAL || e.kind == Q38_EPI_ALLREDUCE_RESIDUAL) {
      e.residual += (size_t)r0 * w->n;
      e.xbf += (size_t)r0 * w->n;
      e.partials_out += (size_t)r0 * (w->n / 128);
    } else if (e.kind == Q38_EPI_STORE_F32) {
      e.out = static_cast<float*>(e.out) + (size_t)r0 * e.ldo;
    } else {
      e.out = static_cast<q38_bf16*>(e.out) + (size_t)r0 * e.ldo;
    }
    if (e.partials_in) e.partials_in += (size_t)r0 * (e.hidden / 128);
    const int mb = kConfigs[config].mblocks;
    const int rc = kConfigs[config].umma ? qgemm_umma_launch(tm / mb, mb, kConfigs[config].a_in_tmem, ap + (size_t)r0 * w->k, rows, *w, e, ws, s)
                                         : qgemm_stream_launch(tm / 8, ap + (size_t)r0 * w->k, rows, *w, e, ws, s);
    if (rc != Q38_OK) return rc;
  }
  return Q38_OK;
}

extern "C" int q38_bq_dequant(const q38_bq_weight* w, q38_bf16* out, void* stream) {
  Q38_REQUIRE(w && out, "bq_dequant: null argument");
  Q38_REQUIRE(w->n % 64 == 0 && w->k % 64 == 0, "bq_dequant: shape");
  const long long slabs = (long long)(w->n / 64) * (w->k / 16);
  const int warps = 8;
  const unsigned grid = unsigned((slabs + warps - 1) / warps);
  const uint8_t* sc = reinterpret_cast<const uint8_t*>(w->scales);
  __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(out);
  const cudaStream_t s = as_stream(stream);
  switch (w->bits) {
    case 4: (void)launch_kernel(bq_dequant_kernel<4>, dim3(grid), dim3(warps * 32), 0, s, w->lo, w->hi, sc, w->n, w->k, o); break;
    case 5: (void)launch_kernel(bq_dequant_kernel<5>, dim3(grid), dim3(warps * 32), 0, s, w->lo, w->hi, sc, w->n, w->k, o); break;
    case 6: (void)launch_kernel(bq_dequant_kernel<6>, dim3(grid), dim3(warps * 32), 0, s, w->lo, w->hi, sc, w->n, w->k, o); break;
    case 8: (void)launch_kernel(bq_dequant_kernel<8>, dim3(grid), dim3(warps * 32), 0, s, w->lo, w->hi, sc, w->n, w->k, o); break;
    default: Q38_REQUIRE(false, "bq_dequant: unsupported bit width %d", w->bits);
  }
  Q38_LAUNCH_OK("bq_dequant_kernel");
  return Q38_OK;
}

// ---------------------------------------------------------------------------------------------------
// q38_qgemm_static: the decode GEMM for callers that cannot allocate device memory.
//
// q38_qgemm needs a caller-provided stream-K workspace (partial tiles + arrival counters). Some hosts have no
// way to provide one: a plugin that is only handed its input and output buffers, a runtime whose memory pool is
// closed once serving starts, code running inside a region where cudaMalloc is forbidden. For them the workspace
// lives in this library as a fixed array in device memory (about 3.2 MB, held by every GPU that loads the library
// until the process exits). Limits that follow from the fixed size: m <= 16 tokens (the streaming kernel),
// n <= 128 * kStaticCounters columns, and a GPU with at most kStaticCtas SMs. All calls on a device share the one
// array: calls that overlap on the GPU (different streams, or graphs replayed concurrently) race on it and
// must be serialised by the caller. The arrival counters have to be zero when a launch starts, so every call
// clears them on `stream` first (a memset node, no allocation).
// ---------------------------------------------------------------------------------------------------
namespace {
constexpr int kStaticCtas = 192;        // persistent CTAs (= SMs) the partial-tile area is sized for
constexpr int kStaticM = 16;            // largest token count served
constexpr int kStaticCounters = 4096;   // 128-column tiles: n <= 524288
constexpr size_t kStaticPartialFloats = size_t(kStaticCtas) * 2 * kStaticM * 128;

static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];
static __device__ __align__(256) int g_static_counters[kStaticCounters];

struct StaticWs {
  std::once_flag once;      // the lookup runs once per device, also with several host threads calling
  float* partials = nullptr;
  int* counters = nullptr;
  int sms = 0;              // SM count of this device (the cached count of the library is the first device's)
  cudaError_t status = cudaSuccess;
};
constexpr int kMaxDevices = 64;
StaticWs g_static_ws[kMaxDevices];

// The array names above are host-side stand-ins; the device addresses come from cudaGetSymbolAddress, looked up
// once per device with that device current.
int static_ws_for_current_device(const StaticWs** out) {
  int dev = 0;
  Q38_CUDA_OK(cudaGetDevice(&dev));
  Q38_REQUIRE(dev >= 0 && dev < kMaxDevices, "qgemm_static: device index %d out of range", dev);
  StaticWs& ws = g_static_ws[dev];
  std::call_once(ws.once, [&ws, dev] {
    void* p = nullptr;
    void* c = nullptr;
    ws.status = cudaGetSymbolAddress(&p, g_static_partials);
    if (ws.status == cudaSuccess) ws.status = cudaGetSymbolAddress(&c, g_static_counters);
    if (ws.status == cudaSuccess) ws.status = cudaDeviceGetAttribute(&ws.sms, cudaDevAttrMultiProcessorCount, dev);
    ws.partials = static_cast<float*>(p);
    ws.counters = static_cast<int*>(c);
  });
  Q38_CUDA_OK(ws.status);
  *out = &ws;
  return Q38_OK;
}
}  // namespace

extern "C" int q38_qgemm_static(const q38_bf16* a, int m, const q38_bq_weight* w, const q38_gemm_epilogue* ep,
                                void* stream) {
  Q38_REQUIRE(a && w && ep, "qgemm_static: null argument");
  Q38_REQUIRE(m > 0 && m <= kStaticM, "qgemm_static: m = %d is outside the built-in workspace (1..%d tokens)", m,
              kStaticM);
  Q38_REQUIRE(w->n > 0 && w->n / 128 <= kStaticCounters, "qgemm_static: n = %d exceeds the built-in workspace (%d columns)",
              w->n, 128 * kStaticCounters);
  const StaticWs* sws = nullptr;
  const int rc = static_ws_for_current_device(&sws);
  if (rc != Q38_OK) return rc;
  Q38_REQUIRE(sws->sms <= kStaticCtas, "qgemm_static: %d SMs exceed the built-in workspace (%d)", sws->sms, kStaticCtas);
  Q38_CUDA_OK(cudaMemsetAsync(sws->counters, 0, sizeof(int) * kStaticCounters, as_stream(stream)));
  const q38_gemm_workspace ws{sws->partials, kStaticPartialFloats, sws->counters, kStaticCounters};
  return q38_qgemm(a, m, w, ep, &ws, stream, Q38_GEMM_CONFIG_AUTO);
}

namespace q38 {
unsigned int qgemm_dispatch_error(bool clear) { return read_tu_error(clear); }
unsigned int* qgemm_dispatch_error_address() { return tu_error_address(); }
}
