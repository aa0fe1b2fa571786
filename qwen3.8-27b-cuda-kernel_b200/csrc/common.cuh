// Device-side building blocks shared by every kernel of the library (sm_100a only):
// bounded mbarrier waits, 1-D bulk (TMA) copies, tensor-map loads, ldmatrix / mma.sync wrappers,
// L2 cache policies, and the per-translation-unit device error word.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace q38 {

// Every spin-wait in this library gives up after this many polls, records the site in the error word
// and lets the kernel run to its end (results of that launch are then meaningless, the context stays
// usable). The host reads the word through q38_device_error().
constexpr uint32_t kSpinLimit = 1u << 22;

// One error word per translation unit; each .cu exports a reader that c_abi.cu sums up.
static __device__ unsigned int g_tu_error = 0;

__device__ __forceinline__ void report_error(unsigned int code) { atomicCAS(&g_tu_error, 0u, code); }

static inline unsigned int read_tu_error(bool clear) {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_tu_error, sizeof(v));
  if (clear && v) {
    const unsigned int zero = 0;
    cudaMemcpyToSymbol(g_tu_error, &zero, sizeof(zero));
  }
  return v;
}

// Device address of this translation unit's error word (host code cannot use the symbol's name as an address).
static inline unsigned int* tu_error_address() {
  void* p = nullptr;
  return cudaGetSymbolAddress(&p, g_tu_error) == cudaSuccess ? static_cast<unsigned int*>(p) : nullptr;
}

// Programmatic dependent launch: let the next kernel of the stream be scheduled / wait until everything the
// previous kernels of the stream wrote is visible. Both are no-ops for a kernel launched without the attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return uint32_t(__cvta_generic_to_shared(p)); }

// ---- mbarrier -------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
#ifndef Q38_WAIT_HINT_NS
#define Q38_WAIT_HINT_NS 1000
#endif
constexpr uint32_t kWaitHintNs = Q38_WAIT_HINT_NS;  // upper bound of one parked poll, nanoseconds

// One poll of the barrier phase. The hint lets the hardware park the thread for up to about a microsecond while the
// phase is incomplete (it resumes as soon as the phase completes), so that waiting warps do not take issue slots from
// the warps that compute.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
#if Q38_WAIT_HINT_NS > 0
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitHintNs)
      : "memory");
#else
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
#endif
  return ok != 0;
}
// Bounded wait: false after kSpinLimit polls (the caller must then stop using the pipeline).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int site) {
  for (uint32_t i = 0; i < kSpinLimit; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  report_error(site);
  return false;
}

// ---- L2 policies, bulk copies ---------------------------------------------------------------------
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_normal() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_normal.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// global -> shared 1-D bulk copy; both addresses 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
      : "memory");
}

// 2-D tiled tensor-map load into this CTA only. x is the innermost coordinate: x * elem_size % 16 == 0.
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// ---- warp-level tensor ops (legacy path, used where M is too small for tcgen05) ----------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Folded-RMSNorm row scales rs[t] = rsqrt(sum_b partials[t][b] / hidden + eps) for t < rows, written to
// shared memory by `nthreads` cooperating threads (thread index `tix`): eight lanes share a token so that all of a
// token's partials are requested in one round trip to L2. Call from whole warps only.
__device__ __forceinline__ void row_scales_to_smem(const float* __restrict__ partials, int rows, int cap, int hidden,
                                                   float eps, float* rs_sm, int tix, int nthreads) {
  const int blocks = hidden / 128;
  for (int base = 0; base < cap; base += nthreads / 8) {
    const int t = base + tix / 8, sub = tix & 7;
    float sum = 0.0f;
    if (partials && t < rows)
      for (int b = sub; b < blocks; b += 8) sum += partials[(size_t)t * blocks + b];
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if (sub == 0 && t < cap) rs_sm[t] = (partials && t < rows) ? 1.0f / sqrtf(sum / float(hidden) + eps) : 1.0f;
  }
}

__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

}  // namespace q38
