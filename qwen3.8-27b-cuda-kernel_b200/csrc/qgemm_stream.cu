// Decode-sized BQ GEMM (M <= 16 tokens per pass): a weight-streaming kernel.
//
//   C[M][N] = A[M][K] (bf16) * W^T, W in BQ 4/5/6/8-bit planes; fused epilogues StoreBF16 / SwiGLU /
//   Residual (+ bf16 copy + next-norm partial sums) / StoreF32 with the folded-RMSNorm row scale.
//   Replaces kernels::qgemm of the reference (src/kernels/kernels.h:119-121, src/kernels/qgemm.cu) for
//   decode batches; the arithmetic contract is the reference's (bf16 x bf16 -> fp32 accumulate, weights
//   bf16(code * scale), epilogue in fp32).
//
// Design (B200):
//   * BQ planes are n-block-major: for one 64-column block all of K is one contiguous byte run in each
//     plane. A tile is 128 columns (2 blocks); the work list is (tile, 64-wide k-group) in memory order,
//     cut over one persistent CTA per SM (whole tiles, s CTAs inside each tile, or an even cut: the
//     launcher decides), so each CTA streams two contiguous runs per plane with large 1-D bulk (TMA)
//     copies into a multi-stage shared-memory ring (mbarrier full/empty pairs, one producer warp).
//     Weights carry an L2 evict-first policy: they are read once.
//   * The activation chunk of a stage arrives through a 2-D tensor map with the 128-byte swizzle, rows
//     beyond M zero-filled by the TMA unit.
//   * 16 consumer warps = 2 column blocks x 8 k-groups of a stage (the decode chain is latency-bound per warp,
//     so four warps per scheduler are needed to keep the issue slots busy). A lane's 16 bytes of a slab are
//     decoded in registers (bq_dequant.cuh) and are directly the A fragment (16 columns x 16 k) of
//     mma.sync.m16n8k16 with the tokens as the 8-wide N operand, so M <= 8 costs 4 MMAs per slab.
//   * A tile segment ends with a fixed-order reduction of the 8 k-warps into a shared C tile; segments
//     that do not cover all of K go to the workspace and the last-arriving CTA sums them in CTA order
//     (self-resetting counter): results are bit-reproducible from run to run.
#include <algorithm>

#include "bq_dequant.cuh"
#include "common.cuh"
#include "host_util.h"
#include "qgemm.h"

namespace q38 {
namespace {

constexpr int kTileN = 128;
constexpr int kGroupsPerStage = 8;
constexpr int kConsumerWarps = 16;
constexpr int kKWarps = kConsumerWarps / 2;
constexpr int kConsumers = kConsumerWarps * 32;
constexpr int kThreads = kConsumers + 32;
constexpr int kLdc = 132;  // floats per row of the shared C tile (bank-conflict-free fragment stores)
constexpr int kSmemBudget = 225 * 1024;

template <int BITS, int MT>
struct Cfg {
  using G = BqGeom<BITS>;
  static constexpr int kMpad = 8 * MT;
  static constexpr int kXGroup = kMpad * 128;  // bytes of one [kMpad][64] bf16 swizzled sub-tile
  static constexpr int kXOff = 0;
  static constexpr int kLoOff = kXOff + kGroupsPerStage * kXGroup;
  static constexpr int kHiOff = kLoOff + 2 * kGroupsPerStage * G::kLoGroupBytes;
  static constexpr int kScOff = kHiOff + 2 * kGroupsPerStage * G::kHiGroupBytes;
  static constexpr int kStageRaw = kScOff + 2 * kGroupsPerStage * G::kScGroupBytes;
  static constexpr int kStageBytes = (kStageRaw + 1023) / 1024 * 1024;
  static constexpr int kCBytes = kMpad * kLdc * 4;
  static constexpr int kTailBytes = kCBytes + kMpad * 4 + 256;  // C tile, row scales, barriers + flags
  static constexpr int kStagesFit = (kSmemBudget - 1024 - kTailBytes) / kStageBytes;
  static constexpr int kStages = kStagesFit > 6 ? 6 : kStagesFit;
  static constexpr int kSmemBytes = 1024 + kStages * kStageBytes + kTailBytes;
  static_assert(kStages >= 2, "pipeline needs two stages");
};

// Q38_EPI_ALLREDUCE_RESIDUAL: the ranks' buffers as this process sees them (entry `rank` is local memory)
struct AllreduceArgs {
  int world, rank;
  float* recv[Q38_MAX_PEERS];
  unsigned int* flags[Q38_MAX_PEERS];
  unsigned int* seq;
  unsigned int poll_limit;
};

struct StreamArgs {
  const uint8_t* lo;
  const uint8_t* hi;
  const uint8_t* sc;
  int n, k, m;
  int kind;
  void* out;
  int ldo;
  int n_store;
  float* residual;
  __nv_bfloat16* xbf;
  float* partials_out;
  const float* partials_in;
  int hidden;
  float eps;
  float* ws;
  int* counters;
  int tiles, kg;
  long long units;
  int split;
  int cps;  // split with every CTA inside one tile: CTAs per tile (grid = tiles * cps); 0 otherwise
  DecodeConsts dc;
  AllreduceArgs ar;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ long long cta_begin(const StreamArgs& a, int cta, int grid) {
  if (a.split) return (long long)cta * a.units / grid;
  return ((long long)cta * a.tiles / grid) * a.kg;
}

// Waits that give up once any warp of the CTA has given up (control flow stays identical for all warps,
// so the named barriers below still match up).
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned site) {
  if (*abort_flag) return false;
  if (mbar_wait(bar, parity, site)) return true;
  *abort_flag = 1;
  return false;
}

template <int BITS, int MT>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_stream_kernel(const __grid_constant__ CUtensorMap xmap, const StreamArgs a) {
  pdl_wait();               // everything written by earlier kernels of the stream is visible from here on
  pdl_launch_dependents();  // the next kernel may be scheduled now; it holds its own dependent work back the same way
  using C = Cfg<BITS, MT>;
  using G = BqGeom<BITS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint8_t* stages = smem;
  float* csm = reinterpret_cast<float*>(smem + C::kStages * C::kStageBytes);
  float* rs_sm = csm + C::kMpad * kLdc;
  uint64_t* full = reinterpret_cast<uint64_t*>(rs_sm + C::kMpad);
  uint64_t* empty = full + C::kStages;
  volatile int* flags = reinterpret_cast<volatile int*>(empty + C::kStages);  // [0] abort, [1] last-arriver

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long u0 = cta_begin(a, cta, grid), u1 = cta_begin(a, cta + 1, grid);

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], kConsumerWarps);
    }
    flags[0] = 0;
    flags[1] = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kConsumerWarps) {
    // ------------------------------ producer ------------------------------
    // Lane 0 waits for the slot and posts the byte count; then each copy of the stage is issued by its own lane.
    const uint64_t pol_w = policy_evict_first();
    uint32_t it = 0;
    bool alive = true;
    for (long long u = u0; u < u1 && alive;) {
      const int tile = int(u / a.kg), kg_a = int(u % a.kg);
      const int kg_b = int(min((long long)a.kg, kg_a + (u1 - u)));
      for (int g = kg_a; g < kg_b && alive; g += kGroupsPerStage, ++it) {
        const int s = it % C::kStages;
        const int ng = min(kGroupsPerStage, kg_b - g);
        int ok = 1;
        if (lane == 0) {
          ok = wait_or_abort(&empty[s], ((it / C::kStages) & 1) ^ 1, flags, 0x101) ? 1 : 0;
          if (ok)
            mbar_expect_tx(&full[s], uint32_t(ng) * (2u * (G::kLoGroupBytes + G::kHiGroupBytes + G::kScGroupBytes) + C::kXGroup));
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          alive = false;
          break;
        }
        uint8_t* st = stages + (size_t)s * C::kStageBytes;
        if (lane < ng) {
          tma_load_2d(st + C::kXOff + lane * C::kXGroup, &xmap, (g + lane) * 64, 0, &full[s]);
        } else if (lane < ng + 6) {
          const int op = lane - ng, nbl = op / 3, kind = op % 3;
          const size_t grp = (size_t)(tile * 2 + nbl) * a.kg + g;
          if (kind == 0)
            bulk_g2s(st + C::kLoOff + nbl * kGroupsPerStage * G::kLoGroupBytes, a.lo + grp * G::kLoGroupBytes,
                     ng * G::kLoGroupBytes, &full[s], pol_w);
          else if (kind == 1) {
            if constexpr (BITS != 4)
              bulk_g2s(st + C::kHiOff + nbl * kGroupsPerStage * G::kHiGroupBytes, a.hi + grp * G::kHiGroupBytes,
                       ng * G::kHiGroupBytes, &full[s], pol_w);
          } else
            bulk_g2s(st + C::kScOff + nbl * kGroupsPerStage * G::kScGroupBytes, a.sc + grp * G::kScGroupBytes,
                     ng * G::kScGroupBytes, &full[s], pol_w);
        }
        __syncwarp();
      }
      u += kg_b - kg_a;
    }
    return;
  }

  // ------------------------------ consumers ------------------------------
  // row scales of the folded RMSNorm: needed only by the epilogue, so they are fetched while the producer
  // already fills the ring
  row_scales_to_smem(a.partials_in, a.m, C::kMpad, a.hidden, a.eps, rs_sm, tid, kConsumers);
  named_bar_sync(1, kConsumers);
  const int wn = warp & 1, wk = warp >> 1;
  const int gl = lane >> 2, tl = lane & 3;
  const DecodeConsts dc = a.dc;
  uint32_t it = 0;
  for (long long u = u0; u < u1;) {
    const int tile = int(u / a.kg), kg_a = int(u % a.kg);
    const int kg_b = int(min((long long)a.kg, kg_a + (u1 - u)));
    float acc[4][MT][4];
#pragma unroll
    for (int jj = 0; jj < 4; ++jj)
#pragma unroll
      for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[jj][mt][c] = 0.0f;

    for (int g = kg_a; g < kg_b; g += kGroupsPerStage, ++it) {
      const int s = it % C::kStages;
      const uint32_t ph = (it / C::kStages) & 1;
      const bool ok = wait_or_abort(&full[s], ph, flags, 0x102);
      if (ok && g + wk < kg_b) {
        const uint8_t* st = stages + (size_t)s * C::kStageBytes;
        const int slot = wn * kGroupsPerStage + wk;
        const uint8_t* lo_g = st + C::kLoOff + slot * G::kLoGroupBytes;
        const uint8_t* hi_g = st + C::kHiOff + slot * G::kHiGroupBytes;
        const uint32_t x_g = smem_u32(st + C::kXOff + wk * C::kXGroup);
        uint32_t s2[8];
        expand_scales(*reinterpret_cast<const uint4*>(st + C::kScOff + slot * G::kScGroupBytes + 16 * gl), s2);
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          uint32_t b[MT][4];
          {
            const int mi = lane >> 3, r = lane & 7;
            const int chunk = 4 * half + mi;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
              ldmatrix_x4(b[mt], x_g + (8 * mt + r) * 128 + ((chunk ^ r) << 4));
          }
#pragma unroll
          for (int sl = 0; sl < 2; ++sl) {
            const int slab = 2 * half + sl;
            const uint4 lv = *reinterpret_cast<const uint4*>(lo_g + slab * 512 + lane * 16);
            const uint32_t lo[4] = {lv.x, lv.y, lv.z, lv.w};
            uint32_t hi[4] = {0, 0, 0, 0};
            if constexpr (BITS == 5) {
              hi[0] = *reinterpret_cast<const uint32_t*>(hi_g + slab * 128 + lane * 4);
            } else if constexpr (BITS == 6) {
              const uint2 hv = *reinterpret_cast<const uint2*>(hi_g + slab * 256 + lane * 8);
              hi[0] = hv.x;
              hi[1] = hv.y;
            } else if constexpr (BITS == 8) {
              const uint4 hv = *reinterpret_cast<const uint4*>(hi_g + slab * 512 + lane * 16);
              hi[0] = hv.x;
              hi[1] = hv.y;
              hi[2] = hv.z;
              hi[3] = hv.w;
            }
            uint32_t w[16];
            decode_slab<BITS>(lo, hi, s2, w, dc);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              const uint32_t af[4] = {w[4 * jj], w[4 * jj + 2], w[4 * jj + 1], w[4 * jj + 3]};
#pragma unroll
              for (int mt = 0; mt < MT; ++mt) mma_bf16_16816(acc[jj][mt], af, b[mt][2 * sl], b[mt][2 * sl + 1]);
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty[s]);
    }

    // ---- fixed-order reduction of the k-warps into the shared C tile ----
#pragma unroll 1
    for (int r = 0; r < kKWarps; ++r) {
      if (wk == r) {
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              const int idx = (8 * mt + 2 * tl + (c & 1)) * kLdc + 64 * wn + 16 * jj + gl + 8 * (c >> 1);
              if (r == 0) csm[idx] = acc[jj][mt][c];
              else csm[idx] += acc[jj][mt][c];
            }
      }
      named_bar_sync(1, kConsumers);
    }

    bool run_epilogue = true;
    const bool whole = kg_a == 0 && kg_b == a.kg;
    if (!whole) {
      // ---- stream-K fix-up: publish the partial tile; the last arriver sums all of them in CTA order ----
      constexpr int kTileFloats = C::kMpad * kTileN;
      float* mine = a.ws + ((size_t)cta * 2 + (kg_a != 0 ? 0 : 1)) * kTileFloats;
      for (int i = tid; i < kTileFloats; i += kConsumers) mine[i] = csm[(i >> 7) * kLdc + (i & 127)];
      // Publication: the CTA's stores are ordered before the barrier, and the one thread that then counts the CTA in
      // fences on both sides of its atomic (the fence is cumulative over what the barrier made visible to it), so
      // whoever sees the full count also sees every piece.
      named_bar_sync(1, kConsumers);
      // contributors of this tile: CTAs whose unit range intersects [tile * kg, (tile + 1) * kg); the first of them
      // begins at or before the tile (this piece is the one in its second buffer), the others inside it
      const long long t_begin = (long long)tile * a.kg, t_end = t_begin + a.kg;
      int c_first, c_last;
      if (a.cps > 0) {  // every CTA inside one tile: no 64-bit divisions
        c_first = tile * a.cps;
        c_last = c_first + a.cps - 1;
      } else {
        c_first = int(t_begin * grid / a.units);
        while (c_first > 0 && cta_begin(a, c_first, grid) > t_begin) --c_first;
        while (cta_begin(a, c_first + 1, grid) <= t_begin) ++c_first;
        c_last = c_first;
        while (c_last + 1 < grid && cta_begin(a, c_last + 1, grid) < t_end) ++c_last;
      }
      if (tid == 0) {
        __threadfence();
        const int prev = atomicAdd(&a.counters[tile], 1);
        __threadfence();
        const int last = prev == c_last - c_first;
        if (last) a.counters[tile] = 0;
        flags[1] = last;
      }
      named_bar_sync(1, kConsumers);
      run_epilogue = flags[1] != 0;
      if (run_epilogue) {
        for (int i = tid; i < kTileFloats; i += kConsumers) {
          float sum = 0.0f;
          for (int c = c_first; c <= c_last; ++c) {
            const int which = c != c_first ? 0 : 1;  // c_first begins at or before the tile: its second buffer
            sum += __ldcg(a.ws + ((size_t)c * 2 + which) * kTileFloats + i);
          }
          csm[(i >> 7) * kLdc + (i & 127)] = sum;
        }
      }
      named_bar_sync(1, kConsumers);
    }

    if (run_epilogue && a.kind == Q38_EPI_ALLREDUCE_RESIDUAL) {
      // ---- sum of this tile over the tensor-parallel ranks, inside the GEMM ----
      // Push: every rank stores its finished tile rows into slot `rank` of every rank's receive buffer (plain stores
      // to peer memory; its own buffer included), fences, and raises flag [tile][rank] there to the call's sequence
      // number. Pull: it waits until all flags [tile][*] in its own memory have reached that number - a bounded wait
      // that records an error and goes on - and adds the pieces in rank order, so every rank holds the same bits.
      // Two buffers are used in turn: a rank can be one call ahead of another at most (it needs the other's flag of
      // the call before), so the buffer it writes next is one the other has finished reading.
      __shared__ unsigned int ar_seq;
      const AllreduceArgs& ar = a.ar;
      if (tid == 0) ar_seq = ar.seq[tile] + 1u;
      named_bar_sync(1, kConsumers);
      const unsigned int seq = ar_seq;
      const size_t slot_floats = (size_t)Q38_ALLREDUCE_ROWS * a.n;
      const size_t buf_off = (size_t)(seq & 1u) * ar.world * slot_floats;
      const int col = tile * kTileN + 4 * lane;
      for (int m = warp; m < a.m; m += kConsumerWarps) {
        const float4 cv = *reinterpret_cast<const float4*>(csm + m * kLdc + 4 * lane);
        const size_t off = buf_off + (size_t)ar.rank * slot_floats + (size_t)m * a.n + col;
        for (int p = 0; p < ar.world; ++p) *reinterpret_cast<float4*>(ar.recv[p] + off) = cv;
      }
      __threadfence_system();
      named_bar_sync(1, kConsumers);
      if (tid == 0) ar.seq[tile] = seq;
      if (tid < ar.world) {
        st_release_sys(ar.flags[tid] + (size_t)tile * ar.world + ar.rank, seq);
        const unsigned int* mine = ar.flags[ar.rank] + (size_t)tile * ar.world + tid;
        const unsigned int limit = ar.poll_limit ? ar.poll_limit : (1u << 22);
        bool seen = false;
        for (unsigned int i = 0; i < limit && !seen; ++i) {
          seen = int(ld_acquire_sys(mine) - seq) >= 0;
          if (!seen) __nanosleep(32);
        }
        if (!seen) report_error(0x120);
      }
      named_bar_sync(1, kConsumers);
      for (int m = warp; m < a.m; m += kConsumerWarps) {
        float4 sum = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int p = 0; p < ar.world; ++p) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(ar.recv[ar.rank] + buf_off + (size_t)p * slot_floats +
                                                                  (size_t)m * a.n + col));
          sum.x += v.x;
          sum.y += v.y;
          sum.z += v.z;
          sum.w += v.w;
        }
        *reinterpret_cast<float4*>(csm + m * kLdc + 4 * lane) = sum;
      }
      named_bar_sync(1, kConsumers);
    }

    if (run_epilogue) {
      const int n0 = tile * kTileN + 4 * lane;
      const int n_lim = a.n_store > 0 ? a.n_store : a.n;
      for (int m = warp; m < a.m; m += kConsumerWarps) {
        const float4 cv = *reinterpret_cast<const float4*>(csm + m * kLdc + 4 * lane);
        const float rs = rs_sm[m];
        float v[4] = {cv.x, cv.y, cv.z, cv.w};
        if (a.kind == Q38_EPI_STORE_BF16) {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.out) + (size_t)m * a.ldo + n0;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (n0 + e < n_lim) o[e] = __float2bfloat16_rn(v[e] * rs);
        } else if (a.kind == Q38_EPI_STORE_F32) {
          float* o = static_cast<float*>(a.out) + (size_t)m * a.ldo + n0;
#pragma unroll
          for (int e = 0; e < 4; ++e)
            if (n0 + e < n_lim) o[e] = v[e] * rs;
        } else if (a.kind == Q38_EPI_SWIGLU) {
          __nv_bfloat16* o = static_cast<__nv_bfloat16*>(a.out) + (size_t)m * a.ldo + n0 / 2;
#pragma unroll
          for (int e = 0; e < 2; ++e)
            if (n0 + 2 * e < n_lim) o[e] = __float2bfloat16_rn(silu_f(v[2 * e] * rs) * (v[2 * e + 1] * rs));
        } else {
          float* res = a.residual + (size_t)m * a.n + n0;
          float4 rv = *reinterpret_cast<float4*>(res);
          rv.x += v[0];
          rv.y += v[1];
          rv.z += v[2];
          rv.w += v[3];
          *reinterpret_cast<float4*>(res) = rv;
          __nv_bfloat162 p0 = __floats2bfloat162_rn(rv.x, rv.y), p1 = __floats2bfloat162_rn(rv.z, rv.w);
          uint2 packed;
          packed.x = bf16x2_bits(p0);
          packed.y = bf16x2_bits(p1);
          *reinterpret_cast<uint2*>(a.xbf + (size_t)m * a.n + n0) = packed;
          const float ss = warp_sum(rv.x * rv.x + rv.y * rv.y + rv.z * rv.z + rv.w * rv.w);
          if (lane == 0) a.partials_out[(size_t)m * (a.n / 128) + tile] = ss;
        }
      }
    }
    named_bar_sync(1, kConsumers);
    u += kg_b - kg_a;
  }
}

// ---- host side -------------------------------------------------------------------------------------
using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                              CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeFn encode_fn() {
  static EncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
    return reinterpret_cast<EncodeFn>(p);
  }();
  return fn;
}

template <int BITS, int MT>
int launch_one(const __nv_bfloat16* a_ptr, int m, const q38_bq_weight& w, const q38_gemm_epilogue& ep,
               const q38_gemm_workspace* ws, cudaStream_t stream) {
  using C = Cfg<BITS, MT>;
  static const cudaError_t attr = cudaFuncSetAttribute(qgemm_stream_kernel<BITS, MT>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  Q38_CUDA_OK(attr);
  EncodeFn enc = encode_fn();
  Q38_REQUIRE(enc != nullptr, "qgemm: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {cuuint64_t(w.k), cuuint64_t(m)};
  const cuuint64_t strides[1] = {cuuint64_t(w.k) * 2};
  const cuuint32_t box[2] = {64, cuuint32_t(C::kMpad)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(a_ptr), dims, strides,
                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  Q38_REQUIRE(r == CUDA_SUCCESS, "qgemm: tensor map encode failed (%d)", int(r));

  StreamArgs a{};
  a.lo = w.lo;
  a.hi = w.hi;
  a.sc = reinterpret_cast<const uint8_t*>(w.scales);
  a.n = w.n;
  a.k = w.k;
  a.m = m;
  a.kind = ep.kind;
  a.out = ep.out;
  a.ldo = ep.ldo;
  a.n_store = ep.n_store;
  a.residual = ep.residual;
  a.xbf = reinterpret_cast<__nv_bfloat16*>(ep.xbf);
  a.partials_out = ep.partials_out;
  a.partials_in = ep.partials_in;
  a.hidden = ep.hidden;
  a.eps = ep.eps;
  if (ep.kind == Q38_EPI_ALLREDUCE_RESIDUAL) {
    const q38_peer_allreduce& ar = *ep.allreduce;
    a.ar.world = ar.world;
    a.ar.rank = ar.rank;
    for (int r = 0; r < ar.world; ++r) {
      a.ar.recv[r] = ar.recv[r];
      a.ar.flags[r] = ar.flags[r];
    }
    a.ar.seq = ar.seq;
    a.ar.poll_limit = ar.poll_limit;
  }
  a.tiles = w.n / kTileN;
  a.kg = w.k / 64;
  a.units = (long long)a.tiles * a.kg;
  a.dc = decode_consts(BITS);
  const int sms = num_sms();
  // Cut of the (tile, k-group) list over the CTAs: with fewer tiles than SMs, s = SMs / tiles CTAs per tile and no
  // CTA spanning two tiles (one fix-up per CTA, s partial tiles per reduction); with up to four tiles per SM whole
  // tiles; otherwise an even cut over all SMs (stream-K).
  const bool have_ws = ws && ws->partials && ws->counters && ws->num_counters >= a.tiles;
  int grid;
  if (a.tiles < sms) {
    int s = std::max(1, std::min(sms / a.tiles, a.kg / 8));
    if (!have_ws || ws->partial_floats < (size_t)a.tiles * s * 2 * C::kMpad * kTileN) s = 1;
    grid = a.tiles * s;
    a.split = s > 1;
    a.cps = s > 1 ? s : 0;
  } else {
    grid = sms;
    a.split = have_ws && ws->partial_floats >= (size_t)grid * 2 * C::kMpad * kTileN;
    if (a.tiles < 4 * sms) a.split = 0;  // a few tiles per CTA: two fix-ups per CTA cost more than the uneven last wave
    if (!a.split) grid = std::min(sms, a.tiles);
  }
  if (a.split) {
    a.ws = ws->partials;
    a.counters = ws->counters;
  }
  (void)launch_kernel(qgemm_stream_kernel<BITS, MT>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream, xmap, a);
  Q38_LAUNCH_OK("qgemm_stream_kernel");
  return Q38_OK;
}

template <int BITS>
int launch_bits(int mt, const __nv_bfloat16* a, int m, const q38_bq_weight& w, const q38_gemm_epilogue& ep,
                const q38_gemm_workspace* ws, cudaStream_t s) {
  return mt == 1 ? launch_one<BITS, 1>(a, m, w, ep, ws, s) : launch_one<BITS, 2>(a, m, w, ep, ws, s);
}

}  // namespace

// m <= 8 * mt, mt in {1, 2}. Called by the dispatcher in qgemm.cu.
int qgemm_stream_launch(int mt, const __nv_bfloat16* a, int m, const q38_bq_weight& w, const q38_gemm_epilogue& ep,
                        const q38_gemm_workspace* ws, cudaStream_t s) {
  switch (w.bits) {
    case 4: return launch_bits<4>(mt, a, m, w, ep, ws, s);
    case 5: return launch_bits<5>(mt, a, m, w, ep, ws, s);
    case 6: return launch_bits<6>(mt, a, m, w, ep, ws, s);
    default: return launch_bits<8>(mt, a, m, w, ep, ws, s);
  }
}

unsigned int qgemm_stream_error(bool clear) { return read_tu_error(clear); }
unsigned int* qgemm_stream_error_address() { return tu_error_address(); }

}  // namespace q38
