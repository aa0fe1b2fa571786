// BQ GEMM on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM) for 17 <= M <= 512 tokens
// per launch: large decode batches and prefill chunks. Same contract and epilogues as the streaming kernel
// (qgemm_stream.cu); replaces kernels::qgemm of the reference (src/kernels/kernels.h:119-121) for these M.
//
// Orientation: the weights are the MMA's A operand (M_mma = 128 output columns = two 64-column BQ blocks),
// the tokens are its N operand (N_mma = 32..256; 512 tokens = two MMAs over all 512 TMEM columns), so any token
// count fills the 128 TMEM lanes. One persistent CTA per SM walks a list of (work item, 64-wide k-group), a work
// item being a weight tile (or a (token block, weight tile) pair when a launch covers two token blocks); how the
// list is cut over the CTAs - whole tiles, s CTAs inside each tile, or an even cut - is chosen by the launcher.
// Two rings:
//   raw ring      the BQ planes of 4 k-groups per stage (contiguous per 64-column block: 1-D bulk copies, L2
//                 evict-first), as deep as shared memory allows next to the operand ring;
//   operand ring  units of one or two decoded 64-wide k-groups, each with its activation slices [TOK][64] bf16
//                 (2-D tensor map, 128-byte swizzle, rows >= M zero-filled). One mbarrier per unit collects the
//                 decode warps' arrivals and the activation copies' bytes; one tcgen05.commit hands the unit back.
// Where the decoded weights live distinguishes the two variants of the kernel (template flag ATM):
//   ATM = true    (tmem_* configurations, up to 256 tokens per pass; the dispatcher's choice) in tensor memory: a
//                 decode warp writes its registers with tcgen05.st.16x128b - whose register <-> (lane, column)
//                 mapping is the A-fragment layout of mma.m16n8k16, i.e. the layout the BQ planes are packed for -
//                 and the MMA takes A from TMEM ([128 lanes][8 columns of bf16 pairs] per k16 step). TMEM holds the
//                 accumulator (TOK columns) and the ring (32 columns per k-group); shared memory only the raw
//                 planes and the activations. No bf16 weight tile crosses shared memory;
//   ATM = false   (umma_* configurations, up to 512 tokens) in shared memory as [128 n][64 k] slices in the K-major
//                 128-byte-swizzled layout of a UMMA descriptor, written with 4-byte bank-conflict-free stores.
// Warp roles:
//   warp 0       raw producer (six copies per stage, one lane each);
//   warp 1       stays converged; one elected lane issues tcgen05.mma.kind::f16 (bf16 x bf16 -> fp32), four per
//                k-group in one block (ATM) or one per k16 step, and tcgen05.commit per unit / per accumulator;
//   warp 3       up to 128 tokens a second issuer (an MMA costs its issuing thread more time than the tensor pipe
//                there): warp 1 takes the even units into accumulator 0, warp 3 the odd ones into accumulator 1;
//                idle above that (it keeps the decode warps aligned to the TMEM lane quarters);
//   warp 2       activation producer - the first thread that touches data of earlier kernels (griddepcontrol.wait);
//                everything before it (set-up, TMEM allocation, weight prefetch and decode) overlaps the previous
//                kernel's tail;
//   warps 4-19   decode: lane-owned slab bytes -> bf16(code * scale) in registers (bq_dequant.cuh) -> operand ring.
//                ATM: a warp owns the TMEM lane quarter its index selects (32 of the tile's 128 columns = half a
//                64-column block, all k); with two-group units it takes a whole unit quarter every other stage.
//                The same warps run the epilogue out of TMEM (tcgen05.ld).
// Partial tiles go through the caller's workspace; the tile's last-arriving CTA sums them in CTA order, so
// results are bit-reproducible. Every wait is bounded; TMEM is always released before the kernel ends.
#include <algorithm>

#include "bq_dequant.cuh"
#include "common.cuh"
#include "host_util.h"
#include "qgemm.h"

namespace q38 {
namespace {

constexpr int kTileN = 128;
constexpr int kGroupsPerStage = 4;
constexpr int kDecodeWarps = 16;
constexpr int kFirstDecodeWarp = 4;
constexpr int kDecodeThreads = kDecodeWarps * 32;
constexpr int kThreads = (kFirstDecodeWarp + kDecodeWarps) * 32;
constexpr int kWarpsPerSlice = 8;
constexpr int kSliceBytes = kTileN * 128;  // one [128 n][64 k] bf16 operand slice
constexpr int kSmemBudget = 226 * 1024;

// ATM: the decoded weights go to tensor memory (tcgen05.st) and the MMA reads its A operand from there; shared memory
// then holds only the raw planes and the activation slices.
template <int BITS, int TOK, bool ATM>
struct UCfg {
  using G = BqGeom<BITS>;
  static_assert(!ATM || TOK <= 256, "accumulator and weight ring share the 512 TMEM columns");
  // operand unit: what one barrier round trip hands to the MMA thread = kSpu decoded slices + their activations
  static constexpr int kSpu = TOK <= 128 ? 2 : 1;
#ifndef Q38_TMEM_UNITS_SMALL
#define Q38_TMEM_UNITS_SMALL 6
#endif
  static constexpr int kUnits = ATM ? (TOK <= 64 ? Q38_TMEM_UNITS_SMALL : 4) : (TOK <= 128 ? 2 : TOK <= 256 ? 3 : 2);
  static constexpr int kXBytes = TOK * 128;  // activation k-slice [TOK][64] bf16
  static constexpr int kWBytes = ATM ? 0 : kSliceBytes;  // decoded slice held in shared memory
  static constexpr int kUnitBytes = kSpu * (kWBytes + kXBytes);
  static constexpr int kDecodeWarpsPerUnit = ATM ? 4 : kWarpsPerSlice;
  static constexpr int kRawConsumers = ATM && kSpu == 2 ? kDecodeWarps / 2 : kDecodeWarps;  // warps that release a raw stage
  // tensor memory: accumulator [128 lanes][TOK columns] at column 0, then (ATM) the ring of decoded units, one
  // 64-wide k-group = 128 lanes x 32 columns of packed bf16 pairs
  // Issuing one tcgen05.mma costs the issuing thread 40-60 cycles whatever the token count, which at 128 tokens and
  // fewer is more than the MMA's time in the tensor pipe: two warps issue, each the units of its own parity into
  // its own accumulator (the epilogue adds the two).
  static constexpr int kIssuers = TOK <= 128 ? 2 : 1;
  static constexpr int kAccCols = TOK < 32 ? 32 : TOK;  // columns of one accumulator
  static constexpr int kACol0 = kIssuers * kAccCols;
  // A slot's successive uses must all belong to one issuer: a parity wait cannot tell the fill it expects from the
  // one before, which with an odd ring would be the other issuer's and possibly still outstanding.
  static_assert(kUnits % kIssuers == 0, "operand ring length must be a multiple of the number of issuing warps");
  static constexpr int kUnitCols = kSpu * 32;
  static_assert(!ATM || kACol0 + kUnits * kUnitCols <= 512, "tensor memory columns");
  static constexpr int kLoOff = 0;
  static constexpr int kHiOff = kLoOff + 2 * kGroupsPerStage * G::kLoGroupBytes;
  static constexpr int kScOff = kHiOff + 2 * kGroupsPerStage * G::kHiGroupBytes;
  static constexpr int kStageBytes = kScOff + 2 * kGroupsPerStage * G::kScGroupBytes;  // a multiple of 1024
  static constexpr int kTail = TOK * 4 + TOK * 4 * 4 + 1024;  // row scales, per-quarter partial sums, barriers
  static constexpr int kFit = (kSmemBudget - 1024 - kTail - kUnits * kUnitBytes) / kStageBytes;
  // (two-group TMEM units: a decode warp visits every other stage, so an even ring length keeps it on consecutive
  // uses of the same slots - a parity wait cannot tell uses two apart)
  static constexpr int kStages = kFit > 8 ? 8 : (ATM && kSpu == 2 ? kFit / 2 * 2 : kFit);
  static constexpr int kUnitOff = kStages * kStageBytes;
  static constexpr int kTailOff = kUnitOff + kUnits * kUnitBytes;
  static constexpr int kSmemBytes = 1024 + kTailOff + kTail;
  static constexpr int kTmemCols = ATM ? 512 : kIssuers * kAccCols;  // a power of two (32 ... 512)
  static constexpr int kMmaN = TOK < 256 ? TOK : 256;  // tokens per MMA instruction and per activation box
  static constexpr int kEpiChunks = TOK >= 64 ? 4 : 2;  // decode warps per TMEM lane quarter that run the epilogue
  static constexpr int kColsPerWarp = TOK / kEpiChunks;
  static_assert(kStageBytes % 1024 == 0, "x slots and slices need 1024-byte alignment");
  static_assert(kStages >= 2, "raw ring needs two stages");
  static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");
};

struct UmmaArgs {
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
  int tiles, kg;   // 128-column weight tiles, 64-wide k-groups
  int mblocks;     // token blocks of TOK rows handled in one launch (work item = (token block, weight tile))
  int items;       // tiles * mblocks
  long long units; // items * kg
  int split;
  int cps;         // split with every CTA inside one tile: CTAs per tile (grid = tiles * cps); 0 otherwise
  DecodeConsts dc;
};

__device__ __forceinline__ long long u_begin(const UmmaArgs& a, int cta, int grid) {
  if (a.split) return (long long)cta * a.units / grid;
  return ((long long)cta * a.items / grid) * a.kg;
}

// Bounded wait that also gives up once another thread of the CTA has given up (the flag is polled only on the slow
// path, so a wait that is already satisfied costs one try_wait).
__device__ __forceinline__ bool wait_flag(uint64_t* bar, uint32_t parity, volatile int* abort_flag, unsigned site) {
  if (mbar_try_wait(bar, parity)) return true;
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag) return false;
  }
  report_error(site);
  *abort_flag = 1;
  return false;
}

// ---- tcgen05 wrappers ---------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Both are called by a whole, converged warp with warp-uniform arguments; one elected lane issues. Keeping the
// issuing code warp-uniform lets the descriptors live in uniform registers, which the instruction reads directly.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, leader;\n\t"
      "elect.sync _|leader, 0xffffffff;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "@leader tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// With the A operand in tensor memory an MMA reads [128 lanes][8 columns], column c of lane r = A[r][2c], A[r][2c+1].
// The four MMAs of one 64-wide k-group in one block, so that the election and the operand arithmetic are paid once:
// A = tensor memory columns a_tmem + 8 ks, B = shared-memory descriptor {b_lo + 2 ks, b_hi} (32 bytes per k16 step;
// the 14-bit address field cannot carry), ks = 0..3. The first MMA overwrites the accumulator unless `accumulate`.
__device__ __forceinline__ void umma_group_ta(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p, t, leader;\n\t.reg .b32 a1, a2, a3, l1, l2, l3;\n\t.reg .b64 b0, b1, b2, b3;\n\t"
      "elect.sync _|leader, 0xffffffff;\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "setp.eq.b32 t, %5, %5;\n\t"
      "add.u32 a1, %1, 8;\n\tadd.u32 a2, %1, 16;\n\tadd.u32 a3, %1, 24;\n\t"
      "add.u32 l1, %2, 2;\n\tadd.u32 l2, %2, 4;\n\tadd.u32 l3, %2, 6;\n\t"
      "mov.b64 b0, {%2, %3};\n\tmov.b64 b1, {l1, %3};\n\tmov.b64 b2, {l2, %3};\n\tmov.b64 b3, {l3, %3};\n\t"
      "@leader tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], b0, %4, p;\n\t"
      "@leader tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %4, t;\n\t"
      "@leader tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %4, t;\n\t"
      "@leader tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %4, t;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Registers -> tensor memory, 16 lanes x 32 columns: lane (g = lane >> 2, t = lane & 3) of the warp gives
// r[2 i] to TMEM lane g, column 4 i + t and r[2 i + 1] to TMEM lane g + 8, column 4 i + t - with two bf16 per
// column that is the A fragment of mma.m16n8k16 (rows g / g + 8, k = 2 t + 8 h) for four 16-wide k slabs.
__device__ __forceinline__ void tmem_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile(
      "{\n\t.reg .pred leader;\n\t"
      "elect.sync _|leader, 0xffffffff;\n\t"
      "@leader tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
      ::"r"(smem_u32(bar))
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// K-major operand tile with the 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = uint64_t((addr & 0x3FFFFu) >> 4);
  d |= uint64_t(1) << 16;             // leading byte offset (unused for swizzled K-major)
  d |= uint64_t(1024 >> 4) << 32;     // stride byte offset between 8-row groups
  d |= uint64_t(1) << 46;             // descriptor version of this architecture
  d |= uint64_t(2) << 61;             // 128-byte swizzle
  return d;
}

template <int BITS, int TOK, bool ATM>
__global__ void __launch_bounds__(kThreads, 1)
qgemm_umma_kernel(const __grid_constant__ CUtensorMap xmap, const UmmaArgs a) {
  using C = UCfg<BITS, TOK, ATM>;
  using G = BqGeom<BITS>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = smem_raw + ((1024 - (smem_u32(smem_raw) & 1023)) & 1023);
  uint8_t* stages = smem;
  uint8_t* units = smem + C::kUnitOff;  // per unit: kSpu decoded slices, then kSpu activation slices
  float* rs_sm = reinterpret_cast<float*>(smem + C::kTailOff);
  float* part_sm = rs_sm + TOK;  // [TOK][4]
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(part_sm + TOK * 4);
  uint64_t* raw_empty = raw_full + C::kStages;
  uint64_t* op_full = raw_empty + C::kStages;
  uint64_t* op_empty = op_full + C::kUnits;
  uint64_t* acc_full = op_empty + C::kUnits;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* flags = reinterpret_cast<volatile int*>(tmem_slot + 1);  // [0] abort, [1] last arriver
  static_assert((2 * C::kStages + 2 * C::kUnits + 2) * 8 + 16 <= 1024, "barrier area");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int grid = gridDim.x, cta = blockIdx.x;
  const long long u0 = u_begin(a, cta, grid), u1 = u_begin(a, cta + 1, grid);

  if (tid == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(&raw_full[s], 1);
      mbar_init(&raw_empty[s], C::kRawConsumers);
    }
    for (int s = 0; s < C::kUnits; ++s) {
      mbar_init(&op_full[s], C::kDecodeWarpsPerUnit + 1);  // the unit's decode warps + the activation copies' expect_tx
      mbar_init(&op_empty[s], 1);
    }
    mbar_init(acc_full, C::kIssuers);
    mbar_init(acc_empty, kDecodeWarps);
    flags[0] = 0;
    flags[1] = 0;
    mbar_fence_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, C::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // An allocation of all 512 columns can only start at lane 0, column 0. The weights-in-TMEM variant relies on that:
  // with the base a compile-time constant the MMA's operand addresses are computed in uniform registers, which the
  // instruction reads directly (a base loaded from shared memory costs a register move per operand and MMA).
  const uint32_t tmem_alloc_base = *tmem_slot;
  const bool base_ok = !ATM || tmem_alloc_base == 0;
  const uint32_t tmem_base = ATM ? 0u : tmem_alloc_base;
  if (!base_ok && tid == 0) report_error(0x30A);

  if (!base_ok) {
    // nothing runs; the allocation is released below
  } else if (warp == 0) {
    // ------------------------------ raw-plane producer ------------------------------
    // Lane 0 waits for the slot and posts the byte count; then each copy of the stage is issued by its own lane.
    const uint64_t pol_w = policy_evict_first();
    uint32_t it = 0;
    bool alive = true;
    for (long long u = u0; u < u1 && alive;) {
      const int tile = int(u / a.kg) % a.tiles, kg_a = int(u % a.kg);
      const int kg_b = int(min((long long)a.kg, kg_a + (u1 - u)));
      for (int g = kg_a; g < kg_b && alive; g += kGroupsPerStage, ++it) {
        const int s = it % C::kStages;
        const int ng = min(kGroupsPerStage, kg_b - g);
        int ok = 1;
        if (lane == 0) {
          // a reused stage is free once the decode warps are through with it, and they in turn wait for MMAs that need
          // the previous kernel's output: from here on the bounded waits run on this kernel's time only
          if (it == uint32_t(C::kStages)) pdl_wait();
          ok = wait_flag(&raw_empty[s], ((it / C::kStages) & 1) ^ 1, flags, 0x301) ? 1 : 0;
          if (ok)
            mbar_expect_tx(&raw_full[s], uint32_t(ng) * 2u * (G::kLoGroupBytes + G::kHiGroupBytes + G::kScGroupBytes));
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) {
          alive = false;
          break;
        }
        uint8_t* st = stages + (size_t)s * C::kStageBytes;
        if (lane < 6) {
          const int nbl = lane / 3, kind = lane % 3;
          const size_t grp = (size_t)(tile * 2 + nbl) * a.kg + g;
          if (kind == 0)
            bulk_g2s(st + C::kLoOff + nbl * kGroupsPerStage * G::kLoGroupBytes, a.lo + grp * G::kLoGroupBytes,
                     ng * G::kLoGroupBytes, &raw_full[s], pol_w);
          else if (kind == 1) {
            if constexpr (BITS != 4)
              bulk_g2s(st + C::kHiOff + nbl * kGroupsPerStage * G::kHiGroupBytes, a.hi + grp * G::kHiGroupBytes,
                       ng * G::kHiGroupBytes, &raw_full[s], pol_w);
          } else
            bulk_g2s(st + C::kScOff + nbl * kGroupsPerStage * G::kScGroupBytes, a.sc + grp * G::kScGroupBytes,
                     ng * G::kScGroupBytes, &raw_full[s], pol_w);
        }
        __syncwarp();
      }
      u += kg_b - kg_a;
    }
  } else if (warp == 2) {
    // ------------------------------ activation producer ------------------------------
    // The first thread of the CTA that touches data of earlier kernels: until here the CTA only set itself up and
    // prefetched / decoded weights, which overlaps the previous kernel's tail under programmatic dependent launch.
    if (lane == 0) {
      pdl_wait();
      pdl_launch_dependents();
      uint32_t uc = 0;
      bool alive = true;
      for (long long u = u0; u < u1 && alive;) {
        const int kg_a = int(u % a.kg);
        const int kg_b = int(min((long long)a.kg, kg_a + (u1 - u)));
        const int row0 = (int(u / a.kg) / a.tiles) * TOK;  // first token of this item's token block
        for (int g = kg_a; g < kg_b; g += C::kSpu, ++uc) {
          const int slot = uc % C::kUnits;
          const int nu = min(C::kSpu, kg_b - g);
          alive = wait_flag(&op_empty[slot], ((uc / C::kUnits) & 1) ^ 1, flags, 0x308);
          if (!alive) break;
          uint8_t* xs = units + (size_t)slot * C::kUnitBytes + C::kSpu * C::kWBytes;
          mbar_expect_tx(&op_full[slot], uint32_t(nu) * C::kXBytes);
          for (int gi = 0; gi < nu; ++gi)
#pragma unroll
            for (int nh = 0; nh < TOK / C::kMmaN; ++nh)
              tma_load_2d(xs + gi * C::kXBytes + nh * C::kMmaN * 128, &xmap, (g + gi) * 64, row0 + nh * C::kMmaN,
                          &op_full[slot]);
        }
        u += kg_b - kg_a;
      }
    }
  } else if (warp == 1 || (C::kIssuers == 2 && warp == 3)) {
    // ------------------------------ MMA issuers ------------------------------
    // A warp stays converged and one elected lane issues. Its serial work per unit - one barrier wait, 4 MMAs per
    // slice in one block, one commit - is what bounds the kernel at small TOK (the tensor work of a unit is shorter
    // than any of these), so with two issuers warp 1 takes the even units into accumulator 0 and warp 3 the odd ones
    // into accumulator 1, and ring positions are carried along instead of being derived from counters.
    {
      constexpr uint32_t idesc =
          (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(C::kMmaN >> 3) << 17) | (uint32_t(128 >> 4) << 24);
      constexpr int kI = C::kIssuers;
      const int iss = kI == 2 ? (warp >> 1) : 0;
      const uint32_t d_acc = tmem_base + uint32_t(iss * C::kAccCols);
      const uint64_t desc0 = smem_desc_sw128(smem_u32(units));
      uint32_t seg = 0;
      uint32_t uc0 = 0;  // units of all earlier segments
      bool alive = true;
      // Everything this warp waits for needs the activations, which the previous kernel of the stream produces: the
      // bounded waits below start counting only once that kernel is complete.
      pdl_wait();
      for (long long u = u0; u < u1 && alive; ++seg) {
        const int kg_a = int(u % a.kg);
        const int kg_b = int(min((long long)a.kg, kg_a + (u1 - u)));
        const int nunits = (kg_b - kg_a + C::kSpu - 1) / C::kSpu;
        alive = __all_sync(0xffffffffu, wait_flag(acc_empty, (seg & 1) ^ 1, flags, 0x302));
        tc_fence_after();
        uint32_t accumulate = 0;
        // this warp's first unit of the segment and its ring position
        int i = kI == 2 ? int((uint32_t(iss) - uc0) & 1u) : 0;
        int slot = int((uc0 + uint32_t(i)) % uint32_t(C::kUnits));
        uint32_t par = ((uc0 + uint32_t(i)) / uint32_t(C::kUnits)) & 1u;
        for (; i < nunits && alive; i += kI) {
          const int g = kg_a + i * C::kSpu;
          const int nu = min(C::kSpu, kg_b - g);
          alive = __all_sync(0xffffffffu, wait_flag(&op_full[slot], par, flags, 0x303));
          if (!alive) break;
          tc_fence_after();
          const uint64_t da = desc0 + uint64_t((uint32_t(slot) * C::kUnitBytes) >> 4);
          const uint64_t dx = da + uint64_t((C::kSpu * C::kWBytes) >> 4);
          if constexpr (ATM) {
            static_assert(!ATM || TOK == C::kMmaN, "one MMA covers all tokens");
            const uint32_t ta = tmem_base + uint32_t(C::kACol0 + slot * C::kUnitCols);
            const uint32_t b_lo = uint32_t(dx), b_hi = uint32_t(dx >> 32);
#pragma unroll
            for (int gi = 0; gi < C::kSpu; ++gi) {
              if (gi < nu) {
                umma_group_ta(d_acc, ta + uint32_t(gi * 32), b_lo + uint32_t((gi * C::kXBytes) >> 4), b_hi, idesc,
                              accumulate);
                accumulate = 1;
              }
            }
          } else {
#pragma unroll
            for (int gi = 0; gi < C::kSpu; ++gi) {
              if (gi < nu) {
#pragma unroll
                for (int ks = 0; ks < 4; ++ks) {
#pragma unroll
                  for (int nh = 0; nh < TOK / C::kMmaN; ++nh)
                    umma_bf16(d_acc + uint32_t(nh * C::kMmaN), da + uint64_t((gi * kSliceBytes + ks * 32) >> 4),
                              dx + uint64_t((gi * C::kXBytes + nh * C::kMmaN * 128 + ks * 32) >> 4), idesc, accumulate);
                  accumulate = 1;
                }
              }
            }
          }
          umma_commit(&op_empty[slot]);
          slot += kI;
          if (slot >= C::kUnits) {
            slot -= C::kUnits;
            par ^= 1u;
          }
        }
        umma_commit(acc_full);  // tracks this warp's MMAs only; the barrier counts one arrival per issuer
        uc0 += uint32_t(nunits);
        u += kg_b - kg_a;
      }
    }
  } else if (warp >= kFirstDecodeWarp) {
    // ------------------------------ decode + epilogue warps ------------------------------
    const int dw = warp - kFirstDecodeWarp;
    const int half = dw >> 3;          // which pair of the stage's four k-groups this warp decodes
    const int dnb = (dw >> 2) & 1;     // 64-column block of the tile
    const int ks = dw & 3;             // its k16 slab of the group
    const int gl = lane >> 2, tl = lane & 3;
    DecodeConsts dc;  // in registers: a logic instruction takes only one operand from the constant bank
    asm volatile("mov.b32 %0, %1;" : "=r"(dc.nib) : "r"(a.dc.nib));
    asm volatile("mov.b32 %0, %1;" : "=r"(dc.magic) : "r"(a.dc.magic));
    asm volatile("mov.b32 %0, %1;" : "=r"(dc.himask) : "r"(a.dc.himask));
    const int quarter = dw & 3;        // TMEM lanes this warp may read (warp index modulo 4)
    const int cchunk = dw >> 2;        // which chunk of the token columns it handles in the epilogue
    const bool epi_active = cchunk < C::kEpiChunks;
    const int et = tid - kFirstDecodeWarp * 32;  // 0..511 among the decode threads
    bool dep_passed = false;
    // Wait for an operand slot. Its first use is free; a reused slot is handed back by the MMA warp, whose work needs
    // the previous kernel's output, so the bounded wait starts counting only after that kernel is complete.
    auto wait_slot = [&](int slot, uint32_t par) {
      if (par != 0 && !dep_passed) {
        pdl_wait();
        dep_passed = true;
      }
      return wait_flag(&op_empty[slot], par ^ 1u, flags, 0x306);
    };
    // destination of pair (j, h) of slab ks: row 64 dnb + 8 j + gl, 16-byte chunk (2 ks + h) ^ gl
    const uint32_t row_off = uint32_t(dnb) * 8192u + uint32_t(gl) * 128u + 4u * uint32_t(tl);
    const uint32_t c0_off = row_off + (uint32_t((2 * ks) ^ gl) << 4);
    const uint32_t c1_off = row_off + (uint32_t((2 * ks + 1) ^ gl) << 4);
    // One raw stage (4 k-groups) is decoded in one pass, each warp the same (column block, k16 slab) in two groups.
    // Two-slice units: warps 0-7 take k-groups 0-1 (one unit), warps 8-15 k-groups 2-3, so the slot wait, the proxy
    // fence and the barrier arrival are paid once per two slabs. One-slice units: warps 0-7 take k-groups 0 and 2,
    // warps 8-15 k-groups 1 and 3. Either way a warp's successive units are two apart, so with a ring of two or
    // more units the phase it waits for is never more than one ahead of the barrier (a parity wait cannot tell
    // phases two apart); across a segment boundary the accumulator barrier has seen every earlier commit.
    auto load_raw = [&](const uint8_t* st, int dg, uint32_t (&lo)[4], uint32_t (&hi)[4], uint4& sv) {
      const int rslot = dnb * kGroupsPerStage + dg;
      const uint8_t* lo_g = st + C::kLoOff + rslot * G::kLoGroupBytes;
      const uint8_t* hi_g = st + C::kHiOff + rslot * G::kHiGroupBytes;
      sv = *reinterpret_cast<const uint4*>(st + C::kScOff + rslot * G::kScGroupBytes + 16 * gl);
      const uint4 lv = *reinterpret_cast<const uint4*>(lo_g + ks * 512 + lane * 16);
      lo[0] = lv.x;
      lo[1] = lv.y;
      lo[2] = lv.z;
      lo[3] = lv.w;
      hi[0] = hi[1] = hi[2] = hi[3] = 0;
      if constexpr (BITS == 5) {
        hi[0] = *reinterpret_cast<const uint32_t*>(hi_g + ks * 128 + lane * 4);
      } else if constexpr (BITS == 6) {
        const uint2 hv = *reinterpret_cast<const uint2*>(hi_g + ks * 256 + lane * 8);
        hi[0] = hv.x;
        hi[1] = hv.y;
      } else if constexpr (BITS == 8) {
        const uint4 hv = *reinterpret_cast<const uint4*>(hi_g + ks * 512 + lane * 16);
        hi[0] = hv.x;
        hi[1] = hv.y;
        hi[2] = hv.z;
        hi[3] = hv.w;
      }
    };
    auto store_slice = [&](uint8_t* base, const uint32_t (&w)[16]) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        *reinterpret_cast<uint32_t*>(base + c0_off + j * 1024) = w[2 * j];
        *reinterpret_cast<uint32_t*>(base + c1_off + j * 1024) = w[2 * j + 1];
      }
    };
    // ring positions are carried along (slot + phase bit) instead of being derived from counters by division
    uint32_t seg = 0;
    uint32_t units_done = 0;     // operand units produced so far (all segments): its parity names the issuing warp
    uint32_t stage_no = 0;       // raw stages consumed so far (all segments)
    int s = 0;                   // raw stage and the parity of its current use
    uint32_t s_par = 0;
    int u_slot = 0;              // operand slot of the first unit of the current stage, parity of its current use
    uint32_t u_par = 0;
    auto unit_at = [&](int delta, int& slot, uint32_t& par) {  // ring position `delta` units after (u_slot, u_par)
      slot = u_slot + delta;
      par = u_par;
      while (slot >= C::kUnits) {
        slot -= C::kUnits;
        par ^= 1u;
      }
    };
    for (long long u = u0; u < u1; ++seg) {
      const int item = int(u / a.kg), kg_a = int(u % a.kg);
      const int tile = item % a.tiles;          // weight tile
      const int row0 = (item / a.tiles) * TOK;  // first token of the token block
      const int kg_b = int(min((long long)a.kg, kg_a + (u1 - u)));
      const uint32_t first_unit = units_done;
      if constexpr (ATM) {
        // A warp owns one TMEM lane quarter: 32 of the tile's 128 columns, i.e. half of a 64-column block (pairs
        // j = 4 fh .. 4 fh + 3 of every slab: lo words 2 fh, 2 fh + 1), and decodes whole 64-wide k-groups of it.
        // Two-group units: a stage's two units x four quarters occupy eight warps; warps 0-7 take the even stages of
        // the kernel and warps 8-15 the odd ones, so a warp pays its barrier round trips once per two k-groups and has
        // two stage times for them. One-group units: sixteen warps = four k-groups x four quarters, every stage.
        // The warp walks its own stages only; every stage before a segment's last is full, so the ring positions of
        // its stage and unit follow from the segment's first ones by fixed steps (one wrap at most per step).
        constexpr int kNG = C::kSpu;                      // k-groups per unit
        constexpr int kUPS = kGroupsPerStage / kNG;       // units of a full stage
        constexpr int kStep = kNG == 2 ? 2 : 1;           // distance between this warp's stages
        static_assert(kUPS * kStep <= C::kUnits && kStep <= C::kStages, "one wrap per step");
        const int ui = kNG == 2 ? ((dw >> 2) & 1) : (dw >> 2);
        const int anb = quarter >> 1, fh = quarter & 1;
        const int nst = (kg_b - kg_a + kGroupsPerStage - 1) / kGroupsPerStage;
        const int j0 = kNG == 2 ? int((uint32_t(dw >> 3) - stage_no) & 1u) : 0;
        // ring positions of this warp's first stage and unit of the segment
        int ws = s + j0;
        uint32_t ws_par = s_par;
        if (ws >= C::kStages) {
          ws -= C::kStages;
          ws_par ^= 1u;
        }
        int slot = u_slot + kUPS * j0 + ui;
        uint32_t par = u_par;
        if (slot >= C::kUnits) {
          slot -= C::kUnits;
          par ^= 1u;
        }
        // byte offsets of this lane's words inside a stage (k-group e of the unit adds whole groups)
        const uint32_t lo_off = uint32_t(C::kLoOff + (anb * kGroupsPerStage + ui * kNG) * G::kLoGroupBytes + lane * 16 + fh * 8);
        const uint32_t hi_off = uint32_t(C::kHiOff + (anb * kGroupsPerStage + ui * kNG) * G::kHiGroupBytes);
        const uint32_t sc_off = uint32_t(C::kScOff + (anb * kGroupsPerStage + ui * kNG) * G::kScGroupBytes + 16 * gl + 8 * fh);
        bool alive = true;
        for (int j = j0; j < nst && alive; j += kStep) {
          const int ng = min(kGroupsPerStage, kg_b - kg_a - j * kGroupsPerStage);
          const uint8_t* st = stages + (size_t)ws * C::kStageBytes;
          // Also a warp whose unit does not exist in a partial last stage waits for the stage before it releases
          // it: an arrival that did not wait could be counted with the previous use of the stage (the warp may be
          // a whole turn ahead of a slower one), and the producer would refill a stage that is still being read.
          alive = wait_flag(&raw_full[ws], ws_par, flags, 0x305);
          if (alive && ui * kNG < ng) {
            const uint32_t ta = tmem_base + (uint32_t(32 * quarter) << 16) + uint32_t(C::kACol0 + slot * C::kUnitCols);
#pragma unroll
            for (int e = 0; e < kNG; ++e) {
              if (ui * kNG + e < ng) {  // a unit at the end of a segment may lack its second k-group
                // raw words of the k-group: the lane's two lo words of this half for the four k16 slabs, the matching
                // hi words, the four scales
                uint2 lv[4];
                uint32_t h0[4], h1[4];
                uint32_t s2[8];
                const uint8_t* lo_g = st + lo_off + e * G::kLoGroupBytes;
                const uint8_t* hi_g = st + hi_off + e * G::kHiGroupBytes;
                const uint2 sv = *reinterpret_cast<const uint2*>(st + sc_off + e * G::kScGroupBytes);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  lv[k4] = *reinterpret_cast<const uint2*>(lo_g + k4 * 512);
                  h0[k4] = h1[k4] = 0;
                  if constexpr (BITS == 5) {
                    h0[k4] = *reinterpret_cast<const uint32_t*>(hi_g + k4 * 128 + lane * 4) >> (8 * fh);
                  } else if constexpr (BITS == 6) {
                    h0[k4] = *reinterpret_cast<const uint32_t*>(hi_g + k4 * 256 + lane * 8 + fh * 4);
                  } else if constexpr (BITS == 8) {
                    const uint2 hv = *reinterpret_cast<const uint2*>(hi_g + k4 * 512 + lane * 16 + fh * 8);
                    h0[k4] = hv.x;
                    h1[k4] = hv.y;
                  }
                }
                s2[0] = __byte_perm(sv.x, 0, 0x1010);
                s2[1] = __byte_perm(sv.x, 0, 0x3232);
                s2[2] = __byte_perm(sv.y, 0, 0x1010);
                s2[3] = __byte_perm(sv.y, 0, 0x3232);
                s2[4] = s2[5] = s2[6] = s2[7] = 0;
                if (e == 0) {
                  alive = wait_slot(slot, par);
                  tc_fence_after();
                }
                // rows 0-15 of the quarter (pairs j' = 0, 1), then rows 16-31 (j' = 2, 3): an mma A fragment per slab
                uint32_t f[16];
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  const uint32_t lo[4] = {lv[k4].x, lv[k4].y, 0, 0};
                  const uint32_t hi[4] = {h0[k4], h1[k4], 0, 0};
                  decode_fragment<BITS, 0>(lo, hi, s2, dc, f[4 * k4], f[4 * k4 + 1], f[4 * k4 + 2], f[4 * k4 + 3]);
                }
                if (alive) tmem_st_16x128b_x8(ta + uint32_t(e * 32), f);
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) {
                  const uint32_t lo[4] = {lv[k4].x, lv[k4].y, 0, 0};
                  const uint32_t hi[4] = {h0[k4], h1[k4], 0, 0};
                  decode_fragment<BITS, 1>(lo, hi, s2, dc, f[4 * k4], f[4 * k4 + 1], f[4 * k4 + 2], f[4 * k4 + 3]);
                }
                if (alive) tmem_st_16x128b_x8(ta + (16u << 16) + uint32_t(e * 32), f);
              }
            }
            tmem_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&op_full[slot]);
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(&raw_empty[ws]);
          ws += kStep;
          if (ws >= C::kStages) {
            ws -= C::kStages;
            ws_par ^= 1u;
          }
          slot += kUPS * kStep;
          if (slot >= C::kUnits) {
            slot -= C::kUnits;
            par ^= 1u;
          }
        }
        // the segment's stages and units, for the next segment's first positions
        const uint32_t nun = uint32_t((kg_b - kg_a + kNG - 1) / kNG);
        const uint32_t sn = uint32_t(s) + uint32_t(nst), un = uint32_t(u_slot) + nun;
        s_par ^= (sn / uint32_t(C::kStages)) & 1u;
        s = int(sn % uint32_t(C::kStages));
        u_par ^= (un / uint32_t(C::kUnits)) & 1u;
        u_slot = int(un % uint32_t(C::kUnits));
        stage_no += uint32_t(nst);
        units_done += nun;
      } else {
      for (int g = kg_a; g < kg_b; g += kGroupsPerStage) {
        const int ng = min(kGroupsPerStage, kg_b - g);
        const uint8_t* st = stages + (size_t)s * C::kStageBytes;
        {
          const bool ok = wait_flag(&raw_full[s], s_par, flags, 0x305);
          const int g0 = C::kSpu == 2 ? 2 * half : half;  // first of this warp's two k-groups of the stage
          constexpr int kGStep = C::kSpu == 2 ? 1 : 2;      // distance to its second one
          if (g0 < ng) {
            const bool two = g0 + kGStep < ng;
            uint32_t lo0[4] = {0, 0, 0, 0}, hi0[4] = {0, 0, 0, 0}, lo1[4] = {0, 0, 0, 0}, hi1[4] = {0, 0, 0, 0};
            uint4 sv0 = make_uint4(0, 0, 0, 0), sv1 = sv0;
            if (ok) {
              load_raw(st, g0, lo0, hi0, sv0);
              if (two) load_raw(st, g0 + kGStep, lo1, hi1, sv1);
            }
            uint32_t s2[8], w[16];
            expand_scales(sv0, s2);
            decode_slab<BITS>(lo0, hi0, s2, w, dc);
            if constexpr (C::kSpu == 2) {
              int slot;
              uint32_t par;
              unit_at(half, slot, par);
              const bool free_slot = wait_slot(slot, par);
              uint8_t* base = units + (size_t)slot * C::kUnitBytes;
              if (ok && free_slot) store_slice(base, w);
              if (two) {
                expand_scales(sv1, s2);
                decode_slab<BITS>(lo1, hi1, s2, w, dc);
                if (ok && free_slot) store_slice(base + kSliceBytes, w);
              }
              fence_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(&op_full[slot]);
            } else {
  #pragma unroll
              for (int e = 0; e < 2; ++e) {
                if (e == 0 || two) {
                  if (e == 1) {
                    expand_scales(sv1, s2);
                    decode_slab<BITS>(lo1, hi1, s2, w, dc);
                  }
                  int slot;
                  uint32_t par;
                  unit_at(g0 + kGStep * e, slot, par);
                  const bool free_slot = wait_slot(slot, par);
                  if (ok && free_slot) store_slice(units + (size_t)slot * C::kUnitBytes, w);
                  fence_async_smem();
                  __syncwarp();
                  if (lane == 0) mbar_arrive(&op_full[slot]);
                }
              }
            }
          }
        }
        if constexpr (!ATM) {
          __syncwarp();
          if (lane == 0) mbar_arrive(&raw_empty[s]);
        }
        if (++s == C::kStages) {
          s = 0;
          s_par ^= 1u;
        }
        ++stage_no;
        unit_at((ng + C::kSpu - 1) / C::kSpu, u_slot, u_par);
        units_done += uint32_t((ng + C::kSpu - 1) / C::kSpu);
      }
      }

      // ---- epilogue of this tile segment ----
      if (seg == 0) pdl_wait();  // the accumulator needs the previous kernel's output; so do the row scales below
      const bool got = __all_sync(0xffffffffu, wait_flag(acc_full, seg & 1, flags, 0x307));
      tc_fence_after();
      if (seg == 0 || a.mblocks > 1) {  // the row scales of the folded RMSNorm for this token block
        row_scales_to_smem(a.partials_in ? a.partials_in + (size_t)row0 * (a.hidden / 128) : nullptr, a.m - row0, TOK,
                           a.hidden, a.eps, rs_sm, et, kDecodeThreads);
        named_bar_sync(1, kDecodeThreads);
      }
      const int m_here = a.m - row0;  // valid tokens of this block (may exceed TOK)
      const bool whole = kg_a == 0 && kg_b == a.kg;
      const int n_row = 32 * quarter + lane;  // row of the tile this thread reads from TMEM
      const int n_glob = tile * kTileN + n_row;
      const int n_lim = a.n_store > 0 ? a.n_store : a.n;
      constexpr int kColsPerWarp = C::kColsPerWarp;
      const int col_base = cchunk * kColsPerWarp;
      constexpr int kTileFloats = TOK * kTileN;
      // which accumulators this segment wrote: with two issuers, unit j of the kernel goes to accumulator j & 1, so a
      // segment of one unit leaves the other accumulator with an earlier segment's sums
      const bool acc0_live = C::kIssuers == 1 || units_done - first_unit >= 2u || (first_unit & 1u) == 0u;
      const bool acc1_live = C::kIssuers == 2 && (units_done - first_unit >= 2u || (first_unit & 1u) == 1u);
      // 16 accumulator columns of this thread's row: the sum over the issuers' accumulators
      auto load_acc = [&](int col, float (&v)[16]) {
        const uint32_t taddr = tmem_base + (uint32_t(32 * quarter) << 16) + uint32_t(col);
        uint32_t r[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = 0.0f;
        if (acc0_live) {
          tmem_ld16(taddr, r);
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
        }
        if constexpr (C::kIssuers == 2) {
          if (acc1_live) {
            tmem_ld16(taddr + uint32_t(C::kAccCols), r);
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] += __uint_as_float(r[j]);
          }
        }
      };

      auto finish_chunk = [&](const float (&v)[16], int col0) {
        if (a.kind == Q38_EPI_RESIDUAL) {
          // the old values are requested four at a time before the first new one of the four is stored: a load
          // placed after a store to the same array has to wait for it, and the chunk took sixteen round trips to memory
          constexpr int kRG = 8;
          float rv[kRG];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            if ((j & (kRG - 1)) == 0) {
#pragma unroll
              for (int i = 0; i < kRG; ++i)
                rv[i] = col0 + j + i < m_here ? __ldcg(a.residual + (size_t)(row0 + col0 + j + i) * a.n + n_glob) : 0.0f;
            }
            const int col = col0 + j;
            float r = 0.0f;
            if (col < m_here) {
              r = rv[j & (kRG - 1)] + v[j];
              a.residual[(size_t)(row0 + col) * a.n + n_glob] = r;
              a.xbf[(size_t)(row0 + col) * a.n + n_glob] = __float2bfloat16_rn(r);
            }
            const float ss = warp_sum(r * r);
            if (lane == 0) part_sm[col * 4 + quarter] = ss;
          }
          return;
        }
        // every value is finished before the first store: a shared-memory read placed after a store through a
        // pointer it might alias is held back until that store has left, once per column
        float x[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) x[j] = v[j] * rs_sm[col0 + j];
        const bool n_ok = n_glob < n_lim;
        // bf16 results leave as pairs of neighbouring columns: two lanes that hold neighbouring columns exchange
        // every other token, so that each stores 4 bytes for half of the tokens instead of 2 bytes for all of them.
        // `bit` is the lane distance of the partner, `c` this lane's output column (even in the lower lane of a pair).
        auto store_pairs = [&](int bit, int c, int c_lim, bool lane_on) {
          __nv_bfloat16* base = static_cast<__nv_bfloat16*>(a.out) + (size_t)(row0 + col0) * a.ldo;
          const bool upper = (lane & bit) != 0;
          const bool paired = (a.ldo & 1) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 3u) == 0;  // 4-byte aligned pairs
          if (paired) {
            const int c0p = upper ? c - 1 : c;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const float mine = upper ? x[2 * jj + 1] : x[2 * jj];
              const float theirs = __shfl_xor_sync(0xffffffffu, upper ? x[2 * jj] : x[2 * jj + 1], bit);
              const int tok = 2 * jj + (upper ? 1 : 0);
              const __nv_bfloat162 pr = upper ? __floats2bfloat162_rn(theirs, mine) : __floats2bfloat162_rn(mine, theirs);
              if (lane_on && col0 + tok < m_here) {
                __nv_bfloat16* d = base + (size_t)tok * a.ldo + c0p;
                if (c0p + 1 < c_lim)
                  *reinterpret_cast<__nv_bfloat162*>(d) = pr;
                else if (c0p < c_lim)
                  *d = pr.x;
              }
            }
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
              if (lane_on && col0 + j < m_here && c < c_lim) base[(size_t)j * a.ldo + c] = __float2bfloat16_rn(x[j]);
          }
        };
        if (a.kind == Q38_EPI_SWIGLU) {
          // Lanes 2i / 2i + 1 hold the gate / up column of output column n / 2 for sixteen tokens. They split the tokens
          // (the even lane takes the even ones): each sends the other what it needs and computes eight products, then
          // lanes two apart (neighbouring output columns) exchange every other product and store column pairs.
          const bool odd = (lane & 1) != 0;
          float y[8];
#pragma unroll
          for (int jj = 0; jj < 8; ++jj) {
            const float got_v = __shfl_xor_sync(0xffffffffu, odd ? x[2 * jj] : x[2 * jj + 1], 1);
            y[jj] = odd ? silu_f(got_v) * x[2 * jj + 1] : silu_f(x[2 * jj]) * got_v;
          }
          const int c = n_glob / 2, c_lim = (n_lim + 1) / 2;
          __nv_bfloat16* base = static_cast<__nv_bfloat16*>(a.out) + (size_t)(row0 + col0) * a.ldo;
          if ((a.ldo & 1) == 0 && (reinterpret_cast<uintptr_t>(a.out) & 3u) == 0) {
            const bool upper = (lane & 2) != 0;
            const int c0p = upper ? c - 1 : c;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float theirs = __shfl_xor_sync(0xffffffffu, upper ? y[2 * q] : y[2 * q + 1], 2);
              const int tok = 2 * (2 * q + (upper ? 1 : 0)) + (odd ? 1 : 0);
              const __nv_bfloat162 pr =
                  upper ? __floats2bfloat162_rn(theirs, y[2 * q + 1]) : __floats2bfloat162_rn(y[2 * q], theirs);
              if (col0 + tok < m_here) {
                __nv_bfloat16* d = base + (size_t)tok * a.ldo + c0p;
                if (c0p + 1 < c_lim)
                  *reinterpret_cast<__nv_bfloat162*>(d) = pr;
                else if (c0p < c_lim)
                  *d = pr.x;
              }
            }
          } else {
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
              const int tok = 2 * jj + (odd ? 1 : 0);
              if (col0 + tok < m_here && c < c_lim) base[(size_t)tok * a.ldo + c] = __float2bfloat16_rn(y[jj]);
            }
          }
        } else if (a.kind == Q38_EPI_STORE_BF16) {
          store_pairs(1, n_glob, n_lim, true);
        } else {
          float* dst = static_cast<float*>(a.out) + (size_t)(row0 + col0) * a.ldo + n_glob;
#pragma unroll
          for (int j = 0; j < 16; ++j)
            if (col0 + j < m_here && n_ok) dst[(size_t)j * a.ldo] = x[j];
        }
      };

      bool run_epilogue = true;
      if (whole) {
        if (epi_active) {
#pragma unroll 1
          for (int c0 = 0; c0 < kColsPerWarp; c0 += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            if (got) load_acc(col_base + c0, v);
            finish_chunk(v, col_base + c0);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty);
      } else {
        // stream-K: publish this CTA's partial accumulator [token][128 n], then the last arriver reduces
        float* mine = a.ws + ((size_t)cta * 2 + (kg_a != 0 ? 0 : 1)) * kTileFloats;
        // with one 16-column chunk per warp the thread's own partial sums stay in registers for the reduction
        constexpr bool kKeepOwn = kColsPerWarp == 16;
        float own[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) own[j] = 0.0f;
        if (epi_active) {
#pragma unroll 1
          for (int c0 = 0; c0 < kColsPerWarp; c0 += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            if (got) load_acc(col_base + c0, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) mine[(size_t)(col_base + c0 + j) * kTileN + n_row] = v[j];
            if constexpr (kKeepOwn) {
#pragma unroll
              for (int j = 0; j < 16; ++j) own[j] = v[j];
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(acc_empty);
        // Publication: the CTA's stores are ordered before the barrier, and the one thread that then counts the CTA in
        // fences on both sides of its atomic (the fence is cumulative over what the barrier made visible to it), so
        // whoever sees the full count also sees every piece.
        named_bar_sync(1, kDecodeThreads);
        // the CTAs that hold pieces of this tile: c_first .. c_last; the first of them may have started before the tile
        const long long t_begin = (long long)tile * a.kg, t_end = t_begin + a.kg;
        int c_first, c_last;
        if (a.cps > 0) {  // every CTA inside one tile: no 64-bit divisions
          c_first = tile * a.cps;
          c_last = c_first + a.cps - 1;
        } else {
          c_first = int(t_begin * grid / a.units);
          while (c_first > 0 && u_begin(a, c_first, grid) > t_begin) --c_first;
          while (u_begin(a, c_first + 1, grid) <= t_begin) ++c_first;
          c_last = c_first;
          while (c_last + 1 < grid && u_begin(a, c_last + 1, grid) < t_end) ++c_last;
        }
        if (et == 0) {
          __threadfence();
          const int prev = atomicAdd(&a.counters[tile], 1);
          __threadfence();
          const int last = prev == c_last - c_first;
          if (last) a.counters[tile] = 0;
          flags[1] = last;
        }
        named_bar_sync(1, kDecodeThreads);
        run_epilogue = flags[1] != 0;
        if (run_epilogue && epi_active) {
#pragma unroll 1
          for (int c0 = 0; c0 < kColsPerWarp; c0 += 16) {
            float v[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) v[j] = 0.0f;
            // in CTA order (the sum is the same whichever CTA arrives last); this CTA's own piece comes from registers
            for (int c = c_first; c <= c_last; ++c) {
              if (kKeepOwn && c == cta) {
#pragma unroll
                for (int j = 0; j < 16; ++j) v[j] += own[j];
                continue;
              }
              // c_first begins at or before the tile (this piece is in its second buffer), the others inside it
              const float* src = a.ws + ((size_t)c * 2 + (c != c_first ? 0 : 1)) * kTileFloats;
#pragma unroll
              for (int j = 0; j < 16; ++j) v[j] += __ldcg(src + (size_t)(col_base + c0 + j) * kTileN + n_row);
            }
            finish_chunk(v, col_base + c0);
          }
        }
      }
      if (a.kind == Q38_EPI_RESIDUAL) {
        named_bar_sync(2, kDecodeThreads);
        if (run_epilogue && et < m_here && et < TOK) {
          const float* p = part_sm + et * 4;
          a.partials_out[(size_t)(row0 + et) * (a.n / 128) + tile] = (p[0] + p[1]) + (p[2] + p[3]);
        }
      }
      named_bar_sync(2, kDecodeThreads);
      u += kg_b - kg_a;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_alloc_base, C::kTmemCols);
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

template <int BITS, int TOK, bool ATM>
int launch_one(const __nv_bfloat16* a_ptr, int m, int mblocks, const q38_bq_weight& w, const q38_gemm_epilogue& ep,
               const q38_gemm_workspace* ws, cudaStream_t stream) {
  using C = UCfg<BITS, TOK, ATM>;
  static const cudaError_t attr = cudaFuncSetAttribute(qgemm_umma_kernel<BITS, TOK, ATM>,
                                                       cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
  Q38_CUDA_OK(attr);
  EncodeFn enc = encode_fn();
  Q38_REQUIRE(enc != nullptr, "qgemm: cuTensorMapEncodeTiled is not available from this driver");
  CUtensorMap xmap;
  const cuuint64_t dims[2] = {cuuint64_t(w.k), cuuint64_t(m)};
  const cuuint64_t strides[1] = {cuuint64_t(w.k) * 2};
  const cuuint32_t box[2] = {64, cuuint32_t(C::kMmaN)};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(&xmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<__nv_bfloat16*>(a_ptr), dims, strides,
                         box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  Q38_REQUIRE(r == CUDA_SUCCESS, "qgemm: tensor map encode failed (%d)", int(r));

  UmmaArgs a{};
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
  a.tiles = w.n / kTileN;
  a.kg = w.k / 64;
  a.mblocks = mblocks;
  a.items = a.tiles * mblocks;
  a.units = (long long)a.items * a.kg;
  a.dc = decode_consts(BITS);
  const int sms = num_sms();
  // How the (tile, k-group) list is cut over the CTAs. Every cut inside a tile costs a partial-tile round trip
  // through the workspace and a serial sum by the tile's last CTA, so:
  //   * fewer tiles than SMs: s = SMs / tiles CTAs per tile, every CTA inside one tile (grid = tiles * s makes the
  //     even cut land on tile boundaries); s is capped where the partial tiles are large;
  //   * tiles >= SMs: whole tiles while a CTA gets fewer than four of them or the partial tiles are large (>= 256
  //     tokens), an even cut over all SMs (stream-K) otherwise.
  const bool have_ws = ws && ws->partials && ws->counters && ws->num_counters >= a.tiles;
  int grid;
  if (mblocks > 1) {  // several token blocks per launch: enough whole items to spread, no cut inside a tile
    grid = std::min(sms, a.items);
    a.split = 0;
  } else if (a.tiles < sms) {
    int s = sms / a.tiles;
    s = std::min(s, TOK >= 256 ? 3 : 8);
    s = std::max(1, std::min(s, a.kg / 8));
    if (!have_ws || ws->partial_floats < (size_t)a.tiles * s * 2 * TOK * kTileN) s = 1;
    grid = a.tiles * s;
    a.split = s > 1;
    a.cps = s > 1 ? s : 0;
  } else {
    grid = sms;
    a.split = TOK <= 128 && have_ws && ws->partial_floats >= (size_t)grid * 2 * TOK * kTileN;
    if (a.tiles < 4 * sms) a.split = 0;  // a few tiles per CTA: two fix-ups per CTA cost more than the uneven last wave
  }
  if (a.split) {
    a.ws = ws->partials;
    a.counters = ws->counters;
  }
  (void)launch_kernel(qgemm_umma_kernel<BITS, TOK, ATM>, dim3(grid), dim3(kThreads), C::kSmemBytes, stream, xmap, a);
  Q38_LAUNCH_OK("qgemm_umma_kernel");
  return Q38_OK;
}

template <int BITS>
int launch_bits(int tok, int mblocks, bool a_in_tmem, const __nv_bfloat16* a, int m, const q38_bq_weight& w,
                const q38_gemm_epilogue& ep, const q38_gemm_workspace* ws, cudaStream_t s) {
  if (a_in_tmem) {
    switch (tok) {
      case 32: return launch_one<BITS, 32, true>(a, m, mblocks, w, ep, ws, s);
      case 64: return launch_one<BITS, 64, true>(a, m, mblocks, w, ep, ws, s);
      case 128: return launch_one<BITS, 128, true>(a, m, mblocks, w, ep, ws, s);
      case 256: return launch_one<BITS, 256, true>(a, m, mblocks, w, ep, ws, s);
      default: set_error("qgemm: the weights-in-TMEM kernel serves up to 256 tokens per pass"); return Q38_ERR_INVALID;
    }
  }
  switch (tok) {
    case 32: return launch_one<BITS, 32, false>(a, m, mblocks, w, ep, ws, s);
    case 64: return launch_one<BITS, 64, false>(a, m, mblocks, w, ep, ws, s);
    case 128: return launch_one<BITS, 128, false>(a, m, mblocks, w, ep, ws, s);
    case 256: return launch_one<BITS, 256, false>(a, m, mblocks, w, ep, ws, s);
    default:
      if constexpr (BITS == 8) {
        set_error("qgemm: the 512-token configuration is not built for 8-bit weights");
        return Q38_ERR_INVALID;
      } else {
        return launch_one<BITS, 512, false>(a, m, 1, w, ep, ws, s);
      }
  }
}

}  // namespace

// m <= tok * mblocks, tok in {32, 64, 128, 256, 512} (mblocks > 1: that many token blocks of `tok` rows in one
// launch, whole tiles per CTA; not with tok = 512). Called by the dispatcher in qgemm.cu.
int qgemm_umma_launch(int tok, int mblocks, bool a_in_tmem, const __nv_bfloat16* a, int m, const q38_bq_weight& w,
                      const q38_gemm_epilogue& ep, const q38_gemm_workspace* ws, cudaStream_t s) {
  switch (w.bits) {
    case 4: return launch_bits<4>(tok, mblocks, a_in_tmem, a, m, w, ep, ws, s);
    case 5: return launch_bits<5>(tok, mblocks, a_in_tmem, a, m, w, ep, ws, s);
    case 6: return launch_bits<6>(tok, mblocks, a_in_tmem, a, m, w, ep, ws, s);
    default: return launch_bits<8>(tok, mblocks, a_in_tmem, a, m, w, ep, ws, s);
  }
}

unsigned int qgemm_umma_error(bool clear) { return read_tu_error(clear); }
unsigned int* qgemm_umma_error_address() { return tu_error_address(); }

}  // namespace q38
