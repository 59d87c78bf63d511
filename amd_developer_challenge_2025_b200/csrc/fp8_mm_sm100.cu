// FP8 (e4m3fn) block-scaled GEMM for NVIDIA B200 (sm_100a), bf16 output.
//
// Replaces the reference's HIP/MFMA kernels fp8_mm_128x128_ft2, fp8_mm_128x128_pt,
// insitu_transpose_128x128, fp8_mm_128x128_ft2_split4(+_merge) and
// fp8_mm_32x32_16x16_ft2 (1-amd-fp8-mm/amd-fp8-mm-submission.py:18-511) and the host
// dispatcher fp8_mm (same file, 514-579). The arithmetic kept from the reference is its
// K loop (same file, 302-357): per 128-wide K block the matrix unit accumulates
// P = sum a*b in fp32 from zero, then acc += P * a_scale[row,kb] * b_scale[col/128,kb]
// in fp32 on the vector ALU, and one fp32 -> bf16 rounding at the end.
//
// Structure of one CTA (384 threads, one CTA per SM, persistent over work items):
//   warp 0      TMA producer: A (128 x 128 B) and B tiles of one K block into a SWIZZLE_128B
//               shared-memory ring, completion on an mbarrier per stage
//   warp 1      MMA issuer: 4 x tcgen05.mma.kind::f8f6f4 (K=32 each) per K block into one of
//               the TMEM partial buffers, then ONE tcgen05.commit to the stage's "done" barrier,
//               which both frees the stage for the producer and publishes the buffer to the
//               promotion warps. It waits on ONE barrier per K block: a stage's "full" barrier also
//               collects the promotion warps' release of the TMEM buffer that K block will
//               overwrite (K block j uses stage j mod stages and buffer j mod buffers; a warp that
//               has drained the buffer of K block j arrives on the barrier of K block j + buffers)
//   warp 2      allocates / frees TMEM; its first lane is a second MMA issuer (the two issuers take
//               alternate K blocks)
//   warp 3      scale loader: cp.async of the a_scale / b_scale values of FOUR K blocks at a time
//               into a small shared-memory ring, up to 16 K blocks ahead
//   warps 4-11  promotion + store: tcgen05.ld the partial, fma into register accumulators with
//               the per-row, per-block scale; at the end of a tile the bf16 result goes through a
//               swizzled shared-memory staging buffer and out by TMA store (32 columns x 128 rows
//               per box), or, for split-K, as fp32 partials + last-arriver reduction
// While the tensor core streams operands, shared memory is nearly saturated and every
// shared-memory operation of a warp (mbarrier probe, ld.shared) takes hundreds of clocks, so
// the promotion warps touch shared memory as rarely as possible: one barrier wait and one
// arrive per K block, and the scales of four K blocks fetched with three vector loads.
// Either operand may also be stored MN-major (a as [K][M], b as [K][N]: the layout the reference's
// harness hands over). Such a tile is loaded as K rows of 128 (or 64) contiguous M/N bytes and
// described to the tensor core as an MN-major operand; nothing is transposed in memory.
// Grouped form (one launch for G independent problems of the same N and K, e.g. the experts of an MoE layer):
// a, b, the scales and c carry a leading group dimension, the work list runs over (group, tile), the tensor
// maps are three-dimensional, and an optional device array gives the number of valid rows per group
// (tiles past it are skipped by every role, rows past it are never written).
// With PAIR, two CTAs of a cluster share one 256-row tile: each loads its own 128 rows of A and
// half of the B rows, the leader CTA issues tcgen05.mma.cta_group::2 for both, and each CTA
// promotes and stores its own 128 rows. No TMA load uses cluster multicast.
// Every mbarrier wait is bounded: when it expires the kernel writes a status word and all roles
// leave their loops; nothing traps and nothing spins without limit.

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "b200_fp8_mm.h"

namespace {

constexpr int kBlockM = 128;  // rows of C per CTA
constexpr int kBlockK = 128;  // bytes of e4m3 per row of a stage = one scale block = one 128B swizzle row
constexpr int kMmasPerBlock = 4;  // K = 32 per instruction
constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // default limit of every mbarrier wait: 2 s
constexpr int kCounterBytes = 4096;
constexpr int kMaxCounters = kCounterBytes / 4;
constexpr int kMaxStages = 8;
constexpr int kStoreBoxCols = 32;                                // bf16 columns per TMA store box (64 bytes)
constexpr int kStoreBufBytes = kBlockM * kStoreBoxCols * 2;      // one staging buffer: 128 rows x 64 B
constexpr int kScaleGroup = 4;  // K blocks per scale-ring slot (4 or 8; 8 measured no faster, 10 % slower at BN=128)
constexpr int kScaleSlots = 4;                                   // ring depth (16 K blocks)
constexpr int kScaleSlotFloats = kBlockM * kScaleGroup + 4 * kScaleGroup;  // a[128][4] + b[4][4]
constexpr int kBarrierBytes = 512;                                         // mbarriers and flags
constexpr int kHeaderBytes = ((kBarrierBytes + kScaleSlots * kScaleSlotFloats * 4 + 1023) / 1024) * 1024;

struct KernelParams {
  const float* a_scale;
  const float* b_scale;
  __nv_bfloat16* c;
  float* partials;  // split-K planes, tile-blocked
  int* counters;    // one per (tile, CTA of the pair), zero between launches
  int* status;      // may be null
  long long sa_m, sa_k, sb_n, sb_k, ldc;
  int M, N, K;
  int n_phase;
  int tiles_m, tiles_n, split_k, kblocks;
  int full_tiles;  // tiles [0, full_tiles) run unsplit; the rest are split split_k ways along K
  int raster_group;
  // Reciprocals for decode_work's divisions (see div_small): 1 / (raster_group * tiles_n), 1 / raster_group,
  // 1 / (rows of the last, shorter raster group), 1 / split_k, 1 / (tiles_m * tiles_n).
  float rcp_per_group, rcp_raster, rcp_raster_last, rcp_split, rcp_per_problem;
  int b_scale_rows;
  int vec_store;  // 1 when c, ldc and N allow 16-byte stores
  int stages;
  int tmem_bufs;  // TMEM partial buffers in use: divides stages, at most TileCfg::kTmemBufs
  int issuers;     // MMA-issuing threads in use: 1 or 2
  int store_bufs;  // staging buffers per promotion warpgroup for the TMA store of c: 0 (plain stores), 1 .. 4
  // Operand layout, as the values the producer and the MMA threads need (see OperandLayout below).
  int a_mn, b_mn;            // 1: the operand is MN-major in global and shared memory
  int b_boxes;               // TMA boxes per stage of b (1 when K-major)
  int b_box_cols;            // rows of b (columns of c) per box
  int b_box_bytes;           // shared-memory bytes per box
  uint32_t a_desc_lo, a_desc_hi, a_kstep;  // descriptor bits beside the address; address step per K=32 MMA
  uint32_t b_desc_lo, b_desc_hi, b_kstep;
  uint32_t idesc_major;      // instruction-descriptor bits 15 / 16: a / b is MN-major
  // Grouped launches (groups > 0): M, tiles_m, a_scale/b_scale/c strides are per group.
  int groups;
  const int* m_valid;        // device int[groups]: rows of each group that exist (null: all M)
  long long sa_g, sb_g, c_g; // group strides of a_scale, b_scale (floats) and c (elements)
  unsigned long long wait_limit_ns;  // every mbarrier wait gives up after this long
  // Self-test of the give-up path (b200_fp8_mm_selftest_wait_expiry): the producer of the plain 64-wide
  // single-CTA kernel leaves this K block of the launch's first tile out (no expect_tx, no copy), so the waits
  // that depend on it run into the limit. -1 in every other launch.
  int selftest_skip_kblock;
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}

// shared::cluster address of the same shared-memory location in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}

__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Arrive + expect_tx on a barrier given by its shared::cluster address (own CTA or the peer).
// Default (CTA-scope release) semantics: a cluster-scope release here costs about 0.4 us per call.
__device__ __forceinline__ void mbar_expect_tx_cluster(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}

// One probe of the barrier. The suspend-time hint (nanoseconds) lets the hardware park the thread
// until the phase completes instead of returning at once, so a waiting role costs few issue slots
// and few shared-memory probes.
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(200000)
      : "memory");
  return ok;
}

// Non-blocking probe of the barrier.
__device__ __forceinline__ uint32_t mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Shared flag every role polls while it waits; set by the first wait that expires.
struct AbortCtx {
  volatile int* abort_flag;  // shared memory
  int* status;               // global, may be null
  unsigned long long limit_ns;
};

// Bounded wait. Returns false when the wait expired here or in another role.
__device__ __forceinline__ bool mbar_wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                               unsigned long long limit_ns, int where) {
  const unsigned long long t0 = global_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3u) == 0) {
      if (*abort_flag) return false;
      if (global_ns() - t0 > limit_ns) {
        *abort_flag = 1;
        if (status != nullptr) {
          if (atomicCAS(status, 0, B200_FP8_MM_DEV_WAIT_EXPIRED) == 0) {
            status[1] = where;
            status[2] = static_cast<int>(blockIdx.x);
            status[3] = static_cast<int>(parity);
          }
        }
        return false;
      }
    }
  }
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtx& ctx, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  return mbar_wait_slow(bar, parity, ctx.abort_flag, ctx.status, ctx.limit_ns, where);
}

// TMA tile load into this CTA's shared memory; completion bytes go to `bar`.
template <bool PAIR>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int c0, int c1, uint32_t bar) {
  if constexpr (PAIR) {
    // cta_group::2 form: the mbarrier may live in the peer CTA (the pair's leader).
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            dst),
        "l"(map), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
  }
}

// Three-dimensional forms for grouped launches: the third coordinate is the group.
template <bool PAIR>
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  if constexpr (PAIR) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            dst),
        "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
        : "memory");
  }
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(map), "r"(c0),
               "r"(c1), "r"(c2), "r"(src)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// TMA store of one staged box to c; out-of-range rows and columns are clipped by the hardware.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, uint32_t src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];" ::"l"(map), "r"(c0),
               "r"(c1), "r"(src)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// Waits until at most N of this thread's bulk store groups still read their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void wg_bar_sync(int wg) {
  asm volatile("bar.sync %0, 128;" ::"r"(2 + wg) : "memory");
}

__device__ __forceinline__ void cp_async_4(uint32_t dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}

// The barrier receives one arrival from this thread when all its earlier cp.async have landed.
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Descriptors are passed as their 32-bit halves: only the low word (start address) changes from one
// instruction to the next, which keeps the issuing thread's arithmetic to one add per operand.
template <bool PAIR>
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t a_hi, uint32_t b_hi,
                                        uint32_t idesc, uint32_t accumulate) {
  if constexpr (PAIR) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %4};\n\t"
        "setp.ne.b32 p, %6, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
        "r"(a_lo), "r"(b_lo), "r"(a_hi), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}

// Arrives on `bar` (same shared-memory offset in both CTAs of a pair) when all MMAs issued so
// far by this thread have completed.
template <bool PAIR>
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  if constexpr (PAIR) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
        "h"(static_cast<uint16_t>(3))
        : "memory");
  } else {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  }
}

// 32 lanes x 32 columns of fp32: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// Waits for this thread's outstanding tcgen05.ld; the registers pass through the statement so
// that no use of them can be scheduled above it.
__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
        "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
        "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31])
      :
      : "memory");
}

// 64-column variants.
__device__ __forceinline__ void tmem_ld(uint32_t taddr, uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31]),
        "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]),
        "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]),
        "=r"(v[48]), "=r"(v[49]), "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]),
        "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]), "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
      : "r"(taddr)
      : "memory");
}

__device__ __forceinline__ void tmem_ld_wait(uint32_t (&v)[64]) {
  asm volatile(
      "tcgen05.wait::ld.sync.aligned;"
      : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
        "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15]),
        "+r"(v[16]), "+r"(v[17]), "+r"(v[18]), "+r"(v[19]), "+r"(v[20]), "+r"(v[21]), "+r"(v[22]), "+r"(v[23]),
        "+r"(v[24]), "+r"(v[25]), "+r"(v[26]), "+r"(v[27]), "+r"(v[28]), "+r"(v[29]), "+r"(v[30]), "+r"(v[31]),
        "+r"(v[32]), "+r"(v[33]), "+r"(v[34]), "+r"(v[35]), "+r"(v[36]), "+r"(v[37]), "+r"(v[38]), "+r"(v[39]),
        "+r"(v[40]), "+r"(v[41]), "+r"(v[42]), "+r"(v[43]), "+r"(v[44]), "+r"(v[45]), "+r"(v[46]), "+r"(v[47]),
        "+r"(v[48]), "+r"(v[49]), "+r"(v[50]), "+r"(v[51]), "+r"(v[52]), "+r"(v[53]), "+r"(v[54]), "+r"(v[55]),
        "+r"(v[56]), "+r"(v[57]), "+r"(v[58]), "+r"(v[59]), "+r"(v[60]), "+r"(v[61]), "+r"(v[62]), "+r"(v[63])
      :
      : "memory");
}

template <int THREADS>
__device__ __forceinline__ void epi_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(THREADS) : "memory");
}

// Two fp32 accumulators live in one 64-bit register: acc.{lo,hi} += p.{0,1} * s.{lo,hi} with one
// packed instruction (half the issue slots of two scalar fmas; the pack of p0/p1 costs nothing when
// they are adjacent registers, which the outputs of one tcgen05.ld are).
__device__ __forceinline__ void fma2(unsigned long long& acc, uint32_t p0, uint32_t p1, unsigned long long s2) {
  asm("{\n\t.reg .b64 pp;\n\t"
      "mov.b64 pp, {%1, %2};\n\t"
      "fma.rn.f32x2 %0, pp, %3, %0;\n\t}"
      : "+l"(acc)
      : "r"(p0), "r"(p1), "l"(s2));
}

__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
  unsigned long long r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}

__device__ __forceinline__ float2 unpack2(unsigned long long v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// Shared-memory matrix descriptor (sm_100 format), as two 32-bit words.
// Low word: start address in 16-byte units (bits 0-13), leading byte offset in 16-byte units (bits 16-29).
// High word: stride byte offset in 16-byte units (bits 0-13), version 1 (bit 14), swizzle mode (bits 29-31:
// 2 = 128-byte, 4 = 64-byte).
// K-major, 128-byte swizzle (a stage row = 128 bytes of K of one matrix row): 8-row groups 1024 bytes apart
// (stride offset), leading offset unused (1); the next K=32 slice starts 32 bytes further in the row.
// MN-major (a stage row = 128 or 64 contiguous bytes along M/N of one k): the 8-row groups along K are the
// stride offset (8 x row pitch), the leading offset is the distance between blocks of 128 (64) M/N values
// (one TMA box each); the next K=32 slice starts 32 rows further.
__device__ __forceinline__ uint32_t smem_desc_addr(uint32_t smem_addr) { return (smem_addr >> 4) & 0x3fffu; }

struct OperandLayout {
  uint32_t desc_lo, desc_hi, kstep;
  int boxes, box_cols, box_bytes;
};

// rows = M/N extent of the operand's stage tile (128 for a, block_n for b).
inline OperandLayout operand_layout(bool mn_major, int rows) {
  OperandLayout L;
  if (!mn_major) {
    L.desc_lo = 1u << 16;
    L.desc_hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    L.kstep = 32u >> 4;
    L.boxes = 1;
    L.box_cols = rows;
    L.box_bytes = rows * kBlockK;
    return L;
  }
  const int span = (rows % 128 == 0) ? 128 : 64;  // bytes of M/N per shared-memory row = swizzle span
  L.boxes = rows / span;
  L.box_cols = span;
  L.box_bytes = span * kBlockK;                   // 128 k-rows
  L.desc_lo = static_cast<uint32_t>(L.box_bytes >> 4) << 16;
  L.desc_hi = static_cast<uint32_t>((8 * span) >> 4) | (1u << 14) | ((span == 128 ? 2u : 4u) << 29);
  L.kstep = static_cast<uint32_t>((32 * span) >> 4);
  return L;
}

// kind::f8f6f4 instruction descriptor: D = fp32, A = B = e4m3, both K-major, M x N as given.
__host__ __device__ constexpr uint32_t make_idesc(int umma_m, int umma_n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | (0u << 15) | (0u << 16) |
         (static_cast<uint32_t>(umma_n >> 3) << 17) | (static_cast<uint32_t>(umma_m >> 4) << 24);
}

template <int BN, bool PAIR>
struct TileCfg {
  static constexpr int kTileM = PAIR ? 2 * kBlockM : kBlockM;  // rows of C per tile
  static constexpr int kRowsB = PAIR ? BN / 2 : BN;            // rows of B this CTA loads per stage
  static constexpr int kStageBytesA = kBlockM * kBlockK;
  static constexpr int kStageBytesB = kRowsB * kBlockK;
  static constexpr int kStageBytes = kStageBytesA + kStageBytesB;
  static constexpr int kTmemBufs = (BN <= 128) ? 4 : 2;
  static constexpr int kTmemColsUsed = kTmemBufs * BN;
  static constexpr int kTmemCols = kTmemColsUsed <= 256 ? 256 : 512;  // power of two >= 32
  // Promotion warps: groups of four (one per TMEM lane quarter), each group owning a share of the
  // tile's columns. Two groups everywhere: a third group for the 192-wide tile (64 columns per
  // thread instead of 96) was measured 6-15 % slower, more warps meaning more shared-memory
  // barrier traffic on an already saturated shared-memory path.
  static constexpr int kEpiWarps = 8;
  static constexpr int kEpiGroups = kEpiWarps / 4;
  static constexpr int kEpiThreads = kEpiWarps * 32;
  static constexpr int kThreads = 128 + kEpiThreads;
  static constexpr int kColsPerThread = BN / kEpiGroups;
  // Register split after setmaxnreg (light: producer / MMA / loader warps, heavy: promotion warps):
  // 128 * light + kEpiThreads * heavy is at most the allocation the CTA is launched with
  // (384 threads x 168 registers).
  // The 256-wide pair tile trades registers of the light warps for a 64-register landing area in the promotion
  // warps (128 accumulators + 64 + addressing): two 64-column fetches per K block instead of four 32-column
  // ones measured 1.7 % faster on the headline GEMM. The single-CTA 256-wide kernel keeps the old split: its
  // light warps spill at 56 registers and it ran 40 % slower.
  static constexpr bool kWideLanding = (BN == 256) && PAIR;
  static constexpr int kRegsLight = kWideLanding ? 56 : 104;
  static constexpr int kRegsHeavy = kWideLanding ? 224 : 200;
  // Columns fetched from TMEM per tcgen05.ld: as wide as the registers allow without spilling
  // next to the accumulators. tcgen05.wait::ld waits for every outstanding fetch; keeping two
  // 32-column fetches in flight with two landing areas was measured 5-8 % slower than one at a time.
  static constexpr int kChunkCols = (kColsPerThread == 64 || kWideLanding) ? 64 : 32;
  static constexpr int kChunks = kColsPerThread / kChunkCols;
  // Accumulators as packed pairs (fma.rn.f32x2: half the issue slots) or as scalars. With 128 columns per
  // thread the packed form spills (the pairs want aligned 64-bit registers next to a 32-register landing
  // area); scalars fit, and the 256-wide pair plan went from 442 to 262 us on the headline GEMM.
  static constexpr bool kScalarAcc = (BN == 256);
  // At BN=256 the first 64 of a thread's 128 columns stay packed (no spill, 1 % faster than all scalar);
  // 96 packed columns spill again.
  static constexpr int kPackedCols = kScalarAcc ? 64 : kColsPerThread;
  // Narrow tiles: the promotion warps probe the next K block's barrier (non-blocking) right after they
  // release a buffer, so the answer arrives during the fmas and the blocking wait is skipped when the
  // block is already there. Measured -3 % at 64 and 128 columns, 0 at 256, +2.6 % on 192-wide pairs.
  static constexpr bool kEarlyProbe = (BN <= 128);


  static_assert(BN % 64 == 0 && BN >= 64 && BN <= 256, "block_n must be 64, 128, 192 or 256");
};

struct WorkItem {
  int m0, n0, tile, split, nsplit, kb_begin, kb_end;
  int group;    // 0 unless grouped
  int m_limit;  // rows [0, m_limit) of the group exist; a tile with m0 >= m_limit is skipped by every role
  bool skip;
};

// n / d for 0 <= n < 2^22 and d >= 1, with rcp = 1.0f / d: the float quotient is off by at most one, which the
// remainder corrects. Every role decodes one work item per tile; the hardware has no integer divide, and the
// compiler's division sequences (the 64-bit ones above all) cost about a thousand clocks per item, which tiles of
// two to four K blocks feel.
__device__ __forceinline__ int div_small(int n, int d, float rcp) {
  int q = __float2int_rz(__int2float_rn(n) * rcp);
  const int r = n - q * d;
  if (r < 0) {
    --q;
  } else if (r >= d) {
    ++q;
  }
  return q;
}
constexpr int kDivSmallLimit = 1 << 22;

// Work item w -> tile and K range. Tiles are walked in groups of raster_group tile rows, column
// by column inside a group, so that the CTAs running at one time share A and B tiles in L2.
template <bool GENERIC>
__device__ __forceinline__ WorkItem decode_work(const KernelParams& p, int w, int tile_m, int block_n) {
  WorkItem it;
  int t;
  if (w < p.full_tiles) {
    t = w;
    it.split = 0;
    it.nsplit = 1;
  } else {
    // The tail: tiles that would fill only part of a last wave are cut along K so that every CTA
    // gets a share of them.
    const int r = w - p.full_tiles;
    const int q = (r < kDivSmallLimit) ? div_small(r, p.split_k, p.rcp_split) : r / p.split_k;
    t = p.full_tiles + q;
    it.split = r - q * p.split_k;
    it.nsplit = p.split_k;
  }
  const bool small = t < kDivSmallLimit;
  it.tile = t;
  it.group = 0;
  it.m_limit = p.M;
  if (GENERIC && p.groups > 0) {
    const int per_problem = p.tiles_m * p.tiles_n;
    it.group = small ? div_small(t, per_problem, p.rcp_per_problem) : t / per_problem;
    t -= it.group * per_problem;
    if (p.m_valid != nullptr) it.m_limit = max(0, min(p.M, __ldg(p.m_valid + it.group)));
  }
  const int per_group = p.raster_group * p.tiles_n;
  const int group = small ? div_small(t, per_group, p.rcp_per_group) : t / per_group;
  const int first_m = group * p.raster_group;
  const bool whole = first_m + p.raster_group <= p.tiles_m;
  const int gsize = whole ? p.raster_group : p.tiles_m - first_m;
  const int within = t - group * per_group;
  const int tn = small ? div_small(within, gsize, whole ? p.rcp_raster : p.rcp_raster_last) : within / gsize;
  const int tm = first_m + (within - tn * gsize);
  it.m0 = tm * tile_m;
  it.n0 = tn * block_n;
  it.skip = GENERIC && it.m0 >= it.m_limit;
  if (it.nsplit == 1) {
    it.kb_begin = 0;
    it.kb_end = p.kblocks;
  } else {
    // split < nsplit <= 64 and kblocks < 2^24: the products fit 32 bits
    it.kb_begin = static_cast<int>((static_cast<unsigned>(it.split) * static_cast<unsigned>(p.kblocks)) /
                                   static_cast<unsigned>(it.nsplit));
    it.kb_end = static_cast<int>((static_cast<unsigned>(it.split + 1) * static_cast<unsigned>(p.kblocks)) /
                                 static_cast<unsigned>(it.nsplit));
  }
  return it;
}

// ---------------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------------

// GENERIC = false is the plain case (K-major a and b, one problem): operand layout and work list are
// compile-time facts and none of the MN-major / grouped code is in the instruction stream of the
// single-thread roles, whose per-K-block instruction count is on the critical path of narrow tiles.
template <int BN, bool PAIR, bool GENERIC>
__global__ void __launch_bounds__((TileCfg<BN, PAIR>::kThreads), 1)
fp8_mm_blockscaled_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                          const __grid_constant__ CUtensorMap tmap_c, const KernelParams p) {
  using Cfg = TileCfg<BN, PAIR>;
  extern __shared__ uint8_t smem_raw[];
  // SWIZZLE_128B tiles need 1024-byte alignment.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int stages = p.stages;
  const int nbufs = p.tmem_bufs;
  // Barriers, flags and the scale ring sit at fixed offsets in front of the operand ring, so that every
  // role can form their addresses from one base register.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  float* scale_ring = reinterpret_cast<float*>(smem + kBarrierBytes);
  uint8_t* ring = smem + kHeaderBytes;
  uint64_t* full_bar = bars;                                 // [kMaxStages]
  uint64_t* done_bar = bars + kMaxStages;                    // [kMaxStages]
  uint64_t* scale_full_bar = bars + 2 * kMaxStages + 8;      // [kScaleSlots]
  uint64_t* scale_empty_bar = scale_full_bar + kScaleSlots;  // [kScaleSlots]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(scale_empty_bar + kScaleSlots);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  volatile int* last_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 2);
  // staging for the TMA store of c: [warpgroup][buffer][128 rows x 64 B], behind the ring (1024-byte aligned:
  // the header and every stage are multiples of 1024 bytes)
  uint8_t* staging = ring + stages * Cfg::kStageBytes;

  const int warp = static_cast<int>(threadIdx.x) >> 5;
  const int lane = static_cast<int>(threadIdx.x) & 31;
  const AbortCtx ctx{abort_flag, p.status, p.wait_limit_ns};
  const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kMaxStages; ++s) {
      // one arrive.expect_tx per producing CTA + one release per promotion warp (of both CTAs)
      mbar_init(smem_u32(&full_bar[s]), (PAIR ? 2 : 1) * (1 + Cfg::kEpiWarps));
      mbar_init(smem_u32(&done_bar[s]), 1);  // the MMA thread's commit
    }
    for (int s = 0; s < kScaleSlots; ++s) {
      mbar_init(smem_u32(&scale_full_bar[s]), 32);
      mbar_init(smem_u32(&scale_empty_bar[s]), Cfg::kEpiWarps);
    }
    *abort_flag = 0;
    *last_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b) : "memory");
    if (p.store_bufs > 0) asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_c) : "memory");
  }
  if (warp == 2) {
    if constexpr (PAIR) {
      asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_base_slot)),
                   "r"(Cfg::kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    } else {
      asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                       smem_u32(tmem_base_slot)),
                   "r"(Cfg::kTmemCols)
                   : "memory");
      asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();  // the peer's barriers are initialised before any remote arrive
  tcgen05_fence_after();
  // The TMEM base address is read again inside each role instead of being carried across the register
  // re-allocation below: a value that is live in every role at once gets one register for all of them, which
  // the promotion warps' accumulators then push out to local memory for everybody.

  // The extent of the work list (kept out of registers across the role split for the same reason).
  auto work_total = [&]() {
    const int all_tiles = p.tiles_m * p.tiles_n * ((GENERIC && p.groups > 0) ? p.groups : 1);
    return p.full_tiles + (all_tiles - p.full_tiles) * p.split_k;
  };
  auto work_begin = [&]() { return PAIR ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x); };
  auto work_stride = [&]() { return PAIR ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x); };

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(Cfg::kRegsLight));
    if (warp == 0) {
      // ---------------- TMA producer ----------------
      if (lane == 0) {
        const int total_work = work_total(), work_step = work_stride();
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int w = work_begin(); w < total_work && ok; w += work_step) {
          const WorkItem it = decode_work<GENERIC>(p, w, Cfg::kTileM, BN);
          if (it.skip) continue;
          const int a_row = it.m0 + static_cast<int>(cta_rank) * kBlockM;
          const int b_row = it.n0 + static_cast<int>(cta_rank) * (PAIR ? Cfg::kRowsB : 0);
          for (int kb = it.kb_begin; kb < it.kb_end; ++kb) {
            if (!mbar_wait(smem_u32(&done_bar[stage]), phase ^ 1u, ctx, 0x100 | stage)) {
              ok = false;
              break;
            }
            if constexpr (BN == 64 && !PAIR && !GENERIC) {
              if (kb == p.selftest_skip_kblock && w == work_begin()) {  // self-test only: this block never arrives
                if (++stage == stages) {
                  stage = 0;
                  phase ^= 1u;
                }
                continue;
              }
            }
            // Both CTAs of a pair report to the leader's barrier: its MMA thread consumes the stage.
            const uint32_t fb = PAIR ? map_to_cta(smem_u32(&full_bar[stage]), 0) : smem_u32(&full_bar[stage]);
#ifdef FP8MM_X_NOTMA
            mbar_expect_tx_cluster(fb, 0);
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
            continue;
#endif
            mbar_expect_tx_cluster(fb, Cfg::kStageBytes);
            const uint32_t sa = smem_u32(ring + stage * Cfg::kStageBytes);
            // K-major: x = byte of K, y = matrix row. MN-major: x = matrix row (a multiple of 64), y = k.
            if (GENERIC && p.groups > 0) {
              tma_load_3d<PAIR>(sa, &tmap_a, kb * kBlockK, a_row, it.group, fb);
              tma_load_3d<PAIR>(sa + Cfg::kStageBytesA, &tmap_b, kb * kBlockK, b_row, it.group, fb);
            } else {
            if (!GENERIC || !p.a_mn) {
              tma_load_2d<PAIR>(sa, &tmap_a, kb * kBlockK, a_row, fb);
            } else {
              tma_load_2d<PAIR>(sa, &tmap_a, a_row, kb * kBlockK, fb);
            }
            if (!GENERIC || !p.b_mn) {
              tma_load_2d<PAIR>(sa + Cfg::kStageBytesA, &tmap_b, kb * kBlockK, b_row, fb);
            } else {
              for (int i = 0; i < p.b_boxes; ++i)
                tma_load_2d<PAIR>(sa + Cfg::kStageBytesA + static_cast<uint32_t>(i * p.b_box_bytes), &tmap_b,
                                  b_row + i * p.b_box_cols, kb * kBlockK, fb);
            }
            }
            if (++stage == stages) {
              stage = 0;
              phase ^= 1u;
            }
          }
        }
        if (!ok || *abort_flag) {
          // Some wait ran out. Copies this thread issued may still be landing in shared memory: give them far
          // longer than a copy takes (a bounded pause, not a wait on anything) before the CTA is torn down.
          const unsigned long long t0 = global_ns();
          while (global_ns() - t0 < 100000ull) __nanosleep(2000);
        }
      }
      __syncwarp();
    } else if (warp == 1 || warp == 2) {
      // ---------------- MMA issuers (the leader CTA of a pair issues for both) ----------------
      // Up to two threads, one in each warp, take alternate K blocks. A K block's MMAs go to a TMEM
      // buffer of their own, so the two streams need no ordering between them; one thread alone spends
      // about 700 clocks per K block on its barrier wait and on issuing (an MMA costs the issuing
      // thread roughly 100 clocks), more than the tensor pipe needs for a narrow tile's block.
      if (lane == 0 && cta_rank == 0 && warp - 1 < p.issuers) {
        constexpr uint32_t kHiK = (1024u >> 4) | (1u << 14) | (2u << 29);  // K-major, 128-byte swizzle
        const uint32_t idesc = make_idesc(Cfg::kTileM, BN) | (GENERIC ? p.idesc_major : 0u);
        const uint32_t a_hi = GENERIC ? p.a_desc_hi : kHiK, b_hi = GENERIC ? p.b_desc_hi : kHiK;
        const uint32_t a_kstep = GENERIC ? p.a_kstep : 2u, b_kstep = GENERIC ? p.b_kstep : 2u;
        const uint32_t a_lo_bits = GENERIC ? p.a_desc_lo : (1u << 16), b_lo_bits = GENERIC ? p.b_desc_lo : (1u << 16);
        const int me = warp - 1;
        const int total_work = work_total(), work_step = work_stride();
        const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);
        // Each issuer visits only its own K blocks (every issuers-th one of the CTA's whole sequence, across
        // tile boundaries) and keeps its ring position with add-and-wrap only: no division and no work for
        // the other issuer's blocks on this thread, whose scalar instructions are on the critical path.
        const int step = p.issuers;
        int my_stage = me % stages, my_buf = me % nbufs;
        uint32_t my_phase = (me / stages) & 1u;
        int first = me;  // offset of this issuer's next K block from the start of the next tile
        bool ok = true;
        for (int w = work_begin(); w < total_work && ok; w += work_step) {
          const WorkItem it = decode_work<GENERIC>(p, w, Cfg::kTileM, BN);
          if (it.skip) continue;
          int kb = it.kb_begin + first;
          for (; kb < it.kb_end; kb += step) {
            const uint32_t sa = smem_u32(ring + my_stage * Cfg::kStageBytes);
            const uint32_t a_lo = smem_desc_addr(sa) | a_lo_bits;
            const uint32_t b_lo = smem_desc_addr(sa + Cfg::kStageBytesA) | b_lo_bits;
            const uint32_t d_addr = tmem_base + static_cast<uint32_t>(my_buf * BN);
            // operands landed AND the TMEM buffer of this K block drained (see the promotion warps)
            if (!mbar_wait(smem_u32(&full_bar[my_stage]), my_phase, ctx, 0x300 | my_stage)) {
              ok = false;
              break;
            }
            tcgen05_fence_after();
#ifndef FP8MM_X_NOMMA
#pragma unroll
            for (int k = 0; k < kMmasPerBlock; ++k) {
              // next K=32 slice: 32 bytes further inside the swizzle row (K-major) or 32 rows further
              umma_f8<PAIR>(d_addr, a_lo + a_kstep * k, b_lo + b_kstep * k, a_hi, b_hi, idesc, k > 0 ? 1u : 0u);
            }
#endif
            umma_commit<PAIR>(smem_u32(&done_bar[my_stage]));
            my_stage += step;
            if (my_stage >= stages) {
              my_stage -= stages;
              my_phase ^= 1u;
            }
            my_buf += step;
            while (my_buf >= nbufs) my_buf -= nbufs;
          }
          first = kb - it.kb_end;
        }
      }
      __syncwarp();
    } else if (warp == 3) {
      // ---------------- scale loader ----------------
      // One ring slot holds the scales of kScaleGroup consecutive K blocks of the current tile:
      // a[row][u] for the CTA's 128 rows and b[j][u] for the (up to 4) b_scale rows the tile touches.
      const int total_work = work_total(), work_step = work_stride();
      int slot = 0;
      uint32_t sphase = 0;
      bool ok = true;
      for (int w = work_begin(); w < total_work && ok; w += work_step) {
        const WorkItem it = decode_work<GENERIC>(p, w, Cfg::kTileM, BN);
        if (it.skip) continue;
        const int row0 = it.m0 + static_cast<int>(cta_rank) * kBlockM;
        const float* a_base = p.a_scale + static_cast<long long>(it.group) * p.sa_g;
        const float* a_src[4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
          a_src[r] = a_base + static_cast<long long>(min(row0 + lane + 32 * r, p.M - 1)) * p.sa_m;
        // lanes 0..15: b_scale row (n0 + n_phase)/128 + lane/4 (clamped), K block offset lane%4
        const int jb = min(((it.n0 + p.n_phase) >> 7) + ((lane / kScaleGroup) & 3), p.b_scale_rows - 1);
        const float* b_src = p.b_scale + static_cast<long long>(it.group) * p.sb_g + static_cast<long long>(jb) * p.sb_n;
        for (int kb = it.kb_begin; kb < it.kb_end; kb += kScaleGroup) {
          if (!mbar_wait(smem_u32(&scale_empty_bar[slot]), sphase ^ 1u, ctx, 0x500 | slot)) {
            ok = false;
            break;
          }
          const uint32_t dst = smem_u32(scale_ring + slot * kScaleSlotFloats);
#pragma unroll
          for (int r = 0; r < 4; ++r) {
#pragma unroll
            for (int u = 0; u < kScaleGroup; ++u) {
              const int kk = min(kb + u, it.kb_end - 1);  // the tail of a K range repeats its last block
              cp_async_4(dst + static_cast<uint32_t>(4 * ((lane + 32 * r) * kScaleGroup + u)),
                         a_src[r] + static_cast<long long>(kk) * p.sa_k);
            }
          }
          if (lane < 4 * kScaleGroup) {
            const int kk = min(kb + (lane % kScaleGroup), it.kb_end - 1);
            cp_async_4(dst + static_cast<uint32_t>(4 * (kBlockM * kScaleGroup + lane)),
                       b_src + static_cast<long long>(kk) * p.sb_k);
          }
          cp_async_arrive_noinc(smem_u32(&scale_full_bar[slot]));
          if (++slot == kScaleSlots) {
            slot = 0;
            sphase ^= 1u;
          }
        }
      }
      // Nothing may still be writing shared memory when the CTA exits.
      asm volatile("cp.async.wait_all;" ::: "memory");
    }
  } else {
    // ---------------- promotion + store ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(Cfg::kRegsHeavy));
    const int ew = warp - 4;
    const int total_work = work_total(), work_step = work_stride();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);
    const int quarter = warp & 3;  // TMEM lanes [32*quarter, +32) belong to warps with this id mod 4
    const int half = ew >> 2;      // column group of this warp: which share of the tile's columns
    const int row_in_tile = quarter * 32 + lane;
    const int col_base = half * Cfg::kColsPerThread;
    const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
    const int epi_tid = static_cast<int>(threadIdx.x) - 128;
    // "Buffer drained" is reported to the full barrier of the stage whose K block will overwrite the
    // buffer: kTmemBufs K blocks after the one just read. The MMA thread that waits on it lives in
    // the leader CTA.
    const uint32_t full_base = PAIR ? map_to_cta(smem_u32(&full_bar[0]), 0) : smem_u32(&full_bar[0]);
    const uint32_t ready_base = smem_u32(&done_bar[0]);
    auto release_to = [&](int st) {
      if (lane == 0) {
        if constexpr (PAIR) {
          mbar_arrive_cluster(full_base + static_cast<uint32_t>(st * 8));
        } else {
          mbar_arrive(full_base + static_cast<uint32_t>(st * 8));
        }
      }
    };
    // A wait of the whole warp, with the same outcome in every lane (the warp-wide TMEM fetches need all 32).
    // (Every lane probes the barrier itself: one lane probing for the warp and broadcasting its answer measured
    // 5 % slower, and one arrival per warpgroup behind a named barrier instead of one per warp 2 % slower.)
    auto warp_wait = [&](uint32_t bar, uint32_t parity, int where) -> bool {
      return __all_sync(0xffffffffu, mbar_wait(bar, parity, ctx, where));
    };
    // Nothing was read before the first kTmemBufs K blocks: their buffers start out drained.
    for (int b = 0; b < nbufs; ++b) release_to(b);
    int rel_stage = nbufs % stages;

    int buf = 0, slot = 0, cstage = 0;
    uint32_t ready_next = 0;  // kEarlyProbe: the next K block's barrier was seen complete
    uint32_t scale_ready = 0;  // the next scale slot's barrier was seen complete
    uint32_t cphase = 0, sphase = 0;
    bool ok = true;

    // `ok` turns false when a wait of this warp ran out (or another role's did: the shared abort flag). The
    // warp then stops waiting, fetching and storing but still walks the remaining tiles and takes part in
    // every named barrier of their epilogues, so that warps which have not noticed yet are never left alone
    // at a barrier; they notice at their next wait.
    for (int w = work_begin(); w < total_work; w += work_step) {
      const WorkItem it = decode_work<GENERIC>(p, w, Cfg::kTileM, BN);
      if (it.skip) continue;
      const int row = it.m0 + static_cast<int>(cta_rank) * kBlockM + row_in_tile;
      // Index of this thread's first b_scale row inside a ring slot (at most 2 rows per 128 columns).
      const int gcol0 = it.n0 + col_base + p.n_phase;
      const int jb0 = gcol0 >> 7;
      const int bi0 = jb0 - ((it.n0 + p.n_phase) >> 7);

      constexpr int kPackedCols = Cfg::kPackedCols;
      constexpr int kScalarCols = Cfg::kColsPerThread - kPackedCols;
      unsigned long long acc2[kPackedCols / 2 > 0 ? kPackedCols / 2 : 1];
      float accf[kScalarCols > 0 ? kScalarCols : 1];
#pragma unroll
      for (int j = 0; j < (kPackedCols / 2 > 0 ? kPackedCols / 2 : 1); ++j) acc2[j] = 0ull;
#pragma unroll
      for (int j = 0; j < (kScalarCols > 0 ? kScalarCols : 1); ++j) accf[j] = 0.f;

      // One K block's fmas on CC landed columns starting at column offset ch * CC of this thread's share.
      auto fma_cols = [&](auto& vv, int ch, float slo, float shi) {
        constexpr int CC = sizeof(vv) / sizeof(uint32_t);
        // 32 columns at a time: a scale-row boundary can fall on any multiple of 32 columns
#pragma unroll
        for (int q = 0; q < CC / 32; ++q) {

          const int cb = ch * CC + 32 * q;  // offset inside this thread's columns
          const float s = (((gcol0 + cb) >> 7) == jb0) ? slo : shi;
          if (cb < kPackedCols) {
            const unsigned long long s2 = pack2(s, s);
#pragma unroll
            for (int j = 0; j < 16; ++j) fma2(acc2[cb / 2 + j], vv[32 * q + 2 * j], vv[32 * q + 2 * j + 1], s2);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              accf[cb - kPackedCols + j] = fmaf(__uint_as_float(vv[32 * q + j]), s, accf[cb - kPackedCols + j]);
          }
        }
      };
      for (int kb0 = it.kb_begin; kb0 < it.kb_end && ok; kb0 += kScaleGroup) {
        // Scales of the next (up to) four K blocks: three 16-byte shared-memory loads, then the
        // slot goes back to the loader.
        // (the vote makes the outcome the same in every lane: the warp-wide TMEM fetches below need all 32)
        // (the barrier was probed during the previous group's last fmas: scale_ready)
        if (!__all_sync(0xffffffffu, scale_ready)) {
          if (!warp_wait(smem_u32(&scale_full_bar[slot]), sphase, 0x600 | slot)) {
            ok = false;
            break;
          }
        }
        scale_ready = 0;
        const float4* sl = reinterpret_cast<const float4*>(scale_ring + slot * kScaleSlotFloats);
        constexpr int kQ = kScaleGroup / 4;  // float4s per row of a slot
        float s_lo[kScaleGroup], s_hi[kScaleGroup];
#pragma unroll
        for (int q = 0; q < kQ; ++q) {
          const float4 a4 = sl[row_in_tile * kQ + q];
          const float4 blo4 = sl[(kBlockM + bi0) * kQ + q];
          const float4 bhi4 = sl[(kBlockM + bi0 + 1) * kQ + q];
          s_lo[4 * q + 0] = a4.x * blo4.x;
          s_lo[4 * q + 1] = a4.y * blo4.y;
          s_lo[4 * q + 2] = a4.z * blo4.z;
          s_lo[4 * q + 3] = a4.w * blo4.w;
          s_hi[4 * q + 0] = a4.x * bhi4.x;
          s_hi[4 * q + 1] = a4.y * bhi4.y;
          s_hi[4 * q + 2] = a4.z * bhi4.z;
          s_hi[4 * q + 3] = a4.w * bhi4.w;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(smem_u32(&scale_empty_bar[slot]));
        if (++slot == kScaleSlots) {
          slot = 0;
          sphase ^= 1u;
        }

#pragma unroll
        for (int u = 0; u < kScaleGroup; ++u) {
          if (kb0 + u >= it.kb_end) break;
          if (!(Cfg::kEarlyProbe && ready_next)) {
            if (!warp_wait(ready_base + static_cast<uint32_t>(cstage * 8), cphase, 0x400 | cstage)) {
              ok = false;
              break;
            }
          }
          tcgen05_fence_after();
          const uint32_t taddr = tmem_base + lane_addr + static_cast<uint32_t>(buf * BN + col_base);
          constexpr int CC = Cfg::kChunkCols;
          uint32_t v[CC];
#ifdef FP8MM_X_NOPROMO
#pragma unroll
          for (int j = 0; j < CC; ++j) v[j] = 0;
#else
          tmem_ld(taddr, v);
#endif
#pragma unroll
          for (int ch = 0; ch < Cfg::kChunks; ++ch) {
#ifndef FP8MM_X_NOPROMO
            tmem_ld_wait(v);
#endif
            if (ch + 1 == Cfg::kChunks) {
              // Every column of this buffer is in registers (tcgen05.wait::ld has returned in every
              // lane once __syncwarp is passed): hand it back to the MMA warp.
              __syncwarp();
              release_to(rel_stage);
              if (++rel_stage == stages) rel_stage = 0;
              if constexpr (Cfg::kEarlyProbe) {
                int ns = cstage + 1;
                uint32_t np = cphase;
                if (ns == stages) {
                  ns = 0;
                  np ^= 1u;
                }
                ready_next = mbar_test(ready_base + static_cast<uint32_t>(ns * 8), np);
              }
              // The next group's scales: a non-blocking probe of their slot's barrier, issued here so that its
              // answer arrives under this K block's fmas. The loader runs slots ahead, so the answer is normally
              // yes and the blocking wait (a few hundred clocks even on a complete barrier while the
              // shared-memory path is busy) is skipped.
              if (u == kScaleGroup - 1) scale_ready = mbar_test(smem_u32(&scale_full_bar[slot]), sphase);
            }
#ifdef FP8MM_X_NOPROMO
            if (ch > 0) continue;
#endif
            fma_cols(v, ch, s_lo[u], s_hi[u]);
#ifndef FP8MM_X_NOPROMO
            if (ch + 1 < Cfg::kChunks) tmem_ld(taddr + static_cast<uint32_t>((ch + 1) * CC), v);
#endif
          }
          if (++buf == nbufs) buf = 0;
          if (++cstage == stages) {
            cstage = 0;
            cphase ^= 1u;
          }
        }
      }
      float2 acc[Cfg::kColsPerThread / 2];
#pragma unroll
      for (int j = 0; j < Cfg::kColsPerThread / 2; ++j) {
        if constexpr (Cfg::kScalarAcc) {
          if (2 * j < kPackedCols) {
            acc[j] = unpack2(acc2[j]);
          } else {
            acc[j] = make_float2(accf[2 * j - kPackedCols], accf[2 * j + 1 - kPackedCols]);
          }
        } else {
          acc[j] = unpack2(acc2[j]);
        }
      }
      const int col0 = it.n0 + col_base;  // first column of this thread inside (the shard of) c
      bool do_store = true;  // the same in every promotion thread of the CTA
      if (it.nsplit > 1) {
        // Split-K: publish this K range's fp32 tile; the last CTA to arrive for the tile then sums the
        // ranges in order 0..nsplit-1 (so the result does not depend on arrival order) and stores the
        // tile like an unsplit one. Plane layout per (split tile, CTA of the pair, range): float4 index
        // (col/4)*128 + row, so that a warp's accesses cover 512 contiguous bytes.
        const size_t plane_floats = static_cast<size_t>(kBlockM) * BN;
        const size_t unit = static_cast<size_t>(it.tile - p.full_tiles) * (PAIR ? 2 : 1) + cta_rank;
        float* unit_base = p.partials + unit * p.split_k * plane_floats;
        float4* mine = reinterpret_cast<float4*>(unit_base + static_cast<size_t>(it.split) * plane_floats);
#pragma unroll
        for (int j = 0; j < Cfg::kColsPerThread / 4; ++j) {
          const int c4 = (col_base >> 2) + j;
          mine[c4 * kBlockM + row_in_tile] =
              make_float4(acc[2 * j].x, acc[2 * j].y, acc[2 * j + 1].x, acc[2 * j + 1].y);
        }
        __threadfence();
        epi_bar_sync<Cfg::kEpiThreads>();
        if (epi_tid == 0) {
          int last = 0;
          if (*abort_flag == 0) {
            const int prev = atomicAdd(p.counters + unit, 1);
            last = (prev == it.nsplit - 1) ? 1 : 0;
            if (last) p.counters[unit] = 0;  // leave the counters zero for the next launch
          }
          *last_flag = last;
        }
        epi_bar_sync<Cfg::kEpiThreads>();
        do_store = (*last_flag != 0);
        epi_bar_sync<Cfg::kEpiThreads>();  // everyone has read the flag before thread 0 can overwrite it
        if (do_store) {
          __threadfence();
          const float4* base = reinterpret_cast<const float4*>(unit_base);
#pragma unroll
          for (int j = 0; j < Cfg::kColsPerThread / 2; ++j) acc[j] = make_float2(0.f, 0.f);
          for (int sp = 0; sp < it.nsplit; ++sp) {
            // all of one range's loads are independent: they are in flight together
            const float4* plane = base + static_cast<size_t>(sp) * (plane_floats / 4);
#pragma unroll
            for (int j = 0; j < Cfg::kColsPerThread / 4; ++j) {
              const float4 t = __ldcg(plane + ((col_base >> 2) + j) * kBlockM + row_in_tile);
              acc[2 * j].x += t.x;
              acc[2 * j].y += t.y;
              acc[2 * j + 1].x += t.z;
              acc[2 * j + 1].y += t.w;
            }
          }
        }
      }
      // The TMA store clips at the tensor's edges only: a tile that a group's row count cuts short goes out
      // through the guarded plain stores instead.
      const bool tma_rows_ok = !GENERIC || (it.m_limit == p.M) || (it.m0 + Cfg::kTileM <= it.m_limit);
      if (do_store && p.store_bufs > 0 && tma_rows_ok) {
        // bf16 tile -> swizzled staging -> TMA store, 32 columns at a time per warpgroup. The
        // 16-byte piece q of row r sits at r*64 + ((q ^ ((r >> 1) & 3)) * 16) (SWIZZLE_64B), which
        // spreads a warp's stores over all banks.
        const int wg_tid = epi_tid & 127;
        uint8_t* my_stage = staging + half * p.store_bufs * kStoreBufBytes;
        const int sw = (row_in_tile >> 1) & 3;
        constexpr int kBoxes = Cfg::kColsPerThread / kStoreBoxCols;
        auto stage_box = [&](int ch, int bufi) {
#ifdef FP8MM_X_NOSTAGE
          return;
#endif
          uint8_t* rowp = my_stage + bufi * kStoreBufBytes + row_in_tile * 64;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int j = ch * 16 + q * 4;
            uint4 o;
            o.x = pack_bf16x2(acc[j + 0].x, acc[j + 0].y);
            o.y = pack_bf16x2(acc[j + 1].x, acc[j + 1].y);
            o.z = pack_bf16x2(acc[j + 2].x, acc[j + 2].y);
            o.w = pack_bf16x2(acc[j + 3].x, acc[j + 3].y);
            *reinterpret_cast<uint4*>(rowp + ((q ^ sw) << 4)) = o;
          }
        };
        auto store_box = [&](int ch, int bufi) {
#ifdef FP8MM_X_NOSTOREISSUE
          return;
#endif
          if (GENERIC && p.groups > 0) {
            tma_store_3d(&tmap_c, smem_u32(my_stage + bufi * kStoreBufBytes), col0 + ch * kStoreBoxCols,
                         it.m0 + static_cast<int>(cta_rank) * kBlockM, it.group);
          } else {
            tma_store_2d(&tmap_c, smem_u32(my_stage + bufi * kStoreBufBytes), col0 + ch * kStoreBoxCols,
                         it.m0 + static_cast<int>(cta_rank) * kBlockM);
          }
        };
        if (p.store_bufs >= kBoxes) {
          // A staging buffer for every box of the warpgroup's share: the whole share is staged between two
          // barriers and leaves as kBoxes bulk stores that drain while the next tile's K loop runs; the
          // wait below is for the previous tile's stores, issued a tile ago. Box ch is issued (and later waited
          // for) by lane 0 of the warpgroup's warp ch % 4: a bulk store costs its issuing thread about 200
          // clocks, which four warps pay side by side instead of one thread four times in a row.
          if (lane == 0) tma_store_wait_read<0>();
          wg_bar_sync(half);
#pragma unroll
          for (int ch = 0; ch < kBoxes; ++ch) stage_box(ch, ch);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          wg_bar_sync(half);
          if (lane == 0 && *abort_flag == 0) {
#pragma unroll
            for (int ch = 0; ch < kBoxes; ++ch) {
              if ((ch & 3) == (wg_tid >> 5)) store_box(ch, ch);
            }
          }
        } else {
#pragma unroll
          for (int ch = 0; ch < kBoxes; ++ch) {
            const int bufi = (p.store_bufs == 2) ? (ch & 1) : 0;
            // the store that last used this buffer has finished reading it
            if (wg_tid == 0) {
              if (p.store_bufs == 2) {
                tma_store_wait_read<1>();
              } else {
                tma_store_wait_read<0>();
              }
            }
            wg_bar_sync(half);
            stage_box(ch, bufi);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            wg_bar_sync(half);
            if (wg_tid == 0 && *abort_flag == 0) store_box(ch, bufi);
          }
        }
      } else if (do_store && ok) {
        if (row < it.m_limit) {
          __nv_bfloat16* crow = p.c + static_cast<long long>(it.group) * p.c_g + static_cast<long long>(row) * p.ldc;
#pragma unroll
          for (int j = 0; j < Cfg::kColsPerThread / 8; ++j) {
            const int col = col0 + j * 8;
            if (p.vec_store && col + 8 <= p.N) {
              uint4 o;
              o.x = pack_bf16x2(acc[j * 4 + 0].x, acc[j * 4 + 0].y);
              o.y = pack_bf16x2(acc[j * 4 + 1].x, acc[j * 4 + 1].y);
              o.z = pack_bf16x2(acc[j * 4 + 2].x, acc[j * 4 + 2].y);
              o.w = pack_bf16x2(acc[j * 4 + 3].x, acc[j * 4 + 3].y);
              *reinterpret_cast<uint4*>(crow + col) = o;
            } else {
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                if (col + 2 * e < p.N) crow[col + 2 * e] = __float2bfloat16_rn(acc[j * 4 + e].x);
                if (col + 2 * e + 1 < p.N) crow[col + 2 * e + 1] = __float2bfloat16_rn(acc[j * 4 + e].y);
              }
            }
          }
        }
      }
    }
  }

  if (warp >= 4) {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");  // none in flight past here
    // the staging buffers must outlive the bulk stores that read them
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");  // every thread that issued stores
  }
  // Teardown: every role has left its loop (normally or through an expired wait). In a pair no
  // CTA may exit while its peer can still signal its barriers or use its shared memory.
  tcgen05_fence_before();
  __syncthreads();
  if constexpr (PAIR) cluster_sync_all();
  if (warp == 2) {
    tcgen05_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_base_slot);
    if constexpr (PAIR) {
      asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols)
                   : "memory");
    } else {
      asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(Cfg::kTmemCols)
                   : "memory");
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// The only mutable state of the library's host side: per-device facts looked up once (SM count, kernels
// opted in to the large shared-memory carve-out, address of the built-in scratch array) and the cache of
// encoded tensor maps. All of it is guarded by this mutex, so entry points may be called from several threads.
std::mutex g_host_mutex;

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess) {
      return nullptr;
    }
    return reinterpret_cast<EncodeTiledFn>(ptr);
  }();
  return fn;
}

// Everything a tiled tensor map is made from. A map is a pure function of these values (it holds the base
// address, not the memory), so an encoded map is kept and handed out again for the same key: the weights of
// a layer, and any buffer a caller reuses, are encoded once instead of on every call (the driver's encoder
// costs the host about as much as a small GEMM runs on the device).
struct MapKey {
  const void* base;
  cuuint64_t dims[3];
  cuuint64_t strides[2];
  cuuint32_t box[3];
  int rank;
  int dtype;
  int swizzle;
  int l2;
  bool operator==(const MapKey& o) const { return memcmp(this, &o, sizeof(MapKey)) == 0; }
};

struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    const unsigned char* p = reinterpret_cast<const unsigned char*>(&k);
    uint64_t h = 1469598103934665603ull;  // FNV-1a over the key's bytes
    for (size_t i = 0; i < sizeof(MapKey); ++i) h = (h ^ p[i]) * 1099511628211ull;
    return static_cast<size_t>(h);
  }
};

constexpr size_t kMapCacheEntries = 4096;  // the cache is emptied when it reaches this size

bool encode_map(CUtensorMap* map, const MapKey& key_in) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return false;
  MapKey key;
  memset(&key, 0, sizeof(key));  // padding bytes take part in the comparison
  key.base = key_in.base;
  for (int i = 0; i < 3; ++i) {
    key.dims[i] = key_in.dims[i];
    key.box[i] = key_in.box[i];
  }
  key.strides[0] = key_in.strides[0];
  key.strides[1] = key_in.strides[1];
  key.rank = key_in.rank;
  key.dtype = key_in.dtype;
  key.swizzle = key_in.swizzle;
  key.l2 = key_in.l2;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  // B200_FP8_MM_NO_MAP_CACHE=1 encodes on every call (to measure what the cache saves).
  static const bool cache_on = getenv("B200_FP8_MM_NO_MAP_CACHE") == nullptr;
  if (cache_on) {
    std::lock_guard<std::mutex> lock(g_host_mutex);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *map = it->second;
      return true;
    }
  }
  const cuuint32_t elem_strides[3] = {1, 1, 1};
  const CUresult r = fn(map, static_cast<CUtensorMapDataType>(key.dtype), static_cast<cuuint32_t>(key.rank),
                        const_cast<void*>(key.base), key.dims, key.strides, key.box, elem_strides,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, static_cast<CUtensorMapSwizzle>(key.swizzle),
                        static_cast<CUtensorMapL2promotion>(key.l2), CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  if (!cache_on) return true;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (cache.size() >= kMapCacheEntries) cache.clear();
  cache.emplace(key, *map);
  return true;
}

// e4m3 matrix of `rows` rows (M or N) and K columns. K-major (K contiguous, row pitch ld): box = 128 bytes of
// K x box_rows rows, 128-byte swizzle. MN-major (rows contiguous, ld bytes between consecutive k): box =
// box_rows (128 or 64) bytes of rows x 128 k, swizzle span = the box's inner extent.
bool encode_operand_map(CUtensorMap* map, const void* base, int rows, int K, long long ld, int box_rows,
                        bool mn_major) {
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.base = base;
  k.rank = 2;
  k.dims[0] = static_cast<cuuint64_t>(mn_major ? rows : K);
  k.dims[1] = static_cast<cuuint64_t>(mn_major ? K : rows);
  k.strides[0] = static_cast<cuuint64_t>(ld);
  k.box[0] = static_cast<cuuint32_t>(mn_major ? box_rows : kBlockK);
  k.box[1] = static_cast<cuuint32_t>(mn_major ? kBlockK : box_rows);
  k.dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  k.swizzle = (mn_major && box_rows == 64) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  k.l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  return encode_map(map, k);
}

// bf16 matrix c [M, N] with N contiguous: box = 32 columns (64 bytes) x 128 rows, 64-byte swizzle.
bool encode_output_map(CUtensorMap* map, void* base, int M, int N, long long ldc) {
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.base = base;
  k.rank = 2;
  k.dims[0] = static_cast<cuuint64_t>(N);
  k.dims[1] = static_cast<cuuint64_t>(M);
  k.strides[0] = static_cast<cuuint64_t>(ldc) * 2;
  k.box[0] = static_cast<cuuint32_t>(kStoreBoxCols);
  k.box[1] = static_cast<cuuint32_t>(kBlockM);
  k.dtype = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  k.swizzle = CU_TENSOR_MAP_SWIZZLE_64B;
  k.l2 = CU_TENSOR_MAP_L2_PROMOTION_NONE;
  return encode_map(map, k);
}

// Grouped operands: e4m3 [groups][rows][K] with K contiguous, row pitch ld and group pitch lg (bytes);
// box = 128 bytes of K x box_rows rows of one group.
bool encode_operand_map_3d(CUtensorMap* map, const void* base, int groups, int rows, int K, long long ld,
                           long long lg, int box_rows) {
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.base = base;
  k.rank = 3;
  k.dims[0] = static_cast<cuuint64_t>(K);
  k.dims[1] = static_cast<cuuint64_t>(rows);
  k.dims[2] = static_cast<cuuint64_t>(groups);
  k.strides[0] = static_cast<cuuint64_t>(ld);
  k.strides[1] = static_cast<cuuint64_t>(lg);
  k.box[0] = static_cast<cuuint32_t>(kBlockK);
  k.box[1] = static_cast<cuuint32_t>(box_rows);
  k.box[2] = 1;
  k.dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  k.swizzle = CU_TENSOR_MAP_SWIZZLE_128B;
  k.l2 = CU_TENSOR_MAP_L2_PROMOTION_L2_256B;
  return encode_map(map, k);
}

// Grouped output: bf16 [groups][M][N]; rows past M of a group are clipped by the store.
bool encode_output_map_3d(CUtensorMap* map, void* base, int groups, int M, int N, long long ldc, long long c_g) {
  MapKey k;
  memset(&k, 0, sizeof(k));
  k.base = base;
  k.rank = 3;
  k.dims[0] = static_cast<cuuint64_t>(N);
  k.dims[1] = static_cast<cuuint64_t>(M);
  k.dims[2] = static_cast<cuuint64_t>(groups);
  k.strides[0] = static_cast<cuuint64_t>(ldc) * 2;
  k.strides[1] = static_cast<cuuint64_t>(c_g) * 2;
  k.box[0] = static_cast<cuuint32_t>(kStoreBoxCols);
  k.box[1] = static_cast<cuuint32_t>(kBlockM);
  k.box[2] = 1;
  k.dtype = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  k.swizzle = CU_TENSOR_MAP_SWIZZLE_64B;
  k.l2 = CU_TENSOR_MAP_L2_PROMOTION_NONE;
  return encode_map(map, k);
}

int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Rows of b per TMA box of one CTA (K-major b): a CTA of a pair loads half of the tile's rows.
int b_box_rows_for(int block_n, int pair) { return pair ? block_n / 2 : block_n; }

int epi_warps_for(int block_n) {
  (void)block_n;
  return 8;  // keep in step with TileCfg::kEpiWarps
}

int smem_bytes_for(int block_n, int stages, int pair, int store_bufs) {
  const int stage = kBlockM * kBlockK + (pair ? block_n / 2 : block_n) * kBlockK;
  int bytes = 1024 /* alignment slack */ + kHeaderBytes /* barriers, flags, scale ring */ + stages * stage;
  // staging of c for the TMA store: one area of store_bufs buffers per group of four promotion warps
  if (store_bufs > 0) bytes += (epi_warps_for(block_n) / 4) * store_bufs * kStoreBufBytes;
  return bytes;
}

constexpr int kMaxSmem = 232448;  // 227 KiB opt-in limit per CTA on sm_100

int tmem_bufs_for(int block_n) { return block_n <= 128 ? 4 : 2; }

// K block j uses ring stage j mod stages and TMEM buffer j mod buffers; the two counts are independent
// (the promotion warps release a buffer to the barrier of the stage that the K block `buffers` later will
// use), except that a buffer cannot be re-used before its stage is: buffers <= stages.
int tmem_bufs_in_use(int block_n, int stages) {
  const int d = tmem_bufs_for(block_n);
  return d < stages ? d : stages;
}

// Deepest ring that fits. The 256-wide tiles stop at four stages: a fifth measured 5 % slower (their
// promotion warps still spill a little, and local memory loses L1 to every extra stage).
int max_stages_for(int block_n, int pair, int store_bufs) {
  int s = block_n == 256 ? 4 : kMaxStages;
  while (s > 2 && smem_bytes_for(block_n, s, pair, store_bufs) > kMaxSmem) --s;
  return s;
}

// Staging buffers per warpgroup for the TMA store of c. Where the ring keeps four stages (or as many as a
// tile has K blocks) beside it: one buffer for every 32-column box of the warpgroup's share, so that the whole
// tile is staged between two barriers and its stores drain under the next tile. Otherwise two (the store of
// one box overlaps the staging of the next) unless that too would leave fewer than four ring stages.
int store_boxes_per_group(int block_n) { return block_n / (epi_warps_for(block_n) / 4) / kStoreBoxCols; }

int store_bufs_for(int block_n, int pair, int kblocks_per_item) {
  const int all = store_boxes_per_group(block_n);
  const int two = 2 < all ? 2 : all;
  const int need = kblocks_per_item < 4 ? kblocks_per_item : 4;
  if (max_stages_for(block_n, pair, all) >= need || max_stages_for(block_n, pair, all) == max_stages_for(block_n, pair, two))
    return all;
  if (kblocks_per_item <= 8) return two;
  // measured: a second staging buffer is worth more than a fifth (single CTA) or seventh (pair) ring stage
  const int with_two = max_stages_for(block_n, pair, 2);
  return (with_two >= 4 || with_two == max_stages_for(block_n, pair, 1)) ? two : 1;
}

bool valid_block_n(int bn) { return bn == 64 || bn == 128 || bn == 192 || bn == 256; }

size_t plan_workspace_bytes(const b200_fp8_mm_plan& pl) {
  if (pl.split_k <= 1) return 0;
  return static_cast<size_t>(kCounterBytes) + static_cast<size_t>(pl.tiles - pl.full_tiles) *
                                                  (pl.cta_pair ? 2 : 1) * pl.split_k * kBlockM * pl.block_n *
                                                  sizeof(float);
}

// Tile/launch selection: a pure function of the problem and the SM count.
//
// Cost model, in SM clocks, fitted by least squares (median error 2-3 %) to CUDA-event timings of every
// plan over the 36 benchmark shapes on B200. Per tile width 64/128/192/256: clocks per K block (bounded
// by the promotion warps' chain of barrier probe, TMEM fetch and fmas, not by the tensor pipe), clocks
// per tile for the bf16 output, and for split-K a constant plus a per-range cost of the fp32 round
// trip and the last-arriver reduction.
struct WidthCost {
  double per_kblock, per_tile, split_const, per_split;
};

WidthCost width_cost(int bn, int pair) {
  // CTA pairs: each CTA loads half of the B tile, which pays per K block at the wide tiles (192: 5 % fewer
  // clocks than single CTAs, 256: 12 % fewer; K <= 512 loses 2-5 % to the dearer tile turnaround). At 128
  // columns pairs measured slower throughout; at 64 columns they are 3-6 % faster when no tile is split (2048 x
  // 576, 2048 x 512 and 512 x 1536 with K = 7168: one wave of 72, 64 and 48 pair tiles) and about 10 % slower
  // with split K. Plans with a split-K tail measured about 7 % above this model, hence the larger constant.
  if (pair && bn == 192) return {775.0, 3600.0, 12000.0, 1000.0};
  if (pair && bn == 256) return {930.0, 3600.0, 14000.0, 1500.0};
  switch (bn) {
    case 64: return {400.0, 1850.0, 6500.0, 750.0};
    case 128: return {585.0, 2500.0, 9000.0, 1100.0};
    case 192: return {815.0, 3300.0, 8500.0, 1000.0};
    default: return {1050.0, 4400.0, 11000.0, 1500.0};
  }
}

// What a pair plan's cost is multiplied by, for the widths without a table of their own.
double pair_penalty(int bn, int split) {
  if (bn >= 192) return 1.0;
  if (bn == 64) return split > 1 ? 1.08 : 0.96;
  return 1.04;
}

struct Candidate {
  int bn, pair, split, full_tiles;
  double cost;
};

// Three ways to lay a problem out, for one tile shape: every tile whole; every tile split along K
// (few tiles, long K: the tiles alone would leave SMs idle); or whole tiles for the full waves and a
// split-K tail for the tiles that would fill only part of a last wave.
Candidate evaluate(int M, int N, int kblocks, int sm_count, int bn, int pair, int forced_split) {
  const int tiles = ceil_div(M, pair ? 2 * kBlockM : kBlockM) * ceil_div(N, bn);
  const int units = pair ? sm_count / 2 : sm_count;
  const WidthCost wc = width_cost(bn, pair);
  const int per_unit = pair ? 2 : 1;
  auto cap_split = [&](int s) {
    if (s > kblocks / 4) s = kblocks / 4;
    if (s > 16) s = 16;
    return s < 1 ? 1 : s;
  };
  Candidate best{bn, pair, 1, tiles, ceil_div(tiles, units) * (kblocks * wc.per_kblock + wc.per_tile)};
  if (forced_split == 1 || kblocks < 8) {
    if (pair) best.cost *= pair_penalty(bn, best.split);
    return best;
  }
  if (tiles * 2 <= units || (forced_split > 1 && tiles <= units)) {
    // all tiles split
    const int split = forced_split > 1 ? forced_split : cap_split(units / tiles);
    if (split > 1 && tiles * per_unit <= kMaxCounters) {
      const double cost = ceil_div(tiles * split, units) * (ceil_div(kblocks, split) * wc.per_kblock + wc.per_tile) +
                          wc.split_const + wc.per_split * split;
      if (cost < best.cost || forced_split > 1) best = Candidate{bn, pair, split, 0, cost};
    }
  } else if (tiles > units && (tiles % units) != 0) {
    // split-K tail
    const int tail = tiles % units;
    const int split = forced_split > 1 ? forced_split : cap_split(units / tail);
    if (split > 1 && (tail * split <= units || forced_split > 1) && tail * per_unit <= kMaxCounters) {
      const double cost = (tiles / units) * (kblocks * wc.per_kblock + wc.per_tile) +
                          ceil_div(tail * split, units) * (ceil_div(kblocks, split) * wc.per_kblock + wc.per_tile) +
                          wc.split_const + wc.per_split * split;
      if (cost < best.cost || forced_split > 1) best = Candidate{bn, pair, split, tiles - tail, cost};
    }
  }
  if (pair) best.cost *= pair_penalty(bn, best.split);
  return best;
}

double choose_plan(int M, int N, int K, int sm_count, const b200_fp8_mm_plan* forced, b200_fp8_mm_plan* out) {
  const int kblocks = K / kBlockK;
  const int f_bn = (forced && forced->block_n) ? forced->block_n : 0;
  const int f_pair = (forced && forced->cta_pair) ? (forced->cta_pair > 0 ? 1 : 0) : -1;  // -1: choose
  const int f_split = (forced && forced->split_k) ? forced->split_k : 0;
  Candidate best{0, 0, 1, 0, 1e300};
  const int cands[4] = {256, 192, 128, 64};
  for (int pair = 1; pair >= 0; --pair) {
    if (f_pair >= 0 && pair != f_pair) continue;
    if (f_pair < 0 && pair == 1 && M <= kBlockM) continue;  // a pair needs two row blocks to be useful
    for (int i = 0; i < 4; ++i) {
      if (f_bn && cands[i] != f_bn) continue;
      const Candidate c = evaluate(M, N, kblocks, sm_count, cands[i], pair, f_split);
      if (c.cost < best.cost - 1e-9) best = c;
    }
  }
  if (best.bn == 0) best = Candidate{f_bn, f_pair > 0 ? 1 : 0, 1, 0, 0.0};  // invalid forced width
  const int pair = best.pair;
  const int bn = best.bn;
  const int tiles = ceil_div(M, pair ? 2 * kBlockM : kBlockM) * ceil_div(N, bn > 0 ? bn : 1);
  const int units = pair ? sm_count / 2 : sm_count;
  const int full_tiles = best.split > 1 ? best.full_tiles : tiles;
  int store_bufs = (forced && forced->store_bufs) ? (forced->store_bufs > 0 ? forced->store_bufs : 0) : -1;
  if (store_bufs < 0)
    store_bufs = (full_tiles == 0 || !valid_block_n(bn)) ? 0 : store_bufs_for(bn, pair, kblocks);
  if (full_tiles == 0 && best.split > 1) store_bufs = 0;  // every tile leaves through the fp32 planes first
  const int stages =
      (forced && forced->stages) ? forced->stages : (valid_block_n(bn) ? max_stages_for(bn, pair, store_bufs) : 2);
  out->block_m = kBlockM;
  out->block_n = bn;
  out->cta_pair = pair;
  out->split_k = best.split;
  out->stages = stages;
  out->tiles = tiles;
  out->full_tiles = full_tiles;
  const int work = full_tiles + (tiles - full_tiles) * best.split;
  const int used = work < units ? work : units;
  out->grid = pair ? 2 * used : used;
  out->store_bufs = store_bufs;
  out->smem_bytes = valid_block_n(bn) ? smem_bytes_for(bn, stages, pair, store_bufs) : 0;
  return best.cost;
}

// The reciprocals decode_work divides with (tiles_m, tiles_n, split_k, raster_group and groups are set).
void set_decode_reciprocals(KernelParams& kp) {
  const int last = kp.tiles_m % kp.raster_group;
  kp.rcp_per_group = 1.0f / static_cast<float>(kp.raster_group * kp.tiles_n);
  kp.rcp_raster = 1.0f / static_cast<float>(kp.raster_group);
  kp.rcp_raster_last = 1.0f / static_cast<float>(last > 0 ? last : kp.raster_group);
  kp.rcp_split = 1.0f / static_cast<float>(kp.split_k > 0 ? kp.split_k : 1);
  kp.rcp_per_problem = 1.0f / static_cast<float>(kp.tiles_m * kp.tiles_n);
}

// decode_work forms (split + 1) * kblocks in 32 bits; the selector itself never splits more than 16 ways.
constexpr int kMaxSplitK = 64;

bool plan_is_supported(const b200_fp8_mm_plan& pl, int kblocks) {
  if (!valid_block_n(pl.block_n)) return false;
  if (pl.cta_pair != 0 && pl.cta_pair != 1) return false;
  if (pl.stages < 2 || pl.stages > kMaxStages) return false;
  if (pl.store_bufs < 0 || pl.store_bufs > 4) return false;
  if (pl.smem_bytes > kMaxSmem) return false;
  if (pl.split_k < 1 || pl.split_k > kblocks || pl.split_k > kMaxSplitK) return false;
  if (pl.split_k > 1 && (pl.tiles - pl.full_tiles) * (pl.cta_pair ? 2 : 1) > kMaxCounters) return false;
  if (pl.full_tiles < 0 || pl.full_tiles > pl.tiles) return false;
  return true;
}

typedef void (*KernelFn)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const KernelParams);

// generic: MN-major operands or a grouped launch (CTA pairs at the 192- and 256-wide tiles only).
KernelFn kernel_for(int block_n, int pair, bool generic) {
  if (generic) {
    if (pair) {
      // grouped launches on the two widths where pairs pay
      if (block_n == 192) return fp8_mm_blockscaled_kernel<192, true, true>;
      if (block_n == 256) return fp8_mm_blockscaled_kernel<256, true, true>;
      return nullptr;
    }
    switch (block_n) {
      case 64: return fp8_mm_blockscaled_kernel<64, false, true>;
      case 128: return fp8_mm_blockscaled_kernel<128, false, true>;
      case 192: return fp8_mm_blockscaled_kernel<192, false, true>;
      case 256: return fp8_mm_blockscaled_kernel<256, false, true>;
      default: return nullptr;
    }
  }
  switch (block_n) {
    case 64: return pair ? fp8_mm_blockscaled_kernel<64, true, false> : fp8_mm_blockscaled_kernel<64, false, false>;
    case 128: return pair ? fp8_mm_blockscaled_kernel<128, true, false> : fp8_mm_blockscaled_kernel<128, false, false>;
    case 192: return pair ? fp8_mm_blockscaled_kernel<192, true, false> : fp8_mm_blockscaled_kernel<192, false, false>;
    case 256: return pair ? fp8_mm_blockscaled_kernel<256, true, false> : fp8_mm_blockscaled_kernel<256, false, false>;
    default: return nullptr;
  }
}

int device_sm_count() {
  // Looked up once per device (the current one) and kept; B200 has 148.
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (cached[dev] == 0) {
    int n = 0, major = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
    if (major != 10) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// SM count the size functions plan for: the current device's when there is one (so that the size matches the
// plan b200_fp8_mm will make on it), else B200's 148.
int sm_count_for_sizing() {
  const int n = device_sm_count();
  if (n <= 0) (void)cudaGetLastError();
  return n > 0 ? n : 148;
}

int launch(KernelFn fn, const b200_fp8_mm_plan& pl, const CUtensorMap& map_a, const CUtensorMap& map_b,
           const CUtensorMap& map_c, const KernelParams& kp, void* stream);

// Storage of one fp8 operand from its two element strides: K-major (k stride 1) or MN-major (row stride 1).
// Returns false when it is neither, or when the pitch is one the TMA unit cannot address.
bool classify_operand(long long s_row, long long s_k, int rows, int K, bool* mn_major, long long* ld) {
  if (s_k == 1 && s_row >= K) {
    *mn_major = false;
    *ld = s_row;
  } else if (s_row == 1 && s_k >= rows) {
    *mn_major = true;
    *ld = s_k;
  } else {
    return false;
  }
  return (*ld % 16) == 0;
}

// What the special-purpose entry points change about a run.
struct RunOptions {
  bool zero_counters = false;                       // clear the workspace's tile counters on the stream, once every check has passed
  unsigned long long wait_limit_ns = kWaitLimitNs;  // limit of every mbarrier wait in the kernel
  int selftest_skip_kblock = -1;                    // see KernelParams::selftest_skip_kblock
};

int run(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c, int M, int N, int K,
        long long a_sm, long long a_sk, long long b_sn, long long b_sk, long long sa_m, long long sa_k,
        long long sb_n, long long sb_k, long long ldc, int n_phase, void* workspace, size_t workspace_bytes,
        int* device_status, void* stream, const b200_fp8_mm_plan* forced_in, const RunOptions& opts = RunOptions()) {
  if (a == nullptr || b == nullptr || a_scale == nullptr || b_scale == nullptr || c == nullptr)
    return B200_FP8_MM_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return B200_FP8_MM_ERR_SHAPE;
  bool a_mn = false, b_mn = false;
  long long lda = 0, ldb = 0;
  if (!classify_operand(a_sm, a_sk, M, K, &a_mn, &lda) || !classify_operand(b_sn, b_sk, N, K, &b_mn, &ldb) ||
      ldc < N)
    return B200_FP8_MM_ERR_STRIDE;
  if ((reinterpret_cast<uintptr_t>(a) % 16) != 0 || (reinterpret_cast<uintptr_t>(b) % 16) != 0)
    return B200_FP8_MM_ERR_ALIGN;
  if (n_phase < 0 || n_phase >= 128 || (n_phase % 32) != 0) return B200_FP8_MM_ERR_PHASE;

  const int sm_count = device_sm_count();
  if (sm_count <= 0) return B200_FP8_MM_ERR_DRIVER;

  // MN-major operands run the GENERIC kernels, which exist for CTA pairs at the 192- and 256-wide tiles. An
  // MN-major b needs the CTA's half of the tile's columns to be whole 64-byte boxes, i.e. the 256-wide pair
  // (128 columns per CTA). Where the chosen pair plan has no such kernel, single CTAs are planned instead.
  const bool generic = a_mn || b_mn;
  auto pair_plan_runs = [&](const b200_fp8_mm_plan& q) {
    if (!generic || !q.cta_pair) return true;
    if (kernel_for(q.block_n, 1, true) == nullptr) return false;
    return !b_mn || ((q.block_n / 2) % 64) == 0;
  };
  const b200_fp8_mm_plan* forced = forced_in;
  b200_fp8_mm_plan pl;
  choose_plan(M, N, K, sm_count, forced, &pl);
  b200_fp8_mm_plan forced_copy;
  if (!pair_plan_runs(pl)) {
    if (forced_in != nullptr && forced_in->cta_pair > 0) return B200_FP8_MM_ERR_PLAN;
    if (forced_in != nullptr) {
      forced_copy = *forced_in;
    } else {
      memset(&forced_copy, 0, sizeof(forced_copy));
    }
    forced_copy.cta_pair = -1;
    forced = &forced_copy;
    choose_plan(M, N, K, sm_count, forced, &pl);
  }
  const int kblocks = K / kBlockK;
  if (!plan_is_supported(pl, kblocks)) return B200_FP8_MM_ERR_PLAN;
  const size_t need = plan_workspace_bytes(pl);
  if (need > 0 && (workspace == nullptr || workspace_bytes < need ||
                   (reinterpret_cast<uintptr_t>(workspace) % 256) != 0))
    return B200_FP8_MM_ERR_WORKSPACE;

  KernelFn fn = kernel_for(pl.block_n, pl.cta_pair, generic);
  if (fn == nullptr) return B200_FP8_MM_ERR_PLAN;

  CUtensorMap map_a, map_b, map_c;
  // The TMA store of c needs a 16-byte aligned base and row pitch; otherwise plain stores are used.
  int store_bufs = pl.store_bufs;
  if ((reinterpret_cast<uintptr_t>(c) % 16) != 0 || (ldc % 8) != 0) store_bufs = 0;
  if (store_bufs > 0) {
    if (!encode_output_map(&map_c, c, M, N, ldc)) return B200_FP8_MM_ERR_DRIVER;
  } else {
    memset(&map_c, 0, sizeof(map_c));
  }
  const OperandLayout la = operand_layout(a_mn, kBlockM);
  const OperandLayout lb = operand_layout(b_mn, b_box_rows_for(pl.block_n, pl.cta_pair));
  if (!encode_operand_map(&map_a, a, M, K, lda, la.box_cols, a_mn)) return B200_FP8_MM_ERR_DRIVER;
  if (!encode_operand_map(&map_b, b, N, K, ldb, lb.box_cols, b_mn)) return B200_FP8_MM_ERR_DRIVER;

  KernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.a_scale = a_scale;
  kp.b_scale = b_scale;
  kp.c = static_cast<__nv_bfloat16*>(c);
  kp.counters = static_cast<int*>(workspace);
  kp.partials = need > 0 ? reinterpret_cast<float*>(static_cast<char*>(workspace) + kCounterBytes) : nullptr;
  kp.status = device_status;
  kp.sa_m = sa_m;
  kp.sa_k = sa_k;
  kp.sb_n = sb_n;
  kp.sb_k = sb_k;
  kp.ldc = ldc;
  kp.M = M;
  kp.N = N;
  kp.K = K;
  kp.n_phase = n_phase;
  kp.tiles_m = ceil_div(M, pl.cta_pair ? 2 * kBlockM : kBlockM);
  kp.tiles_n = ceil_div(N, pl.block_n);
  kp.split_k = pl.split_k;
  kp.full_tiles = pl.full_tiles;
  kp.kblocks = kblocks;
  kp.stages = pl.stages;
  kp.tmem_bufs = tmem_bufs_in_use(pl.block_n, pl.stages);
  kp.store_bufs = store_bufs;
  kp.a_mn = a_mn ? 1 : 0;
  kp.b_mn = b_mn ? 1 : 0;
  kp.b_boxes = lb.boxes;
  kp.b_box_cols = lb.box_cols;
  kp.b_box_bytes = lb.box_bytes;
  kp.a_desc_lo = la.desc_lo;
  kp.a_desc_hi = la.desc_hi;
  kp.a_kstep = la.kstep;
  kp.b_desc_lo = lb.desc_lo;
  kp.b_desc_hi = lb.desc_hi;
  kp.b_kstep = lb.kstep;
  kp.idesc_major = (a_mn ? (1u << 15) : 0u) | (b_mn ? (1u << 16) : 0u);
  // Two issuing threads pay off where the MMAs are short (narrow tiles: 25 % faster at block_n 64,
  // 10 % at 128); the wide tiles are bound by the promotion warps and run 1 % better with one.
  kp.issuers = pl.block_n <= 128 ? 2 : 1;
  {
    // Tile rows per raster group: the tiles running at one time form a block as square as possible.
    const int units = pl.cta_pair ? sm_count / 2 : sm_count;
    int g = (units + kp.tiles_n / 2) / kp.tiles_n;
    if (g < 1) g = 1;
    if (g > 16) g = 16;
    kp.raster_group = g;
  }
  set_decode_reciprocals(kp);
  kp.b_scale_rows = ceil_div(N + n_phase, 128);
  kp.vec_store =
      ((reinterpret_cast<uintptr_t>(c) % 16) == 0 && (ldc % 8) == 0 && (N % 8) == 0) ? 1 : 0;
  kp.wait_limit_ns = opts.wait_limit_ns;
  kp.selftest_skip_kblock = opts.selftest_skip_kblock;

  if (opts.zero_counters && need > 0) {
    // Nothing has been put on the stream before this point: a call that is refused leaves the stream untouched.
    if (cudaMemsetAsync(workspace, 0, kCounterBytes, static_cast<cudaStream_t>(stream)) != cudaSuccess) {
      (void)cudaGetLastError();
      return B200_FP8_MM_ERR_LAUNCH;
    }
  }
  return launch(fn, pl, map_a, map_b, map_c, kp, stream);
}

int launch(KernelFn fn, const b200_fp8_mm_plan& pl, const CUtensorMap& map_a, const CUtensorMap& map_b,
           const CUtensorMap& map_c, const KernelParams& kp, void* stream) {
  // Opt every kernel in to the full 227 KiB of dynamic shared memory once per device.
  cudaError_t err = cudaSuccess;
  {
    static unsigned char opted_in[64][16] = {};
    int dev = 0;
    (void)cudaGetDevice(&dev);
    const bool generic = kp.groups > 0 || kp.a_mn || kp.b_mn;
    const int slot = (generic ? 8 : 0) + (pl.block_n / 64 - 1) * 2 + (pl.cta_pair ? 1 : 0);
    std::lock_guard<std::mutex> lock(g_host_mutex);
    if (dev < 0 || dev >= 64 || !opted_in[dev][slot]) {
      err = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 kMaxSmem);
      if (err != cudaSuccess) {
        (void)cudaGetLastError();
        return B200_FP8_MM_ERR_LAUNCH;
      }
      if (dev >= 0 && dev < 64) opted_in[dev][slot] = 1;
    }
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(static_cast<unsigned>(pl.grid), 1, 1);
  cfg.blockDim = dim3(static_cast<unsigned>(128 + 32 * epi_warps_for(pl.block_n)), 1, 1);
  cfg.dynamicSmemBytes = static_cast<size_t>(pl.smem_bytes);
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  if (pl.cta_pair) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  err = cudaLaunchKernelEx(&cfg, fn, map_a, map_b, map_c, kp);
  if (err != cudaSuccess) {
    (void)cudaGetLastError();
    return B200_FP8_MM_ERR_LAUNCH;
  }
  return B200_FP8_MM_OK;
}

// Grouped launch: `groups` problems of the same N and K in one kernel. Every tile is a whole tile (no
// split-K, no CTA pairs); the tile width is chosen as for one GEMM with all groups' row blocks stacked.
int run_grouped(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c, int groups, int M,
                int N, int K, long long lda, long long a_g, long long ldb, long long b_g, long long sa_g,
                long long sa_m, long long sa_k, long long sb_g, long long sb_n, long long sb_k, long long ldc,
                long long c_g, const int* m_valid, int* device_status, void* stream,
                const b200_fp8_mm_plan* forced_in) {
  if (a == nullptr || b == nullptr || a_scale == nullptr || b_scale == nullptr || c == nullptr)
    return B200_FP8_MM_ERR_NULL;
  if (groups <= 0 || M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return B200_FP8_MM_ERR_SHAPE;
  if (static_cast<long long>(groups) * ceil_div(M, kBlockM) > (1 << 20)) return B200_FP8_MM_ERR_SHAPE;
  if (lda < K || ldb < K || (lda % 16) != 0 || (ldb % 16) != 0 || ldc < N || (a_g % 16) != 0 || (b_g % 16) != 0 ||
      a_g < lda || b_g < ldb || c_g < ldc)
    return B200_FP8_MM_ERR_STRIDE;
  if ((reinterpret_cast<uintptr_t>(a) % 16) != 0 || (reinterpret_cast<uintptr_t>(b) % 16) != 0)
    return B200_FP8_MM_ERR_ALIGN;
  const int sm_count = device_sm_count();
  if (sm_count <= 0) return B200_FP8_MM_ERR_DRIVER;

  b200_fp8_mm_plan forced;
  if (forced_in != nullptr) {
    if (forced_in->split_k > 1) return B200_FP8_MM_ERR_PLAN;
    forced = *forced_in;
  } else {
    memset(&forced, 0, sizeof(forced));
  }
  forced.split_k = 1;
  // CTA pairs work on 256-row tiles inside each group: considered when a group's rows fill them to at
  // least 7/8 (or when forced), and only at the widths that have a paired grouped kernel.
  const int rows256 = ceil_div(M, 2 * kBlockM) * 2 * kBlockM;
  const bool pair_fits = (rows256 - M) * 8 <= M;
  if (forced.cta_pair == 0 && !pair_fits) forced.cta_pair = -1;
  b200_fp8_mm_plan pl;
  choose_plan(groups * rows256, N, K, sm_count, &forced, &pl);
  if (pl.cta_pair && pl.block_n != 192 && pl.block_n != 256) {
    if (forced_in != nullptr && forced_in->cta_pair > 0) return B200_FP8_MM_ERR_PLAN;
    forced.cta_pair = -1;
  }
  if (!pl.cta_pair || forced.cta_pair < 0) {
    forced.cta_pair = -1;
    choose_plan(groups * ceil_div(M, kBlockM) * kBlockM, N, K, sm_count, &forced, &pl);
  }
  if (!plan_is_supported(pl, K / kBlockK) || pl.split_k != 1) return B200_FP8_MM_ERR_PLAN;
  const int tiles_m = ceil_div(M, pl.cta_pair ? 2 * kBlockM : kBlockM);
  KernelFn fn = kernel_for(pl.block_n, pl.cta_pair, true);
  if (fn == nullptr) return B200_FP8_MM_ERR_PLAN;

  CUtensorMap map_a, map_b, map_c;
  int store_bufs = pl.store_bufs;
  if ((reinterpret_cast<uintptr_t>(c) % 16) != 0 || (ldc % 8) != 0 || (c_g % 8) != 0) store_bufs = 0;
  if (store_bufs > 0) {
    if (!encode_output_map_3d(&map_c, c, groups, M, N, ldc, c_g)) return B200_FP8_MM_ERR_DRIVER;
  } else {
    memset(&map_c, 0, sizeof(map_c));
  }
  if (!encode_operand_map_3d(&map_a, a, groups, M, K, lda, a_g, kBlockM)) return B200_FP8_MM_ERR_DRIVER;
  const int b_rows_per_cta = b_box_rows_for(pl.block_n, pl.cta_pair);
  if (!encode_operand_map_3d(&map_b, b, groups, N, K, ldb, b_g, b_rows_per_cta)) return B200_FP8_MM_ERR_DRIVER;

  const OperandLayout la = operand_layout(false, kBlockM);
  const OperandLayout lb = operand_layout(false, b_rows_per_cta);
  KernelParams kp;
  memset(&kp, 0, sizeof(kp));
  kp.a_scale = a_scale;
  kp.b_scale = b_scale;
  kp.c = static_cast<__nv_bfloat16*>(c);
  kp.status = device_status;
  kp.sa_m = sa_m;
  kp.sa_k = sa_k;
  kp.sb_n = sb_n;
  kp.sb_k = sb_k;
  kp.ldc = ldc;
  kp.M = M;
  kp.N = N;
  kp.K = K;
  kp.tiles_m = tiles_m;
  kp.tiles_n = ceil_div(N, pl.block_n);
  kp.split_k = 1;
  kp.full_tiles = groups * kp.tiles_m * kp.tiles_n;
  kp.kblocks = K / kBlockK;
  kp.stages = pl.stages;
  kp.tmem_bufs = tmem_bufs_in_use(pl.block_n, pl.stages);
  kp.store_bufs = store_bufs;
  kp.b_boxes = lb.boxes;
  kp.b_box_cols = lb.box_cols;
  kp.b_box_bytes = lb.box_bytes;
  kp.a_desc_lo = la.desc_lo;
  kp.a_desc_hi = la.desc_hi;
  kp.a_kstep = la.kstep;
  kp.b_desc_lo = lb.desc_lo;
  kp.b_desc_hi = lb.desc_hi;
  kp.b_kstep = lb.kstep;
  kp.issuers = pl.block_n <= 128 ? 2 : 1;
  {
    const int units = pl.cta_pair ? sm_count / 2 : sm_count;
    int g = (units + kp.tiles_n / 2) / kp.tiles_n;
    if (g < 1) g = 1;
    if (g > 16) g = 16;
    kp.raster_group = g;
  }
  set_decode_reciprocals(kp);
  kp.b_scale_rows = ceil_div(N, 128);
  kp.vec_store = ((reinterpret_cast<uintptr_t>(c) % 16) == 0 && (ldc % 8) == 0 && (c_g % 8) == 0 && (N % 8) == 0) ? 1 : 0;
  kp.wait_limit_ns = kWaitLimitNs;
  kp.selftest_skip_kblock = -1;
  kp.groups = groups;
  kp.m_valid = m_valid;
  kp.sa_g = sa_g;
  kp.sb_g = sb_g;
  kp.c_g = c_g;
  pl.tiles = kp.full_tiles;
  pl.full_tiles = kp.full_tiles;
  {
    const int units = pl.cta_pair ? sm_count / 2 : sm_count;
    const int used = kp.full_tiles < units ? kp.full_tiles : units;
    pl.grid = pl.cta_pair ? 2 * used : used;
  }
  return launch(fn, pl, map_a, map_b, map_c, kp, stream);
}

// ---------------------------------------------------------------------------------------------
// Scratch that lives in the library image, for callers that may not allocate
// ---------------------------------------------------------------------------------------------

// Split-K plans need scratch memory (tile counters + fp32 partial planes). Some callers have no
// way to provide it: code that runs where cudaMalloc is off limits (a plug-in whose enqueue hook
// is handed only input and output pointers, a serving loop that must not take the allocator's
// implicit device synchronisation, anything that runs while the process's memory pools are
// frozen). For them the scratch is this fixed array in the library's device image. Every GPU
// that loads the library carries these 8 MiB until the process exits.
constexpr size_t kStaticScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// Device address of g_static_scratch on the current device. In host code the array's name is only
// a handle for the runtime, not an address a kernel could use, so the address is asked for once
// per device (with that device current) and remembered.
int static_scratch_address(void** out) {
  static void* cached[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return B200_FP8_MM_ERR_DRIVER;
  std::lock_guard<std::mutex> lock(g_host_mutex);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t err = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (err != cudaSuccess || ptr == nullptr) {
      (void)cudaGetLastError();
      return B200_FP8_MM_ERR_DRIVER;
    }
    cached[dev] = ptr;
  }
  *out = cached[dev];
  return B200_FP8_MM_OK;
}

}  // namespace

extern "C" {

int b200_fp8_mm(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c, int M, int N,
                int K, long long lda, long long ldb, long long sa_m, long long sa_k, long long sb_n, long long sb_k,
                long long ldc, int n_phase, void* workspace, size_t workspace_bytes, int* device_status,
                void* stream) {
  return run(a, b, a_scale, b_scale, c, M, N, K, lda, 1, ldb, 1, sa_m, sa_k, sb_n, sb_k, ldc, n_phase, workspace,
             workspace_bytes, device_status, stream, nullptr);
}

int b200_fp8_mm_strided(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c, int M,
                        int N, int K, long long a_sm, long long a_sk, long long b_sn, long long b_sk, long long sa_m,
                        long long sa_k, long long sb_n, long long sb_k, long long ldc, int n_phase, void* workspace,
                        size_t workspace_bytes, int* device_status, void* stream, const b200_fp8_mm_plan* forced) {
  return run(a, b, a_scale, b_scale, c, M, N, K, a_sm, a_sk, b_sn, b_sk, sa_m, sa_k, sb_n, sb_k, ldc, n_phase,
             workspace, workspace_bytes, device_status, stream, forced);
}

int b200_fp8_mm_planned(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c, int M,
                        int N, int K, long long lda, long long ldb, long long sa_m, long long sa_k, long long sb_n,
                        long long sb_k, long long ldc, int n_phase, void* workspace, size_t workspace_bytes,
                        int* device_status, void* stream, const b200_fp8_mm_plan* forced) {
  return run(a, b, a_scale, b_scale, c, M, N, K, lda, 1, ldb, 1, sa_m, sa_k, sb_n, sb_k, ldc, n_phase, workspace,
             workspace_bytes, device_status, stream, forced);
}

int b200_fp8_mm_static_scratch(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c,
                               int M, int N, int K, long long lda, long long ldb, long long sa_m, long long sa_k,
                               long long sb_n, long long sb_k, long long ldc, int n_phase, int* device_status,
                               void* stream) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return B200_FP8_MM_ERR_SHAPE;
  const int sm_count = device_sm_count();
  if (sm_count <= 0) return B200_FP8_MM_ERR_DRIVER;
  b200_fp8_mm_plan pl;
  choose_plan(M, N, K, sm_count, nullptr, &pl);
  const size_t need = plan_workspace_bytes(pl);
  if (need > kStaticScratchBytes) return B200_FP8_MM_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);  // first call on a device looks the address up
  if (rc != B200_FP8_MM_OK) return rc;
  // The array still holds whatever the previous call left; the tile counters have to start at zero (a launch
  // that was cut short would leave them mid-count). run() clears them on the stream, after its own checks.
  RunOptions opts;
  opts.zero_counters = true;
  return run(a, b, a_scale, b_scale, c, M, N, K, lda, 1, ldb, 1, sa_m, sa_k, sb_n, sb_k, ldc, n_phase, scratch,
             kStaticScratchBytes, device_status, stream, nullptr, opts);
}

int b200_fp8_mm_selftest_wait_expiry(const void* a, const void* b, const float* a_scale, const float* b_scale,
                                     void* c, int M, int N, int K, long long lda, long long ldb, long long sa_m,
                                     long long sa_k, long long sb_n, long long sb_k, long long ldc,
                                     unsigned long long wait_limit_ns, int skip_kblock, int* device_status,
                                     void* stream) {
  if (device_status == nullptr) return B200_FP8_MM_ERR_NULL;
  if (K <= 0 || (K % kBlockK) != 0 || skip_kblock < 0 || skip_kblock >= K / kBlockK) return B200_FP8_MM_ERR_SHAPE;
  // A wait that runs out must do so soon (the GPU is busy until then) but not so soon that a healthy wait
  // could be mistaken for a dead one.
  if (wait_limit_ns < 1000000ull || wait_limit_ns > 100000000ull) return B200_FP8_MM_ERR_PLAN;
  b200_fp8_mm_plan forced;
  memset(&forced, 0, sizeof(forced));
  forced.block_n = 64;   // the only kernel that honours skip_kblock
  forced.cta_pair = -1;
  forced.split_k = 1;
  RunOptions opts;
  opts.wait_limit_ns = wait_limit_ns;
  opts.selftest_skip_kblock = skip_kblock;
  return run(a, b, a_scale, b_scale, c, M, N, K, lda, 1, ldb, 1, sa_m, sa_k, sb_n, sb_k, ldc, 0, nullptr, 0,
             device_status, stream, &forced, opts);
}

int b200_fp8_mm_grouped(const void* a, const void* b, const float* a_scale, const float* b_scale, void* c, int groups,
                        int M, int N, int K, long long lda, long long a_g, long long ldb, long long b_g,
                        long long sa_g, long long sa_m, long long sa_k, long long sb_g, long long sb_n,
                        long long sb_k, long long ldc, long long c_g, const int* m_valid, int* device_status,
                        void* stream, const b200_fp8_mm_plan* forced) {
  return run_grouped(a, b, a_scale, b_scale, c, groups, M, N, K, lda, a_g, ldb, b_g, sa_g, sa_m, sa_k, sb_g, sb_n,
                     sb_k, ldc, c_g, m_valid, device_status, stream, forced);
}

size_t b200_fp8_mm_static_scratch_limit(void) { return kStaticScratchBytes; }

size_t b200_fp8_mm_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return 0;
  // Covers both the plan for K-major operands and the one for MN-major operands (no CTA pairs).
  b200_fp8_mm_plan pl, single;
  const int sms = sm_count_for_sizing();
  choose_plan(M, N, K, sms, nullptr, &pl);
  memset(&single, 0, sizeof(single));
  single.cta_pair = -1;
  b200_fp8_mm_plan pl2;
  choose_plan(M, N, K, sms, &single, &pl2);
  size_t need = plan_workspace_bytes(pl);
  if (plan_workspace_bytes(pl2) > need) need = plan_workspace_bytes(pl2);
  return ((need + 255) / 256) * 256;
}

size_t b200_fp8_mm_plan_workspace_bytes(int M, int N, int K, const b200_fp8_mm_plan* forced) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return 0;
  b200_fp8_mm_plan pl;
  choose_plan(M, N, K, sm_count_for_sizing(), forced, &pl);
  const size_t need = plan_workspace_bytes(pl);
  return ((need + 255) / 256) * 256;
}

int b200_fp8_mm_describe(int M, int N, int K, int n_phase, int sm_count, b200_fp8_mm_plan* out) {
  if (out == nullptr) return B200_FP8_MM_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return B200_FP8_MM_ERR_SHAPE;
  if (n_phase < 0 || n_phase >= 128 || (n_phase % 32) != 0) return B200_FP8_MM_ERR_PHASE;
  choose_plan(M, N, K, sm_count > 0 ? sm_count : 148, nullptr, out);
  return B200_FP8_MM_OK;
}

double b200_fp8_mm_estimate_clocks(int M, int N, int K, int sm_count) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % kBlockK) != 0) return -1.0;
  b200_fp8_mm_plan pl;
  return choose_plan(M, N, K, sm_count > 0 ? sm_count : 148, nullptr, &pl);
}

const char* b200_fp8_mm_strerror(int code) {
  switch (code) {
    case B200_FP8_MM_OK: return "ok";
    case B200_FP8_MM_ERR_NULL: return "a required pointer is NULL";
    case B200_FP8_MM_ERR_SHAPE: return "bad shape: M, N, K must be positive and K a multiple of 128";
    case B200_FP8_MM_ERR_STRIDE:
      return "unsupported stride: a and b need either K or M/N contiguous and a pitch that is a multiple of 16";
    case B200_FP8_MM_ERR_ALIGN: return "a and b must be 16-byte aligned";
    case B200_FP8_MM_ERR_PHASE: return "n_phase must be 0, 32, 64 or 96";
    case B200_FP8_MM_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case B200_FP8_MM_ERR_PLAN: return "forced plan not supported";
    case B200_FP8_MM_ERR_DRIVER: return "no sm_100 device or tensor-map encode failed";
    case B200_FP8_MM_ERR_LAUNCH: return "kernel launch failed";
    case B200_FP8_MM_ERR_SCRATCH_LIMIT:
      return "this problem needs more scratch than the 8 MiB built into the library; use b200_fp8_mm with a "
             "caller-provided workspace";
    default: return "unknown error";
  }
}

int b200_fp8_mm_abi_version(void) { return 7; }

}  // extern "C"
