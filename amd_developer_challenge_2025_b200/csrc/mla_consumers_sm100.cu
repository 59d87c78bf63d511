// RoPE and scaled softmax for B200 (sm_100a): the two custom kernels around the KV down-projection GEMM in the
// reference's MLA-decode submission (3-amd-mla-decode/amd-mla-submission.py:17-125 and 127-225). Both are
// memory-bound elementwise passes over bf16 data; they are written for HBM throughput: 16-byte accesses where
// the layout allows, enough CTAs to cover every SM several times, no shared-memory staging of the row.

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "b200_fp8_mm.h"
#include "b200_mla_consumers.h"

namespace {

// bf16 arithmetic as the reference writes it: every operation rounds to bf16 (round to nearest even).
__device__ __forceinline__ __nv_bfloat16 bf(float v) { return __float2bfloat16_rn(v); }
__device__ __forceinline__ float fl(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ __nv_bfloat16 bmul(__nv_bfloat16 a, __nv_bfloat16 b) { return bf(fl(a) * fl(b)); }
__device__ __forceinline__ __nv_bfloat16 badd(__nv_bfloat16 a, __nv_bfloat16 b) { return bf(fl(a) + fl(b)); }
__device__ __forceinline__ __nv_bfloat16 bsub(__nv_bfloat16 a, __nv_bfloat16 b) { return bf(fl(a) - fl(b)); }
__device__ __forceinline__ __nv_bfloat16 bdiv(__nv_bfloat16 a, __nv_bfloat16 b) { return bf(__fdiv_rn(fl(a), fl(b))); }

// The rotation's (cos, sin) for position row i1 and pair index j: a function of (i1, j) only
// (3-amd-mla-decode/amd-mla-submission.py:21-31).
// The part that depends on the pair index alone: 10000^(-2j/d2), every step rounded to bf16.
__device__ __forceinline__ __nv_bfloat16 rope_base(int j, int d2) {
  __nv_bfloat16 theta = bf(static_cast<float>(j));
  theta = bmul(theta, bf(-2.0f));
  theta = bdiv(theta, bf(static_cast<float>(d2)));
  return bf(powf(fl(bf(10000.0f)), fl(theta)));
}
__device__ __forceinline__ void rope_rotation(__nv_bfloat16 base, int pos, int i1, __nv_bfloat16* c, __nv_bfloat16* s) {
  const __nv_bfloat16 idx = badd(bf(static_cast<float>(pos)), bf(static_cast<float>(i1)));
  const float theta = fl(bmul(base, idx));
  *c = bf(cosf(theta));
  *s = bf(sinf(theta));
}
__device__ __forceinline__ void rope_angle(int pos, int i1, int j, int d2, __nv_bfloat16* c, __nv_bfloat16* s) {
  rope_rotation(rope_base(j, d2), pos, i1, c, s);
}

// One thread owns one (i1, j) pair and a share of the d0 rows: the angle is computed once and reused for
// every row. Consecutive threads take consecutive j, so a warp reads two runs of 64 contiguous bytes per row.
// grid.x covers the d1 * d2/2 pairs, grid.y cuts d0 so that small d1 (the query: one position) still fills the GPU.
__global__ void __launch_bounds__(256) rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* y, int pos,
                                                   int d0, int d1, int d2, long long xs1, long long xs2,
                                                   long long ys1, long long ys2, int rows_per_block) {
  const int half = d2 >> 1;
  const long long pair = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (pair >= static_cast<long long>(d1) * half) return;
  const int i1 = static_cast<int>(pair / half);
  const int j = static_cast<int>(pair - static_cast<long long>(i1) * half);
  __nv_bfloat16 c, s;
  rope_angle(pos, i1, j, d2, &c, &s);
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(d0, r0 + rows_per_block);
  const __nv_bfloat16* xp = x + static_cast<long long>(i1) * xs2 + j;
  __nv_bfloat16* yp = y + static_cast<long long>(i1) * ys2 + j;
  for (int i0 = r0; i0 < r1; ++i0) {
    const __nv_bfloat16 x1 = xp[i0 * xs1];
    const __nv_bfloat16 x2 = xp[i0 * xs1 + half];
    yp[i0 * ys1] = bsub(bmul(x1, c), bmul(x2, s));
    yp[i0 * ys1 + half] = badd(bmul(x2, c), bmul(x1, s));
  }
}

constexpr int kRopeTable = 256;  // pair indices whose 10000^(-2j/d2) a CTA keeps in shared memory

// The same with eight adjacent pair indices per thread: 16-byte loads and stores. Used when d2/2 is a multiple of 8
// and every row start is 16-byte aligned (checked by the launcher).
__global__ void __launch_bounds__(256) rope_kernel_vec8(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* y, int pos,
                                                        int d0, int d1, int d2, long long xs1, long long xs2,
                                                        long long ys1, long long ys2, int rows_per_block) {
  const int half = d2 >> 1;
  const int groups = half >> 3;  // groups of eight pair indices per position row
  // 10000^(-2j/d2) depends on j alone: the CTA computes the table once (powf is about half of a thread's angle
  // arithmetic) when it fits; every thread then needs only a cosf and a sinf per pair index.
  __shared__ __nv_bfloat16 base_tab[kRopeTable];
  const bool use_tab = half <= kRopeTable;
  if (use_tab) {
    for (int j = threadIdx.x; j < half; j += blockDim.x) base_tab[j] = rope_base(j, d2);
    __syncthreads();
  }
  const long long g = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (g >= static_cast<long long>(d1) * groups) return;
  const int i1 = static_cast<int>(g / groups);
  const int j0 = static_cast<int>(g - static_cast<long long>(i1) * groups) * 8;
  __nv_bfloat16 c[8], s[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) {
    __nv_bfloat16 ce, se;
    rope_rotation(use_tab ? base_tab[j0 + e] : rope_base(j0 + e, d2), pos, i1, &ce, &se);
    c[e] = ce;
    s[e] = se;
  }
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(d0, r0 + rows_per_block);
  const __nv_bfloat16* xp = x + static_cast<long long>(i1) * xs2 + j0;
  __nv_bfloat16* yp = y + static_cast<long long>(i1) * ys2 + j0;
  // Four rows at a time: their eight 16-byte loads are issued before the first result is stored, so a thread keeps
  // 128 bytes in flight instead of 32 (in place is still fine: a row's loads precede its own stores, and rows do
  // not overlap).
  constexpr int kRowsInFlight = 4;
  // The rotation in packed bf16 arithmetic (two elements per instruction). The hardware's bf16 multiply, add and
  // subtract round the exact result once; rounding the fp32 result of the same operation to bf16, which is what
  // the reference's arithmetic amounts to, gives the same value (a bf16 product is exact in fp32, and fp32 carries
  // more than twice bf16's precision plus two bits, so the double rounding of a sum is harmless). The _rn forms
  // are never contracted into a fused multiply-add, which would skip the products' rounding.
  __nv_bfloat162 c2[4], s2[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    c2[e] = __halves2bfloat162(c[2 * e], c[2 * e + 1]);
    s2[e] = __halves2bfloat162(s[2 * e], s[2 * e + 1]);
  }
  auto rotate_store = [&](const uint4& a, const uint4& b, int i0) {
    const __nv_bfloat162* x1 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* x2 = reinterpret_cast<const __nv_bfloat162*>(&b);
    uint4 o1, o2;
    __nv_bfloat162* y1 = reinterpret_cast<__nv_bfloat162*>(&o1);
    __nv_bfloat162* y2 = reinterpret_cast<__nv_bfloat162*>(&o2);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      y1[e] = __hsub2_rn(__hmul2_rn(x1[e], c2[e]), __hmul2_rn(x2[e], s2[e]));
      y2[e] = __hadd2_rn(__hmul2_rn(x2[e], c2[e]), __hmul2_rn(x1[e], s2[e]));
    }
    *reinterpret_cast<uint4*>(yp + i0 * ys1) = o1;
    *reinterpret_cast<uint4*>(yp + i0 * ys1 + half) = o2;
  };
  int i0 = r0;
  for (; i0 + kRowsInFlight <= r1; i0 += kRowsInFlight) {
    uint4 a[kRowsInFlight], b[kRowsInFlight];
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) {
      a[u] = *reinterpret_cast<const uint4*>(xp + (i0 + u) * xs1);
      b[u] = *reinterpret_cast<const uint4*>(xp + (i0 + u) * xs1 + half);
    }
#pragma unroll
    for (int u = 0; u < kRowsInFlight; ++u) rotate_store(a[u], b[u], i0 + u);
  }
  for (; i0 < r1; ++i0) {
    const uint4 a = *reinterpret_cast<const uint4*>(xp + i0 * xs1);
    const uint4 b = *reinterpret_cast<const uint4*>(xp + i0 * xs1 + half);
    rotate_store(a, b, i0);
  }
}

constexpr int kSoftmaxThreads = 512;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < kSoftmaxThreads / 32) ? scratch[lane] : 0.f;
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

// exp(v * scale) as 2^(v * scale * log2 e) with the hardware's exponential (ex2.approx: relative error about
// 2^-22, far inside the bf16 rounding that follows). The correctly rounded expf and the IEEE division of the
// first version cost some thirty instructions per element and made the kernel compute-bound at half the HBM rate.
__device__ __forceinline__ float exp2_fast(float x) {
  float y;
  asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// The two bf16 halves of a 32-bit word as floats, and back (one cvt.rn.bf16x2.f32).
__device__ __forceinline__ float lo_f(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float hi_f(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&v);
}

// One CTA per row. Pass 1 reads the row (16-byte loads between the row's first and last 16-byte boundary), forms e = expf(v * scale)
// and the fp32 row sum; pass 2 reads the row again (it is in L1/L2 now), rounds e to bf16 as the reference keeps
// it, divides by the sum and writes in place. HBM sees one read and one write of the row.
__global__ void __launch_bounds__(kSoftmaxThreads) div_softmax_kernel(__nv_bfloat16* qk, int sl, float scale2) {
  __shared__ float scratch[kSoftmaxThreads / 32];
  __nv_bfloat16* row = qk + static_cast<long long>(blockIdx.x) * sl;
  // A row starts on a 2-byte boundary: `head` elements up to the next 16-byte boundary go one by one, then
  // 16-byte pieces, then the rest.
  const int head = min(sl, static_cast<int>(((16u - (reinterpret_cast<uintptr_t>(row) & 15u)) & 15u) >> 1));
  const int body = ((sl - head) / 8) * 8;
  __nv_bfloat16* vrow = row + head;
  float sum = 0.f;
  for (int i = threadIdx.x * 8; i < body; i += kSoftmaxThreads * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(vrow + i);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) sum += exp2_fast(lo_f(w[e]) * scale2) + exp2_fast(hi_f(w[e]) * scale2);
  }
  const int rest = sl - body;  // head + tail elements, at most 14
  for (int t = threadIdx.x; t < rest; t += kSoftmaxThreads) {
    const int i = t < head ? t : body + t;
    sum += exp2_fast(fl(row[i]) * scale2);
  }
  const float inv = 1.0f / block_sum(sum, scratch);
  for (int i = threadIdx.x * 8; i < body; i += kSoftmaxThreads * 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(vrow + i);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    uint32_t o[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      // e rounded to bf16 as the reference keeps it, then the quotient rounded to bf16
      const uint32_t e16 = pack_bf16(exp2_fast(lo_f(w[e]) * scale2), exp2_fast(hi_f(w[e]) * scale2));
      o[e] = pack_bf16(lo_f(e16) * inv, hi_f(e16) * inv);
    }
    *reinterpret_cast<uint4*>(vrow + i) = make_uint4(o[0], o[1], o[2], o[3]);
  }
  for (int t = threadIdx.x; t < rest; t += kSoftmaxThreads) {
    const int i = t < head ? t : body + t;
    row[i] = bf(fl(bf(exp2_fast(fl(row[i]) * scale2))) * inv);
  }
}

// Rows of up to kRegRowElems elements (the reference's own limit is 8192): the row is read ONCE, its exponentials
// stay in registers (as the bf16 values the reference keeps) across the block-wide sum, and the quotients are
// written back; four independent 16-byte loads per thread are in flight at a time.
constexpr int kRegThreads = 256;
constexpr int kRegVecs = 4;
constexpr int kRegRowElems = kRegThreads * 8 * kRegVecs;  // 8192 elements in 16-byte pieces, + up to 14 stragglers

__device__ __forceinline__ float block_sum_256(float v, float* scratch) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < kRegThreads / 32) ? scratch[lane] : 0.f;
#pragma unroll
  for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return __shfl_sync(0xffffffffu, t, 0);
}

__global__ void __launch_bounds__(kRegThreads, 8) div_softmax_regs_kernel(__nv_bfloat16* qk, int sl, float scale2) {
  __shared__ float scratch[kRegThreads / 32];
  __nv_bfloat16* row = qk + static_cast<long long>(blockIdx.x) * sl;
  const int head = min(sl, static_cast<int>(((16u - (reinterpret_cast<uintptr_t>(row) & 15u)) & 15u) >> 1));
  const int body = ((sl - head) / 8) * 8;
  const int rest = sl - body;  // head + tail elements, at most 14: one per thread
  __nv_bfloat16* vrow = row + head;
  uint4 raw[kRegVecs];
#pragma unroll
  for (int v = 0; v < kRegVecs; ++v) {
    const int i = (static_cast<int>(threadIdx.x) + v * kRegThreads) * 8;
    raw[v] = (i < body) ? *reinterpret_cast<const uint4*>(vrow + i) : make_uint4(0u, 0u, 0u, 0u);
  }
  const int si = static_cast<int>(threadIdx.x) < head ? static_cast<int>(threadIdx.x) : body + static_cast<int>(threadIdx.x);
  __nv_bfloat16 stray = bf(0.f);
  float sum = 0.f;
  if (static_cast<int>(threadIdx.x) < rest) {
    const float e = exp2_fast(fl(row[si]) * scale2);
    sum += e;
    stray = bf(e);
  }
#pragma unroll
  for (int v = 0; v < kRegVecs; ++v) {
    const int i = (static_cast<int>(threadIdx.x) + v * kRegThreads) * 8;
    if (i < body) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&raw[v]);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float a = exp2_fast(lo_f(w[e]) * scale2), b = exp2_fast(hi_f(w[e]) * scale2);
        sum += a + b;
        w[e] = pack_bf16(a, b);  // kept as the bf16 values the reference stores
      }
    }
  }
  const float inv = 1.0f / block_sum_256(sum, scratch);
#pragma unroll
  for (int v = 0; v < kRegVecs; ++v) {
    const int i = (static_cast<int>(threadIdx.x) + v * kRegThreads) * 8;
    if (i < body) {
      uint32_t* w = reinterpret_cast<uint32_t*>(&raw[v]);
#pragma unroll
      for (int e = 0; e < 4; ++e) w[e] = pack_bf16(lo_f(w[e]) * inv, hi_f(w[e]) * inv);
      *reinterpret_cast<uint4*>(vrow + i) = raw[v];
    }
  }
  if (static_cast<int>(threadIdx.x) < rest) row[si] = bf(fl(stray) * inv);
}

}  // namespace

extern "C" {

int b200_mla_rope(const void* x, void* y, int pos, int d0, int d1, int d2, long long xs1, long long xs2,
                  long long ys1, long long ys2, void* stream) {
  if (x == nullptr || y == nullptr) return B200_FP8_MM_ERR_NULL;
  if (d0 <= 0 || d1 <= 0 || d2 <= 0 || (d2 & 1) != 0) return B200_FP8_MM_ERR_SHAPE;
  const int half = d2 / 2;
  const bool vec8 = (half % 8) == 0 && (xs1 % 8) == 0 && (xs2 % 8) == 0 && (ys1 % 8) == 0 && (ys2 % 8) == 0 &&
                    (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (reinterpret_cast<uintptr_t>(y) % 16) == 0;
  const long long pairs = static_cast<long long>(d1) * (vec8 ? half / 8 : half);
  const int threads = 256;
  const long long blocks_x = (pairs + threads - 1) / threads;
  if (blocks_x > 0x7fffffffll) return B200_FP8_MM_ERR_SHAPE;
  // enough CTAs for every SM a few times over, without cutting d0 finer than 4 rows per CTA
  long long want_y = (148 * 2 + blocks_x - 1) / blocks_x;
  if (want_y > (d0 + 3) / 4) want_y = (d0 + 3) / 4;
  if (want_y < 1) want_y = 1;
  if (want_y > 65535) want_y = 65535;
  const int rows_per_block = static_cast<int>((d0 + want_y - 1) / want_y);
  const int blocks_y = (d0 + rows_per_block - 1) / rows_per_block;
  const dim3 grid(static_cast<unsigned>(blocks_x), static_cast<unsigned>(blocks_y));
  if (vec8) {
    rope_kernel_vec8<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), pos, d0, d1, d2, xs1, xs2, ys1, ys2,
        rows_per_block);
  } else {
    rope_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), pos, d0, d1, d2, xs1, xs2, ys1, ys2,
        rows_per_block);
  }
  if (cudaGetLastError() != cudaSuccess) return B200_FP8_MM_ERR_LAUNCH;
  return B200_FP8_MM_OK;
}

int b200_mla_div_softmax(void* qk, int bs, int nh, int sl, int dnope, int drope, void* stream) {
  if (qk == nullptr) return B200_FP8_MM_ERR_NULL;
  if (bs <= 0 || nh <= 0 || sl <= 0 || dnope + drope <= 0) return B200_FP8_MM_ERR_SHAPE;
  const long long rows = static_cast<long long>(bs) * nh;
  if (rows > 0x7fffffffll) return B200_FP8_MM_ERR_SHAPE;
  // exp(v / sqrt(d)) = 2^(v * scale2)
  const float scale2 = 1.4426950408889634f / sqrtf(static_cast<float>(dnope + drope));
  if (sl <= kRegRowElems) {
    div_softmax_regs_kernel<<<static_cast<unsigned>(rows), kRegThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(qk), sl, scale2);
  } else {
    div_softmax_kernel<<<static_cast<unsigned>(rows), kSoftmaxThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<__nv_bfloat16*>(qk), sl, scale2);
  }
  if (cudaGetLastError() != cudaSuccess) return B200_FP8_MM_ERR_LAUNCH;
  return B200_FP8_MM_OK;
}

}  // extern "C"
