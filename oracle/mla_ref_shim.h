// Stand-ins for the HIP names used by the reference's RoPE and scaled-softmax kernels
// (3-amd-mla-decode/amd-mla-submission.py:17-125, 127-225) so that the kernels compile, as written, with g++
// for the host. Test infrastructure; see build_mla_ref.py.
//
// __hip_bfloat16 is modelled as a 16-bit value with round-to-nearest-even conversion from float; the
// half-precision intrinsics compute in float and round once, which is what bf16 hardware arithmetic does.
// __powf (a fast device intrinsic in the reference) is the host's powf here.
#include <math.h>
#include <stdint.h>
#include <string.h>

#define __global__
#define __shared__ static thread_local

struct RefShimDim3 {
  int x, y, z;
};
static thread_local RefShimDim3 blockIdx = {0, 0, 0};
static thread_local RefShimDim3 threadIdx = {0, 0, 0};
static thread_local RefShimDim3 blockDim = {1, 1, 1};

struct __hip_bfloat16 {
  uint16_t bits;
  __hip_bfloat16() : bits(0) {}
  __hip_bfloat16(float f) { bits = from_float(f); }
  __hip_bfloat16(double f) { bits = from_float(static_cast<float>(f)); }
  __hip_bfloat16(int i) { bits = from_float(static_cast<float>(i)); }
  operator float() const {
    uint32_t u = static_cast<uint32_t>(bits) << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
  }
  static uint16_t from_float(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return static_cast<uint16_t>((u >> 16) | 0x40u);  // NaN stays NaN
    const uint32_t lsb = (u >> 16) & 1u;
    u += 0x7fffu + lsb;  // round to nearest, ties to even
    return static_cast<uint16_t>(u >> 16);
  }
};

static inline __hip_bfloat16 __hadd(__hip_bfloat16 a, __hip_bfloat16 b) { return __hip_bfloat16(float(a) + float(b)); }
static inline __hip_bfloat16 __hsub(__hip_bfloat16 a, __hip_bfloat16 b) { return __hip_bfloat16(float(a) - float(b)); }
static inline __hip_bfloat16 __hmul(__hip_bfloat16 a, __hip_bfloat16 b) { return __hip_bfloat16(float(a) * float(b)); }
static inline __hip_bfloat16 __hdiv(__hip_bfloat16 a, __hip_bfloat16 b) { return __hip_bfloat16(float(a) / float(b)); }
// (a macro: the headers of the C library already declare a function of this name)
#define __powf(a, b) powf(static_cast<float>(a), static_cast<float>(b))
