// Stand-ins for the HIP names used by the reference's dqa_kernel / dqb_kernel
// (1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:17-25, 34-42) so that the two functions compile, as
// written, with g++ for the host. Test infrastructure; see build_ref.py.
#include <stdint.h>
#include <string.h>

#define __global__

struct RefShimDim3 {
  int x, y, z;
};
// One "thread" runs at a time per host thread: the driver sets these before each call.
static thread_local RefShimDim3 blockIdx = {0, 0, 0};
static thread_local RefShimDim3 threadIdx = {0, 0, 0};
static thread_local RefShimDim3 blockDim = {1, 1, 1};

// One byte of FP8 storage. The conversion to float decodes e4m3fn: 1 sign, 4 exponent bits with
// bias 7, 3 mantissa bits, subnormals at exponent 0, no infinities, NaN only at 0x7f / 0xff.
// (The name is the AMD "fnuz" type because that is what the reference's text says; the contract
// this repository is built to fixes e4m3fn for both operands.)
struct __hip_fp8_e4m3_fnuz {
  uint8_t bits;
  operator float() const {
    const uint32_t sign = static_cast<uint32_t>(bits & 0x80u) << 24;
    const uint32_t exp = (bits >> 3) & 0xfu;
    const uint32_t man = bits & 0x7u;
    uint32_t u;
    if (exp == 0xfu && man == 0x7u) {
      u = sign | 0x7fc00000u;
    } else if (exp == 0) {
      // subnormal: man * 2^-9, exact in fp32
      float f = static_cast<float>(man) * (1.0f / 512.0f);
      memcpy(&u, &f, 4);
      u |= sign;
    } else {
      u = sign | ((exp - 7u + 127u) << 23) | (man << 20);
    }
    float out;
    memcpy(&out, &u, 4);
    return out;
  }
};
