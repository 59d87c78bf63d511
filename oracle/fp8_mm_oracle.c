/*
 * Plain-C restatement of the FP8 block-scaled GEMM, independent of torch: it carries
 * its own e4m3fn decoder. Test infrastructure only (oracle/fp8_mm_oracle.py says
 * what it is pinned to); nothing in the product links it.
 *
 * fp8mm_oracle_dequant  follows 1-amd-fp8-mm/0-amd-fp8-mm-new-begins.py:17-25, 34-42, 85-89:
 *                       dequantise a and b to fp32, then a plain fp32 dot product per output.
 * fp8mm_oracle_blocks   follows 1-amd-fp8-mm/amd-fp8-mm-submission.py:302-357: per 128-wide
 *                       K block an unscaled fp32 partial from zero, then
 *                       acc += (P * a_scale) * b_scale.
 * Both return fp32 [M,N]; the caller rounds to bf16.
 * Layouts: a [M,K] and b [N,K] row-major bytes; a_scale [M,K/128]; b_scale
 * [ceil((N+n_phase)/128), K/128]; column j uses scale row (j + n_phase)/128.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

/* OCP e4m3fn: 1 sign, 4 exponent (bias 7), 3 mantissa; no infinities; S.1111.111 is NaN. */
float fp8mm_e4m3fn_decode(uint8_t v) {
  const int sign = v >> 7;
  const int exp = (v >> 3) & 0xF;
  const int man = v & 0x7;
  float r;
  if (exp == 0xF && man == 0x7) {
    r = NAN;
  } else if (exp == 0) {
    r = ldexpf((float)man, -9); /* subnormal: man/8 * 2^-6 */
  } else {
    r = ldexpf(1.0f + (float)man / 8.0f, exp - 7);
  }
  return sign ? -r : r;
}

void fp8mm_e4m3fn_table(float* out256) {
  for (int i = 0; i < 256; ++i) out256[i] = fp8mm_e4m3fn_decode((uint8_t)i);
}

int fp8mm_oracle_dequant(const uint8_t* a, const uint8_t* b, const float* a_scale, const float* b_scale,
                         float* c, int M, int N, int K, int n_phase) {
  if (K % 128 != 0) return 1;
  const int KB = K / 128;
  float lut[256];
  fp8mm_e4m3fn_table(lut);
  float* a32 = (float*)malloc((size_t)M * K * sizeof(float));
  float* b32 = (float*)malloc((size_t)N * K * sizeof(float));
  if (!a32 || !b32) { free(a32); free(b32); return 2; }
  for (int i = 0; i < M; ++i)
    for (int kk = 0; kk < K; ++kk)
      a32[(size_t)i * K + kk] = lut[a[(size_t)i * K + kk]] * a_scale[(size_t)i * KB + kk / 128];
  for (int j = 0; j < N; ++j)
    for (int kk = 0; kk < K; ++kk)
      b32[(size_t)j * K + kk] =
          lut[b[(size_t)j * K + kk]] * b_scale[(size_t)((j + n_phase) / 128) * KB + kk / 128];
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float s = 0.0f;
      const float* ar = a32 + (size_t)i * K;
      const float* br = b32 + (size_t)j * K;
      for (int kk = 0; kk < K; ++kk) s += ar[kk] * br[kk];
      c[(size_t)i * N + j] = s;
    }
  free(a32);
  free(b32);
  return 0;
}

int fp8mm_oracle_blocks(const uint8_t* a, const uint8_t* b, const float* a_scale, const float* b_scale,
                        float* c, int M, int N, int K, int n_phase) {
  if (K % 128 != 0) return 1;
  const int KB = K / 128;
  float lut[256];
  fp8mm_e4m3fn_table(lut);
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      float acc = 0.0f;
      for (int kb = 0; kb < KB; ++kb) {
        float p = 0.0f;
        const uint8_t* ar = a + (size_t)i * K + kb * 128;
        const uint8_t* br = b + (size_t)j * K + kb * 128;
        for (int kk = 0; kk < 128; ++kk) p += lut[ar[kk]] * lut[br[kk]];
        acc += (p * a_scale[(size_t)i * KB + kb]) * b_scale[(size_t)((j + n_phase) / 128) * KB + kb];
      }
      c[(size_t)i * N + j] = acc;
    }
  return 0;
}
