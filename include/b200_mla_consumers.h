/*
 * C ABI of the two custom kernels that sit around the KV down-projection GEMM in the reference's
 * MLA-decode submission (3-amd-mla-decode/amd-mla-submission.py), for sm_100a. They live in the same
 * library as the FP8 GEMM (libb200fp8mm.so); the down-projection itself (`x @ wDKV.T`, same file, 269:
 * N = 576, K = 7168) is the GEMM shape b200_fp8_mm is tuned for.
 *
 * Plain pointers and sizes; nothing is allocated; asynchronous on `stream`. Return codes are the
 * B200_FP8_MM_* codes of b200_fp8_mm.h (0 = launched).
 */
#ifndef B200_MLA_CONSUMERS_H_
#define B200_MLA_CONSUMERS_H_

#ifdef __cplusplus
extern "C" {
#endif

/*
 * Rotary position embedding of a bf16 tensor [d0][d1][d2] with arbitrary strides. Replaces the pybind
 * launcher `mla_decode(x, y, pos, xoff, yoff, d0, d1, d2, xs1, xs2, ys1, ys2)` and its four kernels
 * (3-amd-mla-decode/amd-mla-submission.py:8-9, 17-125); x and y here already point at the first element
 * (the launcher's xoff / yoff applied by the caller).
 *
 *   element (i0, i1, j) of x at x + i0*xs1 + i1*xs2 + j, of y at y + i0*ys1 + i1*ys2 + j  (bf16 elements)
 *   position of row i1: pos + i1 (added in bf16, as the reference does)
 *   for j < d2/2:  y[j] = x[j]*cos - x[j+d2/2]*sin,  y[j+d2/2] = x[j+d2/2]*cos + x[j]*sin
 *   angle = bf16(powf(bf16(10000), bf16(j) * -2 / d2)) * position, every step rounded to bf16; each
 *   product and each sum of the rotation rounds to bf16 (same file, 21-33).
 *
 * y may equal x (the reference rotates the query in place). d2 must be even.
 */
int b200_mla_rope(const void* x, void* y, int pos, int d0, int d1, int d2,
                  long long xs1, long long xs2, long long ys1, long long ys2, void* stream);

/*
 * In-place softmax over the last dimension of the contiguous bf16 tensor qk [bs][nh][sl], of
 * qk / sqrt(dnope + drope). Replaces `div_softmax(qk, bs, nh, sl, dnope, drope)` and div_softmax_kernel
 * (3-amd-mla-decode/amd-mla-submission.py:10, 127-225), with its arithmetic: e = exp(float(v) * scale)
 * with no maximum subtracted, the row sum adds e in fp32, the result is bf16(float(bf16(e)) / sum).
 * The exponential is the hardware's 2^x (relative error about 2^-22) and the quotient a multiplication
 * by 1 / sum: a result can differ from a correctly rounded evaluation by one bf16 step, the same as
 * between two math libraries. Any sl (the reference's kernel stops at 8192).
 */
int b200_mla_div_softmax(void* qk, int bs, int nh, int sl, int dnope, int drope, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B200_MLA_CONSUMERS_H_ */
