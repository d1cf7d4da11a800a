/* C ABI of the LayerNorm in front of the MoE block on B200 (sm_100a).
 *
 * The step right before the block in the reference's layer loop: layernorm_fwd / layernorm_bwd
 * (tmt-cuda/src/norm.cu:8-50, 54-110; call sites model.cu:509-510 and the matching backward): bf16 in and out,
 * fp32 gamma / beta and statistics, y = (x - mean) * rstd * gamma + beta, variance = E[x^2] - mean^2, eps = 1e-5.
 * Same argument lists as the reference's two functions, plus a scratch buffer for the backward pass (the reference
 * adds the gamma / beta gradients with atomics; here block partial sums are added in a fixed order, so the
 * result does not depend on timing). Conventions as in tmt_moe.h: 0 / -1, message from tmt_moe_last_error(),
 * device pointers, nothing allocates, nothing calls exit().
 *
 * Arithmetic order (the CPU oracle uses the same, results are bit-identical). A row is read in 16-byte vectors
 * (8 elements); lane l of a warp owns vectors l, l + 32, ...; per lane sum and sum of squares run over its elements
 * in index order (sq = fma(x, x, sq)); lanes combine by the butterfly v += v[lane ^ 16], ^8, ^4, ^2, ^1.
 *   mean = sum / D;  var = sumsq / D - mean * mean;  rstd = 1 / sqrt(var + 1e-5)   (IEEE division and square root)
 *   y = bf16(fma((x - mean) * rstd, gamma, beta))
 * Backward, per row with g = dy * gamma and xh = fma(x, rstd, -(mean * rstd)): thread t of 256 owns vectors t, t + 256,
 * ...; s1 = sum g, s2 = sum g * xh (fma) over its elements, warp butterfly as above, the 8 warp sums added in warp
 * order; a = s1 / D, b = s2 / D, dx = bf16(fma(xh, -(rstd * b), fma(g, rstd, -(rstd * a)))), i.e. the reference's
 * rstd * (g - a - xh * b) with fused multiply-adds; dGamma[d] = fma(dy, xh, dGamma[d]) and dBeta[d] += dy run over the
 * rows of a 128-row block in row order, and the block sums are added in block order. */
#ifndef TMT_NORM_H
#define TMT_NORM_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

/* layernorm_fwd (norm.cu:96-100). X, Y (rows, dim) bf16; gamma, beta (dim) fp32; mean, rstd (rows) fp32 out.
 * dim: a multiple of 8, at most 8192. */
int tmt_ln_forward(const void* X, const float* gamma, const float* beta, void* Y, float* mean, float* rstd, int rows, int dim,
                   void* stream);

/* Bytes of device scratch tmt_ln_backward needs for this shape (block partial sums of dGamma and dBeta). */
size_t tmt_ln_backward_scratch_bytes(int rows, int dim);

/* layernorm_bwd (norm.cu:102-110). dX (rows, dim) bf16 out; dGamma, dBeta (dim) fp32 WRITTEN (the reference zeroes
 * them and accumulates, which is the same). dim: a multiple of 8, at most 8192. */
int tmt_ln_backward(const void* X, const void* dY, const float* gamma, const float* mean, const float* rstd, void* dX,
                    float* dGamma, float* dBeta, int rows, int dim, void* scratch, void* stream);

#ifdef __cplusplus
}
#endif
#endif
