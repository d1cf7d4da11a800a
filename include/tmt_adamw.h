/* C ABI of the multi-tensor AdamW step over the MoE block's parameters on B200 (sm_100a).
 *
 * The step that follows tmt_moe_backward in the reference's training loop: optimizer_step
 * (tmt-cuda/src/model.cu:716-729) over the multi-tensor tables of tmt-cuda/src/adam.cu:44-105
 * (MTParams, mt_sumsq_kernel, mt_adam_kernel, mt_zero_kernel). One handle covers a fixed list of
 * tensors (expert matrices, router); a step computes the global squared gradient norm, clips,
 * applies AdamW to the fp32 master copies and their moments, re-materialises the bf16 working
 * copies the GEMMs read, and clears the gradients, in two passes over the data (the reference makes
 * three: norm, update, zero).
 *
 * Conventions as in tmt_moe.h: opaque handle, 0 / -1, message from tmt_moe_last_error(), device
 * pointers, no allocation after create, nothing calls exit().
 *
 * Arithmetic per element, in this order and with these roundings (fp32, fused multiply-adds where
 * written; the CPU oracle uses the same sequence, so results are bit-identical):
 *   g  = grad * scale                     scale = clip > 0 ? min(1, clip / max(sqrt(sumsq), 1e-12)) : 1
 *   m' = fma(b1, m, (1 - b1) * g)         v' = fma(b2, v, ((1 - b2) * g) * g)
 *   u  = (m' / bc1) / (sqrt(v' / bc2) + eps)          bc1 = 1 - b1^step, bc2 = 1 - b2^step
 *   w' = fma(-lr, fma(wd, w, u), w)       work = bf16(w') round to nearest even
 * (adam.cu:84-99 with the same formulas; the reference passes step + 1, model.cu:722-723).
 * sumsq is accumulated in double, in a fixed order (the reference adds block sums with atomics). */
#ifndef TMT_ADAMW_H
#define TMT_ADAMW_H

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tmt_adamw tmt_adamw;

/* Replaces build of MTParams / MTChunk (adam.cu:44-55): `tensors` parameters of sizes[i] elements each. */
int tmt_adamw_create(int tensors, const long long* sizes, int device, void* stream, tmt_adamw** out);
void tmt_adamw_destroy(tmt_adamw* h);

/* One optimizer step (model.cu:716-729). master / m / v / grad: host arrays of `tensors` device
 * pointers to fp32 data; work: device pointers to the bf16 copies (an entry may be NULL: no copy
 * kept); flags[i] bit 0: tensor i counts in the gradient norm, bit 1: it is updated (adam.cu:49).
 * step >= 1 is the exponent of the bias corrections. zero_grads != 0 clears every gradient that was
 * read (mt_zero_kernel). sumsq_host (may be NULL) receives the squared gradient norm; passing it
 * synchronises the stream, as the reference does once per step (model.cu:726-728). A non-finite
 * norm leaves every tensor untouched (adam.cu:81-82) and the call returns -1 when sumsq_host was
 * given ("non-finite gradient; update refused", model.cu:728). */
int tmt_adamw_step(tmt_adamw* h, float* const* master, float* const* m, float* const* v, float* const* grad,
                   void* const* work, const unsigned char* flags, float clip, float lr, float b1, float b2, float eps,
                   float wd, int step, int zero_grads, double* sumsq_host);

#ifdef __cplusplus
}
#endif
#endif
