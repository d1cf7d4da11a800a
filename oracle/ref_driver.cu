// Builds the reference's own MoE block (tmt-cuda/src/moe.cu) and its two neighbours (norm.cu, adam.cu), compiled
// from where they lie, never copied, into a shared library with C entry points, so that tests can pin the
// oracle and the CUDA path against the reference itself and the benchmark can time it. TEST INFRASTRUCTURE ONLY.
//
// The reference is a GPU-only implementation (cuBLAS per expert); it runs on the GPU box.
// Its fused router kernel is correct only while all experts sit in the first warp
// (experts <= 4: 8 lanes per expert, shuffle mask 0xFF << 8e, moe.cu:15-34), so this
// driver refuses anything else.
#include "moe.cu"
#include "norm.cu"
#include "adam.cu"

#include <cmath>
#include <vector>

extern "C" int ref_moe_run(int N, int E, int K, int D, const void* X_h, const void* Wr_h, const void* Wexp_h,
                           void* Y_h, float beta, const void* dY_h, float aux, float zcoef, float* logits_h,
                           float* probs_h, int* idx_h, int* counts_h, void* dX_h, float* dWr_h, float* dWexp_h,
                           float* aux_out, float* zloss_out) {
    if (E < 1 || E > 4 || K < 1 || K > E) return -2;
    bf16 *X, *Y, *dY, *dX, *Wr;
    float* dWr;
    std::vector<bf16*> Wx(16, nullptr);
    std::vector<float*> dWx(16, nullptr);
    const size_t nd = (size_t)N * D;
    CUDA_CHECK(cudaMalloc(&X, nd * 2));
    CUDA_CHECK(cudaMalloc(&Y, nd * 2));
    CUDA_CHECK(cudaMalloc(&dY, nd * 2));
    CUDA_CHECK(cudaMalloc(&dX, nd * 2));
    CUDA_CHECK(cudaMalloc(&Wr, (size_t)E * D * 2));
    CUDA_CHECK(cudaMalloc(&dWr, (size_t)E * D * 4));
    for (int e = 0; e < E; ++e) {
        CUDA_CHECK(cudaMalloc(&Wx[e], (size_t)D * D * 2));
        CUDA_CHECK(cudaMalloc(&dWx[e], (size_t)D * D * 4));
        CUDA_CHECK(cudaMemcpy(Wx[e], (const bf16*)Wexp_h + (size_t)e * D * D, (size_t)D * D * 2, cudaMemcpyHostToDevice));
        CUDA_CHECK(cudaMemset(dWx[e], 0, (size_t)D * D * 4));
    }
    CUDA_CHECK(cudaMemcpy(X, X_h, nd * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(Y, Y_h, nd * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(Wr, Wr_h, (size_t)E * D * 2, cudaMemcpyHostToDevice));
    MoeKeep keep;
    MoeWs ws;
    moe_keep_alloc(keep, N, E, K, D);
    moe_ws_alloc(ws, N, E, K, D);
    const float a = moe_forward(X, Wr, Wx.data(), Y, keep, ws, N, E, K, D, beta);
    CUDA_CHECK(cudaDeviceSynchronize());
    if (aux_out) *aux_out = a;
    if (zloss_out) *zloss_out = keep.zloss;
    CUDA_CHECK(cudaMemcpy(Y_h, Y, nd * 2, cudaMemcpyDeviceToHost));
    if (E > 1) {
        CUDA_CHECK(cudaMemcpy(logits_h, keep.logits, (size_t)N * E * 4, cudaMemcpyDeviceToHost));
        CUDA_CHECK(cudaMemcpy(probs_h, keep.probs, (size_t)N * E * 4, cudaMemcpyDeviceToHost));
        CUDA_CHECK(cudaMemcpy(idx_h, keep.idx, (size_t)N * K * 4, cudaMemcpyDeviceToHost));
        for (int e = 0; e < E; ++e) counts_h[e] = keep.hcnt[e];
    }
    if (dY_h) {
        CUDA_CHECK(cudaMemcpy(dY, dY_h, nd * 2, cudaMemcpyHostToDevice));
        moe_backward(dY, Wx.data(), Wr, dWr, dWx.data(), dX, keep, ws, aux, zcoef);
        CUDA_CHECK(cudaDeviceSynchronize());
        CUDA_CHECK(cudaMemcpy(dX_h, dX, nd * 2, cudaMemcpyDeviceToHost));
        CUDA_CHECK(cudaMemcpy(dWr_h, dWr, (size_t)E * D * 4, cudaMemcpyDeviceToHost));
        for (int e = 0; e < E; ++e)
            CUDA_CHECK(cudaMemcpy(dWexp_h + (size_t)e * D * D, dWx[e], (size_t)D * D * 4, cudaMemcpyDeviceToHost));
    }
    moe_keep_free(keep);
    moe_ws_free(ws);
    for (void* p : {(void*)X, (void*)Y, (void*)dY, (void*)dX, (void*)Wr, (void*)dWr}) cudaFree(p);
    for (int e = 0; e < E; ++e) { cudaFree(Wx[e]); cudaFree(dWx[e]); }
    return 0;
}

// Steady-state timing of the reference's moe_forward / moe_backward on seeded inputs, the way its own harness
// does it (tmt-cuda/src/profile.cu:34-63: warm-ups, then `iters` calls between two CUDA events on the default
// stream), with allocation and copies outside the timed loops. ms_fwd = forward alone, ms_fwd_bwd = forward +
// backward per iteration. Same shape limits as ref_moe_run.
extern "C" int ref_moe_time(int N, int E, int K, int D, const void* X_h, const void* Wr_h, const void* Wexp_h,
                            const void* dY_h, float aux, float zcoef, int warmup, int iters, float* ms_fwd,
                            float* ms_fwd_bwd) {
    if (E < 1 || E > 4 || K < 1 || K > E || iters < 1) return -2;
    bf16 *X, *Y, *dY, *dX, *Wr;
    float* dWr;
    std::vector<bf16*> Wx(16, nullptr);
    std::vector<float*> dWx(16, nullptr);
    const size_t nd = (size_t)N * D;
    CUDA_CHECK(cudaMalloc(&X, nd * 2));
    CUDA_CHECK(cudaMalloc(&Y, nd * 2));
    CUDA_CHECK(cudaMalloc(&dY, nd * 2));
    CUDA_CHECK(cudaMalloc(&dX, nd * 2));
    CUDA_CHECK(cudaMalloc(&Wr, (size_t)E * D * 2));
    CUDA_CHECK(cudaMalloc(&dWr, (size_t)E * D * 4));
    for (int e = 0; e < E; ++e) {
        CUDA_CHECK(cudaMalloc(&Wx[e], (size_t)D * D * 2));
        CUDA_CHECK(cudaMalloc(&dWx[e], (size_t)D * D * 4));
        CUDA_CHECK(cudaMemcpy(Wx[e], (const bf16*)Wexp_h + (size_t)e * D * D, (size_t)D * D * 2, cudaMemcpyHostToDevice));
    }
    CUDA_CHECK(cudaMemcpy(X, X_h, nd * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(dY, dY_h, nd * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemset(Y, 0, nd * 2));
    CUDA_CHECK(cudaMemcpy(Wr, Wr_h, (size_t)E * D * 2, cudaMemcpyHostToDevice));
    MoeKeep keep;
    MoeWs ws;
    moe_keep_alloc(keep, N, E, K, D);
    moe_ws_alloc(ws, N, E, K, D);
    cudaEvent_t s, e;
    CUDA_CHECK(cudaEventCreate(&s));
    CUDA_CHECK(cudaEventCreate(&e));
    for (int i = 0; i < warmup; ++i) {
        moe_forward(X, Wr, Wx.data(), Y, keep, ws, N, E, K, D);
        moe_backward(dY, Wx.data(), Wr, dWr, dWx.data(), dX, keep, ws, aux, zcoef);
    }
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaEventRecord(s));
    for (int i = 0; i < iters; ++i) moe_forward(X, Wr, Wx.data(), Y, keep, ws, N, E, K, D);
    CUDA_CHECK(cudaEventRecord(e));
    CUDA_CHECK(cudaEventSynchronize(e));
    float ms = 0;
    CUDA_CHECK(cudaEventElapsedTime(&ms, s, e));
    if (ms_fwd) *ms_fwd = ms / iters;
    CUDA_CHECK(cudaEventRecord(s));
    for (int i = 0; i < iters; ++i) {
        moe_forward(X, Wr, Wx.data(), Y, keep, ws, N, E, K, D);
        moe_backward(dY, Wx.data(), Wr, dWr, dWx.data(), dX, keep, ws, aux, zcoef);
    }
    CUDA_CHECK(cudaEventRecord(e));
    CUDA_CHECK(cudaEventSynchronize(e));
    CUDA_CHECK(cudaEventElapsedTime(&ms, s, e));
    if (ms_fwd_bwd) *ms_fwd_bwd = ms / iters;
    cudaEventDestroy(s);
    cudaEventDestroy(e);
    moe_keep_free(keep);
    moe_ws_free(ws);
    for (void* p : {(void*)X, (void*)Y, (void*)dY, (void*)dX, (void*)Wr, (void*)dWr}) cudaFree(p);
    for (int x = 0; x < E; ++x) { cudaFree(Wx[x]); cudaFree(dWx[x]); }
    return 0;
}

// layernorm_fwd + layernorm_bwd (tmt-cuda/src/norm.cu:92-110) on host arrays.
extern "C" int ref_ln_run(int N, int D, const void* X_h, const void* dY_h, const float* gamma_h, const float* beta_h,
                          void* Y_h, float* mean_h, float* rstd_h, void* dX_h, float* dGamma_h, float* dBeta_h) {
    bf16 *X, *dY, *Y, *dX;
    float *gamma, *beta, *mean, *rstd, *dG, *dB;
    const size_t nd = (size_t)N * D;
    CUDA_CHECK(cudaMalloc(&X, nd * 2)); CUDA_CHECK(cudaMalloc(&dY, nd * 2));
    CUDA_CHECK(cudaMalloc(&Y, nd * 2)); CUDA_CHECK(cudaMalloc(&dX, nd * 2));
    CUDA_CHECK(cudaMalloc(&gamma, D * 4)); CUDA_CHECK(cudaMalloc(&beta, D * 4));
    CUDA_CHECK(cudaMalloc(&mean, N * 4)); CUDA_CHECK(cudaMalloc(&rstd, N * 4));
    CUDA_CHECK(cudaMalloc(&dG, D * 4)); CUDA_CHECK(cudaMalloc(&dB, D * 4));
    CUDA_CHECK(cudaMemcpy(X, X_h, nd * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(dY, dY_h, nd * 2, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(gamma, gamma_h, D * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(beta, beta_h, D * 4, cudaMemcpyHostToDevice));
    layernorm_fwd(X, gamma, beta, Y, mean, rstd, N, D);
    layernorm_bwd(X, dY, gamma, mean, rstd, dX, dG, dB, N, D);
    CUDA_CHECK(cudaDeviceSynchronize());
    CUDA_CHECK(cudaMemcpy(Y_h, Y, nd * 2, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(dX_h, dX, nd * 2, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(mean_h, mean, N * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(rstd_h, rstd, N * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(dGamma_h, dG, D * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(dBeta_h, dB, D * 4, cudaMemcpyDeviceToHost));
    for (void* p : {(void*)X, (void*)dY, (void*)Y, (void*)dX, (void*)gamma, (void*)beta, (void*)mean, (void*)rstd, (void*)dG, (void*)dB})
        cudaFree(p);
    return 0;
}

// One optimizer step over `tensors` parameters with the reference's multi-tensor kernels (tmt-cuda/src/adam.cu:44-96:
// mt_sumsq_kernel, mt_adam_kernel, mt_zero_kernel over MT_CHUNK-element chunks) the way optimizer_step drives them
// (model.cu:716-729: step + 1 in the bias corrections is the caller's business here: `step` is used as given).
// All tensors lie back to back in the host arrays (offsets from sizes). In place: master, m, v; work (bf16) and the
// cleared gradient are written; *sumsq_out receives the squared gradient norm.
extern "C" int ref_adam_run(int tensors, const long long* sizes, const unsigned char* flags_h, float* master_h, float* m_h,
                            float* v_h, float* grad_h, void* work_h, float clip, float lr, float b1, float b2, float eps,
                            float wd, int step, double* sumsq_out) {
    long long total = 0;
    for (int i = 0; i < tensors; ++i) total += sizes[i];
    float *master, *m, *v, *grad;
    bf16* work;
    CUDA_CHECK(cudaMalloc(&master, total * 4)); CUDA_CHECK(cudaMalloc(&m, total * 4));
    CUDA_CHECK(cudaMalloc(&v, total * 4)); CUDA_CHECK(cudaMalloc(&grad, total * 4));
    CUDA_CHECK(cudaMalloc(&work, total * 2));
    CUDA_CHECK(cudaMemcpy(master, master_h, total * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(m, m_h, total * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(v, v_h, total * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(grad, grad_h, total * 4, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemset(work, 0, total * 2));
    std::vector<float*> pm(tensors), pmm(tensors), pv(tensors), pg(tensors);
    std::vector<bf16*> pw(tensors);
    std::vector<MTChunk> chunks;
    long long off = 0;
    for (int i = 0; i < tensors; ++i) {
        pm[i] = master + off; pmm[i] = m + off; pv[i] = v + off; pg[i] = grad + off; pw[i] = work + off;
        for (long long st = 0; st < sizes[i]; st += MT_CHUNK) {
            MTChunk c;
            c.param = i; c.start = (long)st; c.len = (int)std::min<long long>(MT_CHUNK, sizes[i] - st);
            chunks.push_back(c);
        }
        off += sizes[i];
    }
    MTParams P;
    CUDA_CHECK(cudaMalloc(&P.master, tensors * sizeof(float*))); CUDA_CHECK(cudaMalloc(&P.m, tensors * sizeof(float*)));
    CUDA_CHECK(cudaMalloc(&P.v, tensors * sizeof(float*))); CUDA_CHECK(cudaMalloc(&P.grad, tensors * sizeof(float*)));
    CUDA_CHECK(cudaMalloc(&P.work, tensors * sizeof(bf16*))); CUDA_CHECK(cudaMalloc(&P.flags, tensors));
    CUDA_CHECK(cudaMalloc(&P.chunks, chunks.size() * sizeof(MTChunk))); CUDA_CHECK(cudaMalloc(&P.sumsq, sizeof(double)));
    CUDA_CHECK(cudaMemcpy(P.master, pm.data(), tensors * sizeof(float*), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(P.m, pmm.data(), tensors * sizeof(float*), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(P.v, pv.data(), tensors * sizeof(float*), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(P.grad, pg.data(), tensors * sizeof(float*), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(P.work, pw.data(), tensors * sizeof(bf16*), cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(P.flags, flags_h, tensors, cudaMemcpyHostToDevice));
    CUDA_CHECK(cudaMemcpy(P.chunks, chunks.data(), chunks.size() * sizeof(MTChunk), cudaMemcpyHostToDevice));
    P.nchunks = (int)chunks.size();
    CUDA_CHECK(cudaMemset(P.sumsq, 0, sizeof(double)));
    mt_sumsq_kernel<<<P.nchunks, 256>>>(P);
    const float bc1 = 1.0f - powf(b1, step), bc2 = 1.0f - powf(b2, step);
    mt_adam_kernel<<<P.nchunks, 256>>>(P, clip, lr, b1, b2, eps, wd, bc1, bc2);
    mt_zero_kernel<<<P.nchunks, 256>>>(P);
    CUDA_CHECK(cudaDeviceSynchronize());
    if (sumsq_out) CUDA_CHECK(cudaMemcpy(sumsq_out, P.sumsq, sizeof(double), cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(master_h, master, total * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(m_h, m, total * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(v_h, v, total * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(grad_h, grad, total * 4, cudaMemcpyDeviceToHost));
    CUDA_CHECK(cudaMemcpy(work_h, work, total * 2, cudaMemcpyDeviceToHost));
    for (void* p : {(void*)master, (void*)m, (void*)v, (void*)grad, (void*)work, (void*)P.master, (void*)P.m, (void*)P.v,
                    (void*)P.grad, (void*)P.work, (void*)P.flags, (void*)P.chunks, (void*)P.sumsq})
        cudaFree(p);
    return 0;
}
