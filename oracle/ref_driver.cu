// Builds the reference's own MoE block (tmt-cuda/src/moe.cu, compiled from where it lies,
// never copied) into a shared library with one C entry point, so that tests can pin the
// oracle and the CUDA path against the reference itself. TEST INFRASTRUCTURE ONLY.
//
// The reference is a GPU-only implementation (cuBLAS per expert); it runs on the GPU box.
// Its fused router kernel is correct only while all experts sit in the first warp
// (experts <= 4: 8 lanes per expert, shuffle mask 0xFF << 8e, moe.cu:15-34), so this
// driver refuses anything else.
#include "moe.cu"

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
