// Source-level drop-in for tmt-cuda/src/moe.cu: the same structs and the same seven inline
// functions (moe_keep_alloc/free, moe_ws_alloc/free, moe_forward, moe_aux_from, moe_backward,
// moe.cu:294-545), implemented on the C ABI of include/tmt_moe.h. A host that `#include`s
// moe.cu today (train.cu:9-17) includes this header instead and links libtmt_moe_b200.so;
// model.cu:252-254, 513, 546, 676 and profile.cu:32-55 compile unchanged.
//
// Differences a caller can observe:
//   * MoeKeep owns an opaque handle instead of raw buffers; the device pointers the reference
//     exposes (logits, probs, idx, ...) are not members. Host copies come from tmt_moe_read.
//   * hcnt / stat / zloss / N,E,K,D,Tk keep their meaning (train_main.cu:207, capi.cu:134,
//     model.cu:257, 547). hcnt is filled when statistics are read (moe_forward without k.stat,
//     or moe_aux_from), not by a blocking copy in the middle of the forward.
//   * experts may exceed 16 (hcnt is sized for 256); dim must be a multiple of 64.
//   * errors throw std::runtime_error with the C ABI's message instead of printf + exit(1)
//     (common.h:26-33).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/tmt_moe.h"

using bf16 = __nv_bfloat16;

struct MoeKeep {   // per layer, persistent forward -> backward (moe.cu:294-315)
    float zloss = 0;
    int hcnt[256] = {0};   // host: tokens per expert
    int N = 0, E = 0, K = 0, D = 0, Tk = 0, Ptk = 0;
    float* stat = nullptr; // optional (E+1)-float device slot owned by the caller (moe.cu:311-314)
    tmt_moe* handle = nullptr;
    int hidden = 0;        // 0 = the reference's single-matrix experts
};
struct MoeWs {     // the reference's shared transient workspace; the handle owns everything now
    int unused = 0;
};

inline void moe_check(int rc) {
    if (rc != 0) throw std::runtime_error(std::string("tmt_moe: ") + tmt_moe_last_error());
}

// moe.cu:330-341. `hidden` > 0 selects the two-matrix FFN (not in the reference).
inline void moe_keep_alloc(MoeKeep& k, int N, int E, int K, int D, int hidden = 0, cudaStream_t stream = nullptr) {
    tmt_moe_desc d{};
    d.tokens = N; d.dim = D; d.hidden = hidden; d.experts = E; d.topk = K;
    d.router_dtype = TMT_MOE_BF16;        // the reference passes the bf16 work copy (model.cu:513)
    d.training = 1; d.gemm_impl = TMT_MOE_GEMM_AUTO;
    int dev = 0;
    cudaGetDevice(&dev);
    d.device = dev; d.host_io = 0; d.stream = stream; d.ep_world = 1; d.ep_rank = 0; d.ep_capacity_factor = 0; d.ep_transport = 0;
    moe_check(tmt_moe_create(&d, &k.handle));
    k.N = N; k.E = E; k.K = K; k.D = D; k.hidden = hidden;
}
inline void moe_keep_free(MoeKeep& k) {
    tmt_moe_destroy(k.handle);
    k = MoeKeep();
}
inline void moe_ws_alloc(MoeWs&, int, int, int, int) {}
inline void moe_ws_free(MoeWs& w) { w = MoeWs(); }

// moe.cu:470-475: aux from host-side statistics; also refreshes hcnt.
inline float moe_aux_from(MoeKeep& k, const float* hsum) {
    k.zloss = hsum[k.E];
    std::vector<int64_t> cnt(k.E);
    moe_check(tmt_moe_stats(k.handle, nullptr, cnt.data(), nullptr));
    float aux = 0;
    int tk = 0;
    for (int e = 0; e < k.E; ++e) {
        k.hcnt[e] = (int)cnt[e];
        tk += k.hcnt[e];
        aux += (hsum[e] / k.N) * (k.hcnt[e] / (float)((long)k.N * k.K));
    }
    k.Tk = tk;
    return k.E == 1 ? 0.0f : k.E * aux;
}

// moe.cu:374-466. Wexp: host array of E device pointers. Returns the switch aux loss when
// k.stat is not set (one synchronisation, as in the reference), otherwise 0 and the E+1
// statistics are copied to k.stat for the owner to read (model.cu:542-549).
inline float moe_forward(const bf16* X, const bf16* Wrouter, bf16** Wexp, bf16* Y, MoeKeep& k, MoeWs&, int N, int E,
                         int K, int D, float beta = 0.0f, bf16** Wdown = nullptr) {
    if (E != k.E || K != k.K || D != k.D) throw std::runtime_error("moe_forward: shape differs from moe_keep_alloc");
    k.N = N;
    moe_check(tmt_moe_forward(k.handle, X, Wrouter, (const void* const*)Wexp, (const void* const*)Wdown, Y, beta, N));
    std::vector<float> st(E + 1);
    if (k.stat) {
        // deferred path: keep the work asynchronous; the statistics land in the caller's device slot
        moe_check(tmt_moe_copy_stats(k.handle, k.stat));
        k.zloss = 0;
        return 0.f;
    }
    std::vector<int64_t> cnt(E);
    float aux = 0;
    moe_check(tmt_moe_stats(k.handle, st.data(), cnt.data(), &aux));
    int tk = 0;
    for (int e = 0; e < E; ++e) { k.hcnt[e] = (int)cnt[e]; tk += k.hcnt[e]; }
    k.Tk = tk;
    k.zloss = st[E];
    return aux;
}

// moe.cu:479-545. dX is written (the reference zeroes and sets it), dWexp[e] and dWrouter are written.
inline void moe_backward(const bf16* dY, bf16** Wexp, const bf16* Wrouter, float* dWrouter, float** dWexp, bf16* dX,
                         MoeKeep& k, MoeWs&, float aux = 0.f, float zcoef = 0.f, bf16** Wdown = nullptr,
                         float** dWdown = nullptr) {
    moe_check(tmt_moe_backward(k.handle, dY, Wrouter, (const void* const*)Wexp, (const void* const*)Wdown, dWrouter,
                               dWexp, dWdown, dX, aux, zcoef));
}
