// Host side of the MoE block behind the C ABI of include/tmt_moe.h: owns every buffer,
// builds the TMA tensor maps, queues the kernels of one forward / backward on the handle's
// stream. Mirrors moe_keep_alloc / moe_ws_alloc / moe_forward / moe_aux_from / moe_backward
// of tmt-cuda/src/moe.cu:330-545; no allocation and no host synchronisation inside a step.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/tmt_moe.h"
#include "gemm.cuh"
#include "kernels.cuh"
#include "moe_internal.h"

namespace tmt {

thread_local std::string g_error;

void set_error(const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_error = buf;
}

namespace {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess || !p)
            throw std::runtime_error("cuTensorMapEncodeTiled is not available from this driver");
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// 2-D tensor of 2-byte (bf16) or 4-byte (fp32) elements, 128-byte swizzle: the output side of the GEMMs.
void make_out_map(CUtensorMap* m, const void* base, bool f32, uint64_t inner, uint64_t rows) {
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner * (f32 ? 4u : 2u)};
    cuuint32_t box[2] = {32u, 128u};                     // fp32: 128 bytes x 128 rows (128-byte swizzle); bf16: 64 bytes x 128 rows (64-byte swizzle)
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base),
                             dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                             CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) throw std::runtime_error("cuTensorMapEncodeTiled failed for an output map (" + std::to_string((int)r) + ")");
}

// 2-D bf16 tensor, `inner` contiguous elements per row, 128-byte swizzle, zero fill.
void make_map(CUtensorMap* m, const void* base, uint64_t inner, uint64_t rows, uint32_t box_inner, uint32_t box_rows) {
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char msg[160];
        snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled failed (%d) for %llux%llu box %ux%u", (int)r,
                 (unsigned long long)inner, (unsigned long long)rows, box_inner, box_rows);
        throw std::runtime_error(msg);
    }
}

// bf16 matrix [rows][inner] read with the `inner` extent as the MMA's M or N (mn-major operand): a 3-D view
// {64 inner elements, rows, inner / 64 blocks} with the block stride (128 B) below the row stride, so ONE
// box {64, 64, blocks} lands as `blocks` consecutive 8 KB swizzle blocks, the layout the shared-memory
// descriptors of the GEMM kernels use (one TMA instruction per operand and k block instead of one per block).
void make_map_mn(CUtensorMap* m, const void* base, uint64_t inner, uint64_t rows, uint32_t blocks) {
    cuuint64_t dims[3] = {64, rows, inner / 64};
    cuuint64_t strides[2] = {inner * 2, 128};
    cuuint32_t box[3] = {64, 64, blocks};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode_fn()(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS || inner % 64 != 0) {
        char msg[160];
        snprintf(msg, sizeof msg, "cuTensorMapEncodeTiled failed (%d) for the mn-major view of %llux%llu, %u blocks", (int)r,
                 (unsigned long long)inner, (unsigned long long)rows, blocks);
        throw std::runtime_error(msg);
    }
}

#define CK(call)                                                                              \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess) {                                                             \
            char m__[256];                                                                    \
            snprintf(m__, sizeof m__, "%s failed: %s", #call, cudaGetErrorString(e__));       \
            throw std::runtime_error(m__);                                                    \
        }                                                                                     \
    } while (0)

template <class T>
T* dalloc(tmt_moe* h, size_t n) {
    void* p = nullptr;
    CK(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)));
    h->allocs.push_back(p);
    h->bytes += n * sizeof(T);
    return reinterpret_cast<T*>(p);
}

enum ActMap { kXgK = 0, kHactK, kDYgK, kDPK, kDYgMN, kHactMN, kDPMN, kXgMN, kDlgMN, kDltK, kXsMN, kDltMN,
              kOutP, kOutHact, kOutYg, kOutDP, kOutDXg, kOutDXr, kOutSplit0, kNumActMaps = kOutSplit0 + kMaxSplits };
enum WMap { kUpK = 0, kDownK, kDownMN, kUpMN, kNumWMaps };   // one more map follows the 4*E weight maps: the router, mn-major

void build_act_maps(tmt_moe* h) {
    const uint64_t D = h->d.dim, H = h->d.hidden, cap = h->gcap;
    const uint32_t ablk = kBM / 64, bblk = (h->two_cta ? kBN / 2 : kBN) / 64;    // 64-wide blocks one CTA stages per k block
    std::vector<CUtensorMap> m(kNumActMaps);
    memset(m.data(), 0, m.size() * sizeof(CUtensorMap));
    make_map(&m[kXgK], h->Xg, D, cap, 64, 128);
    make_map(&m[kDYgK], h->dYg, D, cap, 64, 128);
    make_map_mn(&m[kDYgMN], h->dYg, D, cap, ablk);
    make_map_mn(&m[kXgMN], h->Xg, D, cap, bblk);
    if (H > 0) {
        make_map(&m[kHactK], h->Hact, H, cap, 64, 128);
        make_map(&m[kDPK], h->dP, H, cap, 64, 128);
        make_map_mn(&m[kHactMN], h->Hact, H, cap, bblk);
        make_map_mn(&m[kDPMN], h->dP, H, cap, ablk);
    }
    make_out_map(&m[kOutYg], h->Yg, false, D, cap);
    if (h->dXg) make_out_map(&m[kOutDXg], h->dXg, false, D, cap);
    if (H > 0) {
        make_out_map(&m[kOutHact], h->Hact, false, H, cap);
        if (h->P) make_out_map(&m[kOutP], h->P, false, H, cap);
        if (h->d.training) make_out_map(&m[kOutDP], h->dP, false, H, cap);
    }
    if (h->dXr) {
        make_out_map(&m[kOutDXr], h->dXr, false, D, (uint64_t)(h->d.tokens + h->pad - 1) / h->pad * h->pad);
        for (int i = 0; i < h->splits; ++i) make_out_map(&m[kOutSplit0 + i], h->dwr_partial + (size_t)i * h->mw * D, true, D, h->mw);
    }
    if (h->dl_g) make_map_mn(&m[kDlgMN], h->dl_g, h->mw, h->dims.cap, ablk);
    if (h->dl_t) make_map(&m[kDltK], h->dl_t, h->kw, (uint64_t)(h->d.tokens + h->pad - 1) / h->pad * h->pad, 64, 128);
    CK(cudaMemcpyAsync(h->act_maps, m.data(), m.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, h->stream));
}

// Rebuilds the per-expert weight maps and pointer tables when the caller's pointers changed.
void refresh_weights(tmt_moe* h, const void* const* Wup, const void* const* Wdown) {
    const int E = h->local_experts;
    const uint64_t D = h->d.dim, H = h->d.hidden;
    bool same = (int)h->up_seen.size() == E;
    for (int e = 0; same && e < E; ++e)
        same = h->up_seen[e] == Wup[e] && (H == 0 || h->down_seen[e] == Wdown[e]);
    if (same) return;
    h->up_seen.assign(Wup, Wup + E);
    if (H > 0) h->down_seen.assign(Wdown, Wdown + E);
    for (int e = 0; e < E; ++e)
        if (!Wup[e] || (H > 0 && !Wdown[e])) throw std::runtime_error("null expert weight pointer");
    if (h->tensor_core) {
        const uint64_t brows = h->two_cta ? kBN / 2 : kBN;       // rows of B one CTA stages per k block
        std::vector<CUtensorMap> m((size_t)kNumWMaps * E);
        memset(m.data(), 0, m.size() * sizeof(CUtensorMap));
        for (int e = 0; e < E; ++e) {
            if (H > 0) {
                make_map(&m[kUpK * E + e], Wup[e], D, H, 64, (uint32_t)std::min<uint64_t>(brows, H));     // [H][D], k = D
                make_map(&m[kDownK * E + e], Wdown[e], H, D, 64, (uint32_t)std::min<uint64_t>(brows, D)); // [D][H], k = H
                make_map_mn(&m[kDownMN * E + e], Wdown[e], H, D, (uint32_t)brows / 64);    // dH: k = rows (D), n = H contiguous
                make_map_mn(&m[kUpMN * E + e], Wup[e], D, H, (uint32_t)brows / 64);        // dXg: k = rows (H), n = D contiguous
            } else {
                make_map(&m[kUpK * E + e], Wup[e], D, D, 64, (uint32_t)std::min<uint64_t>(brows, D));
                make_map_mn(&m[kUpMN * E + e], Wup[e], D, D, (uint32_t)brows / 64);
            }
        }
        CK(cudaMemcpyAsync(h->w_maps, m.data(), m.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, h->stream));
    }
    CK(cudaMemcpyAsync(h->up_ptrs, Wup, E * sizeof(void*), cudaMemcpyHostToDevice, h->stream));
    if (H > 0) CK(cudaMemcpyAsync(h->down_ptrs, Wdown, E * sizeof(void*), cudaMemcpyHostToDevice, h->stream));
}

void refresh_grads(tmt_moe* h, float* const* dWup, float* const* dWdown) {
    const int E = h->local_experts;
    const bool two = h->d.hidden > 0;
    bool same = (int)h->gup_seen.size() == E;
    for (int e = 0; same && e < E; ++e) same = h->gup_seen[e] == dWup[e] && (!two || h->gdown_seen[e] == dWdown[e]);
    if (same) return;
    for (int e = 0; e < E; ++e)
        if (!dWup[e] || (two && !dWdown[e])) throw std::runtime_error("null expert gradient pointer");
    h->gup_seen.assign(dWup, dWup + E);
    CK(cudaMemcpyAsync(h->gup_ptrs, dWup, E * sizeof(void*), cudaMemcpyHostToDevice, h->stream));
    if (h->tensor_core) {
        const uint64_t D = h->d.dim, H = h->d.hidden;
        std::vector<CUtensorMap> m((size_t)2 * E);
        memset(m.data(), 0, m.size() * sizeof(CUtensorMap));
        for (int e = 0; e < E; ++e) {
            if (two) {
                make_out_map(&m[e], dWup[e], true, D, H);              // dWup[e]: H x D
                make_out_map(&m[E + e], dWdown[e], true, H, D);        // dWdown[e]: D x H
            } else {
                make_out_map(&m[e], dWup[e], true, D, D);
            }
        }
        CK(cudaMemcpyAsync(h->g_maps, m.data(), m.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, h->stream));
    }
    if (two) {
        h->gdown_seen.assign(dWdown, dWdown + E);
        CK(cudaMemcpyAsync(h->gdown_ptrs, dWdown, E * sizeof(void*), cudaMemcpyHostToDevice, h->stream));
    }
}

GemmParams base_params(tmt_moe* h) {
    GemmParams p;
    memset(&p, 0, sizeof p);
    p.experts = h->local_experts;
    p.tile_expert = h->g_tile_expert;
    p.num_m_tiles = h->g_num_m_tiles;
    p.poff = h->g_poff;
    p.status = h->rb.status;
    p.a_boxes = 1; p.b_boxes = 1;
    p.tile_begin = 0; p.tile_count = -1;
    p.dbg = h->gemm_dbg;
    return p;
}

// C[rows, N] = A[rows, K] * W_e (k-major W_e[N][K] or mn-major W_e[K][N])
GemmParams rows_gemm(tmt_moe* h, ActMap a, const uint16_t* A, WMap w, const uint16_t* const* Wptrs, bool w_mn, int N, int K,
                     int epi) {
    GemmParams p = base_params(h);
    p.mode = kRowsRagged;
    p.mapA = h->act_maps + a; p.a_stride = 0;
    p.mapB = h->w_maps + (size_t)w * h->local_experts; p.b_stride = 1;
    p.A = A; p.lda = K; p.Bexp = Wptrs; p.ldb = w_mn ? N : K;
    p.a_mn = 0; p.b_mn = w_mn;
    p.N = N; p.K = K; p.epi = epi; p.ldc = N;
    const int bcols = h->two_cta ? kBN / 2 : kBN;     // columns of the B tile one CTA stages
    if (w_mn) { p.b_boxes = bcols / 64; p.tx_bytes = kBM * kBK * 2 + p.b_boxes * 8192; }
    else p.tx_bytes = kBM * kBK * 2 + (uint32_t)std::min(bcols, N) * kBK * 2;
    return p;
}

// C_e[M, N] = sum over the group's rows of A[r, M] * B[r, N]
GemmParams red_gemm(tmt_moe* h, ActMap a, const uint16_t* A, int M, ActMap b, const uint16_t* B, int N, float* const* out) {
    GemmParams p = base_params(h);
    p.mode = kRedRagged;
    p.mapA = h->act_maps + a; p.a_stride = 0;
    p.mapB = h->act_maps + b; p.b_stride = 0;
    p.A = A; p.lda = M; p.B = B; p.ldb = N;
    p.a_mn = 1; p.b_mn = 1;
    p.a_boxes = kBM / 64; p.b_boxes = (h->two_cta ? kBN / 2 : kBN) / 64;
    p.tx_bytes = (p.a_boxes + p.b_boxes) * 8192;
    p.M = M; p.N = N; p.epi = kEpiF32; p.outF = out; p.ldc = N;
    return p;
}

void run_tc(tmt_moe* h, const GemmParams& p) {
    const int sms = h->sm_limit > 0 ? std::min(h->sm_limit, h->num_sms) : h->num_sms;
    if (h->two_cta) CK(launch_gemm_tcgen05_2cta(p, sms, h->stream));
    else CK(launch_gemm_tcgen05(p, sms, h->stream));
}

void run_gemm(tmt_moe* h, const GemmParams& p0) {
    GemmParams p = p0;
    if (h->gemm_cyc && h->tensor_core) {
        p.cyc = h->gemm_cyc + (size_t)(h->cyc_slot % kGemmCycLaunches) * kGemmCycCtas * kCycSlots;
        CK(cudaMemsetAsync(p.cyc, 0, sizeof(long long) * kGemmCycCtas * kCycSlots, h->stream));
        h->cyc_slot += 1;
    }
    if (h->tensor_core) run_tc(h, p);
    else CK(launch_gemm_simt(p, h->g_max_tiles, h->stream));
    h->launches += 1;
}

const char* const kPhaseNames[kNumPhases] = {
    "router", "scan", "dispatch", "gemm_up", "gemm_down", "combine", "grad_dispatch", "gemm_dh", "gemm_dwdown",
    "gemm_dwup", "gemm_dx", "router_bwd", "router_dw", "router_dx", "scatter", "exchange"};

void prof_collect(tmt_moe* h) {
    Profiler& pr = h->prof;
    if (pr.marks.empty()) return;
    CK(cudaStreamSynchronize(h->stream));
    for (size_t i = 0; i + 1 < pr.marks.size(); ++i) {
        const int ph = pr.marks[i].first;
        if (ph < 0) continue;
        float ms = 0;
        CK(cudaEventElapsedTime(&ms, pr.pool[pr.marks[i].second], pr.pool[pr.marks[i + 1].second]));
        pr.ms[ph] += ms;
        pr.count[ph] += 1;
    }
    pr.marks.clear();
    pr.used = 0;
}

void check_tokens(tmt_moe* h, int tokens) {
    if (tokens < 1 || tokens > h->d.tokens) throw std::runtime_error("tokens outside [1, desc.tokens]");
}

}  // namespace

// Records an event that closes the previous phase and opens `phase` (-1 closes the step).
void prof_mark(tmt_moe* h, int phase) {
    Profiler& pr = h->prof;
    if (!pr.on) return;
    if (pr.used == pr.pool.size()) {
        cudaEvent_t e;
        CK(cudaEventCreate(&e));
        pr.pool.push_back(e);
    }
    CK(cudaEventRecord(pr.pool[pr.used], h->stream));
    pr.marks.emplace_back(phase, pr.used);
    pr.used += 1;
}

// Router, offset tables and the row copies into `grouped` (token-side grouped layout).
void route_and_dispatch(tmt_moe* h, const uint16_t* X, const void* Wr, uint16_t* grouped) {
    route_only(h, X, Wr);
    prof_mark(h, kPhDispatch);
    CK(launch_dispatch(h->dims, h->rb, X, grouped, h->stream, PeerMap(), h->Xc));
    h->launches += 1;
    if (h->host_hooks) CK(cudaEventRecord(h->host_ev[tmt_moe::kEvXFree], h->stream));      // X has been read for the last time
}

void route_only(tmt_moe* h, const uint16_t* X, const void* Wr) {
    prof_mark(h, kPhRouter);
    bool scanned = false;
    int router_kernels = 1;
    CK(launch_router(h->dims, h->rb, X, Wr, h->has_bias ? h->bias : nullptr, h->stream, h->splits, &scanned, h->ln_gamma,
                     h->ln_beta, h->ln_gamma ? h->xn : nullptr, &router_kernels));
    prof_mark(h, kPhScan);
    if (!scanned) CK(launch_scan(h->dims, h->rb, h->splits, h->stream));
    const int plain = (h->dims.T + h->pad - 1) / h->pad * (h->pad / kPad);     // 128-row tiles, whole pairs for the CTA-pair kernel
    if (h->plain_num && plain != h->plain_num_host) {
        CK(cudaMemcpyAsync(h->plain_num, &plain, sizeof(int), cudaMemcpyHostToDevice, h->stream));
        h->plain_num_host = plain;
    }
    h->launches += router_kernels + (scanned ? 0 : 2);      // the router's one or two kernels, and the scan's two when it ran on its own
}

// Grouped expert products over the rows in h->Xg: Yg = expert(Xg). With gate_in_epilogue the
// down-projection scales each row by its gate weight (single-GPU layout, where slotw is local).
void expert_forward(tmt_moe* h, const void* const* Wup, const void* const* Wdown, bool gate_in_epilogue, int tile_begin,
                    int tile_count) {
    const int D = h->d.dim, H = h->d.hidden;
    refresh_weights(h, Wup, Wdown);
    if (H > 0) {
        GemmParams up = rows_gemm(h, kXgK, h->Xg, kUpK, h->up_ptrs, false, H, D, kEpiUp);
        up.tile_begin = tile_begin; up.tile_count = tile_count;
        up.out0 = h->d.training ? h->P : nullptr;
        up.out1 = h->Hact;
        up.mapC0 = h->act_maps + kOutHact; up.mapC1 = h->d.training ? h->act_maps + kOutP : nullptr;
        if (h->q_expert_scales) up.expert_scale = h->q_scales;
        prof_mark(h, kPhGemmUp);
        run_gemm(h, up);
        GemmParams down = rows_gemm(h, kHactK, h->Hact, kDownK, h->down_ptrs, false, D, H, gate_in_epilogue ? kEpiDown : kEpiBf16);
        down.out0 = h->Yg;
        down.tile_begin = tile_begin; down.tile_count = tile_count;
        down.mapC0 = h->act_maps + kOutYg;
        down.row_scale = h->rb.slotw;
        if (h->q_expert_scales) down.expert_scale = h->q_scales + h->d.experts;
        prof_mark(h, kPhGemmDown);
        run_gemm(h, down);
    } else {
        GemmParams g = rows_gemm(h, kXgK, h->Xg, kUpK, h->up_ptrs, false, D, D, kEpiBf16);
        g.out0 = h->Yg;
        g.tile_begin = tile_begin; g.tile_count = tile_count;
        g.mapC0 = h->act_maps + kOutYg;
        prof_mark(h, kPhGemmUp);
        run_gemm(h, g);
    }
}

void forward_impl(tmt_moe* h, const void* X, const void* Wr, const void* const* Wup, const void* const* Wdown, void* Y,
                  float beta, int tokens) {
    check_tokens(h, tokens);
    if (!X || !Wr || !Wup || !Y || (h->d.hidden > 0 && !Wdown)) throw std::runtime_error("null argument");
    CK(cudaSetDevice(h->d.device));
    h->dims.T = tokens;
    h->last_tokens = tokens;
    route_and_dispatch(h, static_cast<const uint16_t*>(X), Wr, h->Xg);
    expert_forward(h, Wup, Wdown, true);
    prof_mark(h, kPhCombine);
    CK(launch_combine(h->dims, h->rb, h->Yg, static_cast<uint16_t*>(Y), beta, h->d.hidden == 0 ? 1 : 0, h->stream));
    prof_mark(h, -1);
    h->launches += 1;
    h->have_forward = true;
}

// The four (reference mode: two) grouped gradient products over the rows in h->dYg.
void expert_backward(tmt_moe* h, const void* const* Wup, const void* const* Wdown, float* const* dWup,
                     float* const* dWdown, int which, int tile_begin, int tile_count) {
    const int D = h->d.dim, H = h->d.hidden;
    refresh_weights(h, Wup, Wdown);
    refresh_grads(h, dWup, dWdown);
    if (H > 0) {
        if (which & 1) {
            GemmParams dh = rows_gemm(h, kDYgK, h->dYg, kDownMN, h->down_ptrs, true, H, D, kEpiDh);
            dh.out0 = h->dP; dh.P = h->P; dh.sw_part = h->sw_part; dh.sw_ld = h->sw_ld;
            dh.mapC0 = h->act_maps + kOutDP;
            dh.tile_begin = tile_begin; dh.tile_count = tile_count;
            prof_mark(h, kPhGemmDh);
            run_gemm(h, dh);
            GemmParams dx = rows_gemm(h, kDPK, h->dP, kUpMN, h->up_ptrs, true, D, H, kEpiBf16);
            dx.out0 = h->dXg;
            dx.mapC0 = h->act_maps + kOutDXg;
            dx.tile_begin = tile_begin; dx.tile_count = tile_count;
            prof_mark(h, kPhGemmDx);
            run_gemm(h, dx);
        }
        if (which & 2) {
            prof_mark(h, kPhGemmDwDown);
            GemmParams gd = red_gemm(h, kDYgMN, h->dYg, D, kHactMN, h->Hact, H, h->gdown_ptrs);
            gd.mapC0 = h->g_maps + h->local_experts; gd.c_stride = 1;
            run_gemm(h, gd);
            prof_mark(h, kPhGemmDwUp);
            GemmParams gu = red_gemm(h, kDPMN, h->dP, H, kXgMN, h->Xg, D, h->gup_ptrs);
            gu.mapC0 = h->g_maps; gu.c_stride = 1;
            run_gemm(h, gu);
        }
    } else {
        if (which & 1) {
            GemmParams dx = rows_gemm(h, kDYgK, h->dYg, kUpMN, h->up_ptrs, true, D, D, kEpiBf16);
            dx.out0 = h->dXg;
            dx.mapC0 = h->act_maps + kOutDXg;
            prof_mark(h, kPhGemmDx);
            run_gemm(h, dx);
        }
        if (which & 2) {
            prof_mark(h, kPhGemmDwUp);
            GemmParams gu = red_gemm(h, kDYgMN, h->dYg, D, kXgMN, h->Xg, D, h->gup_ptrs);
            gu.mapC0 = h->g_maps; gu.c_stride = 1;
            run_gemm(h, gu);
        }
    }
}

void backward_impl(tmt_moe* h, const void* dY, const void* Wr, const void* const* Wup, const void* const* Wdown,
                   float* dWr, float* const* dWup, float* const* dWdown, void* dX, float aux, float zcoef) {
    if (!h->d.training) throw std::runtime_error("handle was created with training = 0");
    if (!h->have_forward) throw std::runtime_error("backward without a preceding forward");
    if (!dY || !Wr || !Wup || !dWr || !dWup || !dX || (h->d.hidden > 0 && (!Wdown || !dWdown)))
        throw std::runtime_error("null argument");
    CK(cudaSetDevice(h->d.device));
    const int H = h->d.hidden;
    prof_mark(h, kPhGradDispatch);
    CK(launch_grad_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(dY), h->Yg, h->dYg, h->s_j, H == 0 ? 1 : 0, h->stream));
    h->launches += 1;
    if (h->host_hooks) CK(cudaEventRecord(h->host_ev[tmt_moe::kEvDyFree], h->stream));     // dY has been read for the last time
    expert_backward(h, Wup, Wdown, dWup, dWdown);
    router_backward(h, Wr, H > 0 ? h->sw_part : nullptr, h->Xc ? h->Xc : h->Xg, h->Xc != nullptr, h->dXg, dWr,
                    static_cast<uint16_t*>(dX), aux, zcoef, h->rb.counts, (long)h->dims.T);
    prof_mark(h, -1);
}

// Expert parallel: the router weight-gradient product reads X either from the token-side grouped send
// buffer (NCCL transport) or, with peer addressing, from a token-order copy. In token order the
// reduction runs over the tokens themselves: dl_t serves as the mn-major A operand (columns past its
// width read as zero) and the split table is fixed.
void build_ep_maps(tmt_moe* h, const uint16_t* x_rows, bool token_order) {
    h->ep_x_token_order = token_order;
    if (!h->tensor_core || !h->dl_t) return;      // both tcgen05 kernels read these maps; the SIMT cross-check path does not
    const uint64_t tpad = (uint64_t)(h->d.tokens + h->pad - 1) / h->pad * h->pad;
    CUtensorMap m[2];
    memset(m, 0, sizeof m);
    make_map_mn(&m[0], x_rows, h->d.dim, token_order ? tpad : (uint64_t)h->dims.cap, (h->two_cta ? kBN / 2 : kBN) / 64);
    CK(cudaMemcpyAsync(h->act_maps + kXsMN, &m[0], sizeof(CUtensorMap), cudaMemcpyHostToDevice, h->stream));
    if (token_order) {
        make_map_mn(&m[1], h->dl_t, h->kw, tpad, kBM / 64);
        CK(cudaMemcpyAsync(h->act_maps + kDltMN, &m[1], sizeof(CUtensorMap), cudaMemcpyHostToDevice, h->stream));
        std::vector<int> sp(kMaxSplits + 1, 0);
        const long tiles = (long)tpad / kPad;
        for (int i = 0; i <= h->splits; ++i) sp[i] = (int)(tiles * i / h->splits) * kPad;
        h->tok_split_poff = dalloc<int>(h, kMaxSplits + 1);
        CK(cudaMemcpyAsync(h->tok_split_poff, sp.data(), sp.size() * sizeof(int), cudaMemcpyHostToDevice, h->stream));
    }
    CK(cudaStreamSynchronize(h->stream));
}

void router_backward(tmt_moe* h, const void* Wr, const float* sw_part, const uint16_t* grouped_x, bool x_is_ep,
                     const uint16_t* dXg_rows, float* dWr, uint16_t* dX, float aux, float zcoef, const int* counts, long n_norm,
                     PeerMap pm, bool defer_scatter) {
    const bool tok_order = x_is_ep && h->ep_x_token_order;
    const int D = h->d.dim, E = h->d.experts;
    if (E == 1) {      // dense shortcut: no router gradient (moe.cu:488-494)
        CK(cudaMemsetAsync(dWr, 0, (size_t)E * D * sizeof(float), h->stream));
        prof_mark(h, kPhScatter);
        CK(launch_scatter(h->dims, h->rb, h->dlogits, Wr, dXg_rows, nullptr, dX, h->stream, pm));
        h->launches += 1;
        return;
    }
    const bool tc = h->tensor_core;
    prof_mark(h, kPhRouterBwd);
    if (tc && tok_order) {      // rows of an earlier, longer call must not reach the token-order reduction
        if (h->dims.T < h->dl_t_rows)
            CK(cudaMemsetAsync(h->dl_t + (size_t)h->dims.T * h->kw, 0, (size_t)(h->dl_t_rows - h->dims.T) * h->kw * 2, h->stream));
        h->dl_t_rows = h->dims.T;
    }
    if (tc && !tok_order) CK(cudaMemsetAsync(h->dl_g, 0, (size_t)h->dims.cap * h->mw * 2, h->stream));
    CK(launch_router_bwd(h->dims, h->rb, sw_part, h->sw_ld, h->s_j, h->dlogits, aux, zcoef, counts, n_norm,
                         tc ? h->dl_t : nullptr, h->kw, tc && !tok_order ? h->dl_g : nullptr, h->mw, h->stream));
    h->launches += 1;
    if (!tc) {
        prof_mark(h, kPhRouterDw);
        if (tok_order) throw std::runtime_error("the SIMT cross-check path does not support the peer transport");
        CK(launch_router_dw(h->dims, h->rb, h->dlogits, grouped_x, h->dwr_partial, kRouterDwChunks, dWr, h->stream));
        prof_mark(h, kPhScatter);
        CK(launch_scatter(h->dims, h->rb, h->dlogits, Wr, dXg_rows, nullptr, dX, h->stream, pm));
        h->launches += 3;
        return;
    }
    // router weights as a bf16 [E][D] matrix for the token-order product (the reference's work copy, model.cu:513)
    const uint16_t* wr16 = static_cast<const uint16_t*>(Wr);
    if (h->dims.router_f32) {
        CK(launch_to_bf16(static_cast<const float*>(Wr), h->wr_bf16, (long)E * D, h->stream));
        h->launches += 1;
        wr16 = h->wr_bf16;
    }
    if (h->wr_seen != wr16) {
        CUtensorMap m;
        memset(&m, 0, sizeof m);
        make_map_mn(&m, wr16, D, E, (h->two_cta ? kBN / 2 : kBN) / 64);
        CK(cudaMemcpyAsync(h->w_maps + (size_t)kNumWMaps * h->local_experts, &m, sizeof m, cudaMemcpyHostToDevice, h->stream));
        h->wr_seen = wr16;
    }
    prof_mark(h, kPhRouterDw);
    {   // dWr = dl_g^T * X_grouped, reduction split into h->splits row ranges, then summed
        GemmParams p = base_params(h);
        p.mode = kRedRagged;
        p.mapA = h->act_maps + (tok_order ? kDltMN : kDlgMN); p.a_stride = 0;
        p.mapB = h->act_maps + (x_is_ep ? kXsMN : kXgMN); p.b_stride = 0;
        p.a_mn = 1; p.b_mn = 1;
        p.a_boxes = kBM / 64; p.b_boxes = (h->two_cta ? kBN / 2 : kBN) / 64;
        p.tx_bytes = (p.a_boxes + p.b_boxes) * 8192;
        p.M = h->mw; p.N = D; p.experts = h->splits; p.poff = tok_order ? h->tok_split_poff : h->rb.split_poff;
        p.epi = kEpiF32; p.outF = h->dwr_part_ptrs; p.ldc = D;
        p.mapC0 = h->act_maps + kOutSplit0; p.c_stride = 1;
        run_tc(h, p);
        CK(launch_reduce_parts(h->dwr_partial, h->splits, h->mw, E, D, dWr, h->stream));
        h->launches += 2;
    }
    prof_mark(h, kPhRouterDx);
    {   // dXr = dl_t * Wr (one k block per 64 experts), then dX = dXr + sum_j dXg[slot_j]
        GemmParams p = base_params(h);
        p.mode = kRowsRagged;
        p.mapA = h->act_maps + kDltK; p.a_stride = 0;
        p.mapB = h->w_maps + (size_t)kNumWMaps * h->local_experts; p.b_stride = 0;
        p.a_mn = 0; p.b_mn = 1;
        p.b_boxes = (h->two_cta ? kBN / 2 : kBN) / 64;
        p.tx_bytes = kBM * kBK * 2 + p.b_boxes * 8192;
        p.N = D; p.K = h->kw; p.experts = 1;
        p.tile_expert = h->plain_tiles; p.num_m_tiles = h->plain_num;
        p.epi = kEpiBf16; p.out0 = h->dXr; p.ldc = D;
        p.mapC0 = h->act_maps + kOutDXr;
        run_tc(h, p);
        h->launches += 1;
        if (defer_scatter) return;
        prof_mark(h, kPhScatter);
        scatter_rows(h, Wr, dXg_rows, dX, h->stream, pm);
    }
}

void scatter_rows(tmt_moe* h, const void* Wr, const uint16_t* dXg_rows, uint16_t* dX, cudaStream_t stream, PeerMap pm) {
    CK(launch_scatter(h->dims, h->rb, h->dlogits, Wr, dXg_rows, h->tensor_core ? h->dXr : nullptr, dX, stream, pm));
    h->launches += 1;
}

tmt_moe* create_impl(const tmt_moe_desc* dsc) {
    const tmt_moe_desc& d = *dsc;
    if (d.tokens < 1 || d.dim < 64 || d.dim % 64 || d.hidden < 0 || d.hidden % 64)
        throw std::runtime_error("need tokens >= 1, dim and hidden multiples of 64");
    if (d.experts < 1 || d.experts > 256 || d.topk < 1 || d.topk > d.experts || d.topk > 8)
        throw std::runtime_error("require 1 <= topk <= experts <= 256 and topk <= 8");
    if (d.ep_world < 1 || d.ep_rank < 0 || d.ep_rank >= d.ep_world || d.experts % d.ep_world)
        throw std::runtime_error("invalid expert-parallel layout (experts must divide by ep_world)");
    if ((long)d.tokens * d.topk + 256L * d.experts > 0x7fffff00L)
        throw std::runtime_error("tokens * topk exceeds the supported index range");
    CK(cudaSetDevice(d.device));
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, d.device));
    if (prop.major != 10) throw std::runtime_error("this library is built for sm_100a (B200) only");
    std::unique_ptr<tmt_moe, void (*)(tmt_moe*)> hold(new tmt_moe(), [](tmt_moe* p) { tmt_moe_destroy(p); });
    tmt_moe* h = hold.get();
    h->d = d;
    h->stream = static_cast<cudaStream_t>(d.stream);
    h->num_sms = prop.multiProcessorCount;
    h->local_experts = d.experts / d.ep_world;
    const int T = d.tokens, E = d.experts, K = d.topk, D = d.dim, H = d.hidden;
    if (d.gemm_impl < 0 || d.gemm_impl > 3) throw std::runtime_error("unknown gemm_impl");
    h->tensor_core = d.gemm_impl != TMT_MOE_GEMM_SIMT;
    h->two_cta = d.gemm_impl == TMT_MOE_GEMM_TCGEN05_2CTA || d.gemm_impl == TMT_MOE_GEMM_AUTO;
#ifdef TMT_MOE_MEASURE
    if (const char* dbg = getenv("TMT_MOE_GEMM_DEBUG")) h->gemm_dbg = atoi(dbg);     // measurement builds only: results are then wrong
#endif
    if (const char* cyc = getenv("TMT_MOE_GEMM_CYCLES"))                               // measurement only: per-role cycle counters
        if (atoi(cyc) && h->num_sms <= kGemmCycCtas) h->gemm_cyc = dalloc<long long>(h, (size_t)kGemmCycLaunches * kGemmCycCtas * kCycSlots);
    h->pad = h->two_cta ? 2 * kPad : kPad;
    const int pad = h->pad;
    // rows of the grouped buffers: every assignment plus up to pad-1 pad rows per expert (moe.cu:331)
    const long cap = ((long)T * K + pad - 1) / pad * pad + (long)pad * E;
    h->dims = RouteDims{T, D, E, K, (int)cap, (int)(cap / kPad), d.router_dtype == TMT_MOE_F32, pad};
    // rows of the grouped GEMM buffers: the token-side layout on one GPU; under expert parallelism the
    // rows other ranks may route here, bounded by the capacity factor (default 1.5 x tokens x topk)
    long gcap = cap;
    if (d.ep_world > 1) {
        const double f = d.ep_capacity_factor > 0 ? d.ep_capacity_factor : 1.5;
        gcap = ((long)(f * T * K) + pad - 1) / pad * pad + (long)pad * h->local_experts;
        if (gcap > 0x7fffff00L) throw std::runtime_error("expert-side capacity exceeds the supported index range");
    }
    h->gcap = gcap;
    h->x_cap = (int)gcap;
    const int NB = (T + kTokBlock - 1) / kTokBlock;
    RouteBufs& b = h->rb;
    b.logits = dalloc<float>(h, (size_t)T * E);
    b.probs = dalloc<float>(h, (size_t)T * E);
    b.lse = dalloc<float>(h, T);
    b.idx = dalloc<int>(h, (size_t)T * K);
    b.w = dalloc<float>(h, (size_t)T * K);
    b.rank = dalloc<int>(h, (size_t)NB * kTokBlock * K);
    b.block_counts = dalloc<int>(h, (size_t)NB * E);
    b.block_sump = dalloc<float>(h, (size_t)NB * E);
    b.block_z = dalloc<float>(h, NB);
    b.block_base = dalloc<int>(h, (size_t)NB * E);
    b.counts = dalloc<int>(h, E);
    b.off = dalloc<int>(h, E + 1);
    b.poff = dalloc<int>(h, E + 1);
    b.tile_expert = dalloc<int>(h, cap / kPad);
    b.num_m_tiles = dalloc<int>(h, 1);
    b.stat = dalloc<float>(h, E + 1);
    b.slot_of = dalloc<int>(h, (size_t)T * K);
    b.slotw = dalloc<float>(h, cap);
    b.tok_of_slot = dalloc<int>(h, cap);
    b.split_poff = dalloc<int>(h, kMaxSplits + 1);
    b.status = dalloc<int>(h, 1);
    CK(cudaMemsetAsync(b.status, 0, sizeof(int), h->stream));
    b.use_acc = dalloc<long long>(h, E + 1);
    CK(cudaMemsetAsync(b.use_acc, 0, sizeof(long long) * (E + 1), h->stream));
    h->bias = dalloc<float>(h, E);
    h->Xg = dalloc<uint16_t>(h, (size_t)gcap * D);
    h->Yg = dalloc<uint16_t>(h, (size_t)gcap * D);
    if (H > 0) h->Hact = dalloc<uint16_t>(h, (size_t)gcap * H);
    if (d.training) {
        h->dYg = dalloc<uint16_t>(h, (size_t)gcap * D);
        h->dXg = dalloc<uint16_t>(h, (size_t)gcap * D);
        h->s_j = dalloc<float>(h, (size_t)T * K);
        h->dlogits = dalloc<float>(h, (size_t)T * E);
        if (h->tensor_core && E > 1) {
            h->kw = (E + 63) / 64 * 64;
            h->mw = (E + kBM - 1) / kBM * kBM;
            const int tiles = (h->mw / kBM) * ((D + kBN - 1) / kBN);
            h->splits = std::max(1, std::min(kMaxSplits, h->num_sms / tiles));
            const size_t tpad = (size_t)(T + pad - 1) / pad * pad;
            h->dl_t = dalloc<uint16_t>(h, tpad * h->kw);
            CK(cudaMemsetAsync(h->dl_t, 0, tpad * h->kw * 2, h->stream));
            // The router weight gradient reduces over the tokens themselves: X is kept in token order by the dispatch
            // kernel (tokens*D*2 bytes) instead of being read back from the grouped copy (topk times as many rows) through
            // a zero-padded grouped gradient. Expert-parallel handles get their token-order copy in tmt_moe_ep_init.
            if (d.ep_world == 1) {
                h->Xc = dalloc<uint16_t>(h, tpad * D);
                CK(cudaMemsetAsync(h->Xc, 0, tpad * D * 2, h->stream));
            } else {
                h->dl_g = dalloc<uint16_t>(h, (size_t)cap * h->mw);
            }
            h->dXr = dalloc<uint16_t>(h, tpad * D);
            h->wr_bf16 = dalloc<uint16_t>(h, (size_t)E * D);
            h->dwr_partial = dalloc<float>(h, (size_t)h->splits * h->mw * D);
            h->dwr_part_ptrs = dalloc<float*>(h, h->splits);
            std::vector<float*> ptrs(h->splits);
            for (int i = 0; i < h->splits; ++i) ptrs[i] = h->dwr_partial + (size_t)i * h->mw * D;
            CK(cudaMemcpyAsync(h->dwr_part_ptrs, ptrs.data(), ptrs.size() * sizeof(float*), cudaMemcpyHostToDevice, h->stream));
            h->plain_tiles = dalloc<int>(h, tpad / kPad);
            CK(cudaMemsetAsync(h->plain_tiles, 0, tpad / kPad * sizeof(int), h->stream));
            h->plain_num = dalloc<int>(h, 1);
        } else {
            h->dwr_partial = dalloc<float>(h, (size_t)kRouterDwChunks * E * D);
        }
        if (H > 0) {
            h->P = dalloc<uint16_t>(h, (size_t)gcap * H);
            h->dP = dalloc<uint16_t>(h, (size_t)gcap * H);
            h->sw_ld = (H + kEpiCols - 1) / kEpiCols;
            h->sw_part = dalloc<float>(h, (size_t)gcap * h->sw_ld);
        }
    } else {
        // forward-only handles still need valid map bases for the unused gradient maps
        h->dYg = h->Xg; h->dP = h->Hact;
    }
    h->act_maps = dalloc<CUtensorMap>(h, kNumActMaps);
    h->w_maps = dalloc<CUtensorMap>(h, (size_t)kNumWMaps * h->local_experts + 1);
    h->up_ptrs = dalloc<const uint16_t*>(h, h->local_experts);
    h->down_ptrs = dalloc<const uint16_t*>(h, h->local_experts);
    h->gup_ptrs = dalloc<float*>(h, h->local_experts);
    h->gdown_ptrs = dalloc<float*>(h, h->local_experts);
    h->g_maps = dalloc<CUtensorMap>(h, (size_t)2 * h->local_experts);
    h->g_poff = b.poff; h->g_num_m_tiles = b.num_m_tiles; h->g_tile_expert = b.tile_expert; h->g_max_tiles = h->dims.max_tiles;
    if (h->tensor_core) build_act_maps(h);
    if (h->Xc) build_ep_maps(h, h->Xc, true);
    if (d.host_io) {
        CK(cudaStreamCreateWithFlags(&h->in_stream, cudaStreamNonBlocking));
        CK(cudaStreamCreateWithFlags(&h->out_stream, cudaStreamNonBlocking));
        for (cudaEvent_t& e : h->host_ev) CK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        h->Xs = dalloc<uint16_t>(h, (size_t)T * D);
        h->Ys = dalloc<uint16_t>(h, (size_t)T * D);
        if (d.training) {
            h->dYs = dalloc<uint16_t>(h, (size_t)T * D);
            h->dXs = dalloc<uint16_t>(h, (size_t)T * D);
        }
    }
    CK(cudaStreamSynchronize(h->stream));
    return hold.release();
}

}  // namespace tmt

using namespace tmt;

#define GUARD(...)                                                     \
    try { __VA_ARGS__; return 0; }                                     \
    catch (const std::exception& e) { set_error("%s", e.what()); return -1; } \
    catch (...) { set_error("unknown error"); return -1; }

extern "C" {

const char* tmt_moe_last_error(void) { return g_error.c_str(); }

int tmt_moe_create(const tmt_moe_desc* desc, tmt_moe** out) {
    if (!desc || !out) { set_error("null argument"); return -1; }
    *out = nullptr;
    GUARD(*out = create_impl(desc))
}

void tmt_moe_destroy(tmt_moe* h) {
    if (!h) return;
    cudaSetDevice(h->d.device);
    cudaStreamSynchronize(h->stream);
    ep_teardown(h);
    for (cudaEvent_t e : h->prof.pool) cudaEventDestroy(e);
    for (cudaStream_t st : {h->in_stream, h->out_stream}) if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
    for (cudaEvent_t e : h->host_ev) if (e) cudaEventDestroy(e);
    for (void* p : h->allocs) cudaFree(p);
    delete h;
}

int tmt_moe_set_router_bias(tmt_moe* h, const float* bias_host) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        CK(cudaSetDevice(h->d.device));
        h->has_bias = bias_host != nullptr;
        if (bias_host) {
            CK(cudaMemcpyAsync(h->bias, bias_host, h->d.experts * sizeof(float), cudaMemcpyHostToDevice, h->stream));
            CK(cudaStreamSynchronize(h->stream));
        }
    })
}

int tmt_moe_forward(tmt_moe* h, const void* X, const void* Wrouter, const void* const* Wup, const void* const* Wdown,
                    void* Y, float beta, int tokens) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        if (h->d.ep_world > 1) ep_forward(h, X, Wrouter, Wup, Wdown, Y, beta, tokens);
        else forward_impl(h, X, Wrouter, Wup, Wdown, Y, beta, tokens);
    })
}

int tmt_moe_backward(tmt_moe* h, const void* dY, const void* Wrouter, const void* const* Wup, const void* const* Wdown,
                     float* dWrouter, float* const* dWup, float* const* dWdown, void* dX, float aux, float zcoef) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        if (h->d.ep_world > 1) ep_backward(h, dY, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, dX, aux, zcoef);
        else backward_impl(h, dY, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, dX, aux, zcoef);
    })
}

int tmt_moe_stats(tmt_moe* h, float* stat, int64_t* counts, float* aux) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        CK(cudaSetDevice(h->d.device));
        const int E = h->d.experts, K = h->d.topk;
        std::vector<float> st(E + 1);
        std::vector<int> cn(E);
        CK(cudaMemcpyAsync(st.data(), ep_stat(h), (E + 1) * sizeof(float), cudaMemcpyDeviceToHost, h->stream));
        CK(cudaMemcpyAsync(cn.data(), h->ep_world_counts ? h->ep_world_counts : h->rb.counts, E * sizeof(int),
                           cudaMemcpyDeviceToHost, h->stream));
        CK(cudaStreamSynchronize(h->stream));
        const double N = (double)h->last_tokens * h->d.ep_world;
        st[E] /= (float)h->d.ep_world;     // every rank contributed the mean over its own tokens
        if (stat) memcpy(stat, st.data(), (E + 1) * sizeof(float));
        if (counts) for (int e = 0; e < E; ++e) counts[e] = cn[e];
        if (aux) {
            // moe_aux_from, moe.cu:470-475
            float a = 0;
            for (int e = 0; e < E; ++e) a += (st[e] / (float)N) * (cn[e] / (float)(N * K));
            *aux = E == 1 ? 0.0f : E * a;
        }
    })
}

int tmt_moe_copy_stats(tmt_moe* h, float* stat_device) {
    if (!h || !stat_device) { set_error("null argument"); return -1; }
    GUARD({
        CK(cudaSetDevice(h->d.device));
        CK(cudaMemcpyAsync(stat_device, ep_stat(h), (h->d.experts + 1) * sizeof(float), cudaMemcpyDeviceToDevice, h->stream));
    })
}

int tmt_moe_step_host_async(tmt_moe* h, const void* X_host, const void* dY_host, const void* Wrouter, const void* const* Wup,
                            const void* const* Wdown, float* dWrouter, float* const* dWup, float* const* dWdown, void* Y_host,
                            void* dX_host, float* stat_host, float beta, float aux, float zcoef, int tokens) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        if (!h->Xs) throw std::runtime_error("handle was created with host_io = 0");
        if (!X_host || !Y_host) throw std::runtime_error("null argument");
        check_tokens(h, tokens);
        CK(cudaSetDevice(h->d.device));
        const size_t bytes = (size_t)tokens * h->d.dim * 2;
        const bool bwd = dY_host != nullptr;
        if (bwd && (!dX_host || !h->dYs)) throw std::runtime_error("backward needs dX_host and training = 1");
        // Three streams. Uploads wait only until the previous step has consumed the staging buffer (X: after its
        // dispatch, dY: after its gradient dispatch), so they run under the previous step's GEMMs; downloads run under
        // the next phase of compute; the compute stream waits for exactly what it consumes or overwrites. PCIe carries
        // both directions at once. (Waiting on an event that was never recorded returns at once: first step.)
        cudaEvent_t* ev = h->host_ev;
        CK(cudaStreamWaitEvent(h->in_stream, ev[tmt_moe::kEvXFree], 0));
        CK(cudaMemcpyAsync(h->Xs, X_host, bytes, cudaMemcpyHostToDevice, h->in_stream));
        CK(cudaEventRecord(ev[tmt_moe::kEvXReady], h->in_stream));
        if (bwd) {
            CK(cudaStreamWaitEvent(h->in_stream, ev[tmt_moe::kEvDyFree], 0));
            CK(cudaMemcpyAsync(h->dYs, dY_host, bytes, cudaMemcpyHostToDevice, h->in_stream));
            CK(cudaEventRecord(ev[tmt_moe::kEvDyReady], h->in_stream));
        }
        CK(cudaStreamWaitEvent(h->stream, ev[tmt_moe::kEvXReady], 0));
        CK(cudaStreamWaitEvent(h->stream, ev[tmt_moe::kEvYOut], 0));        // the previous Y has left Ys
        if (beta != 0.0f) CK(cudaMemcpyAsync(h->Ys, Y_host, bytes, cudaMemcpyHostToDevice, h->stream));
        h->host_hooks = true;
        struct Off { tmt_moe* h; ~Off() { h->host_hooks = false; } } off{h};
        if (h->d.ep_world > 1) ep_forward(h, h->Xs, Wrouter, Wup, Wdown, h->Ys, beta, tokens);
        else forward_impl(h, h->Xs, Wrouter, Wup, Wdown, h->Ys, beta, tokens);
        CK(cudaEventRecord(ev[tmt_moe::kEvYWritten], h->stream));
        CK(cudaStreamWaitEvent(h->out_stream, ev[tmt_moe::kEvYWritten], 0));
        CK(cudaMemcpyAsync(Y_host, h->Ys, bytes, cudaMemcpyDeviceToHost, h->out_stream));
        if (stat_host)
            CK(cudaMemcpyAsync(stat_host, ep_stat(h), (h->d.experts + 1) * sizeof(float), cudaMemcpyDeviceToHost, h->out_stream));
        CK(cudaEventRecord(ev[tmt_moe::kEvYOut], h->out_stream));
        if (bwd) {
            CK(cudaStreamWaitEvent(h->stream, ev[tmt_moe::kEvDyReady], 0));
            CK(cudaStreamWaitEvent(h->stream, ev[tmt_moe::kEvDxOut], 0));   // the previous dX has left dXs
            if (h->d.ep_world > 1) ep_backward(h, h->dYs, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, h->dXs, aux, zcoef);
            else backward_impl(h, h->dYs, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, h->dXs, aux, zcoef);
            CK(cudaEventRecord(ev[tmt_moe::kEvDxWritten], h->stream));
            CK(cudaStreamWaitEvent(h->out_stream, ev[tmt_moe::kEvDxWritten], 0));
            CK(cudaMemcpyAsync(dX_host, h->dXs, bytes, cudaMemcpyDeviceToHost, h->out_stream));
            CK(cudaEventRecord(ev[tmt_moe::kEvDxOut], h->out_stream));
        }
    })
}

int tmt_moe_host_wait(tmt_moe* h) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        if (!h->Xs) throw std::runtime_error("handle was created with host_io = 0");
        CK(cudaSetDevice(h->d.device));
        CK(cudaStreamSynchronize(h->in_stream));
        CK(cudaStreamSynchronize(h->stream));
        CK(cudaStreamSynchronize(h->out_stream));
    })
}

int tmt_moe_step_host(tmt_moe* h, const void* X_host, const void* dY_host, const void* Wrouter, const void* const* Wup,
                      const void* const* Wdown, float* dWrouter, float* const* dWup, float* const* dWdown, void* Y_host,
                      void* dX_host, float* stat_host, float beta, float aux, float zcoef, int tokens) {
    if (tmt_moe_step_host_async(h, X_host, dY_host, Wrouter, Wup, Wdown, dWrouter, dWup, dWdown, Y_host, dX_host, stat_host, beta,
                                aux, zcoef, tokens) != 0)
        return -1;
    return tmt_moe_host_wait(h);
}

long long tmt_moe_read(tmt_moe* h, const char* name, void* dst, size_t dst_bytes) {
    if (!h || !name || !dst) { set_error("null argument"); return -1; }
    try {
        CK(cudaSetDevice(h->d.device));
        const size_t T = h->last_tokens, E = h->d.experts, K = h->d.topk;
        const void* src = nullptr;
        size_t n = 0;
        const std::string s(name);
        if (s == "logits") { src = h->rb.logits; n = T * E * 4; }
        else if (s == "probs") { src = h->rb.probs; n = T * E * 4; }
        else if (s == "idx") { src = h->rb.idx; n = T * K * 4; }
        else if (s == "slot_of") { src = h->rb.slot_of; n = T * K * 4; }
        else if (s == "w") { src = h->rb.w; n = T * K * 4; }
        else if (s == "lse") { src = h->rb.lse; n = T * 4; }
        else if (s == "counts") { src = h->rb.counts; n = E * 4; }
        else if (s == "poff") { src = h->rb.poff; n = (E + 1) * 4; }
        else if (s == "dlogits") { src = h->dlogits; n = T * E * 4; }
        else if (s == "s_j") { src = h->s_j; n = T * K * 4; }
        else if (s == "cap") { n = 4; int cap = h->dims.cap; if (dst_bytes < 4) throw std::runtime_error("destination too small"); memcpy(dst, &cap, 4); return 4; }
        else if (s == "slotw") { src = h->rb.slotw; n = (size_t)h->dims.cap * 4; }
        else if (s == "tok_of_slot") { src = h->rb.tok_of_slot; n = (size_t)h->dims.cap * 4; }
        else if (s == "tile_expert") { src = h->rb.tile_expert; n = (size_t)h->dims.max_tiles * 4; }
        else if (s == "num_m_tiles") { src = h->rb.num_m_tiles; n = 4; }
        // grouped activations, all gcap rows: the rows of the grouped GEMM buffers ("gcap"; equal to "cap" on one GPU)
        else if (s == "Xg") { src = h->Xg; n = (size_t)h->gcap * h->d.dim * 2; }
        else if (s == "Yg") { src = h->Yg; n = (size_t)h->gcap * h->d.dim * 2; }
        else if (s == "dYg") { src = h->d.training ? h->dYg : nullptr; n = (size_t)h->gcap * h->d.dim * 2; }
        else if (s == "dXg") { src = h->dXg; n = (size_t)h->gcap * h->d.dim * 2; }
        else if (s == "ep_waves") { int w = ep_waves(h); if (dst_bytes < 4) throw std::runtime_error("destination too small"); memcpy(dst, &w, 4); return 4; }
        else if (s == "gcap") { n = 4; int gc = (int)h->gcap; if (dst_bytes < 4) throw std::runtime_error("destination too small"); memcpy(dst, &gc, 4); return 4; }
        else if (s == "P") { src = h->P; n = (size_t)h->gcap * h->d.hidden * 2; }
        else if (s == "Hact") { src = h->Hact; n = (size_t)h->gcap * h->d.hidden * 2; }
        else if (s == "dP") { src = h->d.training ? h->dP : nullptr; n = (size_t)h->gcap * h->d.hidden * 2; }
        else if (s == "sw_part") { src = h->sw_part; n = (size_t)h->gcap * h->sw_ld * 4; }
        else throw std::runtime_error("unknown tensor name: " + s);
        if (!src) throw std::runtime_error("tensor not kept by this handle: " + s);
        if (n > dst_bytes) throw std::runtime_error("destination too small for " + s);
        CK(cudaMemcpyAsync(dst, src, n, cudaMemcpyDeviceToHost, h->stream));
        CK(cudaStreamSynchronize(h->stream));
        return (long long)n;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

int tmt_moe_set_profile(tmt_moe* h, int on) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        CK(cudaSetDevice(h->d.device));
        prof_collect(h);
        h->prof.on = on != 0;
    })
}

int tmt_moe_profile(tmt_moe* h, float* ms, long long* count, int reset) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        CK(cudaSetDevice(h->d.device));
        prof_collect(h);
        for (int i = 0; i < kNumPhases; ++i) {
            if (ms) ms[i] = (float)h->prof.ms[i];
            if (count) count[i] = h->prof.count[i];
            if (reset) { h->prof.ms[i] = 0; h->prof.count[i] = 0; }
        }
    })
}

int tmt_moe_num_phases(void) { return kNumPhases; }
const char* tmt_moe_phase_name(int i) { return i >= 0 && i < kNumPhases ? kPhaseNames[i] : ""; }

int tmt_moe_selftest_bounded_wait(tmt_moe* h, long long limit_cycles) {
    if (!h) { set_error("null handle"); return -1; }
    int out = -1;
    try {
        CK(cudaSetDevice(h->d.device));
        if (limit_cycles < 1 || limit_cycles > 2000000000LL) throw std::runtime_error("limit_cycles outside [1, 2e9]");
        int* words = dalloc<int>(h, 2);          // [0] status of this self-test, [1] where the kernel ended
        CK(cudaMemsetAsync(words, 0, 2 * sizeof(int), h->stream));
        CK(launch_bounded_wait_selftest(words, limit_cycles, words + 1, h->stream));
        int host[2] = {-1, -1};
        CK(cudaMemcpyAsync(host, words, sizeof host, cudaMemcpyDeviceToHost, h->stream));
        CK(cudaStreamSynchronize(h->stream));
        out = (host[0] == kErrWaitTimeout && host[1] == 1) ? kErrWaitTimeout : -2 - host[1];
        return out;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

long long tmt_moe_launch_count(const tmt_moe* h) { return h ? h->launches : -1; }

int tmt_moe_usage(tmt_moe* h, double* min_share, double* max_share, long long* dead, long long* passes, long long* totals,
                  int reset) {
    if (!h) { set_error("null handle"); return -1; }
    GUARD({
        CK(cudaSetDevice(h->d.device));
        const int E = h->d.experts;
        std::vector<long long> acc(E + 1);
        CK(cudaMemcpyAsync(acc.data(), h->rb.use_acc, sizeof(long long) * (E + 1), cudaMemcpyDeviceToHost, h->stream));
        if (reset) CK(cudaMemsetAsync(h->rb.use_acc, 0, sizeof(long long) * (E + 1), h->stream));
        CK(cudaStreamSynchronize(h->stream));
        long long tot = 0;
        for (int e = 0; e < E; ++e) tot += acc[e];
        double mn = 1, mx = 0;                     // train_main.cu:235-243: share 1.0 = uniform, dead below 0.01
        long long nd = 0;
        for (int e = 0; e < E; ++e) {
            const double s = tot ? (double)acc[e] / (double)tot * E : 0;
            mn = std::min(mn, s); mx = std::max(mx, s);
            if (s < 0.01) ++nd;
        }
        if (min_share) *min_share = mn;
        if (max_share) *max_share = mx;
        if (dead) *dead = nd;
        if (passes) *passes = acc[E];
        if (totals) for (int e = 0; e < E; ++e) totals[e] = acc[e];
    })
}

int tmt_moe_debug_gemm_cycles(tmt_moe* h, long long* out, int* launches, int* ctas, int* slots) {
    if (!h) { set_error("null handle"); return -1; }
    if (launches) *launches = kGemmCycLaunches;
    if (ctas) *ctas = kGemmCycCtas;
    if (slots) *slots = kCycSlots;
    if (!h->gemm_cyc) { set_error("cycle counters are off (set TMT_MOE_GEMM_CYCLES=1 before tmt_moe_create)"); return -1; }
    if (!out) return h->cyc_slot;
    cudaSetDevice(h->d.device);
    if (cudaMemcpyAsync(out, h->gemm_cyc, sizeof(long long) * kGemmCycLaunches * kGemmCycCtas * kCycSlots, cudaMemcpyDeviceToHost, h->stream) != cudaSuccess ||
        cudaStreamSynchronize(h->stream) != cudaSuccess) {
        set_error("reading the cycle counters failed: %s", cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    return h->cyc_slot;
}

int tmt_moe_device_status(tmt_moe* h) {
    if (!h) { set_error("null handle"); return -1; }
    int v = -1;
    cudaSetDevice(h->d.device);
    if (cudaMemcpyAsync(&v, h->rb.status, sizeof v, cudaMemcpyDeviceToHost, h->stream) != cudaSuccess ||
        cudaStreamSynchronize(h->stream) != cudaSuccess) {
        set_error("reading the device status failed: %s", cudaGetErrorString(cudaGetLastError()));
        return -1;
    }
    return v;
}

}  // extern "C"
