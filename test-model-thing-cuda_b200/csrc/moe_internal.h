// Internal definition of the opaque handle and of the entry points shared between the
// translation units of the library.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <memory>
#include <string>
#include <vector>

#include "../../include/tmt_moe.h"
#include "kernels.cuh"

struct tmt_ep_state;

namespace tmt {
// Phases of one step, timed with CUDA events on the handle's stream when profiling is on
// (the reference's TMT_PROFILE phases, tmt-cuda/src/moe.cu:380-394, at kernel granularity).
enum Phase : int {
    kPhRouter = 0, kPhScan, kPhDispatch, kPhGemmUp, kPhGemmDown, kPhCombine,
    kPhGradDispatch, kPhGemmDh, kPhGemmDwDown, kPhGemmDwUp, kPhGemmDx, kPhRouterBwd, kPhRouterDw, kPhRouterDx, kPhScatter,
    kPhExchange, kNumPhases
};
struct Profiler {
    bool on = false;
    std::vector<cudaEvent_t> pool;
    size_t used = 0;
    std::vector<std::pair<int, size_t>> marks;   // (phase or -1 = end of step, event index)
    double ms[kNumPhases] = {0};
    long long count[kNumPhases] = {0};
};
}  // namespace tmt

constexpr int kGemmCycLaunches = 16;   // GEMM launches whose cycle counters are kept (a ring)
constexpr int kGemmCycCtas = 160;

struct tmt_moe {
    tmt_moe_desc d{};
    cudaStream_t stream = nullptr;
    int num_sms = 0;
    int local_experts = 0;
    tmt::RouteDims dims{};
    tmt::RouteBufs rb{};
    // layout tables the grouped GEMMs run on: the token-side tables on one GPU, the expert-side ones under EP
    const int* g_poff = nullptr; const int* g_num_m_tiles = nullptr; const int* g_tile_expert = nullptr; int g_max_tiles = 0;
    long gcap = 0;      // rows of the grouped GEMM buffers
    bool two_cta = false; bool tensor_core = true; int gemm_dbg = 0;
    int sm_limit = 0;       // > 0: GEMM launches use this many SMs (leaves room for kernels of another stream)
    long long* gemm_cyc = nullptr; int cyc_slot = 0;   // measurement only: cycle counters of the last kGemmCycLaunches GEMM launches
    int pad = 128;      // group padding (rows)
    int x_cap = 0;
    float* bias = nullptr;
    bool has_bias = false;
    // grouped activations (cap rows): input copies, up-projection pre-activation, SiLU output,
    // down-projection output (reference mode: pre-activation) and their gradients
    uint16_t *Xg = nullptr, *P = nullptr, *Hact = nullptr, *Yg = nullptr;
    uint16_t *dYg = nullptr, *dP = nullptr, *dXg = nullptr;
    float* sw_part = nullptr; int sw_ld = 0;
    float *s_j = nullptr, *dlogits = nullptr, *dwr_partial = nullptr;
    // tensor-core router gradient products: bf16 gradient in token order (kw columns) and in grouped
    // order (mw columns), the router term of dX, the split-reduction partials of dWr and their pointers,
    // a bf16 copy of an fp32 router, and the one-expert tile table of the token-order product
    uint16_t *dl_t = nullptr, *dl_g = nullptr, *dXr = nullptr, *wr_bf16 = nullptr;
    int kw = 0, mw = 0, splits = 1;
    float** dwr_part_ptrs = nullptr;
    int* plain_tiles = nullptr; int* plain_num = nullptr; int plain_num_host = -1;
    const void* wr_seen = nullptr;
    bool ep_x_token_order = false;     // the router dW product reads X in token order (one GPU, and the peer transport)
    uint16_t* Xc = nullptr;            // one GPU, training: X kept in token order by the dispatch kernel for that product
    int dl_t_rows = 0;                 // rows of dl_t that may hold values of an earlier, longer call
    int* tok_split_poff = nullptr;
    CUtensorMap* act_maps = nullptr;
    CUtensorMap* w_maps = nullptr;
    const uint16_t** up_ptrs = nullptr; const uint16_t** down_ptrs = nullptr;
    float** gup_ptrs = nullptr; float** gdown_ptrs = nullptr;
    CUtensorMap* g_maps = nullptr;      // [2][local experts] fp32 output maps of the weight gradients
    std::vector<const void*> up_seen, down_seen;
    std::vector<float*> gup_seen, gdown_seen;
    // staging for the host-buffer entry point
    uint16_t *Xs = nullptr, *Ys = nullptr, *dYs = nullptr, *dXs = nullptr;
    // host_io: uploads on in_stream, downloads on out_stream, both under the compute of this and the next step
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    enum HostEvent { kEvXFree = 0, kEvDyFree, kEvXReady, kEvDyReady, kEvYWritten, kEvDxWritten, kEvYOut, kEvDxOut, kNumHostEvents };
    cudaEvent_t host_ev[kNumHostEvents] = {};
    bool host_hooks = false;     // forward / backward record kEvXFree / kEvDyFree once X / dY have been consumed
    // NVFP4 scratch: dequantised bf16 weights and per-expert tensor scales
    uint16_t* q_up = nullptr; uint16_t* q_down = nullptr; float* q_scales = nullptr;
    std::vector<const void*> q_ptrs_host;
    std::vector<const void*> q_key; std::vector<float> q_scales_host;   // what the scratch was expanded from
    bool q_expert_scales = false;   // forward applies q_scales[e] / q_scales[E+e] to the accumulators
    // small-batch NVFP4 route: device table of the packed weights ([4][E] pointers, then [2][E] scales) and what it was built from
    void* q_table = nullptr;
    std::vector<const void*> q_table_key; std::vector<float> q_table_scales;
    // LayerNorm in front of the block, fused into the per-token router (tmt_moe_forward_nvfp4_ln): the parameters of the
    // call in progress, the normalised rows, and the statistics of the stand-alone kernel for larger batches
    const float* ln_gamma = nullptr; const float* ln_beta = nullptr;
    uint16_t* xn = nullptr; float* ln_stats = nullptr;
    // expert parallelism
    tmt_ep_state* ep = nullptr;
    int* ep_world_counts = nullptr;
    long long launches = 0;
    tmt::Profiler prof;
    int last_tokens = 0;
    bool have_forward = false;
    size_t bytes = 0;
    std::vector<void*> allocs;
};

namespace tmt {
void set_error(const char* fmt, ...);
void forward_impl(tmt_moe* h, const void* X, const void* Wr, const void* const* Wup, const void* const* Wdown, void* Y,
                  float beta, int tokens);
void backward_impl(tmt_moe* h, const void* dY, const void* Wr, const void* const* Wup, const void* const* Wdown,
                   float* dWr, float* const* dWup, float* const* dWdown, void* dX, float aux, float zcoef);
void ep_forward(tmt_moe* h, const void* X, const void* Wr, const void* const* Wup, const void* const* Wdown, void* Y,
                float beta, int tokens);
void ep_backward(tmt_moe* h, const void* dY, const void* Wr, const void* const* Wup, const void* const* Wdown,
                 float* dWr, float* const* dWup, float* const* dWdown, void* dX, float aux, float zcoef);
void ep_teardown(tmt_moe* h);
const float* ep_stat(tmt_moe* h);
int ep_waves(tmt_moe* h);           // expert waves of an expert-parallel step (1: one exchange per pass)
void route_only(tmt_moe* h, const uint16_t* X, const void* Wr);
void route_and_dispatch(tmt_moe* h, const uint16_t* X, const void* Wr, uint16_t* grouped);
// tile_count >= 0: only the 128-row tiles [tile_begin, tile_begin + tile_count) of the grouped buffers.
void expert_forward(tmt_moe* h, const void* const* Wup, const void* const* Wdown, bool gate_in_epilogue, int tile_begin = 0,
                    int tile_count = -1);
// which: bit 0 = the products the input gradient needs (dH, dXg), bit 1 = the weight gradients (dWdown, dWup).
// tile_count >= 0 restricts the bit-0 products to the 128-row tiles [tile_begin, tile_begin + tile_count).
void expert_backward(tmt_moe* h, const void* const* Wup, const void* const* Wdown, float* const* dWup, float* const* dWdown,
                     int which = 3, int tile_begin = 0, int tile_count = -1);
// Router backward after the expert products: dlogits, dWr (local contribution) and dX.
// grouped_x / x_is_ep: the token-side grouped copy of X (Xg, or the send buffer under expert parallelism).
// pm: where the rows of dXg live (expert parallel with peer addressing); x_tokens: grouped_x is X in token order.
void router_backward(tmt_moe* h, const void* Wr, const float* sw_part, const uint16_t* grouped_x, bool x_is_ep,
                     const uint16_t* dXg_rows, float* dWr, uint16_t* dX, float aux, float zcoef, const int* counts, long n_norm,
                     PeerMap pm = PeerMap(), bool defer_scatter = false);
// The last step of the backward pass when router_backward was told to leave it out: dX = router term + sum_j dXg[slot_j], on `stream`.
void scatter_rows(tmt_moe* h, const void* Wr, const uint16_t* dXg_rows, uint16_t* dX, cudaStream_t stream, PeerMap pm);
void build_ep_maps(tmt_moe* h, const uint16_t* x_rows, bool token_order);
void prof_mark(tmt_moe* h, int phase);
}  // namespace tmt
