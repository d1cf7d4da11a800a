// Launchers of the routing / permutation kernels (routing.cu, permute.cu).
#pragma once
#include "common.cuh"

namespace tmt {

struct RouteBufs {
    // shapes: T tokens, E experts, K top-k, NB = ceil(T / kTokBlock) router blocks
    float* logits;        // T*E
    float* probs;         // T*E
    float* lse;           // T
    int* idx;             // T*K   selected experts, best first
    float* w;             // T*K   renormalised gate weights
    int* rank;            // T*K   position of the assignment among its block's assignments to the same expert
    int* block_counts;    // NB*E
    float* block_sump;    // NB*E
    float* block_z;       // NB
    int* block_base;      // NB*E  assignments to expert e in earlier blocks
    int* counts;          // E
    int* off;             // E+1   true group starts (moe.cu:413)
    int* poff;            // E+1   group starts padded to kPad rows (moe.cu:416-419)
    int* tile_expert;     // cap/kPad expert of each 128-row tile, -1 past the end
    int* num_m_tiles;     // 1
    float* stat;          // E+1   sum_p[0..E), mean lse^2
    int* slot_of;         // T*K   row of the assignment in the grouped buffers
    float* slotw;         // cap   gate weight of each grouped row (0 on pad rows)
    int* tok_of_slot;     // cap   token of each grouped row (-1 on pad rows)
    int* split_poff;      // kMaxSplits+1 row ranges (multiples of kPad) the router weight-gradient GEMM splits its reduction into
    int* status;
    long long* use_acc;   // E+1  tokens routed to each expert since the last reset, [E] = forward passes counted (train_main.cu:204-209)
};

struct RouteDims {
    int T, D, E, K;
    int cap;              // rows of the grouped buffers
    int max_tiles;        // cap / kPad
    int router_f32;
    int pad;              // group padding in rows: kPad or 2 * kPad
};

// Expert-parallel addressing: a grouped row of expert e lives in the buffer of the rank that owns e.
// base[g] is that rank's buffer (peer memory mapped into this process, base[own rank] the local one);
// this rank's rows for expert e start at row dest_row0[e] there and keep their token-side order.
// base == nullptr: plain local addressing by token-side slot.
struct PeerMap {
    uint16_t* const* base = nullptr;
    const int* dest_row0 = nullptr;
    int experts_per_rank = 1;
    // Only assignments whose expert's index inside its owner rank lies in [wave_lo, wave_hi) move rows (the expert-
    // parallel step sends the experts in waves so that a wave's transfer runs under the previous wave's GEMMs).
    int wave_lo = 0, wave_hi = 1 << 30;
    // Rows of an owner's grouped buffer; a row at or past it is not touched (the step's capacity check failed: with the
    // exchange plan computed on the device the host learns of it from the status word, after the kernels have run).
    int row_limit = 0;
    int* status = nullptr;
    // launch_combine only: the rows of assignments whose expert's index inside its owner lies below fetched_hi were
    // brought over earlier (mode 3) and are read from `fetched` at their token-side slots, not from the owner.
    const uint16_t* fetched = nullptr;
    int fetched_hi = 0;
    // Extra dynamic shared memory per block (unused by the kernel): with a few KB a block no longer fits beside a
    // resident GEMM CTA, so a kernel launched next to a GEMM stays on the SMs that GEMM left free.
    int pad_smem = 0;
};

// scan_splits > 0 and scanned != NULL: a batch of at most kTokBlock tokens also runs the scan (launch_scan) inside the
// router's last kernel; *scanned tells whether it did.
// ln_gamma / ln_beta / xn (all or none): X holds the rows before the LayerNorm in front of the block; the per-token
// kernel normalises each row itself and writes it to xn. Only where router_takes_layernorm(d) says so.
// kernels (may be NULL): receives the number of kernels launched (1 tiled, 2 per-token).
cudaError_t launch_router(const RouteDims& d, const RouteBufs& b, const uint16_t* X, const void* Wr,
                          const float* bias, cudaStream_t s, int scan_splits = 0, bool* scanned = nullptr,
                          const float* ln_gamma = nullptr, const float* ln_beta = nullptr, uint16_t* xn = nullptr,
                          int* kernels = nullptr);
bool router_takes_layernorm(const RouteDims& d);
// splits: number of reduction ranges written to split_poff (1..kMaxSplits).
cudaError_t launch_scan(const RouteDims& d, const RouteBufs& b, int splits, cudaStream_t s);
// Xg[slot] = X[token]; pad rows zeroed; fills slot_of / slotw / tok_of_slot (moe.cu:103-140).
// x_copy (may be NULL): also keeps X in token order (the expert-parallel path reads it in backward).
cudaError_t launch_dispatch(const RouteDims& d, const RouteBufs& b, const uint16_t* X, uint16_t* Xg, cudaStream_t s,
                            PeerMap pm = PeerMap(), uint16_t* x_copy = nullptr);
// mode 0: Y = beta*Y + sum_j Yg[slot_j]               (two-matrix experts, gate applied by the GEMM)
// mode 1: Y = beta*Y + sum_j w_j * silu(Yg[slot_j])   (reference mode, moe.cu:144-158)
// mode 2: Y = beta*Y + sum_j w_j * Yg[slot_j]         (expert parallel: rows come back unscaled)
// mode 3: no Y; only fetches the rows of pm's wave into y_keep (their token-side slots)
// y_keep (may be NULL): stores every fetched row at its token-side slot (kept for the backward pass).
cudaError_t launch_combine(const RouteDims& d, const RouteBufs& b, const uint16_t* Yg, uint16_t* Y, float beta,
                           int mode, cudaStream_t s, PeerMap pm = PeerMap(), uint16_t* y_keep = nullptr);
// mode 0: dYg[slot] = bf16(w * dY[token]), pad rows zero                         (two-matrix experts)
// mode 1: dYg[slot] = silu_bwd(Yg[slot], w * dY[token]); s_j = <dY, silu(Yg[slot])>  (reference, moe.cu:162-197)
// mode 2: as mode 0 and s_j = <dY, Yg[slot]>                                     (expert parallel)
cudaError_t launch_grad_dispatch(const RouteDims& d, const RouteBufs& b, const uint16_t* dY, const uint16_t* Yg,
                                 uint16_t* dYg, float* s_j, int mode, cudaStream_t s, PeerMap pm = PeerMap());
// One expert wave's row moves beside a resident tensor-core CTA (128-thread blocks, no shared memory, `blocks` = one per
// SM). op 0: owner's Xg row = X[token] (src = X); op 1: owner's dYg row = bf16(w * dY[token]) and s_j = <dY[token],
// kept[slot]> (src = dY); op 2: kept[slot] = owner's Yg row. pm names the owners' buffers and the wave; the slots must
// have been fixed by launch_dispatch before.
cudaError_t launch_wave_rows(const RouteDims& d, const RouteBufs& b, int op, const uint16_t* src, uint16_t* kept, float* s_j,
                             int blocks, cudaStream_t s, PeerMap pm);
// moe.cu:200-234. sw_part (may be NULL): per-row partial sums of w * dL/dw from the dH GEMM.
// counts / n_norm: per-expert counts and token count the aux and z terms are normalised by
// (the local ones on one GPU, the totals over all ranks under expert parallelism).
// dl_t / dl_g (may be NULL): the gradient rounded to bf16 in the two layouts the tensor-core router
// products read: dl_t[t][kw] token order (columns >= E zero), dl_g[slot_of[t,0]][mw] grouped order
// (the buffer is zeroed beforehand, so every other grouped row contributes nothing).
cudaError_t launch_router_bwd(const RouteDims& d, const RouteBufs& b, const float* sw_part, int sw_ld, float* s_j,
                              float* dlogits, float aux, float zcoef, const int* counts, long n_norm,
                              uint16_t* dl_t, int kw, uint16_t* dl_g, int mw, cudaStream_t s);
// dWr[e, :] = sum_t bf16(dlogits[t, e]) * X[t, :] with X[t] read from Xg[slot_of[t, 0]] (moe.cu:519-521).
cudaError_t launch_router_dw(const RouteDims& d, const RouteBufs& b, const float* dlogits, const uint16_t* Xg,
                             float* partial, int chunks, float* dWr, cudaStream_t s);
// dX[t] = sum_e bf16(dlogits[t, e]) * Wr[e] + sum_j dXg[slot_j]   (moe.cu:525-529, 238-249)
// With dXr != NULL the router term was already computed by the tensor-core product: dX[t] = dXr[t] + sum_j ...
cudaError_t launch_scatter(const RouteDims& d, const RouteBufs& b, const float* dlogits, const void* Wr,
                           const uint16_t* dXg, const uint16_t* dXr, uint16_t* dX, cudaStream_t s, PeerMap pm = PeerMap());
// out[i] = bf16(in[i])
cudaError_t launch_to_bf16(const float* in, uint16_t* out, long n, cudaStream_t s);
// dWr[e][d] = sum over `parts` partial products part[p][e][d] (row pitch of a part: mw rows x D)
cudaError_t launch_reduce_parts(const float* parts, int nparts, int mw, int E, int D, float* dWr, cudaStream_t s);

constexpr int kRouterDwChunks = 32;
constexpr int kMaxSplits = 64;

}  // namespace tmt
