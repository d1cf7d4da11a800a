// Dispatch / combine and their backward twins: one warp per token row, 16-byte vector
// loads and stores, every row of X / Y / dY / dX read or written exactly once and the K
// grouped rows of a token touched once each. Replaces fill_kernel, gather_slot_kernel (and
// the memset before it), combine_kernel, combine_bwd_kernel, sdot_kernel,
// router_bwd_kernel, to_bf16_kernel, the two skinny router GEMMs and scatter_add_kernel of
// tmt-cuda/src/moe.cu:103-249, 513-531.
#include "kernels.cuh"

namespace tmt {
namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kMaxK = 8;

__device__ __forceinline__ void unpack8(const uint4 v, float (&f)[8]) {
    f[0] = bf_lo(v.x); f[1] = bf_hi(v.x); f[2] = bf_lo(v.y); f[3] = bf_hi(v.y);
    f[4] = bf_lo(v.z); f[5] = bf_hi(v.z); f[6] = bf_lo(v.w); f[7] = bf_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf2(f[0], f[1]), pack_bf2(f[2], f[3]), pack_bf2(f[4], f[5]), pack_bf2(f[6], f[7]));
}

// Address of grouped row `slot` (token-side numbering) of expert e: local, or in the owner's buffer.
__device__ __forceinline__ uint16_t* group_row(const PeerMap& pm, const uint16_t* local, const int* poff, int e, int slot, int D) {
    if (pm.base == nullptr) return const_cast<uint16_t*>(local) + (long)slot * D;
    const int row = pm.dest_row0[e] + slot - poff[e];
    if (pm.row_limit > 0 && (row < 0 || row >= pm.row_limit)) { report(pm.status, kErrCapacity); return nullptr; }
    return pm.base[e / pm.experts_per_rank] + (long)row * D;
}
__device__ __forceinline__ bool in_wave(const PeerMap& pm, int e) {
    const int le = e % pm.experts_per_rank;
    return le >= pm.wave_lo && le < pm.wave_hi;
}
__device__ __forceinline__ uint16_t* shfl_ptr(uint16_t* p, int lane) {
    return reinterpret_cast<uint16_t*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(p), lane));
}

// Blocks [0, tok_blocks) handle tokens; blocks [tok_blocks, tok_blocks + E) zero the pad rows
// of expert (blockIdx - tok_blocks). The offset table (padded group starts and this router
// block's per-expert base) is staged in shared memory.
__global__ void __launch_bounds__(kWarpsPerBlock * 32) dispatch_kernel(const RouteDims d, const RouteBufs b,
                                                                        const uint16_t* __restrict__ X,
                                                                        uint16_t* __restrict__ Xg, int tok_blocks,
                                                                        const PeerMap pm, uint16_t* __restrict__ x_copy) {
    extern __shared__ int table[];     // [E] poff + block_base of the router block these 8 tokens belong to
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvec = d.D >> 3;
    if ((int)blockIdx.x >= tok_blocks) {
        const int e = blockIdx.x - tok_blocks;
        const int r0 = b.poff[e] + b.counts[e], r1 = b.poff[e + 1];
        for (int r = r0 + warp; r < r1; r += kWarpsPerBlock) {
            if (r >= d.cap) { report(b.status, kErrSlotRange); break; }
            for (int v = lane; v < nvec; v += 32) stg16(Xg + (long)r * d.D + v * 8, make_uint4(0, 0, 0, 0));
            if (lane == 0) { b.slotw[r] = 0.0f; b.tok_of_slot[r] = -1; }
        }
        return;
    }
    // kTokBlock is a multiple of the 8 tokens of this block, so one router block covers them all
    const long t0 = (long)blockIdx.x * kWarpsPerBlock;
    const int rb = (int)(t0 / kTokBlock);
    for (int e = threadIdx.x; e < d.E; e += blockDim.x) table[e] = b.poff[e] + b.block_base[(long)rb * d.E + e];
    __syncthreads();
    const long t = t0 + warp;
    if (t >= d.T) return;
    uint16_t* row = nullptr;
    if (lane < d.K) {
        const int e = b.idx[t * d.K + lane];
        if (e < 0 || e >= d.E) report(b.status, kErrSlotRange);
        else {
            const int slot = table[e] + b.rank[t * d.K + lane];
            if (slot < 0 || slot >= d.cap) report(b.status, kErrSlotRange);
            else {
                b.slot_of[t * d.K + lane] = slot;
                b.slotw[slot] = b.w[t * d.K + lane];
                b.tok_of_slot[slot] = (int)t;
                if (in_wave(pm, e)) row = group_row(pm, Xg, b.poff, e, slot, d.D);
            }
        }
    }
    uint16_t* rows[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) rows[j] = shfl_ptr(row, j);
    const uint16_t* src = X + t * d.D;
    for (int v = lane; v < nvec; v += 32) {
        const uint4 x = ldg16(src + v * 8);
#pragma unroll
        for (int j = 0; j < kMaxK; ++j)
            if (j < d.K && rows[j] != nullptr) stg16(rows[j] + v * 8, x);
        if (x_copy) stg16(x_copy + t * d.D + v * 8, x);
    }
}

template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) combine_kernel(const RouteDims d, const RouteBufs b,
                                                                       const uint16_t* __restrict__ Yg,
                                                                       uint16_t* __restrict__ Y, float beta,
                                                                       const PeerMap pm,
                                                                       uint16_t* __restrict__ y_keep) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long t = (long)blockIdx.x * kWarpsPerBlock + warp;
    if (t >= d.T) return;
    int slot = -1; float wj = 0.0f; uint16_t* row = nullptr;
    if (lane < d.K) {
        slot = b.slot_of[t * d.K + lane];
        const int e = b.idx[t * d.K + lane];
        if (slot < 0 || slot >= d.cap) { report(b.status, kErrSlotRange); slot = -1; }
        else if (!in_wave(pm, e)) slot = -1;
        else if (pm.fetched != nullptr && e % pm.experts_per_rank < pm.fetched_hi) {
            wj = b.slotw[slot]; row = const_cast<uint16_t*>(pm.fetched) + (long)slot * d.D;
        }
        else { wj = b.slotw[slot]; row = group_row(pm, Yg, b.poff, e, slot, d.D); if (row == nullptr) slot = -1; }
    }
    int slots[kMaxK]; float ws[kMaxK]; const uint16_t* rows[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) {
        slots[j] = __shfl_sync(0xffffffffu, slot, j); ws[j] = __shfl_sync(0xffffffffu, wj, j); rows[j] = shfl_ptr(row, j);
    }
    const int nvec = d.D >> 3;
    if constexpr (MODE == 3) {
#pragma unroll 2
        for (int v = lane; v < nvec; v += 32) {
#pragma unroll
            for (int j = 0; j < kMaxK; ++j)
                if (j < d.K && slots[j] >= 0) stg16(y_keep + (long)slots[j] * d.D + v * 8, ldg16(rows[j] + v * 8));
        }
        return;
    }
    uint16_t* dst = Y + t * d.D;
#pragma unroll 2
    for (int v = lane; v < nvec; v += 32) {
        float acc[8];
        if (beta != 0.0f) {
            unpack8(ldg16(dst + v * 8), acc);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = beta * acc[i];
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            if (j < d.K && slots[j] >= 0) {
                float y[8];
                const uint4 raw = ldg16(rows[j] + v * 8);
                if (y_keep && rows[j] != y_keep + (long)slots[j] * d.D) stg16(y_keep + (long)slots[j] * d.D + v * 8, raw);
                unpack8(raw, y);
                if constexpr (MODE == 1) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += ws[j] * silu_f(y[i]);
                } else if constexpr (MODE == 2) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += ws[j] * y[i];
                } else {
#pragma unroll
                    for (int i = 0; i < 8; ++i) acc[i] += y[i];
                }
            }
        }
        stg16(dst + v * 8, pack8(acc));
    }
}

template <int MODE>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) grad_dispatch_kernel(const RouteDims d, const RouteBufs b,
                                                                             const uint16_t* __restrict__ dY,
                                                                             const uint16_t* __restrict__ Yg,
                                                                             uint16_t* __restrict__ dYg,
                                                                             float* __restrict__ s_j,
                                                                             int tok_blocks, const PeerMap pm) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nvec = d.D >> 3;
    if ((int)blockIdx.x >= tok_blocks) {
        const int e = blockIdx.x - tok_blocks;
        const int r0 = b.poff[e] + b.counts[e], r1 = b.poff[e + 1];
        for (int r = r0 + warp; r < r1 && r < d.cap; r += kWarpsPerBlock)
            for (int v = lane; v < nvec; v += 32) stg16(dYg + (long)r * d.D + v * 8, make_uint4(0, 0, 0, 0));
        return;
    }
    const long t = (long)blockIdx.x * kWarpsPerBlock + warp;
    if (t >= d.T) return;
    int slot = -1; float wj = 0.0f; uint16_t* row = nullptr;
    if (lane < d.K) {
        slot = b.slot_of[t * d.K + lane];
        const int e = b.idx[t * d.K + lane];
        if (slot < 0 || slot >= d.cap) { report(b.status, kErrSlotRange); slot = -1; }
        else if (!in_wave(pm, e)) slot = -1;
        else { wj = b.slotw[slot]; row = group_row(pm, dYg, b.poff, e, slot, d.D); if (row == nullptr) slot = -1; }
    }
    int slots[kMaxK]; float ws[kMaxK]; float sdot[kMaxK]; uint16_t* rows[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) {
        slots[j] = __shfl_sync(0xffffffffu, slot, j); ws[j] = __shfl_sync(0xffffffffu, wj, j); sdot[j] = 0.0f;
        rows[j] = shfl_ptr(row, j);
    }
    const uint16_t* src = dY + t * d.D;
#pragma unroll 2
    for (int v = lane; v < nvec; v += 32) {
        float g[8];
        unpack8(ldg16(src + v * 8), g);
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            if (j < d.K && slots[j] >= 0) {
                float o[8];
                if constexpr (MODE == 1) {
                    float pre[8];
                    unpack8(ldg16(Yg + (long)slots[j] * d.D + v * 8), pre);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float sg = sigmoid_f(pre[i]);
                        sdot[j] += g[i] * (pre[i] * sg);
                        o[i] = (ws[j] * g[i]) * sg * (1.0f + pre[i] * (1.0f - sg));     // silu_bwd, common.h:21-24
                    }
                } else {
                    if constexpr (MODE == 2) {
                        float y[8];
                        unpack8(ldg16(Yg + (long)slots[j] * d.D + v * 8), y);
#pragma unroll
                        for (int i = 0; i < 8; ++i) sdot[j] += g[i] * y[i];
                    }
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = ws[j] * g[i];
                }
                stg16(rows[j] + v * 8, pack8(o));
            }
        }
    }
    if constexpr (MODE != 0) {
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            if (j < d.K) {
                float s = sdot[j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                if (lane == 0 && slots[j] >= 0) s_j[t * d.K + j] = s;
            }
        }
    }
}

// The row moves of one expert wave (expert-parallel step), shaped to run BESIDE a resident tensor-core CTA of the
// CTA-pair kernel. Such a CTA leaves 1.9 KB of the SM's shared memory, i.e. room for ONE more block (every block
// reserves 1 KB) that uses none of its own, and, with its registers capped at 128, 4096 registers in each of the four
// scheduler partitions: two warps of 64. So: one block per SM, 256 threads, at most 64 registers, each warp walking
// the tokens with a grid stride and keeping a whole 4 KB row in flight. The slots were fixed by the first wave's
// dispatch (slot_of, slotw), so only rows move here. A warp reads the bookkeeping of 32 / K tokens at once (one
// assignment per lane), so the dependent index loads are paid once per handful of rows, not once per row.
//   OP 0: owner's Xg[row]  = X[token]                                         (dispatch_kernel's copy)
//   OP 1: owner's dYg[row] = bf16(w * dY[token]); s_j = <dY[token], kept[slot]>  (grad_dispatch_kernel, mode 2, same sum order)
//   OP 2: kept[slot]       = owner's Yg[row]                                  (combine_kernel, mode 3)
template <int OP>
__global__ void __launch_bounds__(256, 4) wave_rows_kernel(const RouteDims d, const RouteBufs b,
                                                                                          const uint16_t* __restrict__ src,
                                                                                          uint16_t* __restrict__ kept,
                                                                                          float* __restrict__ s_j, const PeerMap pm) {
    const int lane = threadIdx.x & 31;
    const int nvec = d.D >> 3;
    const int per = 32 / d.K;                                   // tokens a warp looks at together
    const long nchunk = (d.T + per - 1) / per;
    const long nwarp = (long)gridDim.x * (blockDim.x >> 5);
    const int tl = lane / d.K;                                  // this lane's token within the chunk; its assignment is lane % K
    for (long c = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); c < nchunk; c += nwarp) {
        const long t = c * per + tl;
        int slot = -1; float wj = 0.0f; uint16_t* row = nullptr;
        if (tl < per && t < d.T) {
            const long a = c * per * d.K + lane;                // = t * K + lane % K
            const int e = b.idx[a];
            if (e >= 0 && e < d.E && in_wave(pm, e)) {
                slot = b.slot_of[a];
                if (slot < 0 || slot >= d.cap) { report(b.status, kErrSlotRange); slot = -1; }
                else {
                    wj = b.slotw[slot];
                    row = group_row(pm, nullptr, b.poff, e, slot, d.D);
                    if (row == nullptr) slot = -1;
                }
            }
        }
        unsigned todo = __ballot_sync(0xffffffffu, slot >= 0);
        while (todo) {
            const int j = __ffs(todo) - 1;
            todo &= todo - 1;
            const int sl = __shfl_sync(0xffffffffu, slot, j);
            uint16_t* r = shfl_ptr(row, j);
            const long tj = c * per + j / d.K;
            if constexpr (OP == 0) {
                const uint16_t* x = src + tj * d.D;
#pragma unroll 8
                for (int v = lane; v < nvec; v += 32) stg16(r + v * 8, ldg16_stream(x + v * 8));
            } else if constexpr (OP == 2) {
                uint16_t* k = kept + (long)sl * d.D;
#pragma unroll 8
                for (int v = lane; v < nvec; v += 32) stg16(k + v * 8, ldg16_stream(r + v * 8));
            } else {
                const float w = __shfl_sync(0xffffffffu, wj, j);
                const uint16_t* g_row = src + tj * d.D;
                const uint16_t* y_row = kept + (long)sl * d.D;
                float sdot = 0.0f;
#pragma unroll 4
                for (int v = lane; v < nvec; v += 32) {
                    float g[8], y[8], o[8];
                    unpack8(ldg16_stream(g_row + v * 8), g);
                    unpack8(ldg16_stream(y_row + v * 8), y);
#pragma unroll
                    for (int i = 0; i < 8; ++i) sdot += g[i] * y[i];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = w * g[i];
                    stg16(r + v * 8, pack8(o));
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xffffffffu, sdot, o);
                if (lane == 0) s_j[c * per * d.K + j] = sdot;
            }
        }
    }
}

// Router backward through softmax, top-k and renormalisation plus the aux and z terms
// (moe.cu:200-234, same formulas). Eight lanes per token, lane s owns experts s, s+8, ...; only the K
// selected experts carry a non-zero renormalisation gradient, so the softmax correction
// sum_e g_e p_e has K terms and needs no pass over E.
__global__ void __launch_bounds__(256) router_bwd_kernel(const RouteDims d, const RouteBufs b,
                                                         const float* __restrict__ sw_part, int sw_ld,
                                                         float* __restrict__ s_j, float* __restrict__ dlogits, float aux,
                                                         float zcoef, const int* __restrict__ counts, long n_norm,
                                                         uint16_t* __restrict__ dl_t, int kw, uint16_t* __restrict__ dl_g,
                                                         int mw) {
    const int lane = threadIdx.x & 31;
    const int s = lane & 7;
    const unsigned full = 0xffffffffu;
    const long r = ((long)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const bool valid = r < d.T;
    const long rr = valid ? r : 0;
    const int E = d.E, K = d.K;
    const float* probs = b.probs + rr * E;
    const float nk = (float)(n_norm * K);
    const float nn = (float)n_norm;
    // lane j of the group owns selected expert j
    int my_e = -1; float my_p = 0.0f, my_s = 0.0f;
    if (s < K) {
        my_e = b.idx[rr * K + s];
        my_p = probs[my_e];
        if (sw_part) {
            // dH-GEMM partials hold w * dL/dw, one per kEpiCols columns, added in column order
            const int slot = b.slot_of[rr * K + s];
            float acc = 0.0f;
            for (int q = 0; q < sw_ld; ++q) acc += sw_part[(long)slot * sw_ld + q];
            const float wj = b.slotw[slot];
            my_s = wj > 0.0f ? acc / wj : 0.0f;
            if (valid) s_j[rr * K + s] = my_s;
        } else {
            my_s = s_j[rr * K + s];
        }
    }
    float Z = 0.0f, sp = 0.0f;
    int sel_e[8]; float sel_p[8], sel_s[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        sel_e[j] = __shfl_sync(full, my_e, (lane & 24) + j);
        sel_p[j] = __shfl_sync(full, my_p, (lane & 24) + j);
        sel_s[j] = __shfl_sync(full, my_s, (lane & 24) + j);
        if (j < K) { Z += sel_p[j]; sp += sel_s[j] * sel_p[j]; }
    }
    const float Z2 = Z * Z + 1e-12f;
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
        if (j < K) { sel_s[j] = (sel_s[j] * Z - sp) / Z2; acc += sel_s[j] * sel_p[j]; }      // sel_s now holds g_sel
    float expected = 0.0f;
    for (int e = s; e < E; e += 8) expected += probs[e] * counts[e] / nk;
    expected += __shfl_xor_sync(full, expected, 1);
    expected += __shfl_xor_sync(full, expected, 2);
    expected += __shfl_xor_sync(full, expected, 4);
    const float lse = b.lse[rr];
    const int slot0 = b.slot_of[rr * K];
    const bool slot_ok = slot0 >= 0 && slot0 < d.cap;
    for (int e = s; e < max(E, kw); e += 8) {
        float g = 0.0f;
        if (e < E) {
            const float p = probs[e];
            float gs = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) if (j < K && sel_e[j] == e) gs = sel_s[j];
            g = p * (gs - acc) + aux * E / nn * p * (counts[e] / nk - expected) + zcoef * 2.f / nn * lse * p;
            if (valid) {
                dlogits[rr * E + e] = g;
                if (dl_g && slot_ok) dl_g[(long)slot0 * mw + e] = f2bf(g);
            }
        }
        if (valid && dl_t && e < kw) dl_t[rr * kw + e] = e < E ? f2bf(g) : (uint16_t)0;
    }
}

__global__ void to_bf16_kernel(const float* __restrict__ in, uint16_t* __restrict__ out, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = f2bf(in[i]);
}

__global__ void reduce_parts_kernel(const float* __restrict__ parts, int nparts, int mw, int E, int D, float* __restrict__ dWr) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long)E * D) return;
    float s = 0.0f;
    for (int p = 0; p < nparts; ++p) s += parts[(long)p * mw * D + i];     // rows e < E of every part, same [e][d] pitch
    dWr[i] = s;
}

// Partial router weight gradient of one token chunk: block = 256 threads x 2 columns.
template <int EC>
__global__ void __launch_bounds__(256) router_dw_kernel(const RouteDims d, const RouteBufs b,
                                                         const float* __restrict__ dlogits,
                                                         const uint16_t* __restrict__ Xg, float* __restrict__ partial,
                                                         int chunks) {
    __shared__ float dl[32 * 64];      // 32 tokens x EC (<= 64) rounded gradients
    __shared__ int srow[32];
    const int d0 = (blockIdx.x * 256 + threadIdx.x) * 2;
    const int chunk = blockIdx.y;
    const long per = (d.T + chunks - 1) / chunks;
    const long tbeg = chunk * per, tend = min((long)d.T, tbeg + per);
    const bool dok = d0 < d.D;
    for (int ec0 = 0; ec0 < d.E; ec0 += EC) {
        float a0[EC], a1[EC];
#pragma unroll
        for (int e = 0; e < EC; ++e) { a0[e] = 0.0f; a1[e] = 0.0f; }
        for (long tb = tbeg; tb < tend; tb += 32) {
            __syncthreads();
            for (int i = threadIdx.x; i < 32 * EC; i += 256) {
                const int tt = i / EC, e = i - tt * EC;
                const long t = tb + tt;
                dl[tt * EC + e] = (t < tend && ec0 + e < d.E) ? round_bf(dlogits[t * d.E + ec0 + e]) : 0.0f;
            }
            if (threadIdx.x < 32) {
                const long t = tb + threadIdx.x;
                srow[threadIdx.x] = t < tend ? b.slot_of[t * d.K] : -1;
            }
            __syncthreads();
            if (dok) {
                for (int tt = 0; tt < 32; ++tt) {
                    const int row = srow[tt];
                    if (row < 0) break;
                    const uint32_t xv = __ldg(reinterpret_cast<const uint32_t*>(Xg + (long)row * d.D + d0));
                    const float x0 = bf_lo(xv), x1 = bf_hi(xv);
#pragma unroll
                    for (int e = 0; e < EC; ++e) {
                        const float gq = dl[tt * EC + e];
                        a0[e] += gq * x0; a1[e] += gq * x1;
                    }
                }
            }
        }
        if (dok) {
#pragma unroll
            for (int e = 0; e < EC; ++e)
                if (ec0 + e < d.E) {
                    float* dst = partial + ((long)chunk * d.E + ec0 + e) * d.D + d0;
                    dst[0] = a0[e]; dst[1] = a1[e];
                }
        }
    }
}

__global__ void router_dw_reduce_kernel(const float* __restrict__ partial, float* __restrict__ dWr, long n, int chunks) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.0f;
    for (int c = 0; c < chunks; ++c) s += partial[(long)c * n + i];
    dWr[i] = s;
}

template <bool WF32>
__global__ void __launch_bounds__(kWarpsPerBlock * 32) scatter_kernel(const RouteDims d, const RouteBufs b,
                                                                       const float* __restrict__ dlogits,
                                                                       const void* __restrict__ Wr,
                                                                       const uint16_t* __restrict__ dXg,
                                                                       const uint16_t* __restrict__ dXr,
                                                                       uint16_t* __restrict__ dX, const PeerMap pm) {
    extern __shared__ float dls[];     // [warps][E]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long t = (long)blockIdx.x * kWarpsPerBlock + warp;
    if (t >= d.T) return;
    float* mine = dls + warp * d.E;
    const bool router = d.E > 1 && dXr == nullptr;     // dense shortcut has no router gradient (moe.cu:488-494)
    if (router)
        for (int e = lane; e < d.E; e += 32) mine[e] = round_bf(dlogits[t * d.E + e]);
    uint16_t* row = nullptr;
    if (lane < d.K) {
        const int slot = b.slot_of[t * d.K + lane];
        if (slot < 0 || slot >= d.cap) report(b.status, kErrSlotRange);
        else row = group_row(pm, dXg, b.poff, b.idx[t * d.K + lane], slot, d.D);
    }
    const uint16_t* rows[kMaxK];
#pragma unroll
    for (int j = 0; j < kMaxK; ++j) rows[j] = shfl_ptr(row, j);
    __syncwarp();
    const int nvec = d.D >> 3;
    for (int v = lane; v < nvec; v += 32) {
        float acc[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
        if (dXr != nullptr && d.E > 1) unpack8(ldg16(dXr + t * d.D + v * 8), acc);
        if (router) {
            for (int e = 0; e < d.E; ++e) {
                const float gq = mine[e];
                float wv[8];
                if constexpr (WF32) {
                    const float4* wp = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(Wr) + (long)e * d.D + v * 8);
                    const float4 w0 = __ldg(wp), w1 = __ldg(wp + 1);
                    wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w; wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
                } else {
                    unpack8(ldg16(reinterpret_cast<const uint16_t*>(Wr) + (long)e * d.D + v * 8), wv);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += gq * wv[i];
            }
        }
#pragma unroll
        for (int j = 0; j < kMaxK; ++j) {
            if (j < d.K && rows[j] != nullptr) {
                float x[8];
                unpack8(ldg16(rows[j] + v * 8), x);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += x[i];
            }
        }
        stg16(dX + t * d.D + v * 8, pack8(acc));
    }
}

inline int tok_blocks_of(int T) { return (T + kWarpsPerBlock - 1) / kWarpsPerBlock; }

}  // namespace

cudaError_t launch_dispatch(const RouteDims& d, const RouteBufs& b, const uint16_t* X, uint16_t* Xg, cudaStream_t s,
                            PeerMap pm, uint16_t* x_copy) {
    const int tb = tok_blocks_of(d.T);
    // with peer addressing the pad rows belong to the owners, who zero their own
    dispatch_kernel<<<tb + (pm.base ? 0 : d.E), kWarpsPerBlock * 32, d.E * sizeof(int) + pm.pad_smem, s>>>(d, b, X, Xg, tb, pm, x_copy);
    return cudaGetLastError();
}

cudaError_t launch_combine(const RouteDims& d, const RouteBufs& b, const uint16_t* Yg, uint16_t* Y, float beta,
                           int mode, cudaStream_t s, PeerMap pm, uint16_t* y_keep) {
    const dim3 grid(tok_blocks_of(d.T)), block(kWarpsPerBlock * 32);
    if (mode == 3) combine_kernel<3><<<grid, block, pm.pad_smem, s>>>(d, b, Yg, Y, beta, pm, y_keep);
    else if (mode == 1) combine_kernel<1><<<grid, block, pm.pad_smem, s>>>(d, b, Yg, Y, beta, pm, y_keep);
    else if (mode == 2) combine_kernel<2><<<grid, block, pm.pad_smem, s>>>(d, b, Yg, Y, beta, pm, y_keep);
    else combine_kernel<0><<<grid, block, pm.pad_smem, s>>>(d, b, Yg, Y, beta, pm, y_keep);
    return cudaGetLastError();
}

cudaError_t launch_grad_dispatch(const RouteDims& d, const RouteBufs& b, const uint16_t* dY, const uint16_t* Yg,
                                 uint16_t* dYg, float* s_j, int mode, cudaStream_t s, PeerMap pm) {
    const int tb = tok_blocks_of(d.T);
    const dim3 grid(tb + (pm.base ? 0 : d.E)), block(kWarpsPerBlock * 32);
    if (mode == 1) grad_dispatch_kernel<1><<<grid, block, pm.pad_smem, s>>>(d, b, dY, Yg, dYg, s_j, tb, pm);
    else if (mode == 2) grad_dispatch_kernel<2><<<grid, block, pm.pad_smem, s>>>(d, b, dY, Yg, dYg, s_j, tb, pm);
    else grad_dispatch_kernel<0><<<grid, block, pm.pad_smem, s>>>(d, b, dY, Yg, dYg, s_j, tb, pm);
    return cudaGetLastError();
}

cudaError_t launch_router_bwd(const RouteDims& d, const RouteBufs& b, const float* sw_part, int sw_ld, float* s_j,
                              float* dlogits, float aux, float zcoef, const int* counts, long n_norm,
                              uint16_t* dl_t, int kw, uint16_t* dl_g, int mw, cudaStream_t s) {
    router_bwd_kernel<<<(d.T + 31) / 32, 256, 0, s>>>(d, b, sw_part, sw_ld, s_j, dlogits, aux, zcoef, counts, n_norm,
                                                      dl_t, kw, dl_g, mw);
    return cudaGetLastError();
}

cudaError_t launch_wave_rows(const RouteDims& d, const RouteBufs& b, int op, const uint16_t* src, uint16_t* kept, float* s_j,
                             int blocks, cudaStream_t s, PeerMap pm) {
    if (d.K < 1 || d.K > kMaxK || (d.D & 7) != 0 || pm.base == nullptr || blocks < 1) return cudaErrorInvalidValue;
    switch (op) {
        case 0: wave_rows_kernel<0><<<blocks, 256, 0, s>>>(d, b, src, kept, s_j, pm); break;
        case 1: wave_rows_kernel<1><<<blocks, 256, 0, s>>>(d, b, src, kept, s_j, pm); break;
        case 2: wave_rows_kernel<2><<<blocks, 256, 0, s>>>(d, b, src, kept, s_j, pm); break;
        default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

cudaError_t launch_to_bf16(const float* in, uint16_t* out, long n, cudaStream_t s) {
    to_bf16_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(in, out, n);
    return cudaGetLastError();
}

cudaError_t launch_reduce_parts(const float* parts, int nparts, int mw, int E, int D, float* dWr, cudaStream_t s) {
    const long n = (long)E * D;
    reduce_parts_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(parts, nparts, mw, E, D, dWr);
    return cudaGetLastError();
}

cudaError_t launch_router_dw(const RouteDims& d, const RouteBufs& b, const float* dlogits, const uint16_t* Xg,
                             float* partial, int chunks, float* dWr, cudaStream_t s) {
    dim3 grid((d.D / 2 + 255) / 256, chunks);
    if (d.E <= 8) router_dw_kernel<8><<<grid, 256, 0, s>>>(d, b, dlogits, Xg, partial, chunks);
    else if (d.E <= 16) router_dw_kernel<16><<<grid, 256, 0, s>>>(d, b, dlogits, Xg, partial, chunks);
    else if (d.E <= 32) router_dw_kernel<32><<<grid, 256, 0, s>>>(d, b, dlogits, Xg, partial, chunks);
    else router_dw_kernel<64><<<grid, 256, 0, s>>>(d, b, dlogits, Xg, partial, chunks);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    const long n = (long)d.E * d.D;
    router_dw_reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, dWr, n, chunks);
    return cudaGetLastError();
}

cudaError_t launch_scatter(const RouteDims& d, const RouteBufs& b, const float* dlogits, const void* Wr,
                           const uint16_t* dXg, const uint16_t* dXr, uint16_t* dX, cudaStream_t s, PeerMap pm) {
    // the staged router gradient is only read when the kernel computes the router term itself; without it a block
    // needs no shared memory and fits beside a resident GEMM CTA
    const size_t smem = (dXr != nullptr ? 0 : (size_t)kWarpsPerBlock * d.E * sizeof(float)) + pm.pad_smem;
    if (d.router_f32) scatter_kernel<true><<<tok_blocks_of(d.T), kWarpsPerBlock * 32, smem, s>>>(d, b, dlogits, Wr, dXg, dXr, dX, pm);
    else scatter_kernel<false><<<tok_blocks_of(d.T), kWarpsPerBlock * 32, smem, s>>>(d, b, dlogits, Wr, dXg, dXr, dX, pm);
    return cudaGetLastError();
}

}  // namespace tmt
