// Fused router (logits, softmax, top-k, gate weights, per-block counts and statistics
// partials) and the single-block scan that turns the per-block counts into the offset
// tables. Replaces router_topk_kernel, count_kernel, the host prefix sum, aux_sum_kernel
// and zloss_kernel of tmt-cuda/src/moe.cu:10-68, 97-101, 411-421, 258-278: no host round
// trip, no global atomics, deterministic.
//
// Not compiled with fast-math: the logits must be bit-identical to the CPU statement.
// Stated order of a router dot product: element d belongs to chain (d/8)%8; a chain is a
// sequential fp32 FMA in increasing d; chains are added ((c0+c1)+(c2+c3))+((c4+c5)+(c6+c7)).
// Here a chain is one lane of an 8-lane group reading 16-byte vectors, and the tree is
// the xor-butterfly 1, 2, 4 (fp32 addition is commutative, so every lane ends equal).
// The products themselves run as a register-tiled fp32 FMA GEMM on the CUDA cores (tensor
// cores would fix their own accumulation order, which the CPU statement could not mirror).
#include <cstdlib>

#include "kernels.cuh"
#include "launch_pdl.cuh"

namespace tmt {
namespace {

constexpr int kDC = 128;            // d elements staged per pipeline step (16 vectors of 8)
constexpr int kTT = 4;              // tokens per thread

// Compile-time loop: f(integral_constant<int, 0>) ... f(integral_constant<int, N-1>)
template <int V> struct IntC { static constexpr int value = V; };
template <int N, int I = 0, class F>
__device__ __forceinline__ void static_for(F& f) {
    if constexpr (I < N) { f(IntC<I>{}); static_for<N, I + 1>(f); }
}

struct RouterArgs {
    const uint16_t* X; const void* Wr; const float* bias;
    int T, D, E, K;
    RouteBufs b;
    // fused LayerNorm in front of the router (per-token kernel only): X holds the rows BEFORE the normalisation, the
    // normalised rows are written to xn (what the expert products read). NULL: X is the block's input as it is.
    const float* ln_gamma; const float* ln_beta; uint16_t* xn;
};

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = valid ? 16 : 0;      // src-size 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// 16-byte shared-memory load from a 32-bit shared address plus a compile-time offset (keeps the
// address arithmetic of the unrolled expert loop in the instruction's immediate field)
template <int OFF>
__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4 + %5];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr), "n"(OFF));
    return v;
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Second half of the router, on the logits of one block of kTokBlock tokens in shared memory (lg, [kTokBlock][E]):
// softmax, top-k, gate weights, then the block's stable ranks, counts and statistics partials.
// keep_cnt / keep_sp / keep_z (shared memory, may be NULL): the block's counts, probability sums and z partial stay on
// chip as well, for a caller that goes on to the scan itself.
template <int NTHR>
__device__ __forceinline__ void route_block_finish(const RouterArgs& a, float* lg, int* sidx, float* zs, long tok0,
                                                   int* keep_cnt = nullptr, float* keep_sp = nullptr, float* keep_z = nullptr) {
    const int E = a.E, K = a.K;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = lane & 7, g = lane >> 3;
    const unsigned full = 0xffffffffu;
    // ---- softmax, top-k (on logits, lowest index wins ties), gate weights: 8 lanes per token ----
    for (int tb = warp * 4 + g; tb < kTokBlock; tb += (NTHR / 32) * 4) {
        const long t = tok0 + tb;
        const bool valid = t < a.T;
        float* L = lg + tb * E;
        float mx = -INFINITY;
        for (int e = s; e < E; e += 8) mx = fmaxf(mx, L[e]);
        mx = fmaxf(mx, __shfl_xor_sync(full, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(full, mx, 2));
        mx = fmaxf(mx, __shfl_xor_sync(full, mx, 4));
        float se = 0.0f;
        for (int e = s; e < E; e += 8) se += expf(L[e] - mx);
        se += __shfl_xor_sync(full, se, 1);
        se += __shfl_xor_sync(full, se, 2);
        se += __shfl_xor_sync(full, se, 4);
        unsigned used = 0;
        for (int j = 0; j < K; ++j) {
            float bv = -INFINITY; int bi = 0x7fffffff;
            for (int e = s, i = 0; e < E; e += 8, ++i)
                if (!(used >> i & 1) && (bi == 0x7fffffff || L[e] > bv)) { bv = L[e]; bi = e; }
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) {
                const float ov = __shfl_xor_sync(full, bv, o);
                const int oi = __shfl_xor_sync(full, bi, o);
                const bool take = (oi != 0x7fffffff) && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi));
                if (take) { bv = ov; bi = oi; }
            }
            if ((bi & 7) == s) used |= 1u << (bi >> 3);
            if (s == 0) sidx[tb * K + j] = valid ? bi : -1;
        }
        for (int e = s; e < E; e += 8) {
            const float l = L[e];
            const float pr = expf(l - mx) / se;
            if (valid) { a.b.logits[t * E + e] = l; a.b.probs[t * E + e] = pr; }
            L[e] = valid ? pr : 0.0f;
        }
        __syncwarp();
        if (s == 0) {
            const float lse = mx + logf(se);
            zs[tb] = valid ? lse * lse : 0.0f;
            if (valid) {
                a.b.lse[t] = lse;
                float z = 0.0f;
                for (int j = 0; j < K; ++j) z += L[sidx[tb * K + j]];
                for (int j = 0; j < K; ++j) {
                    a.b.idx[t * K + j] = sidx[tb * K + j];
                    a.b.w[t * K + j] = L[sidx[tb * K + j]] / z;
                }
            }
        }
    }
    __syncthreads();
    // ---- block level: stable ranks, counts, statistics partials ----
    // rank of an assignment = number of earlier assignments of the block to the same expert: a warp walks the
    // block's assignments 32 at a time for one expert (invalid tokens carry -1 and never match)
    const int n_asg = kTokBlock * K;            // a multiple of 32
    for (int e = warp; e < E; e += NTHR / 32) {
        int running = 0;
        for (int c0 = 0; c0 < n_asg; c0 += 32) {
            const bool hit = sidx[c0 + lane] == e;
            const unsigned m = __ballot_sync(full, hit);
            if (hit) a.b.rank[(long)blockIdx.x * n_asg + c0 + lane] = running + __popc(m & ((1u << lane) - 1));
            running += __popc(m);
        }
        if (lane == 0) { a.b.block_counts[(long)blockIdx.x * E + e] = running; if (keep_cnt) keep_cnt[e] = running; }
    }
    for (int e = threadIdx.x; e < E; e += NTHR) {
        float sp = 0.0f;
        for (int tb = 0; tb < kTokBlock; ++tb) sp += lg[tb * E + e];
        a.b.block_sump[(long)blockIdx.x * E + e] = sp;
        if (keep_sp) keep_sp[e] = sp;
    }
    if (threadIdx.x == NTHR - 1) {
        float z = 0.0f;
        for (int tb = 0; tb < kTokBlock; ++tb) z += zs[tb];
        a.b.block_z[blockIdx.x] = z;
        if (keep_z) *keep_z = z;
    }
}

// Block = 64 tokens x (TE * ESLABS) experts per expert pass; 4 * ESLABS warps. Warp = one slab of 16
// tokens x TE experts; lane = (chain s = lane & 7, token group g = lane >> 3); a thread keeps
// kTT x TE accumulators of its chain, as kTT x TE/2 PAIRS of neighbouring experts: the products run on the packed
// fp32 FMA of sm_100 (fma.rn.f32x2: two chains per issued instruction; each half is one round-to-nearest FMA of its
// own chain, so the logits keep the stated bits). X (bf16) is staged in shared memory by cp.async; the router rows
// travel through registers (loaded one chunk ahead) and are stored as fp32, two experts interleaved element by element
// in four 16-byte planes [plane][pair][vector], so that one 16-byte load returns {w_e[d], w_e+1[d], w_e[d+1], w_e+1[d+1]}
// and the 8 chains of a group read 128 contiguous bytes. Both double buffered, kDC columns at a time.
template <int TE, int ESLABS, bool WF32>
__global__ void __launch_bounds__(128 * ESLABS) router_kernel(const RouterArgs a) {
    static_assert(TE % 2 == 0, "experts are processed in pairs");
    constexpr int EP = TE * ESLABS;                 // experts per pass
    constexpr int NP = EP / 2, TP = TE / 2;         // expert pairs per pass / per thread
    constexpr int NTHR = 128 * ESLABS;
    constexpr int XS_BYTES = kTokBlock * kDC * 2;
    constexpr int WS_BYTES = EP * kDC * 4;
    constexpr int WITEMS = (EP * (kDC / 8) + NTHR - 1) / NTHR;      // (expert row, 8-column vector) items a thread stages per chunk
    extern __shared__ __align__(16) uint8_t smem[];
    uint8_t* stage[2] = {smem, smem + XS_BYTES + WS_BYTES};
    float* lg = reinterpret_cast<float*>(smem + 2 * (XS_BYTES + WS_BYTES));     // [kTokBlock][E]
    __shared__ int sidx[kTokBlock * 8];
    __shared__ float zs[kTokBlock];
    const int E = a.E, D = a.D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = lane & 7, g = lane >> 3;
    const int tslab = warp & 3, eslab = warp >> 2;
    const int nvec = D >> 3;
    const int nchunks = (D + kDC - 1) / kDC;
    const long tok0 = (long)blockIdx.x * kTokBlock;
    const unsigned full = 0xffffffffu;

    for (int ep0 = 0; ep0 < E; ep0 += EP) {
        // X: 64 rows x 16 vectors of 16 bytes by cp.async. A thread copies the same vector column of every (NTHR / 16)-th
        // row, so its source and destination advance by constants (no per-piece index arithmetic).
        auto load_x = [&](int k, uint8_t* buf) {
            constexpr int kRowStep = NTHR / 16, kPieces = kTokBlock / kRowStep;
            const int xv = threadIdx.x & 15, xr = threadIdx.x >> 4;
            const bool col_ok = k * (kDC / 8) + xv < nvec;
            const uint16_t* src = a.X + (tok0 + xr) * D + (long)(k * (kDC / 8) + xv) * 8;
            uint8_t* dst = buf + (xr * (kDC / 8) + xv) * 16;
#pragma unroll
            for (int j = 0; j < kPieces; ++j) {
                const bool ok = col_ok && tok0 + xr + j * kRowStep < a.T;
                cp_async16(dst + j * kRowStep * (kDC / 8) * 16, ok ? src + (long)j * kRowStep * D : a.X, ok);
            }
            cp_async_commit();
        };
        // router rows: item = (expert row of the pass, vector of 8 columns) -> 8 fp32 values in registers
        float wreg[WITEMS][8];
        auto load_w = [&](int k) {
            const int v0 = k * (kDC / 8);
#pragma unroll
            for (int it = 0; it < WITEMS; ++it) {
                const int q = threadIdx.x + it * NTHR;
                const int row = q >> 4, v = q & 15;
                const bool ok = q < EP * (kDC / 8) && ep0 + row < E && v0 + v < nvec;
                if (ok) {
                    if constexpr (WF32) {
                        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.Wr) + (long)(ep0 + row) * D + (long)(v0 + v) * 8);
                        const float4 w0 = __ldg(src), w1 = __ldg(src + 1);
                        wreg[it][0] = w0.x; wreg[it][1] = w0.y; wreg[it][2] = w0.z; wreg[it][3] = w0.w;
                        wreg[it][4] = w1.x; wreg[it][5] = w1.y; wreg[it][6] = w1.z; wreg[it][7] = w1.w;
                    } else {
                        const uint4 w = ldg16(reinterpret_cast<const uint16_t*>(a.Wr) + (long)(ep0 + row) * D + (long)(v0 + v) * 8);
                        wreg[it][0] = bf_lo(w.x); wreg[it][1] = bf_hi(w.x); wreg[it][2] = bf_lo(w.y); wreg[it][3] = bf_hi(w.y);
                        wreg[it][4] = bf_lo(w.z); wreg[it][5] = bf_hi(w.z); wreg[it][6] = bf_lo(w.w); wreg[it][7] = bf_hi(w.w);
                    }
                } else {
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8) wreg[it][q8] = 0.0f;
                }
            }
        };
        // element (row, column 8v + q) -> plane q / 2, pair row / 2, vector v, float (q % 2) * 2 + row % 2
        auto store_w = [&](uint8_t* buf) {
            float* wsm = reinterpret_cast<float*>(buf + XS_BYTES);
#pragma unroll
            for (int it = 0; it < WITEMS; ++it) {
                const int q = threadIdx.x + it * NTHR;
                if (q < EP * (kDC / 8)) {
                    const int row = q >> 4, v = q & 15;
                    float* dst = wsm + ((row >> 1) * (kDC / 8) + v) * 4 + (row & 1);
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8) dst[(q8 >> 1) * (NP * (kDC / 8) * 4) + (q8 & 1) * 2] = wreg[it][q8];
                }
            }
        };
        float2 acc[kTT][TP];
#pragma unroll
        for (int i = 0; i < kTT; ++i)
#pragma unroll
            for (int e = 0; e < TP; ++e) acc[i][e] = make_float2(0.0f, 0.0f);
        load_x(0, stage[0]);
        load_w(0);
        store_w(stage[0]);
        for (int k = 0; k < nchunks; ++k) {
            const bool more = k + 1 < nchunks;
            if (more) { load_x(k + 1, stage[(k + 1) & 1]); load_w(k + 1); cp_async_wait<1>(); }
            else cp_async_wait<0>();
            __syncthreads();
            const uint32_t xb = (uint32_t)__cvta_generic_to_shared(stage[k & 1]);
            const uint32_t wb = xb + XS_BYTES;
#pragma unroll 1
            for (int c = 0; c < 2; ++c) {
                const int v = c * 8 + s;                         // this chain's vector inside the chunk
                if (k * (kDC / 8) + c * 8 < nvec) {              // uniform: nvec is a multiple of 8
                    const uint32_t xa = xb + (uint32_t)(((tslab * 16 + g * kTT) * (kDC / 8) + v) * 16);
                    const uint32_t wa = wb + (uint32_t)(((eslab * TP) * (kDC / 8) + v) * 16);
                    static_assert(kTT == 4, "token rows are unrolled by hand");
                    uint4 xp[kTT];
                    xp[0] = lds16<0 * (kDC / 8) * 16>(xa);
                    xp[1] = lds16<1 * (kDC / 8) * 16>(xa);
                    xp[2] = lds16<2 * (kDC / 8) * 16>(xa);
                    xp[3] = lds16<3 * (kDC / 8) * 16>(xa);
                    // the 8 columns of the vector in two halves of 4, in column order: the chain of (token, expert) stays sequential
                    auto half = [&](auto H_) {
                        constexpr int hq = decltype(H_)::value;
                        float2 xd[kTT][4];                       // x broadcast to both halves of the packed operand
#pragma unroll
                        for (int i = 0; i < kTT; ++i) {
                            const uint32_t w0 = hq == 0 ? xp[i].x : xp[i].z, w1 = hq == 0 ? xp[i].y : xp[i].w;
                            const float f0 = bf_lo(w0), f1 = bf_hi(w0), f2 = bf_lo(w1), f3 = bf_hi(w1);
                            xd[i][0] = make_float2(f0, f0); xd[i][1] = make_float2(f1, f1);
                            xd[i][2] = make_float2(f2, f2); xd[i][3] = make_float2(f3, f3);
                        }
                        auto pair = [&](auto P_) {
                            constexpr int pp = decltype(P_)::value;
                            const uint4 wlo = lds16<((2 * hq) * NP + pp) * (kDC / 8) * 16>(wa);        // columns 4hq, 4hq+1
                            const uint4 whi = lds16<((2 * hq + 1) * NP + pp) * (kDC / 8) * 16>(wa);    // columns 4hq+2, 4hq+3
                            const float2 w[4] = {make_float2(__uint_as_float(wlo.x), __uint_as_float(wlo.y)),
                                                 make_float2(__uint_as_float(wlo.z), __uint_as_float(wlo.w)),
                                                 make_float2(__uint_as_float(whi.x), __uint_as_float(whi.y)),
                                                 make_float2(__uint_as_float(whi.z), __uint_as_float(whi.w))};
#pragma unroll
                            for (int i = 0; i < kTT; ++i)
#pragma unroll
                                for (int q = 0; q < 4; ++q) acc[i][pp] = __ffma2_rn(xd[i][q], w[q], acc[i][pp]);
                        };
                        static_for<TP>(pair);
                    };
                    static_for<2>(half);
                }
            }
            if (more) store_w(stage[(k + 1) & 1]);               // that buffer was last read in iteration k - 1
            __syncthreads();
        }
        // chain tree ((c0+c1)+(c2+c3))+((c4+c5)+(c6+c7)), then lane s keeps every 8th value
#pragma unroll
        for (int i = 0; i < kTT; ++i)
#pragma unroll
            for (int e = 0; e < TE; ++e) {
                float v = (e & 1) ? acc[i][e >> 1].y : acc[i][e >> 1].x;
                v = __fadd_rn(v, __shfl_xor_sync(full, v, 1));
                v = __fadd_rn(v, __shfl_xor_sync(full, v, 2));
                v = __fadd_rn(v, __shfl_xor_sync(full, v, 4));
                const int ge = ep0 + eslab * TE + e;
                if (((i * TE + e) & 7) == s && ge < E) {
                    if (a.bias) v = __fadd_rn(v, a.bias[ge]);
                    lg[(tslab * 16 + g * kTT + i) * E + ge] = v;
                }
            }
    }
    __syncthreads();
    route_block_finish<NTHR>(a, lg, sidx, zs, tok0);
}

// Scan, part 1: one warp per expert. Exclusive scan of that expert's per-block counts (the base of
// every router block inside the group), the expert's total and its probability sum; warp 0 of
// block 0 also reduces the z-loss partials. Fixed orders throughout: results are deterministic.
// This warp handles experts e_first, e_first + e_stride, ...; `with_z`: it also reduces the z-loss partials.
__device__ __forceinline__ void scan_columns_dev(const RouteDims& d, const RouteBufs& b, int NB, int e_first, int e_stride,
                                                 bool with_z) {
    const int lane = threadIdx.x & 31;
    const unsigned full = 0xffffffffu;
    const int E = d.E;
    for (int e = e_first; e < E; e += e_stride) {
        int running = 0;
        float fs = 0.0f;
        for (int b0 = 0; b0 < NB; b0 += 32) {
            const int blk = b0 + lane;
            const int c = blk < NB ? b.block_counts[(long)blk * E + e] : 0;
            int incl = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int n = __shfl_up_sync(full, incl, o);
                if (lane >= o) incl += n;
            }
            if (blk < NB) b.block_base[(long)blk * E + e] = running + incl - c;
            running += __shfl_sync(full, incl, 31);
            if (blk < NB) fs += b.block_sump[(long)blk * E + e];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) fs += __shfl_xor_sync(full, fs, o);
        if (lane == 0) {
            b.counts[e] = running;
            b.stat[e] = E == 1 ? 0.0f : fs;     // dense shortcut reports no statistics (moe.cu:397-403)
        }
    }
    if (with_z) {
        float z = 0.0f;
        for (int blk = lane; blk < NB; blk += 32) z += b.block_z[blk];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(full, z, o);
        if (lane == 0) b.stat[E] = E == 1 ? 0.0f : z / (float)d.T;
    }
}
__global__ void __launch_bounds__(256) scan_columns_kernel(const RouteDims d, const RouteBufs b, int NB) {
    const int warp = threadIdx.x >> 5;
    scan_columns_dev(d, b, NB, blockIdx.x * (blockDim.x >> 5) + warp, 1 << 30, blockIdx.x == 0 && warp == 0);
}

// Scan, part 2: one block. True and padded group starts (moe.cu:413-419), tile -> expert table,
// number of tiles in use, split table of the router weight-gradient product.
__device__ __forceinline__ void scan_finish_dev(const RouteDims& d, const RouteBufs& b, int splits, int* poff_s, int* cnt_s,
                                                bool counts_ready = false) {
    const int E = d.E;
    // counts first, all at once: read one by one between the stores below, every load would wait a full round trip
    if (!counts_ready) {
        for (int e = threadIdx.x; e < E; e += blockDim.x) cnt_s[e] = b.counts[e];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        int tk = 0, ptk = 0;
        for (int e = 0; e < E; ++e) {
            const int c = cnt_s[e];
            b.off[e] = tk; tk += c;
            poff_s[e] = ptk; b.poff[e] = ptk;
            ptk += (c + d.pad - 1) / d.pad * d.pad;
        }
        b.off[E] = tk; poff_s[E] = ptk; b.poff[E] = ptk;
        if (ptk > d.cap) { report(b.status, kErrSlotRange); ptk = 0; }
        *b.num_m_tiles = ptk / kPad;
        if (b.use_acc) b.use_acc[E] += 1;
    }
    if (b.use_acc)      // router-balance telemetry: usage accumulated on the device, read when the host asks
        for (int e = threadIdx.x; e < E; e += blockDim.x) b.use_acc[e] += cnt_s[e];
    __syncthreads();
    const int used = poff_s[E] <= d.cap ? poff_s[E] / kPad : 0;
    for (int i = threadIdx.x; i < d.max_tiles; i += blockDim.x) {
        int e = -1;
        if (i < used) {
            const int row = i * kPad;
            int lo = 0, hi = E;                       // last e with poff[e] <= row
            while (hi - lo > 1) { const int mid = (lo + hi) >> 1; if (poff_s[mid] <= row) lo = mid; else hi = mid; }
            e = lo;
            while (e < E && poff_s[e + 1] <= row) ++e;  // skip empty groups that share the start
        }
        b.tile_expert[i] = e;
    }
    // even split of the rows in use into `splits` ranges of whole tiles
    for (int i = threadIdx.x; i <= splits; i += blockDim.x) b.split_poff[i] = (int)((long)used * i / splits) * kPad;
}
__global__ void __launch_bounds__(256) scan_finish_kernel(const RouteDims d, const RouteBufs b, int splits) {
    __shared__ int poff_s[257], cnt_s[256];
    scan_finish_dev(d, b, splits, poff_s, cnt_s);
}

// Few tokens (sampler steps, short sequences): the 64-token block above would leave all but a handful of SMs idle.
// Here one block computes the logits of ONE token: 16 groups of 8 lanes, lane s = chain s, group q = experts q, q + 16,
// ...; the same chains, in the same order, added by the same butterfly, so the logits are bit-identical. The second
// half then runs per 64-token block on the stored logits (router_finish_kernel).
// LN: the LayerNorm in front of the block (tmt-cuda/src/norm.cu:8-50, model.cu:509-510) runs here as well: warp 0
// normalises the token's row with the arithmetic of the stand-alone forward kernel (lane l owns vectors l, l + 32, ...;
// sums in index order, butterfly 16..1, IEEE division and square root), leaves it in shared memory for the chains and
// writes it once for the expert products, so the fused step gives the bits of LayerNorm followed by the router.
template <bool WF32, bool LN>
__global__ void __launch_bounds__(128) router_logits_small_kernel(const RouterArgs a) {
    extern __shared__ __align__(16) uint16_t xs[];       // LN: the normalised row
    const int s = threadIdx.x & 7, grp = threadIdx.x >> 3;
    const long t = blockIdx.x;
    pdl_begin();
    pdl_wait();
    const int nvec = a.D >> 3;
    const unsigned full = 0xffffffffu;
    const uint16_t* xrow = a.X + t * a.D;
    if constexpr (LN) {
        if (threadIdx.x < 32) {
            const int lane = threadIdx.x;
            float sum = 0.0f, sq = 0.0f;
            for (int v = lane; v < nvec; v += 32) {
                const uint4 r = ldg16(xrow + v * 8);
                const float f[8] = {bf_lo(r.x), bf_hi(r.x), bf_lo(r.y), bf_hi(r.y), bf_lo(r.z), bf_hi(r.z), bf_lo(r.w), bf_hi(r.w)};
#pragma unroll
                for (int q = 0; q < 8; ++q) { sum = __fadd_rn(sum, f[q]); sq = __fmaf_rn(f[q], f[q], sq); }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                sum = __fadd_rn(sum, __shfl_xor_sync(full, sum, o));
                sq = __fadd_rn(sq, __shfl_xor_sync(full, sq, o));
            }
            const float fd = (float)a.D;
            const float m = __fdiv_rn(sum, fd);
            const float var = __fsub_rn(__fdiv_rn(sq, fd), __fmul_rn(m, m));
            const float rs = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, 1e-5f)));
            for (int v = lane; v < nvec; v += 32) {
                const uint4 r = ldg16(xrow + v * 8);
                const float f[8] = {bf_lo(r.x), bf_hi(r.x), bf_lo(r.y), bf_hi(r.y), bf_lo(r.z), bf_hi(r.z), bf_lo(r.w), bf_hi(r.w)};
                float o[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) o[q] = __fmaf_rn(__fmul_rn(__fsub_rn(f[q], m), rs), a.ln_gamma[v * 8 + q], a.ln_beta[v * 8 + q]);
                const uint4 w = make_uint4(pack_bf2(o[0], o[1]), pack_bf2(o[2], o[3]), pack_bf2(o[4], o[5]), pack_bf2(o[6], o[7]));
                *reinterpret_cast<uint4*>(xs + v * 8) = w;
                stg16(a.xn + t * a.D + v * 8, w);
            }
        }
        __syncthreads();
    }
    for (int e0 = 0; e0 < a.E; e0 += 16) {
        const int e = e0 + grp;
        const bool valid = e < a.E;
        const int er = valid ? e : 0;
        float acc = 0.0f;
        constexpr int kB = 8;                   // vectors in flight per lane (the chain itself stays sequential)
        for (int v0 = s; v0 < nvec; v0 += 8 * kB) {
            uint4 xv[kB], wa[kB], wb[kB];
#pragma unroll
            for (int u = 0; u < kB; ++u) {
                const int v = min(v0 + 8 * u, nvec - 8 + s);       // past the end: a valid address, value unused
                if constexpr (LN) xv[u] = *reinterpret_cast<const uint4*>(xs + v * 8);
                else xv[u] = ldg16(xrow + v * 8);
                if constexpr (WF32) {
                    const float* wr = reinterpret_cast<const float*>(a.Wr) + (long)er * a.D + v * 8;
                    wa[u] = ldg16(wr); wb[u] = ldg16(wr + 4);
                } else {
                    wa[u] = ldg16(reinterpret_cast<const uint16_t*>(a.Wr) + (long)er * a.D + v * 8);
                }
            }
#pragma unroll
            for (int u = 0; u < kB; ++u) {
                if (v0 + 8 * u < nvec) {
                    const float x[8] = {bf_lo(xv[u].x), bf_hi(xv[u].x), bf_lo(xv[u].y), bf_hi(xv[u].y),
                                        bf_lo(xv[u].z), bf_hi(xv[u].z), bf_lo(xv[u].w), bf_hi(xv[u].w)};
                    float w[8];
                    if constexpr (WF32) {
                        w[0] = __uint_as_float(wa[u].x); w[1] = __uint_as_float(wa[u].y); w[2] = __uint_as_float(wa[u].z); w[3] = __uint_as_float(wa[u].w);
                        w[4] = __uint_as_float(wb[u].x); w[5] = __uint_as_float(wb[u].y); w[6] = __uint_as_float(wb[u].z); w[7] = __uint_as_float(wb[u].w);
                    } else {
                        w[0] = bf_lo(wa[u].x); w[1] = bf_hi(wa[u].x); w[2] = bf_lo(wa[u].y); w[3] = bf_hi(wa[u].y);
                        w[4] = bf_lo(wa[u].z); w[5] = bf_hi(wa[u].z); w[6] = bf_lo(wa[u].w); w[7] = bf_hi(wa[u].w);
                    }
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc = __fmaf_rn(x[q], w[q], acc);
                }
            }
        }
        acc = __fadd_rn(acc, __shfl_xor_sync(full, acc, 1));
        acc = __fadd_rn(acc, __shfl_xor_sync(full, acc, 2));
        acc = __fadd_rn(acc, __shfl_xor_sync(full, acc, 4));
        if (valid && s == 0) {
            if (a.bias) acc = __fadd_rn(acc, a.bias[e]);
            a.b.logits[t * a.E + e] = acc;
        }
    }
}

constexpr int kFinishThreads = 512;     // 64 groups of 8 lanes: every token of the block at once

// splits > 0 (only with a single block, i.e. at most kTokBlock tokens): the block also does both parts of the scan.
__global__ void __launch_bounds__(kFinishThreads) router_finish_kernel(const RouterArgs a, const RouteDims d, int splits) {
    extern __shared__ __align__(16) uint8_t smem[];
    float* lg = reinterpret_cast<float*>(smem);          // [kTokBlock][E]
    __shared__ int sidx[kTokBlock * 8];
    __shared__ float zs[kTokBlock];
    __shared__ int poff_s[257], cnt_s[256];
    const long tok0 = (long)blockIdx.x * kTokBlock;
    pdl_begin();
    pdl_wait();
    for (int i = threadIdx.x; i < kTokBlock * a.E; i += kFinishThreads) {
        const long t = tok0 + i / a.E;
        lg[i] = t < a.T ? a.b.logits[tok0 * a.E + i] : 0.0f;
    }
    __syncthreads();
    __shared__ float sp_s[256], z_s;
    const bool fused = splits > 0;
    route_block_finish<kFinishThreads>(a, lg, sidx, zs, tok0, fused ? cnt_s : nullptr, fused ? sp_s : nullptr, fused ? &z_s : nullptr);
    if (fused) {
        // One block holds every token: its counts and partial sums ARE the totals (what the first part of the scan
        // computes from a single block: base 0, the same sums with zeros added), and they are still in shared memory.
        __syncthreads();
        const int E = a.E;
        for (int e = threadIdx.x; e < E; e += kFinishThreads) {
            a.b.block_base[e] = 0;
            a.b.counts[e] = cnt_s[e];
            a.b.stat[e] = E == 1 ? 0.0f : sp_s[e];
        }
        if (threadIdx.x == kFinishThreads - 1) a.b.stat[E] = E == 1 ? 0.0f : z_s / (float)d.T;
        scan_finish_dev(d, a.b, splits, poff_s, cnt_s, true);
    }
}

template <int TE, int ESLABS, bool WF32>
cudaError_t launch_router_t(const RouterArgs& a, int nb, cudaStream_t s) {
    constexpr int EP = TE * ESLABS;
    const size_t smem = 2 * ((size_t)kTokBlock * kDC * 2 + (size_t)EP * kDC * 4) + (size_t)kTokBlock * a.E * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(router_kernel<TE, ESLABS, WF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    router_kernel<TE, ESLABS, WF32><<<nb, 128 * ESLABS, smem, s>>>(a);
    return cudaGetLastError();
}

template <bool WF32>
cudaError_t launch_router_w(const RouterArgs& a, int nb, cudaStream_t s) {
    if (a.E <= 4) return launch_router_t<4, 1, WF32>(a, nb, s);
    if (a.E <= 8) return launch_router_t<8, 1, WF32>(a, nb, s);
    if (a.E <= 16) return launch_router_t<16, 1, WF32>(a, nb, s);
    if (a.E <= 32) return launch_router_t<16, 2, WF32>(a, nb, s);
    // more than 32 experts: 64 tokens x 16 experts per pass with 256 threads (73 registers, three blocks per SM) measured
    // faster at 64 experts than one pass of 64 experts with 512 threads (127 registers, one block per SM): 1.66 against
    // 1.83-1.87 ms at 131072 tokens; 16 x 2, 8 x 4 and 8 x 8 slabs gave 1.70, 1.96 and 2.03 ms
    return launch_router_t<8, 2, WF32>(a, nb, s);
}

}  // namespace

// Up to this many logits the per-token kernel is used (TMT_MOE_ROUTER_SMALL = 0 / 1 forces one of the two; both give
// the same bits): beyond it, re-reading the router rows per token costs more than the idle SMs of the tiled kernel.
constexpr long kSmallRouterLogits = 16384;

bool router_takes_layernorm(const RouteDims& d) {
    bool small = (long)d.T * d.E <= kSmallRouterLogits;
    if (const char* f = getenv("TMT_MOE_ROUTER_SMALL")) if (*f) small = *f != '0';
    return small && d.D * 2 <= 48 * 1024;
}

cudaError_t launch_router(const RouteDims& d, const RouteBufs& b, const uint16_t* X, const void* Wr,
                          const float* bias, cudaStream_t s, int scan_splits, bool* scanned, const float* ln_gamma,
                          const float* ln_beta, uint16_t* xn, int* kernels) {
    if (scanned) *scanned = false;
    if (kernels) *kernels = 1;
    RouterArgs a{X, Wr, bias, d.T, d.D, d.E, d.K, b, ln_gamma, ln_beta, xn};
    const int nb = (d.T + kTokBlock - 1) / kTokBlock;
    bool small = (long)d.T * d.E <= kSmallRouterLogits;
    if (const char* f = getenv("TMT_MOE_ROUTER_SMALL")) if (*f) small = *f != '0';
    if (ln_gamma && !(small && router_takes_layernorm(d))) return cudaErrorInvalidValue;     // the caller normalises first
    if (small) {
        if (kernels) *kernels = 2;
        cudaError_t le;
        if (ln_gamma) {
            const size_t row = (size_t)d.D * 2;
            le = d.router_f32 ? launch_pdl(router_logits_small_kernel<true, true>, dim3(d.T), dim3(128), row, s, a)
                              : launch_pdl(router_logits_small_kernel<false, true>, dim3(d.T), dim3(128), row, s, a);
        } else {
            le = d.router_f32 ? launch_pdl(router_logits_small_kernel<true, false>, dim3(d.T), dim3(128), 0, s, a)
                              : launch_pdl(router_logits_small_kernel<false, false>, dim3(d.T), dim3(128), 0, s, a);
        }
        if (le != cudaSuccess) return le;
        const size_t smem = (size_t)kTokBlock * d.E * sizeof(float);
        if (smem > 40 * 1024) {
            cudaError_t e = cudaFuncSetAttribute(router_finish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            if (e != cudaSuccess) return e;
        }
        const bool fuse = nb == 1 && scan_splits > 0 && scanned != nullptr;
        if (fuse) *scanned = true;
        return launch_pdl(router_finish_kernel, dim3(nb), dim3(kFinishThreads), smem, s, a, d, fuse ? scan_splits : 0);
    }
    return d.router_f32 ? launch_router_w<true>(a, nb, s) : launch_router_w<false>(a, nb, s);
}

cudaError_t launch_scan(const RouteDims& d, const RouteBufs& b, int splits, cudaStream_t s) {
    const int nb = (d.T + kTokBlock - 1) / kTokBlock;
    scan_columns_kernel<<<(d.E + 7) / 8, 256, 0, s>>>(d, b, nb);
    scan_finish_kernel<<<1, 256, 0, s>>>(d, b, splits);
    return cudaGetLastError();
}

}  // namespace tmt
