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
#include "kernels.cuh"

namespace tmt {
namespace {

constexpr int kRouterThreads = 256;

struct RouterArgs {
    const uint16_t* X; const void* Wr; const float* bias;
    int T, D, E, K;
    RouteBufs b;
};

template <int EC, bool WF32>
__global__ void __launch_bounds__(kRouterThreads) router_kernel(const RouterArgs a) {
    extern __shared__ float lg[];                 // [kTokBlock][E] logits, later probabilities
    __shared__ int sidx[kTokBlock * 8];
    __shared__ float zs[kTokBlock];
    const int E = a.E, K = a.K, D = a.D;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = lane & 7, g = lane >> 3;
    const int nvec = D >> 3;
    const unsigned full = 0xffffffffu;

    for (int pass = 0; pass < kTokBlock / 32; ++pass) {
        const int tb = pass * 32 + warp * 4 + g;
        const long t = (long)blockIdx.x * kTokBlock + tb;
        const bool valid = t < a.T;
        const uint16_t* xrow = a.X + (valid ? t : 0) * (long)D;
        // ---- dot products, EC experts at a time ----
        for (int ec0 = 0; ec0 < E; ec0 += EC) {
            float acc[EC];
#pragma unroll
            for (int e = 0; e < EC; ++e) acc[e] = 0.0f;
            if (valid) {
                for (int v = s; v < nvec; v += 8) {
                    const uint4 xv = ldg16(xrow + v * 8);
                    float x[8] = {bf_lo(xv.x), bf_hi(xv.x), bf_lo(xv.y), bf_hi(xv.y),
                                  bf_lo(xv.z), bf_hi(xv.z), bf_lo(xv.w), bf_hi(xv.w)};
#pragma unroll
                    for (int e = 0; e < EC; ++e) {
                        if (ec0 + e < E) {
                            float wv[8];
                            if constexpr (WF32) {
                                const float* wp = reinterpret_cast<const float*>(a.Wr) + (long)(ec0 + e) * D + v * 8;
                                const float4 w0 = __ldg(reinterpret_cast<const float4*>(wp));
                                const float4 w1 = __ldg(reinterpret_cast<const float4*>(wp) + 1);
                                wv[0] = w0.x; wv[1] = w0.y; wv[2] = w0.z; wv[3] = w0.w;
                                wv[4] = w1.x; wv[5] = w1.y; wv[6] = w1.z; wv[7] = w1.w;
                            } else {
                                const uint4 w4 = ldg16(reinterpret_cast<const uint16_t*>(a.Wr) + (long)(ec0 + e) * D + v * 8);
                                wv[0] = bf_lo(w4.x); wv[1] = bf_hi(w4.x); wv[2] = bf_lo(w4.y); wv[3] = bf_hi(w4.y);
                                wv[4] = bf_lo(w4.z); wv[5] = bf_hi(w4.z); wv[6] = bf_lo(w4.w); wv[7] = bf_hi(w4.w);
                            }
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[e] = __fmaf_rn(x[i], wv[i], acc[e]);
                        }
                    }
                }
            }
#pragma unroll
            for (int e = 0; e < EC; ++e) {
                float v = acc[e];
                v = __fadd_rn(v, __shfl_xor_sync(full, v, 1));
                v = __fadd_rn(v, __shfl_xor_sync(full, v, 2));
                v = __fadd_rn(v, __shfl_xor_sync(full, v, 4));
                if (ec0 + e < E && (e & 7) == s) {
                    if (a.bias) v = __fadd_rn(v, a.bias[ec0 + e]);
                    lg[tb * E + ec0 + e] = valid ? v : 0.0f;
                }
            }
        }
        __syncwarp();
        // ---- softmax, top-k (on logits, lowest index wins ties), gate weights ----
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
    const int n_asg = kTokBlock * K;
    for (int i = threadIdx.x; i < n_asg; i += blockDim.x) {
        const int e = sidx[i];
        if (e < 0) continue;
        int r = 0;
        for (int q = 0; q < i; ++q) r += (sidx[q] == e);
        a.b.rank[(long)blockIdx.x * n_asg + i] = r;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int c = 0;
        for (int q = 0; q < n_asg; ++q) c += (sidx[q] == e);
        float sp = 0.0f;
        for (int tb = 0; tb < kTokBlock; ++tb) sp += lg[tb * E + e];
        a.b.block_counts[(long)blockIdx.x * E + e] = c;
        a.b.block_sump[(long)blockIdx.x * E + e] = sp;
    }
    if (threadIdx.x == 0) {
        float z = 0.0f;
        for (int tb = 0; tb < kTokBlock; ++tb) z += zs[tb];
        a.b.block_z[blockIdx.x] = z;
    }
}

// One block. Exclusive scan of the per-block counts per expert, totals, true and padded
// group starts, tile -> expert table, statistics.
__global__ void __launch_bounds__(1024) scan_kernel(const RouteDims d, const RouteBufs b, int NB) {
    __shared__ int cnt_s[256];
    __shared__ int poff_s[257];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    const unsigned full = 0xffffffffu;
    const int E = d.E;
    for (int e = warp; e < E; e += nwarps) {
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
            cnt_s[e] = running;
            b.counts[e] = running;
            b.stat[e] = E == 1 ? 0.0f : fs;     // dense shortcut reports no statistics (moe.cu:397-403)
        }
    }
    if (warp == 0) {
        float z = 0.0f;
        for (int blk = lane; blk < NB; blk += 32) z += b.block_z[blk];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) z += __shfl_xor_sync(full, z, o);
        if (lane == 0) b.stat[E] = E == 1 ? 0.0f : z / (float)d.T;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tk = 0, ptk = 0;
        for (int e = 0; e < E; ++e) {
            b.off[e] = tk; tk += cnt_s[e];
            poff_s[e] = ptk; b.poff[e] = ptk;
            ptk += (cnt_s[e] + kPad - 1) / kPad * kPad;
        }
        b.off[E] = tk; poff_s[E] = ptk; b.poff[E] = ptk;
        if (ptk > d.cap) { report(b.status, kErrSlotRange); ptk = 0; }
        *b.num_m_tiles = ptk / kPad;
    }
    __syncthreads();
    const int used = poff_s[E] <= d.cap ? poff_s[E] / kPad : 0;
    for (int i = threadIdx.x; i < d.max_tiles; i += blockDim.x) {
        int e = -1;
        if (i < used) {
            const int row = i * kPad;
            for (int q = 0; q < E; ++q)
                if (row >= poff_s[q] && row < poff_s[q + 1]) { e = q; break; }
        }
        b.tile_expert[i] = e;
    }
}

template <int EC, bool WF32>
cudaError_t launch_router_t(const RouterArgs& a, int nb, cudaStream_t s) {
    const size_t smem = (size_t)kTokBlock * a.E * sizeof(float);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(router_kernel<EC, WF32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    router_kernel<EC, WF32><<<nb, kRouterThreads, smem, s>>>(a);
    return cudaGetLastError();
}

template <bool WF32>
cudaError_t launch_router_w(const RouterArgs& a, int nb, cudaStream_t s) {
    if (a.E <= 4) return launch_router_t<4, WF32>(a, nb, s);
    if (a.E <= 8) return launch_router_t<8, WF32>(a, nb, s);
    if (a.E <= 16) return launch_router_t<16, WF32>(a, nb, s);
    if (a.E <= 32) return launch_router_t<32, WF32>(a, nb, s);
    return launch_router_t<64, WF32>(a, nb, s);
}

}  // namespace

cudaError_t launch_router(const RouteDims& d, const RouteBufs& b, const uint16_t* X, const void* Wr,
                          const float* bias, cudaStream_t s) {
    RouterArgs a{X, Wr, bias, d.T, d.D, d.E, d.K, b};
    const int nb = (d.T + kTokBlock - 1) / kTokBlock;
    return d.router_f32 ? launch_router_w<true>(a, nb, s) : launch_router_w<false>(a, nb, s);
}

cudaError_t launch_scan(const RouteDims& d, const RouteBufs& b, cudaStream_t s) {
    const int nb = (d.T + kTokBlock - 1) / kTokBlock;
    scan_kernel<<<1, 1024, 0, s>>>(d, b, nb);
    return cudaGetLastError();
}

}  // namespace tmt
