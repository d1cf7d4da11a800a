// NVFP4 sampler steps (a few tokens per expert): the expert products straight from the PACKED weights.
//
// With 64 streams x top-2 over 16 experts an expert sees about 8 rows, so the step is bound by how fast
// the 4-bit weights travel (L2 / HBM -> registers), not by arithmetic. Each warp owns 16 weight rows:
// it loads their packed codes with 16-byte loads, expands them in registers to bf16(q * block scale)
// (exact: at most 6 significant bits) and multiplies with the register-operand tensor-core MMA
// (m16n8k16, weights = the 16-row operand, the expert's tokens = the 8 columns). The operand never
// exists in memory in expanded form, which is why the shared-memory-operand tcgen05 path of the grouped
// kernels is not used here. Replaces, for small batches, the dequantise-then-GEMM route of
// tmt-cuda/src/moe.cu:423-462 (forward expert loop) for the sampler of tmt-cuda/src/sample_main.cu.
//
// Expansion of a code: bits (s e1 e0 m) of e2m1, placed at bits 15 and 8..6 of a bf16, read as
// q * 2^-126 (for e = 0 this is a bf16 subnormal, exactly m * 0.5 * 2^-126); one bf16x2 multiply by
// block scale * 2^112 gives q * scale * 2^-14, a normal number; the 2^14 returns with the tensor scale
// in the epilogue. Two codes (nibbles i and i + 4 of a 32-bit word) expand per shift/mask/multiply.
//
// The k order inside one MMA is free as long as both operands agree: a thread takes 32 consecutive k
// (16 bytes of codes = two scale blocks) per 128-k chunk, and the token rows are staged in shared
// memory already permuted to match.
#include <cstdlib>

#include "kernels.cuh"
#include "launch_pdl.cuh"
#include "nvfp4_decode.h"
#include "tc_util.cuh"

namespace tmt {
namespace {

constexpr int kNT = 16;                 // tokens (assignments) of one expert per pass: two MMA column tiles share one expansion
constexpr int kRowsPerCta = 128;        // 8 row groups of 16 weight rows (times RGW)
constexpr int kKSplit = 2;              // warps sharing a row group, each with half of the chunks
constexpr int kThreads = 256 * kKSplit;
constexpr int kListBytes = kDecodeMaxAsg * 4, kLutBytes = 256 * 4;
__host__ __device__ constexpr int red_bytes(int rgw) { return rgw * 8 * 256 * 4; }
constexpr int kSB = 4;                  // staged rows a thread fetches before it stores any
constexpr int kMaxSmem = 227 * 1024;

__device__ __forceinline__ uint32_t mul_bf2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
// codes i and i + 4 of w -> (q_i, q_{i+4}) * scale * 2^-14 as bf16x2
template <int I>
__device__ __forceinline__ uint32_t expand_pair(uint32_t w, uint32_t s2) {
    const uint32_t mag = (I == 0 ? w << 6 : I == 1 ? w << 2 : I == 2 ? w >> 2 : w >> 6) & 0x01C001C0u;
    const uint32_t sgn = (I == 0 ? w << 12 : I == 1 ? w << 8 : I == 2 ? w << 4 : w) & 0x80008000u;
    return mul_bf2(mag | sgn, s2);
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds16u(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts16u(uint32_t addr, uint4 v) {
    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__device__ __forceinline__ uint32_t lds_u16(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
// one row of codes or scales, global -> shared memory, completion counted in bytes on `bar`
__device__ __forceinline__ void bulk_load_row(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// MODE 0: out[asg][row] = bf16(silu(a)), a = bf16(es * acc)          (up-projection; src row = asg / src_div)
// MODE 1: out[asg][row] = bf16(gate[asg] * (es * acc))               (down-projection; src row = asg)
// A block owns 128 * RGW weight rows of one expert (one block per SM). All of them are requested at the start, one bulk
// copy per row of codes and per row of scales into padded shared-memory rows (pitch = row + 64 / + 16 bytes: the 8 rows
// a warp reads together fall on different banks), so the whole tile is in flight at once and no register holds
// prefetched weights. 16 warps = 8 row groups x 2 k halves; RGW row groups per warp, one after the other.
template <int MODE, int RGW>
__global__ void __launch_bounds__(kThreads, 1) fp4_rows_kernel(const Fp4RowsArgs p) {
    extern __shared__ __align__(128) uint8_t smem[];
    int* list = reinterpret_cast<int*>(smem);                         // assignments of this expert, ascending
    const int kdim = p.kdim;
    constexpr int R = kRowsPerCta * RGW;
    const uint32_t cpitch = (uint32_t)(kdim >> 1) + 64, spitch = (uint32_t)(kdim >> 4) + 16;
    const uint32_t rowb = (uint32_t)(kdim / p.kphases) * 2 + 64;      // staged token row pitch
    // [RGW][2][4][256] partial sums of the second k half: a region of their own, or (red_in_stage: when that is what lets
    // whole token rows fit) the start of the staged rows, which are dead by the time the sums are exchanged
    const int redb = p.red_in_stage ? 0 : red_bytes(RGW);
    const uint32_t lut = tc::smem_u32(smem) + kListBytes + redb;      // e4m3 byte -> scale * 2^112 as bf16x2
    const uint32_t codes = lut + kLutBytes;
    const uint32_t scales = codes + R * cpitch;
    const uint32_t stage = scales + R * spitch;
    float* red = reinterpret_cast<float*>(p.red_in_stage ? smem + (stage - tc::smem_u32(smem)) : smem + kListBytes);
    __shared__ __align__(8) uint64_t wbar;
    __shared__ int s_cnt, abort_s;
    __shared__ unsigned masks[kDecodeMaxAsg / 32];
    const int e = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int rgroup = warp & 7, ks = warp >> 3;
    const int row0 = blockIdx.x * R;
    pdl_begin();
    if (threadIdx.x == 0) {
        abort_s = 0;
        tc::mbar_init(tc::smem_u32(&wbar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        tc::fence_async_smem();
        tc::mbar_expect_tx(tc::smem_u32(&wbar), (uint32_t)R * (uint32_t)((kdim >> 1) + (kdim >> 4)));
    }
    if (threadIdx.x < 256) {   // scale table: entry = e4m3 * 2^112 as bf16 in both halves
        const uint32_t byte = threadIdx.x, ex = byte >> 3, m = byte & 7u;
        uint32_t b = (byte << 4) + (232u << 7);                       // normal: exponent ex - 7 + 112 + 127
        if (ex == 0) b = f2bf((float)m * 0x1p103f);                   // subnormal: m * 2^-9 * 2^112
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(lut + byte * 4), "r"(b | (b << 16)) : "memory");
    }
    __syncthreads();
    // The weights do not depend on the kernels before this one: ask for the block's whole tile now, so that it travels
    // while those kernels finish (an expert that turns out to have no tokens pays for the copy and waits for it below).
    if (threadIdx.x < R) {
        bulk_load_row(codes + threadIdx.x * cpitch, p.packed[e] + (size_t)(row0 + threadIdx.x) * (kdim >> 1), (uint32_t)(kdim >> 1),
                      tc::smem_u32(&wbar));
    } else if (threadIdx.x >= 256 && threadIdx.x - 256 < R) {
        const int r = threadIdx.x - 256;
        bulk_load_row(scales + r * spitch, p.scales[e] + (size_t)(row0 + r) * (kdim >> 4), (uint32_t)(kdim >> 4), tc::smem_u32(&wbar));
    }
    pdl_wait();        // everything above read only the weights and wrote only this block's shared memory
    // this warp's first slice of the assignment table, asked for before anything that has to wait for a pointer
    const int first_idx = warp * 32 + lane < p.n_asg ? p.idx[warp * 32 + lane] : -1;
    // token list, ascending: warp w takes the 32-assignment slices w, w + 16, ...; one load latency in all
    for (int sl = warp; sl * 32 < p.n_asg; sl += kThreads / 32) {
        const int i = sl * 32 + lane;
        const int ie = sl == warp ? first_idx : (i < p.n_asg ? p.idx[i] : -1);
        const unsigned m = __ballot_sync(0xffffffffu, ie == e);
        if (lane == 0) masks[sl] = m;
    }
    __syncthreads();
    if (warp == 0) {
        const int nsl = (p.n_asg + 31) >> 5;
        const unsigned m = lane < nsl ? masks[lane] : 0u;
        int incl = __popc(m);
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int n = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += n;
        }
        int pos = incl - __popc(m);
        for (unsigned r = m; r; r &= r - 1) list[pos++] = lane * 32 + (__ffs(r) - 1);
        if (lane == 31) s_cnt = incl;
    }
    __syncthreads();
    const int cnt = TMT_DBG(p, 1) ? 0 : s_cnt;      // measurement only: bit 0 = stop after the token list
    if (cnt == 0) {                                // nothing to do, but the copies must have landed before the block may leave
        tc::mbar_wait(tc::smem_u32(&wbar), 0, &abort_s, p.status);
        return;
    }
    const float es = p.es[e];
    // token rows are staged kstage columns at a time (the whole row when it fits beside the weight tile)
    const int kstage = kdim / p.kphases, cpp = kstage >> 7;          // chunks per phase, split between the two k halves
    const int pieces_per_row = kstage >> 3;
    const int lanes_per_row = min(pieces_per_row, kThreads), rows_per_iter = kThreads / lanes_per_row;
    const int sub = threadIdx.x / lanes_per_row, v0 = threadIdx.x - sub * lanes_per_row;
    const int jl0 = ks * cpp / kKSplit, jl1 = (ks + 1) * cpp / kKSplit;
    bool have_weights = false;

    for (int pass = 0; pass * kNT < cnt; ++pass) {
        const int n_here = min(kNT, cnt - pass * kNT);
        const int ntiles = (n_here + 7) >> 3;
        float acc[RGW][2][4];
#pragma unroll
        for (int rg = 0; rg < RGW; ++rg)
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[rg][t][i] = 0.0f;
        for (int ph = 0; ph < p.kphases; ++ph) {
            if (pass + ph > 0) __syncthreads();                       // everyone has left the rows staged before
            // rows of the pass -> shared memory, permuted; kSB 16-byte loads in flight per thread. Columns past n_here
            // stay as they are: a column of the product depends on nothing but its own token.
            for (int n0 = sub; n0 < (TMT_DBG(p, 4) ? 0 : n_here); n0 += kSB * rows_per_iter) {    // bit 2 = no staging
                for (int v = v0; v < pieces_per_row; v += lanes_per_row) {
                    uint4 x[kSB];
#pragma unroll
                    for (int u = 0; u < kSB; ++u) {
                        const int n = n0 + u * rows_per_iter;
                        if (n < n_here)
                            x[u] = ldg16(p.src + (size_t)(list[pass * kNT + n] / p.src_div) * p.src_ld + (size_t)ph * kstage + v * 8);
                    }
                    const int j = v >> 4, r = v & 15;
#pragma unroll
                    for (int u = 0; u < kSB; ++u) {
                        const int n = n0 + u * rows_per_iter;
                        if (n >= n_here) break;
                        uint4 o;
                        o.x = __byte_perm(x[u].x, x[u].z, 0x5410); o.y = __byte_perm(x[u].x, x[u].z, 0x7632);     // (k0,k4) (k1,k5)
                        o.z = __byte_perm(x[u].y, x[u].w, 0x5410); o.w = __byte_perm(x[u].y, x[u].w, 0x7632);     // (k2,k6) (k3,k7)
                        sts16u(stage + (uint32_t)n * rowb + (uint32_t)(j * 256 + (r & 3) * 64 + (r >> 2) * 16), o);
                    }
                }
            }
            if (!have_weights) {       // bounded wait; a block that gives up reports it in the status word and leaves
                const bool ok = tc::mbar_wait(tc::smem_u32(&wbar), 0, &abort_s, p.status);
                if (!__syncthreads_and(ok)) return;
                have_weights = true;
            } else {
                __syncthreads();
            }
#pragma unroll
            for (int rg = 0; rg < RGW; ++rg) {
                const int lrow = rg * kRowsPerCta + rgroup * 16 + g;  // row inside the block's tile; its partner is 8 further
                const uint32_t crow = codes + (uint32_t)lrow * cpitch + (uint32_t)(c * 16 + ph * cpp * 64);
                const uint32_t srow = scales + (uint32_t)lrow * spitch + (uint32_t)(c * 2 + ph * cpp * 8);
                const uint32_t brow = stage + (uint32_t)g * rowb + (uint32_t)c * 16;
#pragma unroll 2
                for (int j = jl0; j < (TMT_DBG(p, 2) ? jl0 : jl1); ++j) {     // bit 1 = no products
                    const uint4 ca = lds16u(crow + j * 64), cb = lds16u(crow + 8 * cpitch + j * 64);
                    const uint32_t sa = lds_u16(srow + j * 8), sb = lds_u16(srow + 8 * spitch + j * 8);
                    const uint32_t a_w[4] = {ca.x, ca.y, ca.z, ca.w}, b_w[4] = {cb.x, cb.y, cb.z, cb.w};
                    const uint32_t sA[2] = {lds_u32(lut + (sa & 0xffu) * 4), lds_u32(lut + (sa >> 8) * 4)};
                    const uint32_t sB[2] = {lds_u32(lut + (sb & 0xffu) * 4), lds_u32(lut + (sb >> 8) * 4)};
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t wa = a_w[q], wb = b_w[q], s_a = sA[q >> 1], s_b = sB[q >> 1];
                        const uint32_t a00 = expand_pair<0>(wa, s_a), a01 = expand_pair<1>(wa, s_a);
                        const uint32_t a02 = expand_pair<2>(wa, s_a), a03 = expand_pair<3>(wa, s_a);
                        const uint32_t a80 = expand_pair<0>(wb, s_b), a81 = expand_pair<1>(wb, s_b);
                        const uint32_t a82 = expand_pair<2>(wb, s_b), a83 = expand_pair<3>(wb, s_b);
#pragma unroll
                        for (int t = 0; t < 2; ++t) {
                            if (t < ntiles) {
                                const uint4 x = lds16u(brow + (uint32_t)(t * 8) * rowb + (uint32_t)(j * 256 + q * 64));
                                mma_bf16(acc[rg][t], a00, a80, a01, a81, x.x, x.y);
                                mma_bf16(acc[rg][t], a02, a82, a03, a83, x.z, x.w);
                            }
                        }
                    }
                }
            }
        }
        // the second k half hands its sums to the first
        if (p.red_in_stage) __syncthreads();                          // every warp has read its last staged row
        if (ks == 1) {
#pragma unroll
            for (int rg = 0; rg < RGW; ++rg)
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) red[((rg * 2 + t) * 4 + i) * 256 + rgroup * 32 + lane] = acc[rg][t][i];
        }
        __syncthreads();
        if (ks == 0) {
#pragma unroll
            for (int rg = 0; rg < RGW; ++rg)
#pragma unroll
                for (int t = 0; t < 2; ++t)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int n = t * 8 + c * 2 + (i & 1);
                        if (n >= n_here) continue;
                        const int asg = list[pass * kNT + n];
                        const int row = row0 + rg * kRowsPerCta + rgroup * 16 + g + (i >> 1) * 8;
                        const float v = acc[rg][t][i] + red[((rg * 2 + t) * 4 + i) * 256 + rgroup * 32 + lane];
                        float o;
                        if constexpr (MODE == 0) {
                            const float a = round_bf(es * v);
                            o = a * sigmoid_fast(a);
                        } else {
                            o = p.gate[asg] * (es * v);
                        }
                        p.out[(size_t)asg * p.out_ld + row] = f2bf(o);
                    }
        }
    }
}

// Y[t] = beta * Y[t] + sum_j Ya[t * K + j] in increasing j (the gate weight is already applied)
__global__ void __launch_bounds__(256) decode_combine_kernel(const uint16_t* __restrict__ Ya, uint16_t* __restrict__ Y, float beta,
                                                             int T, int D, int K) {
    const int nvec = D >> 3;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    pdl_begin();
    pdl_wait();
    if (i >= (long)T * nvec) return;
    const long t = i / nvec; const int v = (int)(i - t * nvec);
    float acc[8];
    uint16_t* dst = Y + t * D + v * 8;
    if (beta != 0.0f) {
        const uint4 y = ldg16(dst);
        acc[0] = beta * bf_lo(y.x); acc[1] = beta * bf_hi(y.x); acc[2] = beta * bf_lo(y.y); acc[3] = beta * bf_hi(y.y);
        acc[4] = beta * bf_lo(y.z); acc[5] = beta * bf_hi(y.z); acc[6] = beta * bf_lo(y.w); acc[7] = beta * bf_hi(y.w);
    } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.0f;
    }
    for (int j = 0; j < K; ++j) {
        const uint4 y = ldg16(Ya + (t * K + j) * D + v * 8);
        acc[0] += bf_lo(y.x); acc[1] += bf_hi(y.x); acc[2] += bf_lo(y.y); acc[3] += bf_hi(y.y);
        acc[4] += bf_lo(y.z); acc[5] += bf_hi(y.z); acc[6] += bf_lo(y.w); acc[7] += bf_hi(y.w);
    }
    stg16(dst, make_uint4(pack_bf2(acc[0], acc[1]), pack_bf2(acc[2], acc[3]), pack_bf2(acc[4], acc[5]), pack_bf2(acc[6], acc[7])));
}

size_t rows_smem(int kdim, int rgw, int kphases, bool red_in_stage = false) {
    return (size_t)kListBytes + (red_in_stage ? 0 : red_bytes(rgw)) + kLutBytes + (size_t)kRowsPerCta * rgw * ((kdim >> 1) + 64 + (kdim >> 4) + 16) +
           (size_t)kNT * (kdim / kphases * 2 + 64);
}
// Fewest staging phases (1, 2 or 4 slices of whole 256-column units) with which the tile fits; 0: none does.
int pick_phases(int kdim, int rgw) {
    for (int ph = 1; ph <= 4; ph *= 2)
        if (kdim % (256 * ph) == 0 && rows_smem(kdim, rgw, ph) <= (size_t)kMaxSmem) return ph;
    return 0;
}

template <int MODE, int RGW>
cudaError_t launch_rows_t(Fp4RowsArgs a, int experts, cudaStream_t s) {
    a.kphases = pick_phases(a.kdim, RGW);
    // two slices only because of the exchange buffer: put that buffer into the staged rows and keep the rows whole
    a.red_in_stage = a.kphases == 2 && rows_smem(a.kdim, RGW, 1, true) <= (size_t)kMaxSmem && !getenv("TMT_MOE_FP4_TWO_SLICES");
    if (a.red_in_stage) a.kphases = 1;
    const size_t smem = rows_smem(a.kdim, RGW, a.kphases, a.red_in_stage);
    cudaError_t e = cudaFuncSetAttribute(fp4_rows_kernel<MODE, RGW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    return launch_pdl(fp4_rows_kernel<MODE, RGW>, dim3(a.rows / (kRowsPerCta * RGW), experts), dim3(kThreads), smem, s, a);
}

}  // namespace

// A block covers 256 weight rows when the tile fits in shared memory and that still gives about one block per SM,
// else 128 (TMT_MOE_FP4_ROW_GROUPS = 1 / 2 forces the choice where the shape allows it).
cudaError_t launch_fp4_rows(const Fp4RowsArgs& a, int experts, int mode, cudaStream_t s) {
    const bool two_ok = a.rows % (2 * kRowsPerCta) == 0 && pick_phases(a.kdim, 2) == 1;
    int rgw = two_ok && (long)(a.rows / (2 * kRowsPerCta)) * experts >= 120 ? 2 : 1;
    if (const char* f = getenv("TMT_MOE_FP4_ROW_GROUPS")) if (*f == '1' || (*f == '2' && two_ok)) rgw = *f - '0';
    if (mode == 0) return rgw == 2 ? launch_rows_t<0, 2>(a, experts, s) : launch_rows_t<0, 1>(a, experts, s);
    return rgw == 2 ? launch_rows_t<1, 2>(a, experts, s) : launch_rows_t<1, 1>(a, experts, s);
}

cudaError_t launch_decode_combine(const uint16_t* Ya, uint16_t* Y, float beta, int T, int D, int K, cudaStream_t s) {
    const long n = (long)T * (D >> 3);
    return launch_pdl(decode_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s, Ya, Y, beta, T, D, K);
}

bool fp4_rows_shape_ok(int rows, int kdim) {
    return rows % kRowsPerCta == 0 && kdim % 256 == 0 && pick_phases(kdim, 1) > 0;
}

}  // namespace tmt
