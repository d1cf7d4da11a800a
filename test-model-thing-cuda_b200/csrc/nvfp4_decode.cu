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
#include "kernels.cuh"
#include "nvfp4_decode.h"

namespace tmt {
namespace {

constexpr int kNT = 16;                 // tokens (assignments) of one expert per pass: two MMA column tiles
constexpr int kRowsPerCta = 64;         // 4 row groups of 16 weight rows
constexpr int kKSplit = 2;              // warps sharing a row group, each with half of the chunks
constexpr int kThreads = 128 * kKSplit;
constexpr int kSB = 4;                 // staged rows a thread fetches before it stores any

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
// e4m3 (unsigned) * 2^112 as bf16, duplicated into both halves
__device__ __forceinline__ uint32_t scale_bf2(uint32_t byte) {
    const uint32_t e = byte >> 3, m = byte & 7u;
    uint32_t b = (byte << 4) + (232u << 7);                       // normal: exponent e - 7 + 112 + 127
    if (e == 0) b = f2bf((float)m * 0x1p103f);                    // subnormal: m * 2^-9 * 2^112
    return b | (b << 16);
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

struct Chunk { uint4 a, b; uint32_t sa, sb; };      // 32 codes of rows g and g + 8 and their two block scales each

// MODE 0: out[asg][row] = bf16(silu(a)), a = bf16(es * acc)          (up-projection; src row = asg / src_div)
// MODE 1: out[asg][row] = bf16(gate[asg] * (es * acc))               (down-projection; src row = asg)
template <int MODE>
__global__ void __launch_bounds__(kThreads, 4) fp4_rows_kernel(const Fp4RowsArgs p) {
    extern __shared__ __align__(16) uint8_t smem[];
    int* list = reinterpret_cast<int*>(smem);                         // assignments of this expert, ascending
    float* red = reinterpret_cast<float*>(smem + kDecodeMaxAsg * 4);  // [128][8] partial sums of the second k half
    const uint32_t stage = (uint32_t)__cvta_generic_to_shared(smem) + kDecodeMaxAsg * 4 + 128 * 8 * 4;
    __shared__ int s_cnt;
    __shared__ unsigned masks[kDecodeMaxAsg / 32];
    const int e = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, c = lane & 3;
    const int rgroup = warp & 3, ks = warp >> 2;
    const int kdim = p.kdim, nchunks = kdim >> 7;
    const int ch0 = ks * nchunks / kKSplit, ch1 = (ks + 1) * nchunks / kKSplit;
    const uint32_t rowb = (uint32_t)kdim * 2 + 64;                    // staged row pitch: +64 bytes keeps 8 lanes on 32 banks
    const int r0 = blockIdx.x * kRowsPerCta + rgroup * 16;
    const uint8_t* pa = p.packed[e] + (size_t)(r0 + g) * (kdim >> 1) + c * 16;
    const uint8_t* pb = pa + (size_t)8 * (kdim >> 1);
    const uint8_t* sa = p.scales[e] + (size_t)(r0 + g) * (kdim >> 4) + c * 2;
    const uint8_t* sb = sa + (size_t)8 * (kdim >> 4);
    auto load_chunk = [&](int j) {
        Chunk ck;
        ck.a = ldg16(pa + j * 64); ck.b = ldg16(pb + j * 64);
        ck.sa = __ldg(reinterpret_cast<const uint16_t*>(sa + j * 8));
        ck.sb = __ldg(reinterpret_cast<const uint16_t*>(sb + j * 8));
        return ck;
    };
    // the first weights travel while the token list is built and the rows are staged
    Chunk cur = load_chunk(ch0), nxt = cur;
    if (ch0 + 1 < ch1) nxt = load_chunk(ch0 + 1);

    // token list, ascending: warp w takes the 32-assignment slices w, w + 8, ...; one load latency in all
    for (int sl = warp; sl * 32 < p.n_asg; sl += kThreads / 32) {
        const int i = sl * 32 + lane;
        const unsigned m = __ballot_sync(0xffffffffu, i < p.n_asg && p.idx[i] == e);
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
    const int cnt = s_cnt;
    const float es = p.es[e];
    const int pieces_per_row = kdim >> 3;
    const int lanes_per_row = min(pieces_per_row, kThreads), rows_per_iter = kThreads / lanes_per_row;
    const int sub = threadIdx.x / lanes_per_row, v0 = threadIdx.x - sub * lanes_per_row;

    for (int pass = 0; pass * kNT < cnt; ++pass) {
        const int n_here = min(kNT, cnt - pass * kNT);
        const int ntiles = (n_here + 7) >> 3;
        if (pass > 0) __syncthreads();                                // everyone has left the previous rows
        // rows of the pass -> shared memory, permuted; kSB 16-byte loads in flight per thread
        for (int n0 = sub; n0 < ntiles * 8; n0 += kSB * rows_per_iter) {
            for (int v = v0; v < pieces_per_row; v += lanes_per_row) {
                uint4 x[kSB];
#pragma unroll
                for (int u = 0; u < kSB; ++u) {
                    const int n = n0 + u * rows_per_iter;
                    x[u] = make_uint4(0, 0, 0, 0);
                    if (n < n_here) x[u] = ldg16(p.src + (size_t)(list[pass * kNT + n] / p.src_div) * p.src_ld + v * 8);
                }
                const int j = v >> 4, r = v & 15;
#pragma unroll
                for (int u = 0; u < kSB; ++u) {
                    const int n = n0 + u * rows_per_iter;
                    if (n >= ntiles * 8) break;
                    uint4 o;
                    o.x = __byte_perm(x[u].x, x[u].z, 0x5410); o.y = __byte_perm(x[u].x, x[u].z, 0x7632);     // (k0,k4) (k1,k5)
                    o.z = __byte_perm(x[u].y, x[u].w, 0x5410); o.w = __byte_perm(x[u].y, x[u].w, 0x7632);     // (k2,k6) (k3,k7)
                    sts16u(stage + (uint32_t)n * rowb + (uint32_t)(j * 256 + (r & 3) * 64 + (r >> 2) * 16), o);
                }
            }
        }
        __syncthreads();

        float acc[2][4];
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[t][i] = 0.0f;
        if (pass > 0) { cur = load_chunk(ch0); nxt = ch0 + 1 < ch1 ? load_chunk(ch0 + 1) : cur; }
#pragma unroll 1
        for (int j = ch0; j < ch1; ++j) {
            Chunk fut = nxt;
            if (j + 2 < ch1) fut = load_chunk(j + 2);
            const uint32_t a_w[4] = {cur.a.x, cur.a.y, cur.a.z, cur.a.w}, b_w[4] = {cur.b.x, cur.b.y, cur.b.z, cur.b.w};
            const uint32_t sA[2] = {scale_bf2(cur.sa & 0xffu), scale_bf2(cur.sa >> 8)};
            const uint32_t sB[2] = {scale_bf2(cur.sb & 0xffu), scale_bf2(cur.sb >> 8)};
            const uint32_t bbase = stage + (uint32_t)g * rowb + (uint32_t)(j * 256 + c * 16);
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
                        const uint4 x = lds16u(bbase + (uint32_t)(t * 8) * rowb + (uint32_t)q * 64);
                        mma_bf16(acc[t], a00, a80, a01, a81, x.x, x.y);
                        mma_bf16(acc[t], a02, a82, a03, a83, x.z, x.w);
                    }
                }
            }
            cur = nxt; nxt = fut;
        }
        // the second k half hands its sums to the first
        if (ks == 1) {
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int i = 0; i < 4; ++i) red[(t * 4 + i) * 128 + rgroup * 32 + lane] = acc[t][i];
        }
        __syncthreads();
        if (ks == 0) {
#pragma unroll
            for (int t = 0; t < 2; ++t) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int n = t * 8 + c * 2 + (i & 1);
                    if (n >= n_here) continue;
                    const int asg = list[pass * kNT + n];
                    const int row = r0 + g + (i >> 1) * 8;
                    const float v = acc[t][i] + red[(t * 4 + i) * 128 + rgroup * 32 + lane];
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
}

// Y[t] = beta * Y[t] + sum_j Ya[t * K + j] in increasing j (the gate weight is already applied)
__global__ void __launch_bounds__(256) decode_combine_kernel(const uint16_t* __restrict__ Ya, uint16_t* __restrict__ Y, float beta,
                                                             int T, int D, int K) {
    const int nvec = D >> 3;
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
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

size_t rows_smem(int kdim) { return (size_t)kDecodeMaxAsg * 4 + 128 * 8 * 4 + (size_t)kNT * (kdim * 2 + 64); }

}  // namespace

cudaError_t launch_fp4_rows(const Fp4RowsArgs& a, int experts, int mode, cudaStream_t s) {
    const size_t smem = rows_smem(a.kdim);
    cudaError_t e = mode == 0
        ? cudaFuncSetAttribute(fp4_rows_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : cudaFuncSetAttribute(fp4_rows_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    const dim3 grid(a.rows / kRowsPerCta, experts);
    if (mode == 0) fp4_rows_kernel<0><<<grid, kThreads, smem, s>>>(a);
    else fp4_rows_kernel<1><<<grid, kThreads, smem, s>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_decode_combine(const uint16_t* Ya, uint16_t* Y, float beta, int T, int D, int K, cudaStream_t s) {
    const long n = (long)T * (D >> 3);
    decode_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(Ya, Y, beta, T, D, K);
    return cudaGetLastError();
}

bool fp4_rows_shape_ok(int rows, int kdim) {
    return rows % kRowsPerCta == 0 && kdim % 256 == 0 && rows_smem(kdim) <= 200 * 1024;
}

}  // namespace tmt
