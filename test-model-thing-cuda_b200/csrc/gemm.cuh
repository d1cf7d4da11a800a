// Grouped expert GEMM: parameters and the epilogues shared by the tcgen05 kernel and
// by the slow SIMT cross-check kernel.
//
// Two grouping modes.
//   kRowsRagged  C[r, n] = sum_k A[r, k] * W_e[n, k]  (or W_e[k, n]) for the rows r of expert
//                e's group in a grouped activation buffer; 128-row tiles, one expert each.
//                This is linear_fwd / linear_dX of tmt-cuda/src/linalg.cu:9-29 run once over
//                all experts instead of E cuBLAS calls (moe.cu:431-436, 538).
//   kRedRagged   C_e[m, n] = sum_{r in group e} A[r, m] * B[r, n]: the weight gradient,
//                linear_dW (linalg.cu:32-41, moe.cu:537); the reduction runs over the
//                group's rows. Zero rows give a zero gradient.
#pragma once
#include <cuda.h>
#include "common.cuh"

namespace tmt {

enum GemmMode : int { kRowsRagged = 0, kRedRagged = 1 };
enum Epilogue : int {
    kEpiBf16 = 0,   // out0 = bf16(acc)
    kEpiUp = 1,     // out0 = P = bf16(acc * expert_scale); out1 = bf16(silu(P))   (out0 may be NULL)
    kEpiDown = 2,   // out0 = bf16(row_scale[r] * expert_scale * acc)
    kEpiDh = 3,     // acc = dH*w: out0 = bf16(acc * silu'(P)); sw_part[r, col / kEpiCols] = sum acc * silu(P)
    kEpiF32 = 4,    // outF[e][m, n] = acc (fp32)
};

constexpr int kBM = 128;   // tile rows (UMMA M)
constexpr int kBN = 256;   // tile columns (UMMA N)
constexpr int kBK = 64;    // k per stage: 64 bf16 = one 128-byte swizzle span
constexpr int kChunk = 32; // columns one epilogue step handles per row
constexpr int kEpiCols = 128; // columns of a tile one epilogue warp drains; also the width of one gate-gradient partial

// Cycle counters one CTA of a tcgen05 kernel records when GemmParams::cyc is set.
enum CycSlot : int { kCycMmaWaitFull = 0, kCycMmaIssue, kCycMmaWaitAcc, kCycProdWaitEmpty, kCycProdIssue, kCycEpiWaitAcc, kCycEpiWork, kCycTotal, kCycSlots };

struct GemmParams {
    // tensor maps in device memory; map index = expert * stride (stride 0: one shared map)
    const CUtensorMap* mapA; int a_stride;
    const CUtensorMap* mapB; int b_stride;
    uint32_t tx_bytes;            // bytes one pipeline stage receives
    int a_boxes, b_boxes;         // mn-major operands: 64-wide blocks (8 KB each) one CTA stages per k block; their maps are the
                                  // 3-D views {64, k, block}, one box of a_boxes / b_boxes blocks per load
    // raw views of the same operands for the SIMT kernel
    const uint16_t* A; long lda;
    const uint16_t* B; long ldb;              // kRedRagged
    const uint16_t* const* Bexp;              // kRowsRagged: per-expert weights (device array)
    int mode, a_mn, b_mn;
    int M, N, K;                  // kRowsRagged: N, K static (M from the tile table); kRedRagged: M, N static
    int experts;
    const int* tile_expert;       // kRowsRagged: expert of each 128-row tile
    const int* num_m_tiles;       // kRowsRagged: number of 128-row tiles in use (device scalar)
    int tile_begin, tile_count;   // kRowsRagged: tile_count >= 0 restricts the launch to the 128-row tiles [tile_begin,
                                  // tile_begin + tile_count) (host values; whole 256-row pairs for the CTA-pair kernel)
    const int* poff;              // E+1 padded group starts
    // epilogue
    int epi;
    uint16_t* out0; uint16_t* out1; long ldc;
    float* const* outF;           // kEpiF32: per-expert output (device array of pointers)
    const float* row_scale;       // kEpiDown
    const float* expert_scale;    // optional per-expert factor (NVFP4 tensor scale), may be NULL
    const uint16_t* P;            // kEpiDh
    float* sw_part; int sw_ld;    // kEpiDh: per-row partial sums, one per kEpiCols columns
    // output tensor maps (device memory): with mapC0 set, the tcgen05 kernels stage every output chunk in
    // shared memory and write it with TMA stores; index = expert * c_stride. kEpiUp: mapC0 = SiLU output,
    // mapC1 = pre-activation (optional).
    const CUtensorMap* mapC0; const CUtensorMap* mapC1; int c_stride;
    int* status;
    long long* cyc;               // measurement only: 8 cycle counters per CTA (see kCyc*), NULL = off
    int dbg;                      // measurement only: bit 0 = no TMA loads (stale operands), bit 1 = no MMAs, bit 2 = no epilogue stores, bit 3 = epilogue stores straight from registers
};

// One row, kChunk consecutive columns starting at col0 (col0 % 8 == 0). Stores only
// columns < N in groups of 8. `sw` accumulates the gate-gradient partial of this row.
template <int EPI>
__device__ __forceinline__ void epilogue_chunk(const GemmParams& p, int e, long row, int col0,
                                               float (&v)[kChunk], float& sw) {
    if constexpr (EPI == kEpiF32) {
        float* dst = p.outF[e] + row * p.ldc + col0;
#pragma unroll
        for (int q = 0; q < kChunk / 4; ++q)
            if (col0 + q * 4 < p.N)
                *reinterpret_cast<float4*>(dst + q * 4) = make_float4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
        return;
    } else {
        const float es = p.expert_scale ? p.expert_scale[e] : 1.0f;
        if constexpr (EPI == kEpiDown) {
            const float rs = p.row_scale[row];
#pragma unroll
            for (int i = 0; i < kChunk; ++i) v[i] = rs * (es * v[i]);
        }
        if constexpr (EPI == kEpiUp) {
            uint16_t* dp = p.out0 ? p.out0 + row * p.ldc + col0 : nullptr;
            uint16_t* dh = p.out1 + row * p.ldc + col0;
#pragma unroll
            for (int q = 0; q < kChunk / 8; ++q) {
                if (col0 + q * 8 >= p.N) break;
                uint32_t pp[4], hh[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float a = round_bf(es * v[q * 8 + 2 * i]), b = round_bf(es * v[q * 8 + 2 * i + 1]);
                    pp[i] = pack_bf2(a, b);
                    hh[i] = pack_bf2(a * sigmoid_fast(a), b * sigmoid_fast(b));
                }
                if (dp) stg16(dp + q * 8, make_uint4(pp[0], pp[1], pp[2], pp[3]));
                stg16(dh + q * 8, make_uint4(hh[0], hh[1], hh[2], hh[3]));
            }
            return;
        }
        if constexpr (EPI == kEpiDh) {
            const uint16_t* pp = p.P + row * p.ldc + col0;
#pragma unroll
            for (int q = 0; q < kChunk / 8; ++q) {
                if (col0 + q * 8 >= p.N) break;
                uint4 pv = ldg16(pp + q * 8);
                uint32_t pw[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float x0 = bf_lo(pw[i]), x1 = bf_hi(pw[i]);
                    float s0 = sigmoid_fast(x0), s1 = sigmoid_fast(x1);
                    float a0 = v[q * 8 + 2 * i], a1 = v[q * 8 + 2 * i + 1];
                    sw += a0 * (x0 * s0);
                    sw += a1 * (x1 * s1);
                    v[q * 8 + 2 * i] = a0 * (s0 * (1.0f + x0 * (1.0f - s0)));
                    v[q * 8 + 2 * i + 1] = a1 * (s1 * (1.0f + x1 * (1.0f - s1)));
                }
            }
        }
        uint16_t* dst = p.out0 + row * p.ldc + col0;
#pragma unroll
        for (int q = 0; q < kChunk / 8; ++q) {
            if (col0 + q * 8 >= p.N) break;
            stg16(dst + q * 8, make_uint4(pack_bf2(v[q * 8], v[q * 8 + 1]), pack_bf2(v[q * 8 + 2], v[q * 8 + 3]),
                                          pack_bf2(v[q * 8 + 4], v[q * 8 + 5]), pack_bf2(v[q * 8 + 6], v[q * 8 + 7])));
        }
    }
}

// Launchers (gemm_tcgen05.cu / gemm_simt.cu). Both return the cudaError of the launch.
cudaError_t launch_gemm_tcgen05(const GemmParams& p, int num_sms, cudaStream_t stream);
cudaError_t launch_gemm_tcgen05_2cta(const GemmParams& p, int num_sms, cudaStream_t stream);
cudaError_t launch_gemm_simt(const GemmParams& p, int max_m_tiles, cudaStream_t stream);
size_t gemm_tcgen05_smem_bytes();
cudaError_t launch_bounded_wait_selftest(int* status, long long limit_cycles, int* reached_end, cudaStream_t stream);
size_t gemm_tcgen05_2cta_smem_bytes();

}  // namespace tmt
