// Epilogue of the tcgen05 grouped GEMM kernels, shared by the single-CTA and the CTA-pair kernel:
// one 128-row x 256-column accumulator in tensor memory -> registers -> epilogue math ->
// (shared-memory staging -> TMA store | per-thread-row global stores).
//
// Four warps form a group (one warp per 32-lane quarter of TMEM); kernels with eight epilogue
// warps run two groups, each draining 128 of the 256 columns. A group owns one or two staging
// buffers of 128 rows x 128 bytes, written in the 128-byte swizzle the output tensor maps expect.
#pragma once
#include "gemm.cuh"
#include "tc_util.cuh"

namespace tmt {

constexpr int kStagingBytes = 128 * 128;   // one staged output chunk: 128 rows x 128 bytes (64 bf16 or 32 fp32 columns)

struct EpiState {
    uint32_t cbuf;          // shared-memory address of the two staging buffers
    uint32_t gbar;          // this group's meeting barrier (count 4)
    uint32_t gphase = 0;
    int use = 0;
    int quarter, half, lane;
    bool issuer, staged;
    volatile int* abort_flag;
};

// Group-wide meeting point with the same bounded wait as everything else (a hardware named barrier
// could not be left if a warp of the group had given up).
__device__ __forceinline__ bool epi_group_sync(EpiState& s, int* status) {
    __syncwarp();
    if (s.lane == 0) tc::mbar_arrive(s.gbar);
    const bool ok = tc::mbar_wait(s.gbar, s.gphase, s.abort_flag, status);
    s.gphase ^= 1;
    return __all_sync(0xffffffffu, ok);
}

// Drains this warp's share of one tile. `tm` = TMEM address of (this warp's lane quarter, the tile's
// accumulator); `row0` = first output row of the 128-row tile this CTA owns. Returns false when a
// bounded wait ran out.
template <int EPI, int GROUPS>
__device__ __forceinline__ bool epi_drain_tile(const GemmParams& p, EpiState& s, int expert, int row0, int tcol0, int nkb,
                                               uint32_t tm, bool row_ok) {
    using namespace tc;
    if (p.dbg & 16) return true;           // measurement only: no epilogue work at all
    constexpr int kWarpCols = kBN / GROUPS;
    const int r_in_tile = s.quarter * 32 + s.lane;
    const long row = (long)row0 + r_in_tile;
    float sw = 0.0f;
    if (s.staged) {
        constexpr bool kF32 = EPI == kEpiF32;
        constexpr int kCols = kF32 ? 32 : 64;                 // columns per staged chunk: 128 bytes per row
        const bool two = EPI == kEpiUp && p.mapC1 != nullptr;
        const CUtensorMap* m0 = p.mapC0 + (size_t)expert * p.c_stride;
        const CUtensorMap* m1 = two ? p.mapC1 + (size_t)expert * p.c_stride : nullptr;
        const uint32_t rsw = (uint32_t)(r_in_tile & 7);
        const uint32_t rbase = (uint32_t)r_in_tile * 128u;
#pragma unroll 1
        for (int cc = s.half * (kWarpCols / kCols); cc < (s.half + 1) * (kWarpCols / kCols); ++cc) {
            const int ccol0 = tcol0 + cc * kCols;
            if (ccol0 >= p.N) break;
            // buffer choice: two outputs or two groups -> one buffer each, reused every chunk; else alternate
            constexpr bool single = (EPI == kEpiUp) || GROUPS == 2;
            const uint32_t b0 = s.cbuf + (uint32_t)((EPI == kEpiUp) ? 0 : (GROUPS == 2 ? s.half : (s.use & 1))) * kStagingBytes;
            const uint32_t b1 = s.cbuf + kStagingBytes;
            if (s.issuer) { if (single) bulk_wait_read<0>(); else bulk_wait_read<1>(); }
            if (!epi_group_sync(s, p.status)) return false;
            if constexpr (kF32) {
                float v[kChunk];
                if (nkb > 0) tmem_ld32(tm + (uint32_t)(cc * kCols), v);
                else {
#pragma unroll
                    for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
                }
#pragma unroll
                for (int q = 0; q < 8; ++q)
                    st_shared16(b0 + rbase + (((uint32_t)q ^ rsw) << 4), __float_as_uint(v[4 * q]), __float_as_uint(v[4 * q + 1]),
                                __float_as_uint(v[4 * q + 2]), __float_as_uint(v[4 * q + 3]));
            } else {
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const int col0 = ccol0 + sub * kChunk;
                    float v[kChunk];
                    uint32_t w0[kChunk / 2], w1[kChunk / 2];
                    if (nkb > 0) tmem_ld32(tm + (uint32_t)(cc * kCols + sub * kChunk), v);
                    else {
#pragma unroll
                        for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
                    }
                    if (col0 < p.N && row_ok) epilogue_math<EPI>(p, expert, row, col0, v, w0, w1, sw);
                    else {
#pragma unroll
                        for (int i = 0; i < kChunk / 2; ++i) { w0[i] = 0; w1[i] = 0; }
                    }
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t off = rbase + ((((uint32_t)(sub * 4 + q)) ^ rsw) << 4);
                        st_shared16(b0 + off, w0[4 * q], w0[4 * q + 1], w0[4 * q + 2], w0[4 * q + 3]);
                        if (two) st_shared16(b1 + off, w1[4 * q], w1[4 * q + 1], w1[4 * q + 2], w1[4 * q + 3]);
                    }
                }
            }
            fence_async_smem();
            if (!epi_group_sync(s, p.status)) return false;
            if (s.issuer && !(p.dbg & 4)) {
                tma_store_2d(m0, b0, ccol0, row0);
                if (two) tma_store_2d(m1, b1, ccol0, row0);
                bulk_commit();
            }
            ++s.use;
        }
    } else {
#pragma unroll 1
        for (int c = s.half * (kWarpCols / kChunk); c < (s.half + 1) * (kWarpCols / kChunk); ++c) {
            const int col0 = tcol0 + c * kChunk;
            if (col0 >= p.N) break;
            float v[kChunk];
            if (nkb > 0) {
                tmem_ld32(tm + (uint32_t)(c * kChunk), v);
            } else {
#pragma unroll
                for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
            }
            if (row_ok && !(p.dbg & 4)) epilogue_chunk<EPI>(p, expert, row, col0, v, sw);
        }
    }
    if (EPI == kEpiDh && row_ok && tcol0 + s.half * kEpiCols < p.N)
        p.sw_part[row * p.sw_ld + (tcol0 + s.half * kEpiCols) / kEpiCols] = sw;
    return true;
}

}  // namespace tmt
