// Epilogue of the tcgen05 grouped GEMM kernels, shared by the single-CTA and the CTA-pair kernel:
// one 128-row x 256-column accumulator in tensor memory -> registers -> epilogue math ->
// (shared-memory staging -> TMA store | per-thread-row global stores).
//
// Four warps form a group (one warp per 32-lane quarter of TMEM). The bf16 epilogues run two groups,
// each draining 128 of the 256 columns through two 8 KB staging buffers (128 rows x 64 bytes, 64-byte
// swizzle); the fp32 epilogue runs one group with two 16 KB buffers (128 rows x 128 bytes, 128-byte
// swizzle). The swizzles are the ones the output tensor maps expect.
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

// The bf16 epilogues on 32 accumulator columns of one row: v -> packed bf16 words (w0: the main output, w1: the
// pre-activation of kEpiUp). `es` = expert scale, `rs` = row scale (kEpiDown), `pw` = 32 saved pre-activations of this
// row (kEpiDh), `sw` accumulates the gate-gradient partial in column order.
template <int EPI>
__device__ __forceinline__ void epi_math32(float (&v)[kChunk], float es, float rs, const uint4 (&pw)[4],
                                           uint32_t (&w0)[kChunk / 2], uint32_t (&w1)[kChunk / 2], float& sw) {
    if constexpr (EPI == kEpiDown) {
#pragma unroll
        for (int i = 0; i < kChunk; ++i) v[i] = rs * (es * v[i]);
    }
    if constexpr (EPI == kEpiUp) {
#pragma unroll
        for (int i = 0; i < kChunk / 2; ++i) {
            const float a = round_bf(es * v[2 * i]), b = round_bf(es * v[2 * i + 1]);
            w1[i] = pack_bf2(a, b);
            w0[i] = pack_bf2(a * sigmoid_fast(a), b * sigmoid_fast(b));
        }
        return;
    }
    if constexpr (EPI == kEpiDh) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t pq[4] = {pw[q].x, pw[q].y, pw[q].z, pw[q].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float x0 = bf_lo(pq[i]), x1 = bf_hi(pq[i]);
                const float s0 = sigmoid_fast(x0), s1 = sigmoid_fast(x1);
                const float a0 = v[q * 8 + 2 * i], a1 = v[q * 8 + 2 * i + 1];
                sw += a0 * (x0 * s0);
                sw += a1 * (x1 * s1);
                v[q * 8 + 2 * i] = a0 * (s0 * (1.0f + x0 * (1.0f - s0)));
                v[q * 8 + 2 * i + 1] = a1 * (s1 * (1.0f + x1 * (1.0f - s1)));
            }
        }
    }
    if constexpr (EPI != kEpiUp) {
#pragma unroll
        for (int i = 0; i < kChunk / 2; ++i) w0[i] = pack_bf2(v[2 * i], v[2 * i + 1]);
    }
}

// Staged bf16 epilogue: 8 warps in two groups, each group drains 128 of the tile's 256 columns in chunks of 32
// (64 bytes per row, 64-byte swizzle, one 8 KB TMA store per chunk and output). A group owns two 8 KB buffers:
// the two outputs of kEpiUp (single-buffered), or one output double-buffered. Returns false when a wait ran out.
template <int EPI>
__device__ __forceinline__ bool epi_drain_bf16(const GemmParams& p, EpiState& s, int expert, int row0, int tcol0, int nkb,
                                               uint32_t tm, bool row_ok, float& sw) {
    using namespace tc;
    constexpr int kCols = 32;
    const int r_in_tile = s.quarter * 32 + s.lane;
    const long row = (long)row0 + r_in_tile;
    const bool two = EPI == kEpiUp && p.mapC1 != nullptr;
    const CUtensorMap* m0 = p.mapC0 + (size_t)expert * p.c_stride;
    const CUtensorMap* m1 = two ? p.mapC1 + (size_t)expert * p.c_stride : nullptr;
    const uint32_t gbuf = s.cbuf + (uint32_t)s.half * kStagingBytes;
    const uint32_t rbase = (uint32_t)r_in_tile * 64u, rsw = (uint32_t)(r_in_tile >> 1) & 3u;
    const float es = p.expert_scale ? p.expert_scale[expert] : 1.0f;
    float rs = 1.0f;
    if constexpr (EPI == kEpiDown) rs = p.row_scale[row];
    const int c_first = tcol0 + s.half * kEpiCols;
    uint4 pw[4] = {};
    const uint16_t* prow = nullptr;
    if constexpr (EPI == kEpiDh) {
        prow = p.P + row * p.ldc;
        if (c_first < p.N) {
#pragma unroll
            for (int q = 0; q < 4; ++q) pw[q] = ldg16(prow + c_first + q * 8);
        }
    }
#pragma unroll 1
    for (int cc = 0; cc < kEpiCols / kCols; ++cc) {
        const int ccol0 = c_first + cc * kCols;
        if (ccol0 >= p.N) break;
        float v[kChunk];
        if (nkb > 0) tmem_ld32(tm + (uint32_t)(s.half * kEpiCols + cc * kCols), v);
        else {
#pragma unroll
            for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
        }
        uint32_t w0[kChunk / 2], w1[kChunk / 2];
        uint4 pnext[4] = {};
        if constexpr (EPI == kEpiDh) {       // the next chunk's saved pre-activations travel while this chunk is computed
            if (cc + 1 < kEpiCols / kCols && ccol0 + kCols < p.N) {
#pragma unroll
                for (int q = 0; q < 4; ++q) pnext[q] = ldg16(prow + ccol0 + kCols + q * 8);
            }
        }
        if (row_ok) epi_math32<EPI>(v, es, rs, pw, w0, w1, sw);
        else {
#pragma unroll
            for (int i = 0; i < kChunk / 2; ++i) { w0[i] = 0; w1[i] = 0; }
        }
        if constexpr (EPI == kEpiDh) {
#pragma unroll
            for (int q = 0; q < 4; ++q) pw[q] = pnext[q];
        }
        const uint32_t b0 = gbuf + (two ? 0u : (uint32_t)(s.use & 1) * (kStagingBytes / 2));
        const uint32_t b1 = gbuf + kStagingBytes / 2;
        if (two) {      // both buffers are reused every chunk: the previous pair of stores must have read them
            if (s.issuer) bulk_wait_read<0>();
            if (!epi_group_sync(s, p.status)) return false;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t off = rbase + (((uint32_t)q ^ rsw) << 4);
            st_shared16(b0 + off, w0[4 * q], w0[4 * q + 1], w0[4 * q + 2], w0[4 * q + 3]);
            if (two) st_shared16(b1 + off, w1[4 * q], w1[4 * q + 1], w1[4 * q + 2], w1[4 * q + 3]);
        }
        fence_async_smem();
        // double-buffered: the store of the previous chunk has read its buffer before anyone writes the next chunk there
        if (!two && s.issuer) bulk_wait_read<0>();
        if (!epi_group_sync(s, p.status)) return false;
        if (s.issuer && !TMT_DBG(p, 4)) {
            tma_store_2d(m0, b0, ccol0, row0);
            if (two) tma_store_2d(m1, b1, ccol0, row0);
            bulk_commit();
        }
        ++s.use;
    }
    return true;
}

// Drains this warp's share of one tile. `tm` = TMEM address of (this warp's lane quarter, the tile's
// accumulator); `row0` = first output row of the 128-row tile this CTA owns. Returns false when a
// bounded wait ran out.
template <int EPI, int GROUPS>
__device__ __forceinline__ bool epi_drain_tile(const GemmParams& p, EpiState& s, int expert, int row0, int tcol0, int nkb,
                                               uint32_t tm, bool row_ok) {
    using namespace tc;
    if (TMT_DBG(p, 16)) return true;           // measurement only: no epilogue work at all
    constexpr int kWarpCols = kBN / GROUPS;
    const int r_in_tile = s.quarter * 32 + s.lane;
    const long row = (long)row0 + r_in_tile;
    float sw = 0.0f;
    if (s.staged && EPI != kEpiF32) {
        if constexpr (EPI != kEpiF32) {
            static_assert(GROUPS == 2, "the staged bf16 epilogue runs with two groups of four warps");
            if (!epi_drain_bf16<EPI>(p, s, expert, row0, tcol0, nkb, tm, row_ok, sw)) return false;
        }
    } else if (s.staged) {
        // fp32 output (one group of four warps): 32-column chunks, 128 bytes per row, two 16 KB buffers in turn
        constexpr int kCols = 32;
        const CUtensorMap* m0 = p.mapC0 + (size_t)expert * p.c_stride;
        const uint32_t rsw = (uint32_t)(r_in_tile & 7);
        const uint32_t rbase = (uint32_t)r_in_tile * 128u;
#pragma unroll 1
        for (int cc = s.half * (kWarpCols / kCols); cc < (s.half + 1) * (kWarpCols / kCols); ++cc) {
            const int ccol0 = tcol0 + cc * kCols;
            if (ccol0 >= p.N) break;
            const uint32_t b0 = s.cbuf + (uint32_t)(s.use & 1) * kStagingBytes;
            if (s.issuer) bulk_wait_read<1>();         // the store that read this buffer two chunks ago is done
            if (!epi_group_sync(s, p.status)) return false;
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
            fence_async_smem();
            if (!epi_group_sync(s, p.status)) return false;
            if (s.issuer && !TMT_DBG(p, 4)) {
                tma_store_2d(m0, b0, ccol0, row0);
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
            if (row_ok && !TMT_DBG(p, 4)) epilogue_chunk<EPI>(p, expert, row, col0, v, sw);
        }
    }
    if (EPI == kEpiDh && row_ok && tcol0 + s.half * kEpiCols < p.N)
        p.sw_part[row * p.sw_ld + (tcol0 + s.half * kEpiCols) / kEpiCols] = sw;
    return true;
}

}  // namespace tmt
