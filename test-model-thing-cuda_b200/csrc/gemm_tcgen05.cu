// Grouped expert GEMM on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the
// accumulator in tensor memory, operands staged in shared memory by TMA (one destination CTA per load),
// persistent over 128x256 tiles.
//
// Warp roles (192 threads): warp 0 = TMA producer (one lane), warp 1 = TMEM allocator and
// MMA issuer (one lane), warps 2..5 = epilogue (each owns the 32 TMEM lanes warp_id % 4).
// Two 256-column accumulators in TMEM let the epilogue of tile i run under the MMAs of tile
// i+1. Every wait is bounded: when one runs out the kernel records kErrWaitTimeout, all
// roles leave their loops, the producer waits (bounded) for copies still in flight, TMEM is
// freed and the kernel returns.
#include "gemm.cuh"
#include "tc_util.cuh"

namespace tmt {
namespace {

constexpr int kStages = 4;
constexpr int kATile = kBM * kBK * 2;   // 16 KB
constexpr int kBTile = kBN * kBK * 2;   // 32 KB
constexpr int kStageBytes = kATile + kBTile;
// Epilogue warps per CTA: 4 (one per TMEM lane quarter, 256 columns each) or, for the epilogue that
// also reads the saved pre-activation (measured: that one is latency-bound), 8 (two per quarter, 128
// columns each). Threads = TMA warp + MMA warp + epilogue warps.
template <int EPI> __host__ __device__ constexpr int epi_warps() { return EPI == kEpiDh ? 8 : 4; }
template <int EPI> __host__ __device__ constexpr int block_threads() { return 64 + 32 * epi_warps<EPI>(); }
constexpr uint32_t kTmemCols = 512;     // two fp32 accumulators of 256 columns
constexpr int kStagingBytes = 128 * 128;  // one staged output chunk: 128 rows x 128 bytes (64 bf16 or 32 fp32 columns)

using namespace tc;

struct TileInfo {
    int expert, row0, col0, kb0, nkb;   // row0: output row (kRowsRagged) or m offset; kb0/nkb in 64-wide k blocks
};

__device__ __forceinline__ bool get_tile(const GemmParams& p, int t, int m_tiles, int n_tiles, TileInfo& ti) {
    if (p.mode == kRowsRagged) {
        if (t >= m_tiles * n_tiles) return false;
        int mt = t / n_tiles, nt = t - mt * n_tiles;
        ti.expert = p.tile_expert[mt];
        ti.row0 = mt * kBM;
        ti.col0 = nt * kBN;
        ti.kb0 = 0;
        ti.nkb = (p.K + kBK - 1) / kBK;
        return ti.expert >= 0 && ti.expert < p.experts;
    }
    int per = m_tiles * n_tiles;
    if (t >= per * p.experts) return false;
    int e = t / per, r = t - e * per;
    int mt = r / n_tiles, nt = r - mt * n_tiles;
    ti.expert = e;
    ti.row0 = mt * kBM;
    ti.col0 = nt * kBN;
    ti.kb0 = p.poff[e] / kBK;
    ti.nkb = (p.poff[e + 1] - p.poff[e]) / kBK;
    return true;
}

template <int EPI>
__global__ void __launch_bounds__(block_threads<EPI>(), 1) gemm_tcgen05_kernel(const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kStages], empty_bar[kStages], tfull_bar[2], tempty_bar[2], group_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tiles start on a 1024-byte boundary of the shared window (128-byte swizzle atoms)
    const uint32_t tiles_s = (smem_u32(smem_raw) + 1023u) & ~1023u;
    volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kStages; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        for (int a = 0; a < 2; ++a) mbar_init(smem_u32(&group_bar[a]), 4);      // 4 epilogue warps meet here
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 1 * epi_warps<EPI>()); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    int m_tiles, n_tiles = (p.N + kBN - 1) / kBN;
    if (p.mode == kRowsRagged) m_tiles = *p.num_m_tiles; else m_tiles = (p.M + kBM - 1) / kBM;

    if (warp == 0) {
        // ---------------- TMA producer: lane 0 owns the barriers, lanes 0..n-1 each issue one box ----------------
        // (a single thread issuing 6 boxes per k block was measured to be the slowest part of the launches with
        // mn-major operands)
        int s = 0; uint32_t ph = 0;
        uint32_t issued = 0;           // bit s set once stage s has received a load
        uint32_t last_parity = 0;      // parity of the last load issued into stage s
        bool ok = true;
        const int a_n = p.a_mn ? p.a_boxes : 1, b_n = p.b_mn ? p.b_boxes : 1;
        for (int t = blockIdx.x; ok; t += gridDim.x) {
            TileInfo ti;
            if (!get_tile(p, t, m_tiles, n_tiles, ti)) {
                if (lane == 0 && p.mode == kRowsRagged && t < m_tiles * n_tiles) report(p.status, kErrSlotRange);
                break;
            }
            const CUtensorMap* ma = p.mapA + (size_t)ti.expert * p.a_stride;
            const CUtensorMap* mb = p.mapB + (size_t)ti.expert * p.b_stride;
            if (lane == 0) { tensormap_acquire(ma); tensormap_acquire(mb); }
            __syncwarp();
            for (int kb = 0; kb < ti.nkb; ++kb) {
                const uint32_t fb = smem_u32(&full_bar[s]);
                if (lane == 0) {
                    ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status);
                    if (ok) mbar_expect_tx(fb, (p.dbg & 1) ? 0u : p.tx_bytes);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t sa = tiles_s + s * kStageBytes, sb = sa + kATile;
                const int k0 = (ti.kb0 + kb) * kBK;
                if (!(p.dbg & 1)) {
                    if (lane < a_n) {
                        if (p.a_mn) tma_load_2d(sa + lane * 8192, ma, fb, ti.row0 + lane * p.a_box_step, k0);   // 64 m x 64 k
                        else tma_load_2d(sa, ma, fb, k0, ti.row0);                                              // 64 k x 128 rows
                    } else if (lane < a_n + b_n) {
                        const int j = lane - a_n;
                        if (p.b_mn) tma_load_2d(sb + j * 8192, mb, fb, ti.col0 + j * p.b_box_step, k0);
                        else tma_load_2d(sb, mb, fb, k0, ti.col0);
                    }
                }
                __syncwarp();
                issued |= 1u << s;
                last_parity = (last_parity & ~(1u << s)) | (ph << s);
                if (++s == kStages) { s = 0; ph ^= 1; }
            }
        }
        if (!ok && lane == 0) {
            // aborting: wait (bounded, no abort short-cut) until the copies already issued have landed
            for (int q = 0; q < kStages; ++q) {
                if (!(issued >> q & 1)) continue;
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full_bar[q]), (last_parity >> q) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            // ---------------- MMA issuer ----------------
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn != 0) << 15) |
                                   ((uint32_t)(p.b_mn != 0) << 16) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
            const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4);   // descriptor units of 16 B per k = 16
            const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
            int s = 0; uint32_t ph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool ok = true;
            for (int t = blockIdx.x; ok; t += gridDim.x) {
                TileInfo ti;
                if (!get_tile(p, t, m_tiles, n_tiles, ti)) break;
                if (!mbar_wait(smem_u32(&tempty_bar[acc]), acc_ph ^ 1, abort_flag, p.status)) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int kb = 0; kb < ti.nkb; ++kb) {
                    if (!mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, p.status)) { ok = false; break; }
                    tc_fence_after();
                    const uint32_t sa = tiles_s + s * kStageBytes, sb = sa + kATile;
                    const uint64_t da = make_desc(sa, p.a_mn, 8192), db = make_desc(sb, p.b_mn, 8192);
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        if (!(p.dbg & 2)) tc_mma(d_tmem, da + (uint64_t)(k * a_kstep), db + (uint64_t)(k * b_kstep), idesc, (kb | k) != 0);
                    tc_commit(smem_u32(&empty_bar[s]));     // frees the stage once these MMAs have read it
                    if (++s == kStages) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                if (ti.nkb > 0) tc_commit(smem_u32(&tfull_bar[acc]));   // accumulator complete
                else mbar_arrive(smem_u32(&tfull_bar[acc]));            // empty group: nothing to wait for
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: TMEM -> registers -> (shared memory -> TMA store | global) ----------------
        const int quarter = warp & 3;           // TMEM lanes [32*quarter, 32*quarter+32)
        constexpr int kGroups = epi_warps<EPI>() / 4;                // 4 warps form a group with its own staging buffer(s)
        constexpr int kWarpCols = kBN / kGroups;                     // columns of the tile one group drains
        const int half = (warp - 2) >> 2;
        const bool staged = p.mapC0 != nullptr && !(p.dbg & 8);     // bit 3 of the measurement switches: per-thread-row global stores
        const bool issuer = ((warp - 2) & 3) == 0 && lane == 0;      // one thread per group issues the TMA stores
        const uint32_t cbuf = tiles_s + kStages * kStageBytes;       // two staging buffers of kStagingBytes
        const uint32_t gbar = smem_u32(&group_bar[half]);
        uint32_t gphase = 0;
        int use = 0;
        // group-wide meeting point with the same bounded wait as everything else (a hardware barrier could not
        // be left if a warp of the group had given up)
        auto group_sync = [&]() -> bool {
            __syncwarp();
            if (lane == 0) mbar_arrive(gbar);
            const bool ok = mbar_wait(gbar, gphase, abort_flag, p.status);
            gphase ^= 1;
            return __all_sync(0xffffffffu, ok);
        };
        int acc = 0; uint32_t acc_ph = 0;
        bool alive = true;
        for (int t = blockIdx.x; alive; t += gridDim.x) {
            TileInfo ti;
            if (!get_tile(p, t, m_tiles, n_tiles, ti)) break;
            bool ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_ph, abort_flag, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int r_in_tile = quarter * 32 + lane;
            const long row = (long)ti.row0 + r_in_tile;
            const bool row_ok = (p.mode == kRowsRagged) || (row < p.M);
            const uint32_t tm = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kBN);
            float sw = 0.0f;
            if (staged) {
                constexpr bool kF32 = EPI == kEpiF32;
                constexpr int kCols = kF32 ? 32 : 64;                 // columns per staged chunk: 128 bytes per row
                const bool two = EPI == kEpiUp && p.mapC1 != nullptr;
                const CUtensorMap* m0 = p.mapC0 + (size_t)ti.expert * p.c_stride;
                const CUtensorMap* m1 = two ? p.mapC1 + (size_t)ti.expert * p.c_stride : nullptr;
                const uint32_t rsw = (uint32_t)(r_in_tile & 7);
#pragma unroll 1
                for (int cc = half * (kWarpCols / kCols); cc < (half + 1) * (kWarpCols / kCols); ++cc) {
                    const int ccol0 = ti.col0 + cc * kCols;
                    if (ccol0 >= p.N) break;
                    // buffer choice: two outputs or two groups -> one buffer each, reused every chunk; else alternate
                    const bool single = (EPI == kEpiUp) || kGroups == 2;
                    const uint32_t b0 = cbuf + (uint32_t)((EPI == kEpiUp) ? 0 : (kGroups == 2 ? half : (use & 1))) * kStagingBytes;
                    const uint32_t b1 = cbuf + kStagingBytes;
                    if (issuer) { if (single) bulk_wait_read<0>(); else bulk_wait_read<1>(); }
                    if (!group_sync()) { alive = false; break; }
                    const uint32_t rbase = (uint32_t)r_in_tile * 128u;
                    if constexpr (kF32) {
                        float v[kChunk];
                        if (ti.nkb > 0) tmem_ld32(tm + (uint32_t)(cc * kCols), v);
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
                            if (ti.nkb > 0) tmem_ld32(tm + (uint32_t)(cc * kCols + sub * kChunk), v);
                            else {
#pragma unroll
                                for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
                            }
                            if (col0 < p.N && row_ok) epilogue_math<EPI>(p, ti.expert, row, col0, v, w0, w1, sw);
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
                    if (!group_sync()) { alive = false; break; }
                    if (issuer && !(p.dbg & 4)) {
                        tma_store_2d(m0, b0, ccol0, ti.row0);
                        if (two) tma_store_2d(m1, b1, ccol0, ti.row0);
                        bulk_commit();
                    }
                    ++use;
                }
                if (!alive) break;
            } else {
#pragma unroll 1
                for (int c = half * (kWarpCols / kChunk); c < (half + 1) * (kWarpCols / kChunk); ++c) {
                    const int col0 = ti.col0 + c * kChunk;
                    if (col0 >= p.N) break;
                    float v[kChunk];
                    if (ti.nkb > 0) {
                        tmem_ld32(tm + (uint32_t)(c * kChunk), v);
                    } else {
#pragma unroll
                        for (int i = 0; i < kChunk; ++i) v[i] = 0.0f;
                    }
                    if (row_ok && !(p.dbg & 4)) epilogue_chunk<EPI>(p, ti.expert, row, col0, v, sw);
                }
            }
            if (EPI == kEpiDh && row_ok && ti.col0 + half * kEpiCols < p.N) p.sw_part[row * p.sw_ld + (ti.col0 + half * kEpiCols) / kEpiCols] = sw;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (staged && issuer) bulk_wait_all();      // the shared-memory sources and the global writes of this CTA are done
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

template <int EPI>
cudaError_t launch_one(const GemmParams& p, int grid, cudaStream_t stream) {
    const size_t smem = gemm_tcgen05_smem_bytes();
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    gemm_tcgen05_kernel<EPI><<<grid, block_threads<EPI>(), smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

namespace {
// One block waits on a barrier nobody arrives on, with a short limit: exercises the time-out path of
// every bounded wait in the GEMM kernels (status word, abort flag, orderly return) without a real fault.
__global__ void bounded_wait_selftest_kernel(int* status, long long limit, int* reached_end) {
    __shared__ uint64_t bar;
    __shared__ int abort_s;
    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(smem_u32(&bar), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool ok = mbar_wait_limit(smem_u32(&bar), 0, &abort_s, status, limit);
    __syncthreads();
    if (threadIdx.x == 0) *reached_end = ok ? 2 : 1;
}
}  // namespace

cudaError_t launch_bounded_wait_selftest(int* status, long long limit_cycles, int* reached_end, cudaStream_t stream) {
    bounded_wait_selftest_kernel<<<1, 64, 0, stream>>>(status, limit_cycles, reached_end);
    return cudaGetLastError();
}

size_t gemm_tcgen05_smem_bytes() { return (size_t)kStages * kStageBytes + 2 * kStagingBytes + 1024; }

cudaError_t launch_gemm_tcgen05(const GemmParams& p, int num_sms, cudaStream_t stream) {
    // persistent: one CTA per SM (the shared-memory footprint allows no second one)
    switch (p.epi) {
        case kEpiBf16: return launch_one<kEpiBf16>(p, num_sms, stream);
        case kEpiUp: return launch_one<kEpiUp>(p, num_sms, stream);
        case kEpiDown: return launch_one<kEpiDown>(p, num_sms, stream);
        case kEpiDh: return launch_one<kEpiDh>(p, num_sms, stream);
        case kEpiF32: return launch_one<kEpiF32>(p, num_sms, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace tmt
