// Grouped expert GEMM on the 5th-generation tensor cores (sm_100a): tcgen05.mma with the
// accumulator in tensor memory, operands staged in shared memory by TMA (one destination CTA per load),
// persistent over 128x256 tiles.
//
// Warp roles: warp 0 and the last warp = TMA producers (even / odd pipeline stages), warp 1 = TMEM
// allocator and MMA issuer (the whole warp runs the loop, one elected lane issues), warps 2..5 (2..9) = epilogue (each owns the 32 TMEM lanes
// warp_id % 4). Two producers because a TMA load instruction keeps its warp busy for about 300
// cycles (measured), so one warp could not start a 48 KB stage every 512 cycles.
// Two 256-column accumulators in TMEM let the epilogue of tile i run under the MMAs of tile
// i+1. Two consecutive pipeline stages share one "full" barrier (two producer arrivals), so the
// MMA thread waits once per 8 MMAs: measured on a B200, any shared-memory read by the thread that
// issues tcgen05.mma costs it about 370 cycles, and with one wait per 4 MMAs (512 tensor-pipe
// cycles) the thread, not the pipe, set the pace (640 cycles per k block). Stages are still
// released one by one (tcgen05.commit is cheap). Every wait is bounded: when one runs out the kernel records kErrWaitTimeout, all
// roles leave their loops, the producer waits (bounded) for copies still in flight, TMEM is
// freed and the kernel returns.
#include "gemm_epilogue.cuh"

namespace tmt {
namespace {

constexpr int kStages = 4;
constexpr int kATile = kBM * kBK * 2;   // 16 KB
constexpr int kBTile = kBN * kBK * 2;   // 32 KB
constexpr int kStageBytes = kATile + kBTile;
// Epilogue warps per CTA: 8 for the bf16 epilogues (two groups of four, one warp per TMEM lane quarter, 128 columns
// per group: TMEM load -> math -> staging is latency-bound, and with four warps it took longer than the MMAs of a
// K = 2048 tile), 4 for the fp32 one (its tiles have long reductions). Threads = TMA warp + MMA warp + epilogue
// warps + second TMA warp.
template <int EPI> __host__ __device__ constexpr int epi_warps() { return EPI == kEpiF32 ? 4 : 8; }
template <int EPI> __host__ __device__ constexpr int block_threads() { return 96 + 32 * epi_warps<EPI>(); }
constexpr uint32_t kTmemCols = 512;     // two fp32 accumulators of 256 columns

using namespace tc;

struct TileInfo {
    int expert, row0, col0, kb0, nkb;   // row0: output row (kRowsRagged) or m offset; kb0/nkb in 64-wide k blocks
};

__device__ __forceinline__ bool get_tile(const GemmParams& p, int t, int m_tiles, int n_tiles, TileInfo& ti) {
    if (p.mode == kRowsRagged) {
        if (t >= m_tiles * n_tiles) return false;
        int mt = t / n_tiles, nt = t - mt * n_tiles;
        mt += p.tile_begin;
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

// The MMA thread's view of a tile: no expert lookup for row-ragged launches (a global load it would have to wait for).
__device__ __forceinline__ bool get_tile_nkb(const GemmParams& p, int t, int m_tiles, int n_tiles, int& nkb) {
    if (p.mode == kRowsRagged) {
        nkb = (p.K + kBK - 1) / kBK;
        return t < m_tiles * n_tiles;
    }
    const int per = m_tiles * n_tiles;
    if (t >= per * p.experts) return false;
    const int e = t / per;
    nkb = (p.poff[e + 1] - p.poff[e]) / kBK;
    return true;
}

template <int EPI>
__global__ void __launch_bounds__(block_threads<EPI>(), 1) gemm_tcgen05_kernel(const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kStages / 2], empty_bar[kStages], tfull_bar[2], tempty_bar[2], group_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tiles start on a 1024-byte boundary of the shared window (128-byte swizzle atoms)
    const uint32_t tiles_s = (smem_u32(smem_raw) + 1023u) & ~1023u;
    volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&empty_bar[s]), 1);
        for (int s = 0; s < kStages / 2; ++s) mbar_init(smem_u32(&full_bar[s]), 2);   // one producer arrival per stage of the pair
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
    if (p.mode == kRowsRagged) m_tiles = p.tile_count >= 0 ? p.tile_count : *p.num_m_tiles; else m_tiles = (p.M + kBM - 1) / kBM;

    if (warp == 0 || warp == 2 + epi_warps<EPI>()) {
        // ---------------- TMA producers: warp 0 fills the even stages, the last warp the odd ones; lane 0 owns the
        // barriers and loads A, lane 1 loads B ----------------
        const int my = warp == 0 ? 0 : 1;
        // (one box per operand and k block; six 8 KB boxes per k block were measured to be the slowest part of
        // the launches with mn-major operands)
        int s = 0; uint32_t ph = 0;
        uint32_t issued = 0;           // bit q set once stage pair q has received a load
        uint32_t last_parity = 0;      // parity of the last load issued into pair q
        bool ok = true;
        const bool prof = p.cyc != nullptr && my == 0;
        long long c_wait = 0, c_issue = 0, t0 = 0, t1 = 0;
        for (int t = blockIdx.x; ok; t += gridDim.x) {
            TileInfo ti;
            if (!get_tile(p, t, m_tiles, n_tiles, ti)) {
                if (lane == 0 && p.mode == kRowsRagged && t < m_tiles * n_tiles) { report(p.status, kErrSlotRange); *abort_flag = 1; }
                break;
            }
            const CUtensorMap* ma = p.mapA + (size_t)ti.expert * p.a_stride;
            const CUtensorMap* mb = p.mapB + (size_t)ti.expert * p.b_stride;
            if (lane == 0) { tensormap_acquire(ma); tensormap_acquire(mb); }
            __syncwarp();
            for (int kb = 0; kb < ti.nkb; ++kb) {
                if ((s & 1) != my) { if (++s == kStages) { s = 0; ph ^= 1; } continue; }      // the other producer's stage
                const uint32_t fb = smem_u32(&full_bar[s >> 1]);
                if (lane == 0) {
                    if (prof) t0 = clock64();
                    ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status);
                    if (prof) t1 = clock64();
                    if (ok) mbar_expect_tx(fb, TMT_DBG(p, 1) ? 0u : p.tx_bytes);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t sa = tiles_s + s * kStageBytes, sb = sa + kATile;
                const int k0 = (ti.kb0 + kb) * kBK;
                if (!TMT_DBG(p, 1)) {
                    if (lane == 0) {
                        if (p.a_mn) tma_load_3d(sa, ma, fb, 0, k0, ti.row0 >> 6);        // 2 blocks of 64 m x 64 k
                        else tma_load_2d(sa, ma, fb, k0, ti.row0);                       // 64 k x 128 rows
                    } else if (lane == 1) {
                        if (p.b_mn) tma_load_3d(sb, mb, fb, 0, k0, ti.col0 >> 6);        // 4 blocks of 64 n x 64 k
                        else tma_load_2d(sb, mb, fb, k0, ti.col0);
                    }
                }
                __syncwarp();
                if (prof && lane == 0) { c_wait += t1 - t0; c_issue += clock64() - t1; }
                issued |= 1u << (s >> 1);
                last_parity = (last_parity & ~(1u << (s >> 1))) | (ph << (s >> 1));
                if (++s == kStages) { s = 0; ph ^= 1; }
            }
        }
        // An odd number of k blocks leaves the last pair's barrier one arrival short: the odd producer supplies it, after
        // the same wait a real load of that stage would make (the barrier must have left its previous phase first).
        if (ok && lane == 0 && (s & 1) && my == 1 && mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status))
            mbar_expect_tx(smem_u32(&full_bar[s >> 1]), 0);
        if (prof && lane == 0) {
            p.cyc[blockIdx.x * kCycSlots + kCycProdWaitEmpty] = c_wait;
            p.cyc[blockIdx.x * kCycSlots + kCycProdIssue] = c_issue;
        }
        if (!ok && lane == 0) {
            // aborting: wait (bounded, no abort short-cut) until the copies already issued have landed
            for (int q = 0; q < kStages / 2; ++q) {
                if (!(issued >> q & 1)) continue;
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full_bar[q]), (last_parity >> q) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp runs the loop and one elected lane issues: with uniform control flow the descriptors and
        // barrier addresses stay in uniform registers, and a barrier wait costs the warp about 110 cycles; the same
        // loop run by a single lane inside a divergent branch was measured at about 370 cycles per wait.
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn != 0) << 15) |
                               ((uint32_t)(p.b_mn != 0) << 16) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
        const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4);   // descriptor units of 16 B per k = 16
        const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
        int s = 0; uint32_t ph = 0;
        int acc = 0; uint32_t acc_ph = 0;
        bool ok = true;
        const bool prof = p.cyc != nullptr;
        long long c_full = 0, c_issue = 0, c_acc = 0, t0 = 0, t1 = 0;
        const long long t_start = prof ? clock64() : 0;
        for (int t = blockIdx.x; ok; t += gridDim.x) {
            TileInfo ti;
            if (!get_tile_nkb(p, t, m_tiles, n_tiles, ti.nkb)) break;
            if (prof) t0 = clock64();
            ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&tempty_bar[acc]), acc_ph ^ 1, abort_flag, p.status));
            if (!ok) break;
            if (prof) c_acc += clock64() - t0;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * kBN;
            for (int kb = 0; kb < ti.nkb; ++kb) {
                if (prof) t0 = clock64();
                if (!(s & 1) && !TMT_DBG(p, 64)) {          // both stages of the pair (s, s+1) have landed once this barrier completes
                    ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s >> 1]), ph, abort_flag, p.status));
                    if (!ok) break;
                    tc_fence_after();
                }
                if (prof) t1 = clock64();
                const uint32_t sa = tiles_s + s * kStageBytes, sb = sa + kATile;
                const uint64_t da = make_desc(sa, p.a_mn, 8192), db = make_desc(sb, p.b_mn, 8192);
                if (elect_one()) {
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k)
                        if (!TMT_DBG(p, 2)) tc_mma(d_tmem, da + (uint64_t)(k * a_kstep), db + (uint64_t)(k * b_kstep), idesc, (kb | k) != 0);
                    if (!TMT_DBG(p, 128)) tc_commit(smem_u32(&empty_bar[s]));     // frees the stage once these MMAs have read it
                }
                __syncwarp();
                if (prof) { c_full += t1 - t0; c_issue += clock64() - t1; }
                if (++s == kStages) { s = 0; ph ^= 1; }
            }
            if (!ok) break;
            if (elect_one()) {
                if (ti.nkb > 0) tc_commit(smem_u32(&tfull_bar[acc]));   // accumulator complete
                else mbar_arrive(smem_u32(&tfull_bar[acc]));            // empty group: nothing to wait for
            }
            __syncwarp();
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (prof && lane == 0) {
            long long* c = p.cyc + blockIdx.x * kCycSlots;
            c[kCycMmaWaitFull] = c_full; c[kCycMmaIssue] = c_issue; c[kCycMmaWaitAcc] = c_acc; c[kCycTotal] = clock64() - t_start;
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: TMEM -> registers -> (shared memory -> TMA store | global) ----------------
        constexpr int kGroups = epi_warps<EPI>() / 4;                // 4 warps form a group with its own staging buffer(s)
        EpiState es;
        es.quarter = warp & 3;                  // TMEM lanes [32*quarter, 32*quarter+32)
        es.half = (warp - 2) >> 2;
        es.lane = lane;
        es.staged = p.mapC0 != nullptr && !TMT_DBG(p, 8);     // bit 3 of the measurement switches: per-thread-row global stores
        es.issuer = ((warp - 2) & 3) == 0 && lane == 0;     // one thread per group issues the TMA stores
        es.cbuf = tiles_s + kStages * kStageBytes;          // two staging buffers of kStagingBytes
        es.gbar = smem_u32(&group_bar[es.half]);
        es.abort_flag = abort_flag;
        const bool staged = es.staged, issuer = es.issuer;
        int acc = 0; uint32_t acc_ph = 0;
        const bool prof = p.cyc != nullptr && warp == 2 && lane == 0;
        long long c_wait = 0, c_work = 0, t0 = 0, t1 = 0;
        for (int t = blockIdx.x;; t += gridDim.x) {
            TileInfo ti;
            if (!get_tile(p, t, m_tiles, n_tiles, ti)) break;
            if (prof) t0 = clock64();
            bool ok = true;
            if (!TMT_DBG(p, 32) || lane == 0) ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_ph, abort_flag, p.status);   // bit 5: one lane per warp waits
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (prof) t1 = clock64();
            tc_fence_after();
            const bool row_ok = (p.mode == kRowsRagged) || ((long)ti.row0 + es.quarter * 32 + lane < p.M);
            const uint32_t tm = tmem_base + ((uint32_t)(es.quarter * 32) << 16) + (uint32_t)(acc * kBN);
            if (!epi_drain_tile<EPI, kGroups>(p, es, ti.expert, ti.row0, ti.col0, ti.nkb, tm, row_ok)) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&tempty_bar[acc]));
            if (prof) { c_wait += t1 - t0; c_work += clock64() - t1; }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (prof) { p.cyc[blockIdx.x * kCycSlots + kCycEpiWaitAcc] = c_wait; p.cyc[blockIdx.x * kCycSlots + kCycEpiWork] = c_work; }
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
