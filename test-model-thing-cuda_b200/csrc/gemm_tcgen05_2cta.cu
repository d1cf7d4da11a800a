// Grouped expert GEMM with CTA-pair MMA (tcgen05 cta_group::2): two CTAs of a cluster work on
// one 256x256 tile. Each CTA stages its own 128 rows of A and HALF of the B tile (128 of the 256
// columns), the pair's tensor cores read both halves, so shared-memory traffic per flop drops by
// a third against the single-CTA kernel, whose 128x256 tiles are bound by shared-memory
// bandwidth (TMA fill + operand reads) rather than by the tensor pipe.
//
// Protocol. Both CTAs run two TMA producer warps (warp 0: even stages, last warp: odd stages; a TMA load
// instruction keeps its warp busy for about 300 cycles) for their own tiles and signal the LEADER's
// (cluster rank 0) "full" barrier; the leader's warp 1 issues the MMAs and commits to the
// "empty" and "accumulator full" barriers of BOTH CTAs; the
// epilogue warps of both CTAs drain their own 128 TMEM lanes and arrive on the leader's
// "accumulator empty" barrier. Every TMA load has exactly one destination CTA. Waits are bounded as in the single-CTA
// kernel; both CTAs always reach the closing cluster barrier before TMEM is freed.
//
// Pipeline stages are filled in PAIRS: one "full" barrier covers two consecutive stages, so the MMA
// warp waits once per 8 MMAs (a wait costs it 110-370 cycles, measured, and with one per 4 MMAs the
// issuing warp, not the tensor pipe, set the pace). Stages are released one by one: a single
// tcgen05.commit whose mask names both CTAs arrives on the stage's "empty" barrier in each of them. The epilogue is the shared
// one (staged in shared memory, written with TMA stores).
//
// Needs every group padded to 256 rows so that the two 128-row halves of a tile belong to one
// expert (the handle pads accordingly when this kernel is selected).
#include "gemm_epilogue.cuh"

namespace tmt {
namespace {

using namespace tc;

constexpr int kStages2 = 6;                     // three pairs
constexpr int kATile2 = kBM * kBK * 2;          // 16 KB: this CTA's 128 rows
constexpr int kBTile2 = (kBN / 2) * kBK * 2;    // 16 KB: this CTA's 128 of the 256 columns
constexpr int kStageBytes2 = kATile2 + kBTile2;
// Epilogue warps per CTA: 8 for the bf16 epilogues (two groups of four, one warp per TMEM lane quarter, 128 columns
// per group: TMEM load -> math -> staging is latency-bound, and with four warps it took longer than the MMAs of a
// K = 2048 tile), 4 for the fp32 one (its tiles have long reductions). Threads = TMA warp + MMA warp + epilogue
// warps + second TMA warp.
template <int EPI> __host__ __device__ constexpr int epi_warps() { return EPI == kEpiF32 ? 4 : 8; }
template <int EPI> __host__ __device__ constexpr int block_threads() { return 96 + 32 * epi_warps<EPI>(); }
constexpr uint32_t kTmemCols2 = 512;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t local_addr, uint32_t rank) {
    uint32_t a;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(local_addr), "r"(rank));
    return a;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA load into this CTA's shared memory, completion counted on a barrier that may live in the pair's leader.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at the same shared-memory offset in both CTAs of the pair once the MMAs issued so far are
// done (one instruction; the mask names both CTAs of the cluster).
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((uint16_t)3) : "memory");
}

struct Tile2 {
    int expert, row0, col0, kb0, nkb;
};

// t counts 256-row tiles; `rank` selects this CTA's 128-row half and its 128-column share of B.
__device__ __forceinline__ bool get_tile2(const GemmParams& p, int t, int m_pairs, int n_tiles, int rank, Tile2& ti) {
    if (p.mode == kRowsRagged) {
        if (t >= m_pairs * n_tiles) return false;
        const int mp = t / n_tiles, nt = t - mp * n_tiles;
        ti.expert = p.tile_expert[p.tile_begin + 2 * mp];
        ti.row0 = (p.tile_begin + 2 * mp) * kBM + rank * kBM;
        ti.col0 = nt * kBN;
        ti.kb0 = 0;
        ti.nkb = (p.K + kBK - 1) / kBK;
        return ti.expert >= 0 && ti.expert < p.experts;
    }
    const int per = m_pairs * n_tiles;
    if (t >= per * p.experts) return false;
    const int e = t / per, r = t - e * per;
    const int mp = r / n_tiles, nt = r - mp * n_tiles;
    ti.expert = e;
    ti.row0 = mp * 2 * kBM + rank * kBM;
    ti.col0 = nt * kBN;
    ti.kb0 = p.poff[e] / kBK;
    ti.nkb = (p.poff[e + 1] - p.poff[e]) / kBK;
    return true;
}

// The MMA thread's view of a tile: no expert lookup for row-ragged launches (a global load it would have to wait for).
__device__ __forceinline__ bool get_tile2_nkb(const GemmParams& p, int t, int m_pairs, int n_tiles, int& nkb) {
    if (p.mode == kRowsRagged) {
        nkb = (p.K + kBK - 1) / kBK;
        return t < m_pairs * n_tiles;
    }
    const int per = m_pairs * n_tiles;
    if (t >= per * p.experts) return false;
    const int e = t / per;
    nkb = (p.poff[e + 1] - p.poff[e]) / kBK;
    return true;
}

// Register cap: 128 per thread. An SM's register file is four partitions of 16384, one per warp scheduler, and a
// block's warps are dealt round over them: the 11 warps of an up / dH CTA put three into a partition. At the 152 / 168
// registers the compiler takes when left alone those three warps fill a partition (14592 / 16128), and no warp of another
// kernel fits beside the CTA, although a sixth of the file is free in total. At 128 they leave 4096 per partition: two
// more warps of 64 registers, which is what the expert-parallel step's row kernels for the later waves are shaped to
// (wave_rows_kernel, 256 threads x 64 registers, no shared memory). The cap costs nothing measurable: no spills, and
// the full-size step alone takes the same time with and without it (alternating runs on one GPU).
#ifndef TMT_GEMM_MAXNREG
#define TMT_GEMM_MAXNREG 128
#endif
#define TMT_GEMM_BOUNDS __maxnreg__(TMT_GEMM_MAXNREG)
template <int EPI>
__global__ void __cluster_dims__(2, 1, 1) TMT_GEMM_BOUNDS gemm_tcgen05_2cta_kernel(const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kStages2 / 2], empty_bar[kStages2], tfull_bar[2], tempty_bar[2], group_bar[2];
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int rank = (int)cluster_rank();
    const bool leader = rank == 0;
    const uint32_t tiles_s = (smem_u32(smem_raw) + 1023u) & ~1023u;
    volatile int* abort_flag = &abort_s;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kStages2 / 2; ++s) mbar_init(smem_u32(&full_bar[s]), 2);    // one leader arrival per stage of the pair
        for (int s = 0; s < kStages2; ++s) mbar_init(smem_u32(&empty_bar[s]), 1);
        for (int a = 0; a < 2; ++a) mbar_init(smem_u32(&group_bar[a]), 4);
        for (int a = 0; a < 2; ++a) { mbar_init(smem_u32(&tfull_bar[a]), 1); mbar_init(smem_u32(&tempty_bar[a]), 2 * epi_warps<EPI>()); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols2) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();            // both CTAs' barriers are initialised and both hold their TMEM
    tc_fence_after();
    const uint32_t tmem_base = tmem_base_s;

    const int n_tiles = (p.N + kBN - 1) / kBN;
    const int m_tiles_in_use = p.mode == kRowsRagged ? (p.tile_count >= 0 ? p.tile_count : *p.num_m_tiles) : 0;
    const int m_pairs = p.mode == kRowsRagged ? (m_tiles_in_use + 1) / 2 : (p.M + 2 * kBM - 1) / (2 * kBM);
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;

    if (warp == 0 || warp == 2 + epi_warps<EPI>()) {
        const int my = warp == 0 ? 0 : 1;
        // ---------------- TMA producers (both CTAs): lane 0 owns the barriers and loads A, lane 1 loads B ----------------
        int s = 0; uint32_t ph = 0;
        uint32_t issued = 0, last_parity = 0;
        bool ok = true;
        const bool prof = p.cyc != nullptr && my == 0;
        long long c_wait = 0, c_issue = 0, t0 = 0, t1 = 0;
        for (int t = pair; ok; t += npairs) {
            Tile2 ti;
            if (!get_tile2(p, t, m_pairs, n_tiles, rank, ti)) {
                if (lane == 0 && p.mode == kRowsRagged && t < m_pairs * n_tiles) { report(p.status, kErrSlotRange); *abort_flag = 1; }
                break;
            }
            const CUtensorMap* ma = p.mapA + (size_t)ti.expert * p.a_stride;
            const CUtensorMap* mb = p.mapB + (size_t)ti.expert * p.b_stride;
            if (lane == 0) { tensormap_acquire(ma); tensormap_acquire(mb); }
            __syncwarp();
            const int bcol0 = ti.col0 + rank * (kBN / 2);
            for (int kb = 0; kb < ti.nkb; ++kb) {
                if ((s & 1) != my) { if (++s == kStages2) { s = 0; ph ^= 1; } continue; }     // the other producer's stage
                const uint32_t fb_local = smem_u32(&full_bar[s >> 1]);
                const uint32_t fb = map_to_cta(fb_local, 0);              // the leader's barrier
                if (lane == 0) {
                    if (prof) t0 = clock64();
                    ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status);
                    if (prof) t1 = clock64();
                    if (ok && leader) mbar_expect_tx(fb_local, TMT_DBG(p, 1) ? 0u : 2 * p.tx_bytes);      // both CTAs' bytes
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                const uint32_t sa = tiles_s + s * kStageBytes2, sb = sa + kATile2;
                const int k0 = (ti.kb0 + kb) * kBK;
                if (!TMT_DBG(p, 1)) {
                    if (lane == 0) {
                        if (p.a_mn) tma_load_3d_pair(sa, ma, fb, 0, k0, ti.row0 >> 6);
                        else tma_load_2d_pair(sa, ma, fb, k0, ti.row0);
                    } else if (lane == 1) {
                        if (p.b_mn) tma_load_3d_pair(sb, mb, fb, 0, k0, bcol0 >> 6);
                        else tma_load_2d_pair(sb, mb, fb, k0, bcol0);
                    }
                }
                __syncwarp();
                if (prof && lane == 0) { c_wait += t1 - t0; c_issue += clock64() - t1; }
                issued |= 1u << (s >> 1);
                last_parity = (last_parity & ~(1u << (s >> 1))) | (ph << (s >> 1));
                if (++s == kStages2) { s = 0; ph ^= 1; }
            }
        }
        // An odd number of k blocks leaves the last pair's barrier one arrival short: the leader's odd producer supplies it,
        // after the same wait a real load of that stage would make (the barrier must have left its previous phase first).
        if (ok && leader && lane == 0 && (s & 1) && my == 1 && mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, p.status))
            mbar_expect_tx(smem_u32(&full_bar[s >> 1]), 0);
        if (prof && lane == 0) {
            p.cyc[blockIdx.x * kCycSlots + kCycProdWaitEmpty] = c_wait;
            p.cyc[blockIdx.x * kCycSlots + kCycProdIssue] = c_issue;
        }
        if (!ok && leader && lane == 0) {
            // aborting: the leader's barriers count both CTAs' copies; wait (bounded) for what was announced
            for (int q = 0; q < kStages2 / 2; ++q) {
                if (!(issued >> q & 1)) continue;
                const long long t0 = clock64();
                while (!mbar_try_wait(smem_u32(&full_bar[q]), (last_parity >> q) & 1) && clock64() - t0 < kWaitCycles) {}
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (leader) {
            // ---------------- MMA issuer (leader CTA only): the whole warp runs the loop, one elected lane issues ----------------
            const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn != 0) << 15) |
                                   ((uint32_t)(p.b_mn != 0) << 16) | ((uint32_t)(kBN >> 3) << 17) | ((uint32_t)((2 * kBM) >> 4) << 24);
            const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4);
            const uint32_t b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
            int s = 0; uint32_t ph = 0;
            int acc = 0; uint32_t acc_ph = 0;
            bool ok = true;
            const bool prof = p.cyc != nullptr;
            long long c_full = 0, c_issue = 0, c_acc = 0, t0 = 0, t1 = 0;
            const long long t_start = prof ? clock64() : 0;
            for (int t = pair; ok; t += npairs) {
                Tile2 ti;
                if (!get_tile2_nkb(p, t, m_pairs, n_tiles, ti.nkb)) break;
                if (prof) t0 = clock64();
                ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&tempty_bar[acc]), acc_ph ^ 1, abort_flag, p.status));
                if (!ok) break;
                if (prof) c_acc += clock64() - t0;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * kBN;
                for (int kb = 0; kb < ti.nkb; ++kb) {
                    if (prof) t0 = clock64();
                    if (!(s & 1) && !TMT_DBG(p, 64)) {          // both stages of the pair (s, s+1), in both CTAs, have landed once this barrier completes
                        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&full_bar[s >> 1]), ph, abort_flag, p.status));
                        if (!ok) break;
                        tc_fence_after();
                    }
                    if (prof) t1 = clock64();
                    const uint32_t sa = tiles_s + s * kStageBytes2, sb = sa + kATile2;
                    const uint64_t da = make_desc(sa, p.a_mn, 8192), db = make_desc(sb, p.b_mn, 8192);
                    if (elect_one()) {
#pragma unroll
                        for (int k = 0; k < kBK / 16; ++k)
                            if (!TMT_DBG(p, 2)) tc_mma_pair(d_tmem, da + (uint64_t)(k * a_kstep), db + (uint64_t)(k * b_kstep), idesc, (kb | k) != 0);
                        if (!TMT_DBG(p, 128)) tc_commit_pair(smem_u32(&empty_bar[s]));    // releases stage s in both CTAs
                    }
                    __syncwarp();
                    if (prof) { c_full += t1 - t0; c_issue += clock64() - t1; }
                    if (++s == kStages2) { s = 0; ph ^= 1; }
                }
                if (!ok) break;
                if (elect_one()) {
                    if (ti.nkb > 0) tc_commit_pair(smem_u32(&tfull_bar[acc]));
                    else {                       // empty group: nothing to wait for, release both epilogues
                        mbar_arrive(smem_u32(&tfull_bar[acc]));
                        mbar_arrive_cluster(map_to_cta(smem_u32(&tfull_bar[acc]), 1));
                    }
                }
                __syncwarp();
                if (++acc == 2) { acc = 0; acc_ph ^= 1; }
            }
            if (prof && lane == 0) {
                long long* c = p.cyc + blockIdx.x * kCycSlots;
                c[kCycMmaWaitFull] = c_full; c[kCycMmaIssue] = c_issue; c[kCycMmaWaitAcc] = c_acc; c[kCycTotal] = clock64() - t_start;
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (both CTAs): own 128 TMEM lanes ----------------
        constexpr int kGroups = epi_warps<EPI>() / 4;
        EpiState es;
        es.quarter = warp & 3;                  // TMEM lanes [32*quarter, 32*quarter+32)
        es.half = (warp - 2) >> 2;
        es.lane = lane;
        es.staged = p.mapC0 != nullptr && !TMT_DBG(p, 8);
        es.issuer = ((warp - 2) & 3) == 0 && lane == 0;
        es.cbuf = tiles_s + kStages2 * kStageBytes2;
        es.gbar = smem_u32(&group_bar[es.half]);
        es.abort_flag = abort_flag;
        const bool prof = p.cyc != nullptr && warp == 2 && lane == 0;
        long long c_wait = 0, c_work = 0, t0 = 0, t1 = 0;
        int acc = 0; uint32_t acc_ph = 0;
        for (int t = pair;; t += npairs) {
            Tile2 ti;
            if (!get_tile2(p, t, m_pairs, n_tiles, rank, ti)) break;
            if (prof) t0 = clock64();
            bool ok = true;
            if (!TMT_DBG(p, 32) || lane == 0) ok = mbar_wait(smem_u32(&tfull_bar[acc]), acc_ph, abort_flag, p.status);   // bit 5: one lane per warp waits
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            if (prof) t1 = clock64();
            tc_fence_after();
            const long row = (long)ti.row0 + es.quarter * 32 + lane;
            const bool row_ok = (p.mode == kRowsRagged) ? (row < (long)(p.tile_begin + m_tiles_in_use) * kBM) : (row < p.M);
            const uint32_t tm = tmem_base + ((uint32_t)(es.quarter * 32) << 16) + (uint32_t)(acc * kBN);
            if (!epi_drain_tile<EPI, kGroups>(p, es, ti.expert, ti.row0, ti.col0, ti.nkb, tm, row_ok)) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty_bar[acc]), 0));
            if (prof) { c_wait += t1 - t0; c_work += clock64() - t1; }
            if (++acc == 2) { acc = 0; acc_ph ^= 1; }
        }
        if (prof) { p.cyc[blockIdx.x * kCycSlots + kCycEpiWaitAcc] = c_wait; p.cyc[blockIdx.x * kCycSlots + kCycEpiWork] = c_work; }
        if (es.staged && es.issuer) bulk_wait_all();
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync();            // the peer may still be reading this CTA's shared memory or signalling its barriers
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols2) : "memory");
    }
}

template <int EPI>
cudaError_t launch_one(const GemmParams& p, int grid, cudaStream_t stream) {
    const size_t smem = gemm_tcgen05_2cta_smem_bytes();
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    gemm_tcgen05_2cta_kernel<EPI><<<grid, block_threads<EPI>(), smem, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

size_t gemm_tcgen05_2cta_smem_bytes() { return (size_t)kStages2 * kStageBytes2 + 2 * kStagingBytes + 1024; }

cudaError_t launch_gemm_tcgen05_2cta(const GemmParams& p, int num_sms, cudaStream_t stream) {
    const int grid = num_sms & ~1;      // whole CTA pairs
    switch (p.epi) {
        case kEpiBf16: return launch_one<kEpiBf16>(p, grid, stream);
        case kEpiUp: return launch_one<kEpiUp>(p, grid, stream);
        case kEpiDown: return launch_one<kEpiDown>(p, grid, stream);
        case kEpiDh: return launch_one<kEpiDh>(p, grid, stream);
        case kEpiF32: return launch_one<kEpiF32>(p, grid, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace tmt
