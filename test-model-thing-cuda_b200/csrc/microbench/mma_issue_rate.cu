// Micro-benchmark (measurement only, not part of the library): what the thread that issues tcgen05.mma pays for
// the instructions around it. One CTA per SM, operands resident in shared memory, no loads. Variants: MMAs back
// to back with different tcgen05.commit policies (1-CTA and CTA-pair, N = 32 makes everything issue-bound); a
// producer thread that only hands barriers back and forth (the pipeline hand-shake without data), with the MMA
// loop run by ONE LANE inside a divergent branch or by the WHOLE WARP with an elected lane; barrier waits per 4 or
// per 8 MMAs; a long run that shows the clock, not the cycle count per MMA, dropping under the power cap.
// Every wait is bounded (status word), nothing here can hang.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I.. -o mma_issue_rate mma_issue_rate.cu -lcuda && ./mma_issue_rate
//
// Numbers measured on a B200 are in profiles/gemm_tcgen05_config5_32k_tokens.md.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include "tc_util.cuh"
using namespace tmt;
using namespace tmt::tc;

__device__ __forceinline__ uint32_t cl_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t mapa(uint32_t a, uint32_t r) { uint32_t o; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(o) : "r"(a), "r"(r)); return o; }
__device__ __forceinline__ void cl_sync() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
__device__ __forceinline__ void mma2(uint32_t d, uint64_t a, uint64_t b, uint32_t id, uint32_t acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d), "l"(a), "l"(b), "r"(id), "r"(acc) : "memory");
}
__device__ __forceinline__ void commit2(uint32_t bar) { asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory"); }

__device__ __forceinline__ void commit2m(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar), "h"((uint16_t)3) : "memory");
}
struct P { int rnd; int nkb, commit_every, N, a_mn, b_mn, stages, stage_bytes, a_bytes, same_acc, ncommit; long long* out; int* status; };

template <int PAIR>
__global__ void __launch_bounds__(128, 1) k(P p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t bar_end, bar_mid;
    __shared__ uint32_t tmem_s;
    __shared__ int abort_s;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int rank = PAIR ? (int)cl_rank() : 0;
    // fill the operand area with small bf16 values
    for (int i = threadIdx.x; i < p.stages * p.stage_bytes / 4; i += blockDim.x)
    {
        uint32_t v = 0x3c003c00u + (uint32_t)(i & 7) * 0x00010001u;
        if (p.rnd) {   // random bf16 pairs in about [-2, 2]
            uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u; h ^= h >> 15; h *= 2246822519u; h ^= h >> 13;
            v = (h & 0x807f807fu) | 0x3f803f80u ^ ((h >> 3) & 0x00800080u);
        }
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + i * 4), "r"(v));
    }
    if (threadIdx.x == 0) {
        abort_s = 0;
        mbar_init(smem_u32(&bar_end), 1);
        mbar_init(smem_u32(&bar_mid), 1 << 19);     // never completes: nobody waits on it
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        if (PAIR) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_s)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_s)), "r"(512u) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cl_sync();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    long long t_issue = 0, t_total = 0;
    if (threadIdx.x == 32 && rank == 0) {
        const int M = PAIR ? 256 : 128;
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.a_mn != 0) << 15) | ((uint32_t)(p.b_mn != 0) << 16) |
                               ((uint32_t)(p.N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
        const uint32_t a_kstep = p.a_mn ? (2048u >> 4) : (32u >> 4), b_kstep = p.b_mn ? (2048u >> 4) : (32u >> 4);
        const long long t0 = clock64();
        int s = 0;
        for (int kb = 0; kb < p.nkb; ++kb) {
            const uint32_t sa = base + s * p.stage_bytes, sb = sa + p.a_bytes;
            const uint64_t da = make_desc(sa, p.a_mn, 8192), db = make_desc(sb, p.b_mn, 8192);
            const uint32_t d = tmem + (p.same_acc ? 0 : ((kb >> 5) & 1) * 256);
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
                if (PAIR) mma2(d, da + (uint64_t)(k4 * a_kstep), db + (uint64_t)(k4 * b_kstep), idesc, (kb & 31) | k4);
                else tc_mma(d, da + (uint64_t)(k4 * a_kstep), db + (uint64_t)(k4 * b_kstep), idesc, (kb & 31) | k4);
            }
            if (p.commit_every > 0 && (kb + 1) % p.commit_every == 0) {
                for (int c = 0; c < p.ncommit; ++c) {
                    if (PAIR == 3) commit2m(smem_u32(&bar_mid));
                    else if (PAIR) { commit2(smem_u32(&bar_mid)); if (PAIR == 2) commit2(mapa(smem_u32(&bar_mid), 1)); }
                    else tc_commit(smem_u32(&bar_mid));
                }
            }
            if (++s == p.stages) s = 0;
        }
        if (PAIR) { commit2(smem_u32(&bar_end)); commit2(mapa(smem_u32(&bar_end), 1)); }
        else tc_commit(smem_u32(&bar_end));
        t_issue = clock64() - t0;
        mbar_wait(smem_u32(&bar_end), 0, &abort_s, p.status);
        t_total = clock64() - t0;
        p.out[blockIdx.x * 2] = t_issue;
        p.out[blockIdx.x * 2 + 1] = t_total;
    } else if (threadIdx.x == 32) {
        mbar_wait(smem_u32(&bar_end), 0, &abort_s, p.status);
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cl_sync();
    if (threadIdx.x < 32) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

template <int PAIR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(128, 1) k2(P p);



__device__ __forceinline__ uint32_t test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ uint32_t try_wait_relaxed(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.relaxed.cta.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ void wait_loop_ptx(uint32_t bar, uint32_t parity) {
    asm volatile("{\n\t.reg .pred p;\n\tWAIT_LOOP:\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n\t@p bra WAIT_DONE;\n\tbra WAIT_LOOP;\n\tWAIT_DONE:\n\t}" ::"r"(bar), "r"(parity) : "memory");
}
// bounded spin for the scratch variants (about 2 s)
template <int KIND>
__device__ __forceinline__ bool wait_kind(uint32_t bar, uint32_t parity) {
    const long long t0 = clock64();
    for (;;) {
        uint32_t ok = KIND == 1 ? test_wait(bar, parity) : try_wait_relaxed(bar, parity);
        if (ok) return true;
        if (clock64() - t0 > 4000000000LL) return false;
    }
}
struct H { int nkb, stages, fence, stage_bytes, a_bytes, lockstep, N; long long* out; int* status; };
// MMA thread + producer thread hand-shake without loads: producer waits empty[s], arms full[s]; MMA thread waits full[s],
// issues 4 MMAs, commits to empty[s].
__global__ void __launch_bounds__(128, 1) hk(H p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[16], empty_bar[16], bar_end;
    __shared__ uint32_t tmem_s;
    __shared__ int abort_s;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    for (int i = threadIdx.x; i < 4 * 49152 / 4; i += blockDim.x)
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + i * 4), "r"(0x3c003c00u + (uint32_t)(i & 7) * 0x00010001u));
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < 16; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        mbar_init(smem_u32(&bar_end), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    if (threadIdx.x == 64) {          // producer
        int s = 0; uint32_t ph = 0;
        const int n = p.lockstep == 5 ? p.nkb / 2 : (p.lockstep == 7 ? p.nkb / 3 * 3 : p.nkb);
        for (int kb = 0; kb < n; ++kb) {
            if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, &abort_s, p.status)) break;
            mbar_expect_tx(smem_u32(&full_bar[s]), 0);
            if (++s == p.stages) { s = 0; ph ^= 1; }
        }
    } else if (threadIdx.x == 32) {   // MMA
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        long long w = 0;
        const long long t0 = clock64();
        int s = 0; uint32_t ph = 0;
        const int mode = p.lockstep;
        if (mode <= 1) {
            for (int kb = 0; kb < p.nkb; ++kb) {
                long long a = 0;
                if (mode) a = clock64();
                if (!mbar_wait(smem_u32(&full_bar[s]), ph, &abort_s, p.status)) break;
                if (mode) w += clock64() - a;
                if (p.fence) tc_fence_after();
                const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((kb >> 5) & 1) * 256;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 31) | k4);
                tc_commit(smem_u32(&empty_bar[s]));
                if (++s == p.stages) { s = 0; ph ^= 1; }
            }
        } else if (mode == 2 || mode == 3) {
            // probe the NEXT stage's barrier between the MMAs of the current one (mode 2: after 2 MMAs, mode 3: before the first)
            bool ok = mbar_wait(smem_u32(&full_bar[0]), 0, &abort_s, p.status);
            for (int kb = 0; kb < p.nkb && ok; ++kb) {
                if (p.fence) tc_fence_after();
                const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((kb >> 5) & 1) * 256;
                int sn = s + 1; uint32_t phn = ph;
                if (sn == p.stages) { sn = 0; phn ^= 1; }
                uint32_t ready = 0;
                if (mode == 3) ready = mbar_try_wait(smem_u32(&full_bar[sn]), phn);
                tc_mma(d, da, db, idesc, (kb & 31) | 0);
                tc_mma(d, da + 2, db + 2, idesc, 1);
                if (mode == 2) ready = mbar_try_wait(smem_u32(&full_bar[sn]), phn);
                tc_mma(d, da + 4, db + 4, idesc, 1);
                tc_mma(d, da + 6, db + 6, idesc, 1);
                tc_commit(smem_u32(&empty_bar[s]));
                if (!ready && kb + 1 < p.nkb) ok = mbar_wait(smem_u32(&full_bar[sn]), phn, &abort_s, p.status);
                s = sn; ph = phn;
            }
        } else if (mode == 4) {
            // no wait at all on full; commits rotate over the per-stage barriers (producer still running and arming)
            for (int kb = 0; kb < p.nkb; ++kb) {
                const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((kb >> 5) & 1) * 256;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 31) | k4);
                tc_commit(smem_u32(&empty_bar[s]));
                if (++s == p.stages) { s = 0; ph ^= 1; }
            }
        } else if (mode == 5) {
            // plain wait as mode 0, but 8 MMAs (two k blocks' worth, K = 128 per stage) per wait/commit
            for (int kb = 0; kb < p.nkb / 2; ++kb) {
                if (!mbar_wait(smem_u32(&full_bar[s]), ph, &abort_s, p.status)) break;
                if (p.fence) tc_fence_after();
                const uint32_t sa = base + (s & 1) * 2 * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((kb >> 4) & 1) * 256;
#pragma unroll
                for (int k4 = 0; k4 < 8; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 15) | k4);
                tc_commit(smem_u32(&empty_bar[s]));
                if (++s == p.stages) { s = 0; ph ^= 1; }
            }
        } else if (mode == 6 || mode == 7) {
            // wait for TWO (mode 6) or THREE (mode 7) stages' barriers, then their MMAs with a commit per stage
            const int g = mode == 6 ? 2 : 3;
            for (int kb = 0; kb + g <= p.nkb; kb += g) {
                bool ok = true;
                int s2 = s; uint32_t ph2 = ph;
                for (int j = 0; j < g; ++j) {
                    ok = ok && mbar_wait(smem_u32(&full_bar[s2]), ph2, &abort_s, p.status);
                    if (++s2 == p.stages) { s2 = 0; ph2 ^= 1; }
                }
                if (!ok) break;
                if (p.fence) tc_fence_after();
                for (int j = 0; j < g; ++j) {
                    const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                    const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                    const uint32_t d = tmem + (((kb + j) >> 5) & 1) * 256;
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, ((kb + j) & 31) | k4);
                    tc_commit(smem_u32(&empty_bar[s]));
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                }
            }
        } else if (mode >= 10 && mode <= 13) {
            for (int kb = 0; kb < p.nkb; ++kb) {
                const uint32_t fb = smem_u32(&full_bar[s]);
                bool ok = true;
                if (mode == 10) ok = wait_kind<1>(fb, ph);
                else if (mode == 11) ok = wait_kind<2>(fb, ph);
                else if (mode == 12) { if (!test_wait(fb, ph)) ok = mbar_wait(fb, ph, &abort_s, p.status); }
                else { if (!mbar_try_wait(fb, ph)) ok = mbar_wait(fb, ph, &abort_s, p.status); }
                if (!ok) break;
                if (p.fence) tc_fence_after();
                const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((kb >> 5) & 1) * 256;
#pragma unroll
                for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 31) | k4);
                tc_commit(smem_u32(&empty_bar[s]));
                if (++s == p.stages) { s = 0; ph ^= 1; }
            }
        } else if (mode >= 20 && mode <= 23) {
            bool ok = true;
            if (mode == 23) ok = mbar_wait(smem_u32(&full_bar[0]), 0, &abort_s, p.status);
            for (int kb = 0; kb < p.nkb && ok; ++kb) {
                const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((kb >> 5) & 1) * 256;
                if (mode == 20 || mode == 21) {
                    // no barrier wait; a plain shared-memory load feeding a branch, before (20) the MMAs / between MMAs and commit (21)
                    if (mode == 20) { if (*(volatile int*)&abort_s) break; }
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 31) | k4);
                    if (mode == 21) { if (*(volatile int*)&abort_s) break; }
                    tc_commit(smem_u32(&empty_bar[s]));
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                } else if (mode == 22) {
                    // wait, commit of the PREVIOUS stage, then MMAs
                    if (!mbar_wait(smem_u32(&full_bar[s]), ph, &abort_s, p.status)) break;
                    if (kb > 0) tc_commit(smem_u32(&empty_bar[s == 0 ? p.stages - 1 : s - 1]));
                    tc_fence_after();
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 31) | k4);
                    if (kb + 1 == p.nkb) tc_commit(smem_u32(&empty_bar[s]));
                    if (++s == p.stages) { s = 0; ph ^= 1; }
                } else {
                    // MMAs, wait for the next stage, then commit this one
                    int sn = s + 1; uint32_t phn = ph;
                    if (sn == p.stages) { sn = 0; phn ^= 1; }
#pragma unroll
                    for (int k4 = 0; k4 < 4; ++k4) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (kb & 31) | k4);
                    if (kb + 1 < p.nkb) ok = mbar_wait(smem_u32(&full_bar[sn]), phn, &abort_s, p.status);
                    tc_commit(smem_u32(&empty_bar[s]));
                    tc_fence_after();
                    s = sn; ph = phn;
                }
            }
        }
        tc_commit(smem_u32(&bar_end));
        const long long ti = clock64() - t0;
        mbar_wait(smem_u32(&bar_end), 0, &abort_s, p.status);
        p.out[blockIdx.x * 2] = p.lockstep == 1 ? w : ti;
        p.out[blockIdx.x * 2 + 1] = clock64() - t0;
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

// whole-warp variant of the hand-shake kernel: every lane runs the loop (uniform control flow), one elected lane issues
__global__ void __launch_bounds__(128, 1) hku(H p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[16], empty_bar[16], bar_end;
    __shared__ uint32_t tmem_s;
    __shared__ int abort_s;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    for (int i = threadIdx.x; i < 4 * 49152 / 4; i += blockDim.x)
        asm volatile("st.shared.b32 [%0], %1;" ::"r"(base + i * 4), "r"(0x3c003c00u + (uint32_t)(i & 7) * 0x00010001u));
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < 16; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        mbar_init(smem_u32(&bar_end), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x < 32) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_s)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = tmem_s;
    const int warp = threadIdx.x >> 5;
    const int mode = p.lockstep;      // 0: wait+4 MMAs+commit; 4: no wait; 5: wait + 8 MMAs + commit; 6: wait + 2x(4 MMAs + commit)
    if (threadIdx.x == 64) {          // producer
        int s = 0; uint32_t ph = 0;
        const int n = mode == 5 ? p.nkb / 2 : p.nkb;
        for (int kb = 0; kb < n; ++kb) {
            if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, &abort_s, p.status)) break;
            mbar_expect_tx(smem_u32(&full_bar[s]), 0);
            if (++s == p.stages) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1) {           // MMA warp, all lanes
        const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(p.N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const long long t0 = clock64();
        int s = 0; uint32_t ph = 0;
        bool ok = true;
        const int groups = mode == 5 ? p.nkb / 2 : (mode == 6 ? p.nkb / 2 : p.nkb);
        for (int g = 0; g < groups && ok; ++g) {
            if (mode == 6) {
                int s2 = s + 1; uint32_t ph2 = ph; if (s2 == p.stages) { s2 = 0; ph2 ^= 1; }
                ok = mbar_wait(smem_u32(&full_bar[s]), ph, &abort_s, p.status) && mbar_wait(smem_u32(&full_bar[s2]), ph2, &abort_s, p.status);
            } else if (mode != 4) ok = mbar_wait(smem_u32(&full_bar[s]), ph, &abort_s, p.status);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const int reps = mode == 6 ? 2 : 1, per = mode == 5 ? 8 : 4;
            for (int r = 0; r < reps; ++r) {
                const uint32_t sa = base + (s & 3) * p.stage_bytes, sb = sa + p.a_bytes;
                const uint64_t da = make_desc(sa, false, 8192), db = make_desc(sb, false, 8192);
                const uint32_t d = tmem + ((g >> 5) & 1) * 256;
                if (elect_one()) {
#pragma unroll
                    for (int k4 = 0; k4 < 8; ++k4) if (k4 < per) tc_mma(d, da + (uint64_t)(k4 * 2), db + (uint64_t)(k4 * 2), idesc, (g & 31) | k4);
                    tc_commit(smem_u32(&empty_bar[s]));
                }
                __syncwarp();
                if (++s == p.stages) { s = 0; ph ^= 1; }
            }
        }
        if (elect_one()) tc_commit(smem_u32(&bar_end));
        __syncwarp();
        const long long ti = clock64() - t0;
        mbar_wait(smem_u32(&bar_end), 0, &abort_s, p.status);
        if ((threadIdx.x & 31) == 0) { p.out[blockIdx.x * 2] = ti; p.out[blockIdx.x * 2 + 1] = clock64() - t0; }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1); } } while (0)

int main() {
    int sms = 0;
    CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    long long* out; int* status;
    CK(cudaMalloc(&out, sizeof(long long) * 2 * 256));
    CK(cudaMalloc(&status, 4));
    CK(cudaMemset(status, 0, 4));
    const size_t smem = 4 * 49152 + 1024;
    CK(cudaFuncSetAttribute(k<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CK(cudaFuncSetAttribute(k<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CK(cudaFuncSetAttribute(k<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    CK(cudaFuncSetAttribute(k<3>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    {   // long run: does the MMA rate in cycles change once the power cap bites?
        for (int rnd = 0; rnd < 2; ++rnd) {
            P p{}; p.rnd = rnd; p.nkb = 400000; p.commit_every = 0; p.N = 256; p.stages = 4; p.a_bytes = 16384; p.stage_bytes = 49152; p.ncommit = 1; p.out = out; p.status = status;
            cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
            for (int rep = 0; rep < 12; ++rep) {
                CK(cudaEventRecord(e0));
                k<0><<<sms, 128, smem>>>(p);
                CK(cudaEventRecord(e1));
                CK(cudaDeviceSynchronize());
                float ms = 0; CK(cudaEventElapsedTime(&ms, e0, e1));
                std::vector<long long> h(2 * 256);
                CK(cudaMemcpy(h.data(), out, sizeof(long long) * 2 * 256, cudaMemcpyDeviceToHost));
                double st = 0; for (int b = 0; b < sms; ++b) st += h[2 * b + 1];
                const double cyc = st / sms;
                printf("long run %s data rep %2d: %.1f ms, %.1f cyc/MMA, %.0f MHz, %.0f TFLOP/s\n", rnd ? "random" : "constant", rep, ms, cyc / (400000.0 * 4), cyc / ms / 1e3,
                       400000.0 * 4 * 128 * 256 * 16 * 2 * sms / (ms * 1e-3) / 1e12);
            }
        }
    }
    struct V { const char* name; int pair, commit_every, N, a_mn, b_mn, stages, same_acc, ncommit; };
    std::vector<V> vs = {
        {"1cta N32 no commit", 0, 0, 32, 0, 0, 4, 0, 1}, {"1cta N32 1 commit / 4 MMAs", 0, 1, 32, 0, 0, 4, 0, 1},
        {"1cta N32 2 commits / 4 MMAs", 0, 1, 32, 0, 0, 4, 0, 2}, {"1cta N32 4 commits / 4 MMAs", 0, 1, 32, 0, 0, 4, 0, 4},
        {"1cta N32 1 commit / 8 MMAs", 0, 2, 32, 0, 0, 4, 0, 1},
        {"2cta N32 no commit", 1, 0, 32, 0, 0, 4, 0, 1}, {"2cta N32 1 local commit / 4 MMAs", 1, 1, 32, 0, 0, 4, 0, 1},
        {"2cta N32 local+peer commit / 4 MMAs", 2, 1, 32, 0, 0, 4, 0, 1}, {"2cta N32 masked commit / 4 MMAs", 3, 1, 32, 0, 0, 4, 0, 1},
        {"2cta N256 masked commit / 4 MMAs", 3, 1, 256, 0, 0, 4, 0, 1},
    };
    for (const V& v : vs) {
        P p{};
        p.nkb = 4096; p.commit_every = v.commit_every; p.N = v.N; p.a_mn = v.a_mn; p.b_mn = v.b_mn; p.stages = v.stages;
        p.a_bytes = 16384; p.stage_bytes = v.pair ? 32768 : 49152; p.same_acc = v.same_acc; p.ncommit = v.ncommit; p.out = out; p.status = status;
        const int grid = v.pair ? (sms & ~1) : sms;
        for (int rep = 0; rep < 2; ++rep) {
            CK(cudaMemset(out, 0, sizeof(long long) * 2 * 256));
            if (v.pair) {
                cudaLaunchConfig_t cfg{};
                cfg.gridDim = dim3(grid); cfg.blockDim = dim3(128); cfg.dynamicSmemBytes = smem;
                cudaLaunchAttribute at[1]; at[0].id = cudaLaunchAttributeClusterDimension; at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
                cfg.attrs = at; cfg.numAttrs = 1;
                if (v.pair == 1) CK(cudaLaunchKernelEx(&cfg, k<1>, p)); else if (v.pair == 2) CK(cudaLaunchKernelEx(&cfg, k<2>, p)); else CK(cudaLaunchKernelEx(&cfg, k<3>, p));
            } else k<0><<<grid, 128, smem>>>(p);
            CK(cudaGetLastError());
            CK(cudaDeviceSynchronize());
        }
        std::vector<long long> h(2 * 256);
        CK(cudaMemcpy(h.data(), out, sizeof(long long) * 2 * 256, cudaMemcpyDeviceToHost));
        double si = 0, st = 0; int n = 0;
        for (int b = 0; b < grid; ++b) if (h[2 * b + 1] > 0) { si += h[2 * b]; st += h[2 * b + 1]; ++n; }
        int stv = 0; CK(cudaMemcpy(&stv, status, 4, cudaMemcpyDeviceToHost));
        printf("%-36s ctas %3d  issue %.1f cyc/MMA  total %.1f cyc/MMA  (ideal %d) status %d\n", v.name, n, si / n / (4096.0 * 4), st / n / (4096.0 * 4),
               v.N / 2, stv);
    }

    CK(cudaFuncSetAttribute(hk, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    struct HV { const char* name; int stages, fence, lockstep, N, uni; };
    CK(cudaFuncSetAttribute(hku, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    std::vector<HV> hv = {{"lane: wait+4MMA+commit N32", 8, 1, 0, 32, 0}, {"warp: wait+4MMA+commit N32", 8, 1, 0, 32, 1},
                          {"lane: 4MMA+commit N32 (no wait)", 8, 1, 4, 32, 0}, {"warp: 4MMA+commit N32 (no wait)", 8, 1, 4, 32, 1},
                          {"lane: wait+8MMA+commit N32", 8, 1, 5, 32, 0}, {"warp: wait+8MMA+commit N32", 8, 1, 5, 32, 1},
                          {"lane: 2 waits+2x(4MMA+commit) N32", 8, 1, 6, 32, 0}, {"warp: 2 waits+2x(4MMA+commit) N32", 8, 1, 6, 32, 1},
                          {"warp: wait+4MMA+commit N256", 8, 1, 0, 256, 1}, {"warp: 2 waits+2x(4MMA+commit) N256", 8, 1, 6, 256, 1}, {"warp: wait+4MMA+commit N256 4 stages", 4, 1, 0, 256, 1}};
    for (const HV& v : hv) {
        H p{}; p.nkb = 4096; p.stages = v.stages; p.fence = v.fence; p.stage_bytes = 49152; p.a_bytes = 16384; p.lockstep = v.lockstep; p.N = v.N; p.out = out; p.status = status;
        for (int rep = 0; rep < 2; ++rep) {
            CK(cudaMemset(out, 0, sizeof(long long) * 2 * 256));
            if (v.uni) hku<<<sms, 128, smem>>>(p); else hk<<<sms, 128, smem>>>(p);
            CK(cudaGetLastError());
            CK(cudaDeviceSynchronize());
        }
        std::vector<long long> h(2 * 256);
        CK(cudaMemcpy(h.data(), out, sizeof(long long) * 2 * 256, cudaMemcpyDeviceToHost));
        double si = 0, st = 0; int n = 0;
        for (int b = 0; b < sms; ++b) if (h[2 * b + 1] > 0) { si += h[2 * b]; st += h[2 * b + 1]; ++n; }
        int stv = 0; CK(cudaMemcpy(&stv, status, 4, cudaMemcpyDeviceToHost));
        printf("%-40s ctas %3d  %s %.1f cyc/kblock  total %.1f cyc/kblock (ideal 512) status %d\n", v.name, n, v.lockstep == 1 ? "waits" : "issue", si / n / 4096.0, st / n / 4096.0, stv);
    }
    return 0;
}
