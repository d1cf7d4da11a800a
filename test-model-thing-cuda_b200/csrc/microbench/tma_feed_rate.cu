// Micro-benchmark (measurement only, not part of the library): L2 -> shared memory feed rate of TMA box loads per
// SM against box size, boxes per stage, stages in flight, lanes that issue and producer warps. A consumer thread
// hands every stage straight back. The source matrix (64 MB) stays in L2. Every wait is bounded.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I.. -o tma_feed_rate tma_feed_rate.cu -lcuda && ./tma_feed_rate
//
// Numbers measured on a B200 are in profiles/gemm_tcgen05_config5_32k_tokens.md.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <cuda.h>
#include "tc_util.cuh"
using namespace tmt; using namespace tmt::tc;
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1); } } while (0)
typedef CUresult (*EncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                             CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
struct P { const CUtensorMap* map; int pwarps; int nkb, stages, boxes, box_rows, rows, kblocks, issuers; long long* out; int* status; };

// warp 0: producer (lane j < issuers issues boxes j, j+issuers, ...); warp 1 lane 0: consumer (waits full, arrives empty)
__global__ void __launch_bounds__(128, 1) k(P p) {
    extern __shared__ uint8_t raw[];
    __shared__ uint64_t full_bar[8], empty_bar[8];
    __shared__ int abort_s;
    const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < 8; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    const uint32_t box_bytes = p.box_rows * 128, stage_bytes = p.boxes * box_bytes;
    const long long t0 = clock64();
    if (warp == 0 || (warp == 2 && p.pwarps == 2)) {
        const int my = warp == 0 ? 0 : 1;
        if (lane == 0) tensormap_acquire(p.map);
        __syncwarp();
        int s = 0; uint32_t ph = 0; bool ok = true;
        uint32_t h = blockIdx.x * 2654435761u + 12345u;
        for (int kb = 0; kb < p.nkb && ok; ++kb) {
            if (p.pwarps == 2 && (kb & 1) != my) { if (++s == p.stages) { s = 0; ph ^= 1; } continue; }
            if (lane == 0) { ok = mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, &abort_s, p.status); if (ok) mbar_expect_tx(smem_u32(&full_bar[s]), stage_bytes); }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            h = h * 1664525u + 1013904223u;
            const int kblk = (h >> 8) & (p.kblocks - 1);
            for (int j = lane; j < p.boxes; j += p.issuers) {
                if (lane < p.issuers) {
                    const int row = (((h >> 12) + j * 977u) & (p.rows / 256 - 1)) * 256;
                    tma_load_2d(base + s * stage_bytes + j * box_bytes, p.map, smem_u32(&full_bar[s]), kblk * 64, row);
                }
            }
            __syncwarp();
            if (++s == p.stages) { s = 0; ph ^= 1; }
        }
    } else if (warp == 1 && lane == 0) {
        int s = 0; uint32_t ph = 0;
        for (int kb = 0; kb < p.nkb; ++kb) {
            if (!mbar_wait(smem_u32(&full_bar[s]), ph, &abort_s, p.status)) break;
            mbar_arrive(smem_u32(&empty_bar[s]));
            if (++s == p.stages) { s = 0; ph ^= 1; }
        }
        p.out[blockIdx.x] = clock64() - t0;
    }
}
int main() {
    int sms = 0; CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    const int ROWS = 16384, K = 2048;       // 64 MB, stays in L2
    uint16_t* d; CK(cudaMalloc(&d, (size_t)ROWS * K * 2)); CK(cudaMemset(d, 0x3c, (size_t)ROWS * K * 2));
    long long* out; int* status; CK(cudaMalloc(&out, 8 * 256)); CK(cudaMalloc(&status, 4)); CK(cudaMemset(status, 0, 4));
    void* fp = nullptr; cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q));
    CUtensorMap* dmaps; CK(cudaMalloc(&dmaps, 4 * sizeof(CUtensorMap)));
    const int box_rows_opts[3] = {64, 128, 256};
    for (int i = 0; i < 3; ++i) {
        CUtensorMap m; memset(&m, 0, sizeof m);
        cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)ROWS}; cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)box_rows_opts[i]}; cuuint32_t es[2] = {1, 1};
        CUresult r = ((EncodeFn)fp)(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, d, dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); return 1; }
        CK(cudaMemcpy(dmaps + i, &m, sizeof m, cudaMemcpyHostToDevice));
    }
    const size_t smem = 224 * 1024;
    CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    struct V { int box_i, boxes, stages, issuers, pwarps; };
    std::vector<V> vs = {{1, 1, 4, 1, 1}, {1, 2, 4, 1, 1}, {1, 2, 4, 2, 1}, {1, 2, 6, 2, 1}, {1, 3, 4, 3, 1}, {2, 1, 4, 1, 1},
                         {1, 1, 4, 1, 2}, {1, 2, 4, 2, 2}, {1, 2, 6, 2, 2}, {1, 3, 4, 3, 2}, {2, 1, 4, 1, 2}, {2, 1, 6, 1, 2}, {1, 3, 4, 1, 2}};
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (const V& v : vs) {
        P p{}; p.map = dmaps + v.box_i; p.nkb = 20000; p.stages = v.stages; p.boxes = v.boxes; p.box_rows = box_rows_opts[v.box_i]; p.rows = ROWS; p.kblocks = K / 64;
        p.issuers = v.issuers; p.pwarps = v.pwarps; p.out = out; p.status = status;
        if ((size_t)p.stages * p.boxes * p.box_rows * 128 + 1024 > smem) { printf("skip (smem)\n"); continue; }
        float ms = 0;
        for (int rep = 0; rep < 2; ++rep) {
            CK(cudaEventRecord(e0));
            k<<<sms, 128, smem>>>(p);
            CK(cudaEventRecord(e1));
            CK(cudaDeviceSynchronize());
            CK(cudaEventElapsedTime(&ms, e0, e1));
        }
        std::vector<long long> h(256); CK(cudaMemcpy(h.data(), out, 8 * 256, cudaMemcpyDeviceToHost));
        double cyc = 0; for (int b = 0; b < sms; ++b) cyc += h[b]; cyc /= sms;
        int st = 0; CK(cudaMemcpy(&st, status, 4, cudaMemcpyDeviceToHost));
        const double bytes = (double)p.nkb * p.boxes * p.box_rows * 128;
        printf("box %3d rows x %d boxes/stage (%2d KB), %d stages (%3d KB in flight), %d issuing lanes, %d producer warps: %.0f cycles/stage, %.1f B/clk/SM, %.1f TB/s total, %.0f MHz, status %d\n",
               p.box_rows, p.boxes, p.boxes * p.box_rows / 8, p.stages, p.stages * p.boxes * p.box_rows / 8, p.issuers, p.pwarps, cyc / p.nkb, bytes / cyc,
               bytes * sms / (ms * 1e-3) / 1e12, cyc / ms / 1e3, st);
    }
    return 0;
}
