// Router weight gradient for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc at the moment they need a result: a
// training loop whose framework has already handed the whole device to its own caching
// allocator (a further cudaMalloc can fail there, or stall every stream while the driver
// maps memory), a real-time sampler that may not take the driver's allocation lock, code
// that runs between fixed memory budgets checked by an operator. The handle-based entry
// points allocate their scratch once in tmt_moe_create; this one owns no handle and
// allocates nothing at all: its scratch is a fixed array inside the loaded library image.
//
// What it computes is the same product as the router_dw phase of tmt_moe_backward:
//   dWrouter[e, d] = sum over tokens t of bf16(dlogits[t, e]) * X[t, d]
// (the reference's to_bf16_kernel + linear_dW, tmt-cuda/src/moe.cu:519-521), in two kernels:
// kChunks partial sums over token ranges into the scratch array, then a fixed-order reduction.
//
// Rules that follow from the shared array:
//   * experts * dim must not exceed kMaxED (the call is refused with a message otherwise);
//   * every GPU that loads the library holds the kChunks * kMaxED * 4 bytes until exit;
//   * all calls on one GPU use the same array, which keeps whatever the last call left
//     there. Nothing in it has to start at zero: the first kernel overwrites every partial
//     the second one reads. Two calls that overlap on the GPU (different streams, or
//     different host threads without ordering) race on it: order them yourself;
//   * the first call on each device looks the array's device address up
//     (cudaGetSymbolAddress). Make that first call outside any stream capture.
#include <cuda_runtime.h>

#include <mutex>
#include <stdexcept>
#include <string>

#include "../../include/tmt_moe.h"
#include "common.cuh"

namespace tmt {
void set_error(const char* fmt, ...);

namespace {

constexpr int kChunks = 16;
constexpr long kMaxED = 131072;          // experts * dim, e.g. 64 x 2048
constexpr int kMaxDevices = 64;

// 8 MiB of partial sums: [kChunks][experts * dim] floats, laid out densely for the call's sizes.
static __device__ __align__(256) float g_partials[kChunks * kMaxED];

// Host code must not pass `g_partials` itself to a kernel: on the host that name is only a
// stand-in for the symbol. The device address is looked up once per device and cached here.
float* g_partials_dev[kMaxDevices] = {nullptr};
std::mutex g_lookup_mutex;

float* partials_for_current_device() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) throw std::runtime_error(std::string("cudaGetDevice failed: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) throw std::runtime_error("device ordinal out of range for the no-alloc entry point");
    std::lock_guard<std::mutex> lock(g_lookup_mutex);
    if (!g_partials_dev[dev]) {
        float* p = nullptr;
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_partials);
        if (e != cudaSuccess || !p)
            throw std::runtime_error(std::string("cudaGetSymbolAddress(scratch) failed: ") + cudaGetErrorString(e));
        g_partials_dev[dev] = p;
    }
    return g_partials_dev[dev];
}

// One block = 256 threads x 2 columns of one token chunk; 32 tokens of rounded gradients staged
// in shared memory at a time. EC experts are accumulated per pass.
template <int EC>
__global__ void __launch_bounds__(256) partial_kernel(const float* __restrict__ dlogits, const uint16_t* __restrict__ X,
                                                       float* __restrict__ partial, int T, int D, int E) {
    __shared__ float dl[32 * EC];
    const int d0 = (blockIdx.x * 256 + threadIdx.x) * 2;
    const int chunk = blockIdx.y;
    const long per = (T + kChunks - 1) / kChunks;
    const long tbeg = chunk * per, tend = min((long)T, tbeg + per);
    const bool dok = d0 < D;
    for (int ec0 = 0; ec0 < E; ec0 += EC) {
        float a0[EC], a1[EC];
#pragma unroll
        for (int e = 0; e < EC; ++e) { a0[e] = 0.0f; a1[e] = 0.0f; }
        for (long tb = tbeg; tb < tend; tb += 32) {
            __syncthreads();
            for (int i = threadIdx.x; i < 32 * EC; i += 256) {
                const int tt = i / EC, e = i - tt * EC;
                const long t = tb + tt;
                dl[i] = (t < tend && ec0 + e < E) ? round_bf(dlogits[t * E + ec0 + e]) : 0.0f;
            }
            __syncthreads();
            if (dok) {
                const int n = (int)min(32L, tend - tb);
                for (int tt = 0; tt < n; ++tt) {
                    const uint32_t xv = __ldg(reinterpret_cast<const uint32_t*>(X + (tb + tt) * D + d0));
                    const float x0 = bf_lo(xv), x1 = bf_hi(xv);
#pragma unroll
                    for (int e = 0; e < EC; ++e) {
                        const float g = dl[tt * EC + e];
                        a0[e] += g * x0; a1[e] += g * x1;
                    }
                }
            }
        }
        if (dok) {
#pragma unroll
            for (int e = 0; e < EC; ++e)
                if (ec0 + e < E) {
                    float* dst = partial + ((long)chunk * E + ec0 + e) * D + d0;
                    dst[0] = a0[e]; dst[1] = a1[e];
                }
        }
    }
}

__global__ void reduce_kernel(const float* __restrict__ partial, float* __restrict__ dWr, long n) {
    const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.0f;
    for (int c = 0; c < kChunks; ++c) s += partial[(long)c * n + i];
    dWr[i] = s;
}

}  // namespace
}  // namespace tmt

extern "C" int tmt_moe_router_dw_noalloc(const float* dlogits, const void* X, int tokens, int dim, int experts,
                                         float* dWrouter, void* stream) {
    using namespace tmt;
    try {
        if (!dlogits || !X || !dWrouter) throw std::runtime_error("router_dw_noalloc: null argument");
        if (tokens < 1 || dim < 2 || dim % 2 || experts < 1) throw std::runtime_error("router_dw_noalloc: need tokens >= 1, even dim, experts >= 1");
        if ((long)experts * dim > kMaxED)
            throw std::runtime_error("router_dw_noalloc: experts * dim = " + std::to_string((long)experts * dim) +
                                     " exceeds the built-in scratch (" + std::to_string(kMaxED) +
                                     "); use tmt_moe_backward on a handle instead");
        float* partial = partials_for_current_device();
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const dim3 grid((dim / 2 + 255) / 256, kChunks);
        const uint16_t* Xb = static_cast<const uint16_t*>(X);
        if (experts <= 8) partial_kernel<8><<<grid, 256, 0, s>>>(dlogits, Xb, partial, tokens, dim, experts);
        else if (experts <= 16) partial_kernel<16><<<grid, 256, 0, s>>>(dlogits, Xb, partial, tokens, dim, experts);
        else if (experts <= 32) partial_kernel<32><<<grid, 256, 0, s>>>(dlogits, Xb, partial, tokens, dim, experts);
        else partial_kernel<64><<<grid, 256, 0, s>>>(dlogits, Xb, partial, tokens, dim, experts);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) throw std::runtime_error(std::string("router_dw_noalloc: launch failed: ") + cudaGetErrorString(e));
        const long n = (long)experts * dim;
        reduce_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(partial, dWrouter, n);
        e = cudaGetLastError();
        if (e != cudaSuccess) throw std::runtime_error(std::string("router_dw_noalloc: launch failed: ") + cudaGetErrorString(e));
        return 0;
    } catch (const std::exception& ex) { set_error("%s", ex.what()); return -1; }
}
