// Multi-tensor AdamW over the MoE block's parameters: squared gradient norm (double, fixed order), clipping, AdamW on
// the fp32 masters and moments, bf16 working copies, gradient clearing. Two passes over the data; both are bound by HBM.
// Reference: tmt-cuda/src/adam.cu:44-105 and optimizer_step, tmt-cuda/src/model.cu:716-729.
#include <cuda_runtime.h>

#include <cmath>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/tmt_adamw.h"
#include "common.cuh"

namespace tmt {
void set_error(const char* fmt, ...);
}

namespace {

using namespace tmt;

constexpr int kChunk = 8192;          // elements per table entry (a multiple of 4: tensors are read as float4 when aligned)
constexpr int kThreads = 256;

struct Chunk { int tensor; int len; long long start; };

struct Tables {
    float* const* master; float* const* m; float* const* v; float* const* grad; uint16_t* const* work;
    const unsigned char* flags;
    const Chunk* chunks; int nchunks;
};

#define CKA(call)                                                                             \
    do {                                                                                      \
        cudaError_t e__ = (call);                                                             \
        if (e__ != cudaSuccess) throw std::runtime_error(std::string(#call) + " failed: " + cudaGetErrorString(e__)); \
    } while (0)

// Block b sums the chunks b, b + gridDim.x, ... : every thread its elements in index order, then a fixed tree over the
// block. partial[b] gets the block's sum; nothing is added with atomics, so the result does not depend on timing.
__global__ void __launch_bounds__(kThreads) sumsq_kernel(const Tables t, double* __restrict__ partial) {
    __shared__ double buf[kThreads];
    double s = 0.0;
    for (int c = blockIdx.x; c < t.nchunks; c += gridDim.x) {
        const Chunk ch = t.chunks[c];
        if (!(t.flags[ch.tensor] & 1)) continue;
        const float* g = t.grad[ch.tensor] + ch.start;
        if ((reinterpret_cast<uintptr_t>(g) & 15) == 0 && (ch.len & 3) == 0) {
            const float4* g4 = reinterpret_cast<const float4*>(g);
            for (int i = threadIdx.x; i < ch.len / 4; i += kThreads) {
                const float4 x = __ldg(g4 + i);
                s += (double)x.x * x.x; s += (double)x.y * x.y; s += (double)x.z * x.z; s += (double)x.w * x.w;
            }
        } else {
            for (int i = threadIdx.x; i < ch.len; i += kThreads) { const float x = g[i]; s += (double)x * x; }
        }
    }
    buf[threadIdx.x] = s;
    __syncthreads();
    for (int w = kThreads / 2; w > 0; w >>= 1) {
        if (threadIdx.x < w) buf[threadIdx.x] += buf[threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = buf[0];
}

// One block: partial sums in index order -> sumsq[0]; scale (float) -> sumsq[1] as a double.
__global__ void finish_norm_kernel(const double* __restrict__ partial, int n, float clip, double* __restrict__ out) {
    double s = 0.0;
    for (int i = 0; i < n; ++i) s += partial[i];
    out[0] = s;
    float scale = 1.0f;
    if (clip > 0.0f) scale = fminf(1.0f, __fdiv_rn(clip, fmaxf((float)sqrt(s), 1e-12f)));
    out[1] = (double)scale;
}

__device__ __forceinline__ void adamw_one(float& w, float& m, float& v, float g, float scale, float b1, float b2, float omb1,
                                          float omb2, float eps, float wd, float lr, float bc1, float bc2) {
    g = __fmul_rn(g, scale);
    m = __fmaf_rn(b1, m, __fmul_rn(omb1, g));
    v = __fmaf_rn(b2, v, __fmul_rn(__fmul_rn(omb2, g), g));
    const float u = __fdiv_rn(__fdiv_rn(m, bc1), __fadd_rn(__fsqrt_rn(__fdiv_rn(v, bc2)), eps));
    w = __fmaf_rn(-lr, __fmaf_rn(wd, w, u), w);
}

__global__ void __launch_bounds__(kThreads) adamw_kernel(const Tables t, const double* __restrict__ norm, float lr, float b1, float b2,
                                                         float eps, float wd, float bc1, float bc2, int zero_grads) {
    const double s = norm[0];
    const bool finite = isfinite(s);
    const float scale = (float)norm[1];
    const float omb1 = 1.0f - b1, omb2 = 1.0f - b2;
    for (int c = blockIdx.x; c < t.nchunks; c += gridDim.x) {
        const Chunk ch = t.chunks[c];
        const unsigned char fl = t.flags[ch.tensor];
        float* grad = t.grad[ch.tensor] + ch.start;
        if ((fl & 2) && finite) {
            float* master = t.master[ch.tensor] + ch.start;
            float* mm = t.m[ch.tensor] + ch.start;
            float* vv = t.v[ch.tensor] + ch.start;
            uint16_t* work = t.work[ch.tensor] ? t.work[ch.tensor] + ch.start : nullptr;
            const bool vec = ((reinterpret_cast<uintptr_t>(master) | reinterpret_cast<uintptr_t>(mm) | reinterpret_cast<uintptr_t>(vv) |
                               reinterpret_cast<uintptr_t>(grad)) & 15) == 0 &&
                             (work == nullptr || (reinterpret_cast<uintptr_t>(work) & 7) == 0) && (ch.len & 3) == 0;
            if (vec) {
                for (int i = threadIdx.x; i < ch.len / 4; i += kThreads) {
                    float4 w4 = reinterpret_cast<float4*>(master)[i], m4 = reinterpret_cast<float4*>(mm)[i];
                    float4 v4 = reinterpret_cast<float4*>(vv)[i];
                    const float4 g4 = reinterpret_cast<const float4*>(grad)[i];
                    adamw_one(w4.x, m4.x, v4.x, g4.x, scale, b1, b2, omb1, omb2, eps, wd, lr, bc1, bc2);
                    adamw_one(w4.y, m4.y, v4.y, g4.y, scale, b1, b2, omb1, omb2, eps, wd, lr, bc1, bc2);
                    adamw_one(w4.z, m4.z, v4.z, g4.z, scale, b1, b2, omb1, omb2, eps, wd, lr, bc1, bc2);
                    adamw_one(w4.w, m4.w, v4.w, g4.w, scale, b1, b2, omb1, omb2, eps, wd, lr, bc1, bc2);
                    reinterpret_cast<float4*>(master)[i] = w4;
                    reinterpret_cast<float4*>(mm)[i] = m4;
                    reinterpret_cast<float4*>(vv)[i] = v4;
                    if (work) reinterpret_cast<uint2*>(work)[i] = make_uint2(pack_bf2(w4.x, w4.y), pack_bf2(w4.z, w4.w));
                    if (zero_grads) reinterpret_cast<float4*>(grad)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            } else {
                for (int i = threadIdx.x; i < ch.len; i += kThreads) {
                    float w = master[i], m1 = mm[i], v1 = vv[i];
                    adamw_one(w, m1, v1, grad[i], scale, b1, b2, omb1, omb2, eps, wd, lr, bc1, bc2);
                    master[i] = w; mm[i] = m1; vv[i] = v1;
                    if (work) work[i] = f2bf(w);
                    if (zero_grads) grad[i] = 0.0f;
                }
            }
        } else if (zero_grads && finite) {
            for (int i = threadIdx.x; i < ch.len; i += kThreads) grad[i] = 0.0f;
        }
    }
}

}  // namespace

struct tmt_adamw {
    int tensors = 0, device = 0, nchunks = 0, blocks = 0;
    cudaStream_t stream = nullptr;
    std::vector<long long> sizes;
    void** ptrs = nullptr;             // device: 5 pointer arrays of `tensors` entries
    unsigned char* flags = nullptr;
    Chunk* chunks = nullptr;
    double* partial = nullptr;         // [blocks]
    double* norm = nullptr;            // [2]: sumsq, scale
    std::vector<void*> staged;         // host copy of the pointer arrays, compared with the caller's to skip uploads
    std::vector<unsigned char> staged_flags;
};

extern "C" {

int tmt_adamw_create(int tensors, const long long* sizes, int device, void* stream, tmt_adamw** out) {
    if (!out) { set_error("null argument"); return -1; }
    *out = nullptr;
    try {
        if (tensors < 1 || !sizes) throw std::runtime_error("need at least one tensor");
        CKA(cudaSetDevice(device));
        std::unique_ptr<tmt_adamw, void (*)(tmt_adamw*)> h(new tmt_adamw(), [](tmt_adamw* p) { tmt_adamw_destroy(p); });
        h->tensors = tensors; h->device = device; h->stream = static_cast<cudaStream_t>(stream);
        h->sizes.assign(sizes, sizes + tensors);
        std::vector<Chunk> ch;
        for (int i = 0; i < tensors; ++i) {
            if (sizes[i] < 0) throw std::runtime_error("negative tensor size");
            for (long long s = 0; s < sizes[i]; s += kChunk) ch.push_back({i, (int)std::min<long long>(kChunk, sizes[i] - s), s});
        }
        h->nchunks = (int)ch.size();
        int sms = 0;
        CKA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device));
        h->blocks = std::max(1, std::min(h->nchunks, sms * 8));       // a multiple of the SM count, 8 resident blocks each
        CKA(cudaMalloc(&h->ptrs, sizeof(void*) * 5 * tensors));
        CKA(cudaMalloc(&h->flags, tensors));
        CKA(cudaMalloc(&h->chunks, sizeof(Chunk) * std::max<size_t>(ch.size(), 1)));
        CKA(cudaMalloc(&h->partial, sizeof(double) * h->blocks));
        CKA(cudaMalloc(&h->norm, sizeof(double) * 2));
        CKA(cudaMemcpyAsync(h->chunks, ch.data(), sizeof(Chunk) * ch.size(), cudaMemcpyHostToDevice, h->stream));
        CKA(cudaStreamSynchronize(h->stream));
        *out = h.release();
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

void tmt_adamw_destroy(tmt_adamw* h) {
    if (!h) return;
    cudaSetDevice(h->device);
    for (void* p : {(void*)h->ptrs, (void*)h->flags, (void*)h->chunks, (void*)h->partial, (void*)h->norm}) if (p) cudaFree(p);
    delete h;
}

int tmt_adamw_step(tmt_adamw* h, float* const* master, float* const* m, float* const* v, float* const* grad, void* const* work,
                   const unsigned char* flags, float clip, float lr, float b1, float b2, float eps, float wd, int step,
                   int zero_grads, double* sumsq_host) {
    if (!h || !master || !m || !v || !grad || !work || !flags) { set_error("null argument"); return -1; }
    try {
        if (step < 1) throw std::runtime_error("step counts from 1");
        CKA(cudaSetDevice(h->device));
        const int n = h->tensors;
        std::vector<void*> now((size_t)5 * n);
        for (int i = 0; i < n; ++i) {
            now[i] = master[i]; now[n + i] = m[i]; now[2 * n + i] = v[i]; now[3 * n + i] = grad[i]; now[4 * n + i] = work[i];
            if ((flags[i] & 3) && (!master[i] || !m[i] || !v[i] || !grad[i])) throw std::runtime_error("null tensor pointer");
        }
        if (now != h->staged) {
            CKA(cudaMemcpyAsync(h->ptrs, now.data(), sizeof(void*) * now.size(), cudaMemcpyHostToDevice, h->stream));
            CKA(cudaStreamSynchronize(h->stream));       // `now` is a local
            h->staged = now;
        }
        if (std::vector<unsigned char>(flags, flags + n) != h->staged_flags) {
            h->staged_flags.assign(flags, flags + n);
            CKA(cudaMemcpyAsync(h->flags, h->staged_flags.data(), n, cudaMemcpyHostToDevice, h->stream));
        }
        Tables t;
        t.master = reinterpret_cast<float* const*>(h->ptrs);
        t.m = reinterpret_cast<float* const*>(h->ptrs + n);
        t.v = reinterpret_cast<float* const*>(h->ptrs + 2 * n);
        t.grad = reinterpret_cast<float* const*>(h->ptrs + 3 * n);
        t.work = reinterpret_cast<uint16_t* const*>(h->ptrs + 4 * n);
        t.flags = h->flags; t.chunks = h->chunks; t.nchunks = h->nchunks;
        sumsq_kernel<<<h->blocks, kThreads, 0, h->stream>>>(t, h->partial);
        CKA(cudaGetLastError());
        finish_norm_kernel<<<1, 1, 0, h->stream>>>(h->partial, h->blocks, clip, h->norm);
        CKA(cudaGetLastError());
        const float bc1 = 1.0f - powf(b1, (float)step), bc2 = 1.0f - powf(b2, (float)step);
        adamw_kernel<<<h->blocks, kThreads, 0, h->stream>>>(t, h->norm, lr, b1, b2, eps, wd, bc1, bc2, zero_grads);
        CKA(cudaGetLastError());
        if (sumsq_host) {
            CKA(cudaMemcpyAsync(sumsq_host, h->norm, sizeof(double), cudaMemcpyDeviceToHost, h->stream));
            CKA(cudaStreamSynchronize(h->stream));
            if (!std::isfinite(*sumsq_host)) throw std::runtime_error("non-finite gradient; update refused");
        }
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

}  // extern "C"
