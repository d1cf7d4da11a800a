// Checkpoint pass-through of the MoE block's parameters (include/tmt_ckpt.h): one parameter record of the
// reference's V3 payload (tmt-cuda/src/checkpoint.h:142-149) between device memory and a host buffer, the
// re-materialisation of the bf16 working copy at load, and the file checksum (checkpoint.h:11-17).
#include <cuda_runtime.h>

#include <cstring>
#include <stdexcept>
#include <string>

#include "../../include/tmt_ckpt.h"
#include "common.cuh"

namespace tmt {
void set_error(const char* fmt, ...);

namespace {

// work[i] = bf16(master[i]), 8 elements per thread where the pointers allow 16-byte stores
__global__ void __launch_bounds__(256) materialise_bf16_kernel(const float* __restrict__ master, uint16_t* __restrict__ work, long n,
                                                               int vec_ok) {
    const long i0 = ((long)blockIdx.x * blockDim.x + threadIdx.x) * 8;
    if (i0 >= n) return;
    if (vec_ok && i0 + 8 <= n) {
        const float4 a = __ldg(reinterpret_cast<const float4*>(master + i0));
        const float4 b = __ldg(reinterpret_cast<const float4*>(master + i0 + 4));
        stg16(work + i0, make_uint4(pack_bf2(a.x, a.y), pack_bf2(a.z, a.w), pack_bf2(b.x, b.y), pack_bf2(b.z, b.w)));
    } else {
        for (long i = i0; i < n && i < i0 + 8; ++i) work[i] = f2bf(master[i]);
    }
}

void ck(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + " failed: " + cudaGetErrorString(e));
}

}  // namespace
}  // namespace tmt

using namespace tmt;

extern "C" {

uint64_t tmt_ckpt_hash(uint64_t h, const void* data, size_t size) {
    const unsigned char* b = static_cast<const unsigned char*>(data);
    for (size_t i = 0; i < size; ++i) h = (h ^ b[i]) * UINT64_C(1099511628211);
    return h;
}

size_t tmt_ckpt_record_bytes(long long n) { return n < 0 ? 0 : 8 + (size_t)n * 12; }

int tmt_ckpt_save_param(const float* master, const float* m, const float* v, long long n, void* record_host,
                        size_t record_bytes, void* stream) {
    try {
        if (!master || !m || !v || !record_host || n < 1) throw std::runtime_error("ckpt_save_param: null argument or n < 1");
        if (record_bytes < tmt_ckpt_record_bytes(n)) throw std::runtime_error("ckpt_save_param: record buffer too small");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        unsigned char* dst = static_cast<unsigned char*>(record_host);
        const uint64_t n64 = (uint64_t)n;
        memcpy(dst, &n64, 8);
        const size_t bytes = (size_t)n * 4;
        ck(cudaMemcpyAsync(dst + 8, master, bytes, cudaMemcpyDeviceToHost, s), "copy of the master weights");
        ck(cudaMemcpyAsync(dst + 8 + bytes, m, bytes, cudaMemcpyDeviceToHost, s), "copy of the first moments");
        ck(cudaMemcpyAsync(dst + 8 + 2 * bytes, v, bytes, cudaMemcpyDeviceToHost, s), "copy of the second moments");
        ck(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

int tmt_ckpt_load_param(const void* record_host, size_t record_bytes, long long n, float* master, float* m, float* v,
                        void* work_bf16, void* stream) {
    try {
        if (!record_host || !master || n < 1) throw std::runtime_error("ckpt_load_param: null argument or n < 1");
        if (record_bytes < 8) throw std::runtime_error("checkpoint truncated");
        const unsigned char* src = static_cast<const unsigned char*>(record_host);
        uint64_t n64 = 0;
        memcpy(&n64, src, 8);
        if (n64 != (uint64_t)n) throw std::runtime_error("checkpoint parameter shape mismatch");      // checkpoint.h:146
        if (record_bytes < tmt_ckpt_record_bytes(n)) throw std::runtime_error("checkpoint truncated");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const size_t bytes = (size_t)n * 4;
        ck(cudaMemcpyAsync(master, src + 8, bytes, cudaMemcpyHostToDevice, s), "copy of the master weights");
        if (m) ck(cudaMemcpyAsync(m, src + 8 + bytes, bytes, cudaMemcpyHostToDevice, s), "copy of the first moments");
        if (v) ck(cudaMemcpyAsync(v, src + 8 + 2 * bytes, bytes, cudaMemcpyHostToDevice, s), "copy of the second moments");
        if (work_bf16) {
            const int vec_ok = (((uintptr_t)master & 15) == 0 && ((uintptr_t)work_bf16 & 15) == 0) ? 1 : 0;
            const long threads = (n + 7) / 8;
            materialise_bf16_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, s>>>(master, static_cast<uint16_t*>(work_bf16), (long)n, vec_ok);
            ck(cudaGetLastError(), "materialise_bf16_kernel launch");
        }
        ck(cudaStreamSynchronize(s), "cudaStreamSynchronize");
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

}  // extern "C"
