// Shared device helpers of the MoE kernels: bf16 packing, SiLU, status word.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Measurement switches (kernel phases turned off one at a time, results are then wrong) exist only in builds made with
// -DTMT_MOE_MEASURE; in the product build every test of them is the constant 0 and the environment variables that set
// them are not read.
#ifdef TMT_MOE_MEASURE
#define TMT_DBG(p, bit) ((p).dbg & (bit))
#else
#define TMT_DBG(p, bit) 0
#endif

namespace tmt {

// Rows of one GEMM row tile and unit of every tile table. Expert groups start on a multiple of the
// handle's pad (128 rows, or 256 for the CTA-pair GEMM), so a tile never spans two experts (the
// reference pads to 128 to keep its cuBLAS shapes stable, tmt-cuda/src/moe.cu:414-419).
constexpr int kPad = 128;
// Tokens per router block: the unit of the deterministic slot ranking.
constexpr int kTokBlock = 64;

// Codes stored in the device status word (first one wins).
enum Status : int {
    kOk = 0,
    kErrSlotRange = 1,     // a slot / expert / token index left its range
    kErrWaitTimeout = 2,   // a bounded mbarrier wait ran out
    kErrTmemAlloc = 3,
    kErrCapacity = 4,      // expert parallel: more rows were routed to a rank than its grouped buffers hold
};

__device__ __forceinline__ void report(int* status, int code) {
    if (status) atomicCAS(status, 0, code);
}

__device__ __forceinline__ float bf2f(uint16_t v) { return __uint_as_float((uint32_t)v << 16); }
__device__ __forceinline__ float bf_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint16_t f2bf(float f) {
    return __bfloat16_as_ushort(__float2bfloat16_rn(f));
}
// two floats -> packed bf16x2 (lo in the low half), round to nearest even
__device__ __forceinline__ uint32_t pack_bf2(float lo, float hi) {
    return (uint32_t)f2bf(lo) | ((uint32_t)f2bf(hi) << 16);
}
__device__ __forceinline__ float round_bf(float f) { return bf2f(f2bf(f)); }

// tmt-cuda/src/common.h:15-24, same formulas; expf here is the accurate one.
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x * sigmoid_f(x); }
__device__ __forceinline__ float silu_grad_f(float x) {
    float s = sigmoid_f(x);
    return s * (1.0f + x * (1.0f - s));
}
// Epilogue variants (GEMM epilogues run per element on hot tiles): exp and reciprocal
// on the special-function unit. |error| is a few ulp of fp32, far below bf16 rounding.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }

__device__ __forceinline__ uint4 ldg16(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ void stg16(void* p, uint4 v) { *reinterpret_cast<uint4*>(p) = v; }
// 16-byte read-only load that allocates no L1 line: for kernels that share an SM with a CTA whose shared memory leaves the
// L1 a few KB, where lines for rows that are read once would only be fought over.
__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

}  // namespace tmt
