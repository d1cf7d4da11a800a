// NVFP4 expert weights: quantiser (byte-exact with the CPU statement) and the forward
// entry point. e2m1 values, one e4m3 scale per 16 consecutive input elements, one fp32
// scale per tensor:
//   tensor_scale = amax(W) / (6 * 448)      (1 for an all-zero tensor)
//   block scale  = e4m3_rn(amax(block) / 6 / tensor_scale), saturating at 448
//   q            = e2m1_rn(x / (float(block scale) * tensor_scale)), ties to the even code
// Not compiled with fast-math: the divisions must be IEEE.
#include <stdexcept>
#include <cstdlib>

#include "../../include/tmt_norm.h"
#include "moe_internal.h"
#include "nvfp4_decode.h"

namespace tmt {
namespace {

__device__ __forceinline__ float e4m3_to_f(uint8_t v) {
    const int e = (v >> 3) & 15, m = v & 7;
    return e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + m * 0.125f, e - 7);
}
__device__ __forceinline__ uint8_t f_to_e4m3_pos(float f) {
    if (!(f > 0.0f)) return 0;
    if (f >= 448.0f) return 0x7e;
    int ex;
    frexpf(f, &ex);
    int e = ex - 1;
    if (e < -6) e = -6;
    const float q = ldexpf(f, 3 - e);
    const int mant = (int)rintf(q);         // ties to even
    int be = e + 7;
    if (e == -6 && mant < 8) return (uint8_t)mant;
    int mm = mant;
    if (mm == 16) { mm = 8; be += 1; }
    if (be > 15 || (be == 15 && mm - 8 > 6)) return 0x7e;
    return (uint8_t)((be << 3) | (mm - 8));
}
__device__ __forceinline__ uint8_t f_to_e2m1(float x) {
    const uint8_t sign = signbit(x) ? 8 : 0;
    const float a = fabsf(x);
    int code;
    if (a <= 0.25f) code = 0;
    else if (a < 0.75f) code = 1;
    else if (a <= 1.25f) code = 2;
    else if (a < 1.75f) code = 3;
    else if (a <= 2.5f) code = 4;
    else if (a < 3.5f) code = 5;
    else if (a <= 5.0f) code = 6;
    else code = 7;
    return sign | (uint8_t)code;
}

// amax over the tensor: |x| of bf16 as an integer compare (non-negative floats order like ints)
__global__ void amax_kernel(const uint16_t* __restrict__ W, long n, unsigned* __restrict__ out) {
    unsigned m = 0;
    for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x)
        m = max(m, (unsigned)(W[i] & 0x7fffu));
    for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) atomicMax(out, m);
}

// one thread per 16-element block
__global__ void quantize_kernel(const uint16_t* __restrict__ W, long blocks, const unsigned* __restrict__ amax_bits,
                                uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, float* __restrict__ ts_out) {
    const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const float amax = bf2f((uint16_t)*amax_bits);
    const float ts = amax > 0.0f ? amax / (6.0f * 448.0f) : 1.0f;
    if (b == 0) *ts_out = ts;
    if (b >= blocks) return;
    const uint4 v0 = ldg16(W + b * 16), v1 = ldg16(W + b * 16 + 8);
    const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
    float x[16];
    float bmax = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        x[2 * i] = bf_lo(w[i]); x[2 * i + 1] = bf_hi(w[i]);
        bmax = fmaxf(bmax, fmaxf(fabsf(x[2 * i]), fabsf(x[2 * i + 1])));
    }
    const uint8_t sc = f_to_e4m3_pos(bmax / 6.0f / ts);
    scales[b] = sc;
    const float s = e4m3_to_f(sc) * ts;
    uint32_t out[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        const uint32_t q = s > 0.0f ? f_to_e2m1(x[i] / s) : 0;
        out[i >> 3] |= q << ((i & 7) * 4);
    }
    *reinterpret_cast<uint2*>(packed + b * 8) = make_uint2(out[0], out[1]);
}

// bf16(q * block scale): exact (at most 6 significant bits). The tensor scale is applied
// to the GEMM accumulator. This first NVFP4 path keeps the weights packed in the caller's
// memory and expands them once into bf16 scratch for the tensor-core GEMMs; the expansion is
// not fused into the GEMM's operand staging yet.
__global__ void dequantize_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales, long blocks,
                                  uint16_t* __restrict__ W) {
    const long b = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= blocks) return;
    const uint2 pk = *reinterpret_cast<const uint2*>(packed + b * 8);
    const float s = e4m3_to_f(scales[b]);
    const uint32_t wds[2] = {pk.x, pk.y};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float f[2];
#pragma unroll
        for (int hh = 0; hh < 2; ++hh) {
            const uint32_t nib = (wds[(2 * i + hh) >> 3] >> (((2 * i + hh) & 7) * 4)) & 15u;
            const uint32_t c = nib & 7u;
            float v = c < 2 ? 0.5f * c : ldexpf(1.0f + 0.5f * (c & 1u), (int)(c >> 1) - 1);
            f[hh] = (nib & 8u) ? -v * s : v * s;
        }
        o[i] = pack_bf2(f[0], f[1]);
    }
    stg16(W + b * 16, make_uint4(o[0], o[1], o[2], o[3]));
    stg16(W + b * 16 + 8, make_uint4(o[4], o[5], o[6], o[7]));
}

#define CKQ(call)                                                                          \
    do {                                                                                   \
        cudaError_t e__ = (call);                                                          \
        if (e__ != cudaSuccess) throw std::runtime_error(std::string(#call) + " failed: " + cudaGetErrorString(e__)); \
    } while (0)


// Steps of at most this many tokens take the small-batch route (TMT_MOE_DECODE_MAX_TOKENS overrides; 0 turns it off).
int small_batch_limit() {
    const char* s = getenv("TMT_MOE_DECODE_MAX_TOKENS");      // read per call: tests switch routes inside one process
    return s && *s ? atoi(s) : 256;
}

bool small_batch_route(tmt_moe* h, const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown, int tokens) {
    const int E = h->d.experts, D = h->d.dim, H = h->d.hidden;
    if (tokens > small_batch_limit() || (long)tokens * h->d.topk > kDecodeMaxAsg) return false;
    if (!fp4_rows_shape_ok(H, D) || !fp4_rows_shape_ok(D, H)) return false;
    for (int e = 0; e < E; ++e)
        if (((uintptr_t)Wup[e].packed | (uintptr_t)Wup[e].scales | (uintptr_t)Wdown[e].packed | (uintptr_t)Wdown[e].scales) & 15)
            return false;
    return true;
}

// Router and scan as in every forward pass; then the two expert products read the packed weights and the token rows
// directly (no grouped copy of X), one output row per assignment, and a small kernel sums the top-k rows of a token.
void forward_small(tmt_moe* h, const uint16_t* X, const void* Wr, const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown,
                   uint16_t* Y, float beta, int tokens) {
    const int E = h->d.experts, D = h->d.dim, H = h->d.hidden, K = h->d.topk;
    if (!h->q_table) {
        void* p = nullptr;
        CKQ(cudaMalloc(&p, (size_t)E * (4 * sizeof(void*) + 2 * sizeof(float)))); h->allocs.push_back(p); h->q_table = p;
    }
    std::vector<const void*> key(4 * E);
    std::vector<float> sc(2 * E);
    for (int e = 0; e < E; ++e) {
        key[e] = Wup[e].packed; key[E + e] = Wup[e].scales; key[2 * E + e] = Wdown[e].packed; key[3 * E + e] = Wdown[e].scales;
        sc[e] = Wup[e].tensor_scale * 16384.0f; sc[E + e] = Wdown[e].tensor_scale * 16384.0f;     // the kernels carry 2^-14
    }
    const uint8_t* const* tab = static_cast<const uint8_t* const*>(h->q_table);
    float* es = reinterpret_cast<float*>(static_cast<char*>(h->q_table) + (size_t)4 * E * sizeof(void*));
    if (key != h->q_table_key || sc != h->q_table_scales) {
        CKQ(cudaMemcpyAsync(h->q_table, key.data(), key.size() * sizeof(void*), cudaMemcpyHostToDevice, h->stream));
        CKQ(cudaMemcpyAsync(es, sc.data(), sc.size() * sizeof(float), cudaMemcpyHostToDevice, h->stream));
        CKQ(cudaStreamSynchronize(h->stream));      // the host vectors are about to be replaced
        h->q_table_key = key; h->q_table_scales = sc;
    }
    h->dims.T = tokens;
    h->last_tokens = tokens;
    route_only(h, X, Wr);
    Fp4RowsArgs up{};
    up.packed = tab; up.scales = tab + E; up.es = es;
    up.src = h->ln_gamma ? h->xn : X; up.src_ld = D; up.src_div = K;      // fused LayerNorm: the router wrote the normalised rows
    up.out = h->Hact; up.out_ld = H;
    up.idx = h->rb.idx; up.gate = h->rb.w; up.n_asg = tokens * K; up.rows = H; up.kdim = D;
    up.status = h->rb.status;
#ifdef TMT_MOE_MEASURE
    const char* dbg = getenv("TMT_MOE_FP4_DEBUG");            // measurement builds only: results are then wrong
    up.dbg = dbg && *dbg ? atoi(dbg) : 0;
#endif
    prof_mark(h, kPhGemmUp);
    if (!TMT_DBG(up, 8)) CKQ(launch_fp4_rows(up, E, 0, h->stream));        // 8: measurement only, no expert products at all
    Fp4RowsArgs down = up;
    down.packed = tab + 2 * E; down.scales = tab + 3 * E; down.es = es + E;
    down.src = h->Hact; down.src_ld = H; down.src_div = 1;
    down.out = h->Yg; down.out_ld = D; down.rows = D; down.kdim = H;
    prof_mark(h, kPhGemmDown);
    if (!TMT_DBG(up, 8)) CKQ(launch_fp4_rows(down, E, 1, h->stream));
    prof_mark(h, kPhCombine);
    CKQ(launch_decode_combine(h->Yg, Y, beta, tokens, D, K, h->stream));
    prof_mark(h, -1);
    h->launches += 3;
    h->have_forward = true;
}

}  // namespace
}  // namespace tmt

using namespace tmt;

extern "C" {

int tmt_moe_quantize_nvfp4(const void* W, int rows, int cols, void* packed, void* scales, float* tensor_scale_host,
                           void* stream) {
    try {
        if (!W || !packed || !scales || !tensor_scale_host || rows < 1 || cols < 16 || cols % 16)
            throw std::runtime_error("quantize_nvfp4: need non-null pointers and cols % 16 == 0");
        cudaStream_t s = static_cast<cudaStream_t>(stream);
        const long n = (long)rows * cols, blocks = n / 16;
        unsigned* tmp = nullptr;
        CKQ(cudaMalloc(&tmp, 8));
        CKQ(cudaMemsetAsync(tmp, 0, 8, s));
        amax_kernel<<<(unsigned)std::min<long>((n + 255) / 256, 1184), 256, 0, s>>>(static_cast<const uint16_t*>(W), n, tmp);
        quantize_kernel<<<(unsigned)((blocks + 255) / 256), 256, 0, s>>>(static_cast<const uint16_t*>(W), blocks, tmp,
                                                                          static_cast<uint8_t*>(packed),
                                                                          static_cast<uint8_t*>(scales),
                                                                          reinterpret_cast<float*>(tmp + 1));
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpyAsync(tensor_scale_host, tmp + 1, 4, cudaMemcpyDeviceToHost, s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);
        cudaFree(tmp);
        CKQ(e);
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

int tmt_moe_nvfp4_weights_changed(tmt_moe* h) {
    if (!h) { set_error("null handle"); return -1; }
    h->q_key.clear(); h->q_scales_host.clear();             // the next large step expands the weights again
    h->q_table_key.clear(); h->q_table_scales.clear();      // the next small step rebuilds its pointer table
    return 0;
}

int tmt_moe_forward_nvfp4_ln(tmt_moe* h, const void* X, const float* gamma, const float* beta_ln, const void* Wrouter,
                             const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown, void* Y, float beta, int tokens) {
    if (!h) { set_error("null handle"); return -1; }
    try {
        if (!X || !gamma || !beta_ln) throw std::runtime_error("null argument");
        if (tokens < 1 || tokens > h->d.tokens) throw std::runtime_error("tokens outside [1, desc.tokens]");
        if (h->d.dim % 8 || h->d.dim > 8192) throw std::runtime_error("LayerNorm needs dim <= 8192");
        CKQ(cudaSetDevice(h->d.device));
        if (!h->xn) {      // allocated on first use, kept for the handle's lifetime
            void* p = nullptr;
            CKQ(cudaMalloc(&p, (size_t)h->d.tokens * h->d.dim * 2)); h->allocs.push_back(p); h->xn = static_cast<uint16_t*>(p);
            CKQ(cudaMalloc(&p, (size_t)h->d.tokens * 2 * sizeof(float))); h->allocs.push_back(p); h->ln_stats = static_cast<float*>(p);
        }
        RouteDims dd = h->dims;
        dd.T = tokens;
        const bool fused = Wup && Wdown && small_batch_route(h, Wup, Wdown, tokens) && router_takes_layernorm(dd);
        if (fused) {
            struct Clear { tmt_moe* h; ~Clear() { h->ln_gamma = nullptr; h->ln_beta = nullptr; } } clear{h};
            h->ln_gamma = gamma; h->ln_beta = beta_ln;
            return tmt_moe_forward_nvfp4(h, X, Wrouter, Wup, Wdown, Y, beta, tokens);
        }
        // larger batches: the stand-alone LayerNorm kernel, then the block on the normalised rows
        if (tmt_ln_forward(X, gamma, beta_ln, h->xn, h->ln_stats, h->ln_stats + h->d.tokens, tokens, h->d.dim, h->stream) != 0) return -1;
        h->launches += 1;
        return tmt_moe_forward_nvfp4(h, h->xn, Wrouter, Wup, Wdown, Y, beta, tokens);
    } catch (const std::exception& e) { h->ln_gamma = nullptr; h->ln_beta = nullptr; set_error("%s", e.what()); return -1; }
}

int tmt_moe_forward_nvfp4(tmt_moe* h, const void* X, const void* Wrouter, const tmt_nvfp4_weight* Wup,
                          const tmt_nvfp4_weight* Wdown, void* Y, float beta, int tokens) {
    if (!h) { set_error("null handle"); return -1; }
    try {
        const int E = h->d.experts, D = h->d.dim, H = h->d.hidden;
        if (H == 0 || h->d.training || h->d.ep_world > 1)
            throw std::runtime_error("NVFP4 forward needs hidden > 0, training = 0 and a single rank");
        if (!Wup || !Wdown) throw std::runtime_error("null argument");
        CKQ(cudaSetDevice(h->d.device));
        if (!X || !Wrouter || !Y) throw std::runtime_error("null argument");
        if (tokens < 1 || tokens > h->d.tokens) throw std::runtime_error("tokens outside [1, desc.tokens]");
        for (int e = 0; e < E; ++e) {
            if (Wup[e].rows != H || Wup[e].cols != D || Wdown[e].rows != D || Wdown[e].cols != H)
                throw std::runtime_error("NVFP4 weight shape does not match the handle");
            if (!Wup[e].packed || !Wup[e].scales || !Wdown[e].packed || !Wdown[e].scales)
                throw std::runtime_error("null NVFP4 weight pointer");
        }
        if (small_batch_route(h, Wup, Wdown, tokens)) {
            forward_small(h, static_cast<const uint16_t*>(X), Wrouter, Wup, Wdown, static_cast<uint16_t*>(Y), beta, tokens);
            return 0;
        }
        if (!h->q_up) {
            // scratch for the dequantised tiles: allocated on first use, kept for the handle's lifetime
            void* p = nullptr;
            CKQ(cudaMalloc(&p, (size_t)E * H * D * 2)); h->allocs.push_back(p); h->q_up = static_cast<uint16_t*>(p);
            CKQ(cudaMalloc(&p, (size_t)E * H * D * 2)); h->allocs.push_back(p); h->q_down = static_cast<uint16_t*>(p);
            CKQ(cudaMalloc(&p, (size_t)2 * E * sizeof(float))); h->allocs.push_back(p); h->q_scales = static_cast<float*>(p);
            h->q_ptrs_host.resize(2 * E);
            for (int e = 0; e < E; ++e) {
                h->q_ptrs_host[e] = h->q_up + (size_t)e * H * D;
                h->q_ptrs_host[E + e] = h->q_down + (size_t)e * H * D;
            }
        }
        // The dequantised copy is derived data: it is rebuilt only when the caller hands in other weights
        // (other pointers or scales), e.g. once after a checkpoint load; sampling steps reuse it.
        std::vector<const void*> key;
        key.reserve(4 * E);
        std::vector<float> sc(2 * E);
        const long blocks = (long)H * D / 16;
        for (int e = 0; e < E; ++e) {
            sc[e] = Wup[e].tensor_scale; sc[E + e] = Wdown[e].tensor_scale;
            key.push_back(Wup[e].packed); key.push_back(Wup[e].scales); key.push_back(Wdown[e].packed); key.push_back(Wdown[e].scales);
        }
        if (key != h->q_key || sc != h->q_scales_host) {
            for (int e = 0; e < E; ++e) {
                dequantize_kernel<<<(unsigned)((blocks + 255) / 256), 256, 0, h->stream>>>(
                    static_cast<const uint8_t*>(Wup[e].packed), static_cast<const uint8_t*>(Wup[e].scales), blocks,
                    h->q_up + (size_t)e * H * D);
                dequantize_kernel<<<(unsigned)((blocks + 255) / 256), 256, 0, h->stream>>>(
                    static_cast<const uint8_t*>(Wdown[e].packed), static_cast<const uint8_t*>(Wdown[e].scales), blocks,
                    h->q_down + (size_t)e * H * D);
            }
            h->launches += 2 * E;
            CKQ(cudaGetLastError());
            CKQ(cudaMemcpyAsync(h->q_scales, sc.data(), sc.size() * sizeof(float), cudaMemcpyHostToDevice, h->stream));
            h->q_key = key;
            h->q_scales_host = sc;
        }
        h->q_expert_scales = true;
        forward_impl(h, X, Wrouter, h->q_ptrs_host.data(), h->q_ptrs_host.data() + E, Y, beta, tokens);
        h->q_expert_scales = false;
        return 0;
    } catch (const std::exception& e) { h->q_expert_scales = false; set_error("%s", e.what()); return -1; }
}

}  // extern "C"
