// Batched multi-stream sampler session (include/tmt_sampler.h): the NVFP4 MoE decode step of `streams` independent
// byte streams as a replayed CUDA graph over device-resident ring slots, and Generator::sample
// (tmt-cuda/src/generate.h:47-58) as one kernel over all streams. The reference's generator is one stream with five
// blocking copies per byte (generate.h:31-44).
#include <cuda_runtime.h>

#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/tmt_sampler.h"
#include "common.cuh"

namespace tmt {
void set_error(const char* fmt, ...);
}

struct tmt_sampler {
    tmt_sampler_desc d{};
    tmt_moe* moe = nullptr;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    uint16_t* X = nullptr;           // [ring][streams][dim]
    uint16_t* Y = nullptr;           // [ring][streams][dim]
    uint16_t* warm = nullptr;        // [streams][dim] output of the warm-up step
    const void* Wr = nullptr;
    const float* ln_gamma = nullptr; const float* ln_beta = nullptr;     // LayerNorm in front of the block (optional)
    std::vector<tmt_nvfp4_weight> up, down;
    std::vector<cudaGraphExec_t> graphs;     // per slot, nullptr until the slot's first step
    std::vector<float> graph_beta;
    // host rows: uploads and downloads run on streams of their own, ordered against the steps by per-slot events, so the
    // copies of neighbouring decode steps overlap a step's kernels
    cudaStream_t in_stream = nullptr, out_stream = nullptr;
    std::vector<cudaEvent_t> ev_in, ev_step, ev_out;   // upload landed / step done / download done, per slot
    std::vector<unsigned char> pend_in, pend_out, stepped;
    long long steps = 0;
    int recorded = 0;
};

namespace tmt {
namespace {

#define CKS(call)                                                                                  \
    do {                                                                                           \
        cudaError_t e__ = (call);                                                                  \
        if (e__ != cudaSuccess) throw std::runtime_error(std::string(#call) + " failed: " + cudaGetErrorString(e__)); \
    } while (0)

void moe_ok(int rc) {
    if (rc != 0) throw std::runtime_error(tmt_moe_last_error());
}

size_t slot_elems(const tmt_sampler* s) { return (size_t)s->d.streams * s->d.dim; }

// One decode step on the session's stream: with LayerNorm parameters set, X holds the rows before the normalisation.
int queue_step(tmt_sampler* s, const uint16_t* X, uint16_t* Y, float beta) {
    if (s->ln_gamma)
        return tmt_moe_forward_nvfp4_ln(s->moe, X, s->ln_gamma, s->ln_beta, s->Wr, s->up.data(), s->down.data(), Y, beta, s->d.streams);
    return tmt_moe_forward_nvfp4(s->moe, X, s->Wr, s->up.data(), s->down.data(), Y, beta, s->d.streams);
}

void warm_up(tmt_sampler* s) {
    // outside any recording: builds the handle's weight tables (and, for batches above the small-batch limit, the bf16
    // expansion) and the buffer of normalised rows, which involve allocations and host copies a graph cannot hold
    moe_ok(queue_step(s, s->X, s->warm, 0.0f));
    CKS(cudaStreamSynchronize(s->stream));
    if (tmt_moe_device_status(s->moe) != 0) throw std::runtime_error("sampler: device status after the warm-up step");
}

void drop_graphs(tmt_sampler* s) {
    for (cudaGraphExec_t& g : s->graphs)
        if (g) { cudaGraphExecDestroy(g); g = nullptr; }
}

__device__ __forceinline__ unsigned long long splitmix64(unsigned long long x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}

// One block of 256 threads per stream; thread i owns logit i. The sums and the walk along the cumulative
// distribution run in index order in one thread, as the reference's loops do (generate.h:53-56).
__global__ void __launch_bounds__(256) sample_kernel(const uint16_t* __restrict__ logits, float temp, unsigned long long seed,
                                                     long long pos, int* __restrict__ next) {
    __shared__ float l[256];
    __shared__ double p[256];
    __shared__ float wmax[8];
    __shared__ int widx[8];
    const int s = blockIdx.x, i = threadIdx.x, lane = i & 31, warp = i >> 5;
    const float li = bf2f(logits[(long)s * 256 + i]);
    l[i] = li;
    // first maximum (std::max_element, generate.h:50-51): larger value wins, equal values keep the lower index
    float bv = li; int bi = i;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) { wmax[warp] = bv; widx[warp] = bi; }
    __syncthreads();
    float mx = wmax[0]; int best = widx[0];
#pragma unroll
    for (int w = 1; w < 8; ++w)
        if (wmax[w] > mx) { mx = wmax[w]; best = widx[w]; }      // warps are in index order: ties keep the earlier one
    if (temp <= 0.0f) {
        if (i == 0) next[s] = best;
        return;
    }
    p[i] = exp((double)((li - mx) / temp));
    __syncthreads();
    if (i == 0) {
        double sum = 0.0;
        for (int k = 0; k < 256; ++k) sum += p[k];
        const unsigned long long key = splitmix64(seed ^ splitmix64((unsigned long long)s * 0x632BE59BD9B4E019ull + (unsigned long long)pos));
        double r = (double)(key >> 11) * (1.0 / 9007199254740992.0) * sum;
        int pick = 255;
        for (int k = 0; k < 256; ++k)
            if ((r -= p[k]) <= 0) { pick = k; break; }
        next[s] = pick;
    }
}

tmt_sampler* create_impl(const tmt_sampler_desc& d) {
    if (d.streams < 1 || d.ring < 1 || d.ring > 4096) throw std::runtime_error("sampler: need streams >= 1 and 1 <= ring <= 4096");
    if (d.hidden <= 0) throw std::runtime_error("sampler: hidden must be > 0 (NVFP4 experts are two-matrix)");
    std::unique_ptr<tmt_sampler, void (*)(tmt_sampler*)> hold(new tmt_sampler(), [](tmt_sampler* p) { tmt_sampler_destroy(p); });
    tmt_sampler* s = hold.get();
    s->d = d;
    CKS(cudaSetDevice(d.device));
    s->stream = static_cast<cudaStream_t>(d.stream);
    if (!s->stream) {
        CKS(cudaStreamCreateWithFlags(&s->stream, cudaStreamNonBlocking));
        s->own_stream = true;
    }
    tmt_moe_desc md{};
    md.tokens = d.streams; md.dim = d.dim; md.hidden = d.hidden; md.experts = d.experts; md.topk = d.topk;
    md.router_dtype = d.router_dtype; md.training = 0; md.gemm_impl = TMT_MOE_GEMM_AUTO; md.device = d.device;
    md.host_io = 0; md.stream = s->stream; md.ep_world = 1; md.ep_rank = 0;
    moe_ok(tmt_moe_create(&md, &s->moe));
    const size_t n = slot_elems(s);
    CKS(cudaMalloc(&s->X, n * d.ring * 2));
    CKS(cudaMalloc(&s->Y, n * d.ring * 2));
    CKS(cudaMalloc(&s->warm, n * 2));
    CKS(cudaMemsetAsync(s->X, 0, n * d.ring * 2, s->stream));
    CKS(cudaMemsetAsync(s->Y, 0, n * d.ring * 2, s->stream));
    CKS(cudaStreamSynchronize(s->stream));
    s->graphs.assign(d.ring, nullptr);
    s->graph_beta.assign(d.ring, 0.0f);
    CKS(cudaStreamCreateWithFlags(&s->in_stream, cudaStreamNonBlocking));
    CKS(cudaStreamCreateWithFlags(&s->out_stream, cudaStreamNonBlocking));
    s->ev_in.assign(d.ring, nullptr); s->ev_step.assign(d.ring, nullptr); s->ev_out.assign(d.ring, nullptr);
    for (int i = 0; i < d.ring; ++i) {
        CKS(cudaEventCreateWithFlags(&s->ev_in[i], cudaEventDisableTiming));
        CKS(cudaEventCreateWithFlags(&s->ev_step[i], cudaEventDisableTiming));
        CKS(cudaEventCreateWithFlags(&s->ev_out[i], cudaEventDisableTiming));
    }
    s->pend_in.assign(d.ring, 0); s->pend_out.assign(d.ring, 0); s->stepped.assign(d.ring, 0);
    return hold.release();
}

void record_slot(tmt_sampler* s, int slot, float beta) {
    if (s->graphs[slot]) { cudaGraphExecDestroy(s->graphs[slot]); s->graphs[slot] = nullptr; }
    const size_t n = slot_elems(s);
    cudaGraph_t graph = nullptr;
    CKS(cudaStreamBeginCapture(s->stream, cudaStreamCaptureModeThreadLocal));
    const int rc = queue_step(s, s->X + (size_t)slot * n, s->Y + (size_t)slot * n, beta);
    const cudaError_t e = cudaStreamEndCapture(s->stream, &graph);
    if (rc != 0 || e != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        throw std::runtime_error(std::string("sampler: recording the decode step failed: ") +
                                 (rc != 0 ? tmt_moe_last_error() : cudaGetErrorString(e)));
    }
    cudaGraphExec_t exec = nullptr;
    const cudaError_t ie = cudaGraphInstantiate(&exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) throw std::runtime_error(std::string("cudaGraphInstantiate failed: ") + cudaGetErrorString(ie));
    s->graphs[slot] = exec;
    s->graph_beta[slot] = beta;
    s->recorded += 1;
}

void check_slot(const tmt_sampler* s, int slot) {
    if (slot < 0 || slot >= s->d.ring) throw std::runtime_error("sampler: slot outside [0, ring)");
}

}  // namespace
}  // namespace tmt

using namespace tmt;

#define SGUARD(...)                                                      \
    try { __VA_ARGS__; return 0; }                                       \
    catch (const std::exception& e) { set_error("%s", e.what()); return -1; } \
    catch (...) { set_error("unknown error"); return -1; }

extern "C" {

int tmt_sampler_create(const tmt_sampler_desc* desc, tmt_sampler** out) {
    if (!desc || !out) { set_error("null argument"); return -1; }
    *out = nullptr;
    SGUARD(*out = create_impl(*desc))
}

void tmt_sampler_destroy(tmt_sampler* s) {
    if (!s) return;
    cudaSetDevice(s->d.device);
    for (cudaStream_t st : {s->in_stream, s->stream, s->out_stream})
        if (st) cudaStreamSynchronize(st);
    for (auto* v : {&s->ev_in, &s->ev_step, &s->ev_out})
        for (cudaEvent_t e : *v) if (e) cudaEventDestroy(e);
    if (s->in_stream) cudaStreamDestroy(s->in_stream);
    if (s->out_stream) cudaStreamDestroy(s->out_stream);
    drop_graphs(s);
    if (s->moe) tmt_moe_destroy(s->moe);
    for (void* p : {(void*)s->X, (void*)s->Y, (void*)s->warm})
        if (p) cudaFree(p);
    if (s->own_stream && s->stream) cudaStreamDestroy(s->stream);
    delete s;
}

int tmt_sampler_set_weights(tmt_sampler* s, const void* Wrouter, const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown) {
    if (!s) { set_error("null handle"); return -1; }
    SGUARD({
        if (!Wrouter || !Wup || !Wdown) throw std::runtime_error("sampler: null weights");
        CKS(cudaSetDevice(s->d.device));
        drop_graphs(s);
        s->Wr = Wrouter;
        s->up.assign(Wup, Wup + s->d.experts);
        s->down.assign(Wdown, Wdown + s->d.experts);
        moe_ok(tmt_moe_nvfp4_weights_changed(s->moe));
        warm_up(s);
    })
}

int tmt_sampler_set_layernorm(tmt_sampler* s, const float* gamma, const float* beta) {
    if (!s) { set_error("null handle"); return -1; }
    SGUARD({
        if ((gamma == nullptr) != (beta == nullptr)) throw std::runtime_error("sampler: gamma and beta go together");
        CKS(cudaSetDevice(s->d.device));
        drop_graphs(s);
        s->ln_gamma = gamma; s->ln_beta = beta;
        if (s->Wr) warm_up(s);
    })
}

void* tmt_sampler_x(tmt_sampler* s, int slot) { return (!s || slot < 0 || slot >= s->d.ring) ? nullptr : s->X + (size_t)slot * slot_elems(s); }
void* tmt_sampler_y(tmt_sampler* s, int slot) { return (!s || slot < 0 || slot >= s->d.ring) ? nullptr : s->Y + (size_t)slot * slot_elems(s); }
void* tmt_sampler_stream(tmt_sampler* s) { return s ? s->stream : nullptr; }

int tmt_sampler_step(tmt_sampler* s, int slot, float beta) {
    if (!s) { set_error("null handle"); return -1; }
    SGUARD({
        check_slot(s, slot);
        if (!s->Wr) throw std::runtime_error("sampler: tmt_sampler_set_weights has not been called");
        CKS(cudaSetDevice(s->d.device));
        if (!s->graphs[slot] || s->graph_beta[slot] != beta) record_slot(s, slot, beta);
        if (s->pend_in[slot]) { CKS(cudaStreamWaitEvent(s->stream, s->ev_in[slot], 0)); s->pend_in[slot] = 0; }      // the rows have landed
        if (s->pend_out[slot]) { CKS(cudaStreamWaitEvent(s->stream, s->ev_out[slot], 0)); s->pend_out[slot] = 0; }   // the old result has left
        CKS(cudaGraphLaunch(s->graphs[slot], s->stream));
        CKS(cudaEventRecord(s->ev_step[slot], s->stream));
        s->stepped[slot] = 1;
        s->steps += 1;
    })
}

int tmt_sampler_upload(tmt_sampler* s, int slot, const void* X_host) {
    if (!s || !X_host) { set_error("null argument"); return -1; }
    SGUARD({
        check_slot(s, slot);
        CKS(cudaSetDevice(s->d.device));
        if (s->stepped[slot]) CKS(cudaStreamWaitEvent(s->in_stream, s->ev_step[slot], 0));      // the slot's last step has read its rows
        CKS(cudaMemcpyAsync(s->X + (size_t)slot * slot_elems(s), X_host, slot_elems(s) * 2, cudaMemcpyHostToDevice, s->in_stream));
        CKS(cudaEventRecord(s->ev_in[slot], s->in_stream));
        s->pend_in[slot] = 1;
    })
}

int tmt_sampler_download(tmt_sampler* s, int slot, void* Y_host) {
    if (!s || !Y_host) { set_error("null argument"); return -1; }
    SGUARD({
        check_slot(s, slot);
        CKS(cudaSetDevice(s->d.device));
        if (s->stepped[slot]) CKS(cudaStreamWaitEvent(s->out_stream, s->ev_step[slot], 0));     // the slot's last step has written them
        CKS(cudaMemcpyAsync(Y_host, s->Y + (size_t)slot * slot_elems(s), slot_elems(s) * 2, cudaMemcpyDeviceToHost, s->out_stream));
        CKS(cudaEventRecord(s->ev_out[slot], s->out_stream));
        s->pend_out[slot] = 1;
    })
}

int tmt_sampler_sync(tmt_sampler* s) {
    if (!s) { set_error("null handle"); return -1; }
    SGUARD({
        CKS(cudaSetDevice(s->d.device));
        CKS(cudaStreamSynchronize(s->in_stream));
        CKS(cudaStreamSynchronize(s->stream));
        CKS(cudaStreamSynchronize(s->out_stream));
        const int st = tmt_moe_device_status(s->moe);
        if (st != 0) throw std::runtime_error("sampler: device status " + std::to_string(st));
    })
}

int tmt_sampler_sample(tmt_sampler* s, const void* logits, float temp, long long position, int* next_device) {
    if (!s || !logits || !next_device) { set_error("null argument"); return -1; }
    SGUARD({
        CKS(cudaSetDevice(s->d.device));
        sample_kernel<<<s->d.streams, 256, 0, s->stream>>>(static_cast<const uint16_t*>(logits), temp, (unsigned long long)s->d.seed,
                                                           position, next_device);
        CKS(cudaGetLastError());
    })
}

long long tmt_sampler_steps(const tmt_sampler* s) { return s ? s->steps : -1; }
int tmt_sampler_graphs(const tmt_sampler* s) { return s ? s->recorded : -1; }

}  // extern "C"
