// Expert parallelism: experts are partitioned over the ranks of one NCCL communicator (one
// process per GPU, rank g owns experts [g*E/G, (g+1)*E/G)). Every rank routes its own tokens;
// grouped rows travel to the owning rank, run through the grouped GEMMs there and travel back.
// The reference has no counterpart (single GPU, no communication library).
//
// Two transports (desc.ep_transport):
//   TMT_MOE_EP_PEER (default): the four permutation kernels address the owner's buffers directly
//     over NVLink (peer memory mapped with CUDA IPC): dispatch and the gradient dispatch STORE rows
//     into the owner's grouped buffer, combine and scatter LOAD rows from it. No send buffer, no
//     separate exchange pass: the all-to-all is fused into the gather / scatter kernels. Ranks
//     meet at stream-ordered NCCL barriers (a one-word all-reduce) between writer and reader
//     kernels. Only plain loads and stores touch peer memory; TMA reads local memory only.
//   TMT_MOE_EP_NCCL: dispatch into a local send buffer, then ONE NCCL group of point-to-point
//     sends and receives per exchange, one message per (peer, expert) pair, so that rows land
//     directly in their expert group on the owner and come back directly into the token-side
//     slots (no re-permutation pass).
// Both size everything from an all-gather of the per-expert counts, read on the host once per
// step (it doubles as the barrier that separates two steps).
//
// NCCL is bound at run time (dlopen of the process's libnccl.so.2): the library has no link
// dependency on it, and a host program that never uses expert parallelism does not need it.
#include <dlfcn.h>
#include <nccl.h>

#include <algorithm>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "gemm.cuh"
#include "moe_internal.h"

struct tmt_ep_state {
    void* lib = nullptr;
    ncclComm_t comm = nullptr;
    // second stream of the peer transport: rank barriers and row transfers that run under GEMMs of the main stream
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    static constexpr int kMaxWaves = 4;
    cudaEvent_t ev_sent[kMaxWaves] = {}, ev_done[kMaxWaves] = {};     // a wave's rows have landed / its GEMMs are done
    bool overlap = true;              // TMT_MOE_EP_OVERLAP=0 switches the second stream off (measurement)
    int waves = 1;                    // TMT_MOE_EP_WAVES: expert waves of both passes. Peer transport: four from four ranks up (measured
                                      // at 4 GPUs: 2-4 % faster than one exchange per pass), none at two ranks, where half of the
                                      // rows never leave the GPU and the waves cost 1-3 ms more than they hide.
    int fetch_waves = -1;             // TMT_MOE_EP_FETCH: how many of the forward waves' output rows are fetched under later GEMMs
                                      // (the final combine reads the others from their owners itself); -1: all
    bool thin = true;                 // TMT_MOE_EP_THIN=0: the waves after the first use the full-size row kernels again (measurement)
    int side_sms = 0;                 // TMT_MOE_EP_SMS: > 0 keeps that many SMs for the side stream's row kernels instead of
                                      // letting their blocks share SMs with the GEMM CTAs
    int G = 1, r = 0, EL = 0;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    // token side (cap rows, padded layout by global expert)
    uint16_t *Xs = nullptr, *Yr = nullptr, *dYs = nullptr, *dXr = nullptr;
    // expert side layout (x_cap rows): tables live in one device block, filled from the host each step
    int x_cap = 0, x_max_tiles = 0;
    int* x_tables = nullptr;          // [EL+1] poff | [EL] counts | [1] num tiles | [x_max_tiles] tile -> expert
    std::vector<int> x_tables_host;
    int* cnt_all_dev = nullptr;       // [G][E]
    std::vector<int> cnt_all, tok_poff, x_counts, x_poff, src_off;
    float* stat_global = nullptr;     // E+1
    // peer transport: owners' buffers as seen from this process, [G] pointers each, on the device
    bool peer = false;
    bool dma = false;                 // TMT_MOE_EP_DMA: rows cross NVLink as peer-to-peer copies of the copy engines
    std::vector<uint16_t*> peer_tab_host;   // [4][G] the same addresses on the host (sources / destinations of those copies)
    std::vector<cudaStream_t> copy_streams; // DMA transport: one stream per owner, so that several copy engines and links work at once
    std::vector<cudaEvent_t> copy_done;
    cudaEvent_t copy_go = nullptr;
    uint16_t** peer_Xg = nullptr; uint16_t** peer_Yg = nullptr; uint16_t** peer_dYg = nullptr; uint16_t** peer_dXg = nullptr;
    std::vector<void*> opened;        // cudaIpcOpenMemHandle results to close
    int* dest_row0 = nullptr;         // [E] this rank's first row inside the owner's group of expert e
    std::vector<int> dest_row0_host;
    uint16_t* Xc = nullptr;           // [T_pad][D] X in token order (router weight gradient)
    int* bar_word = nullptr;
    // Peer transport without expert waves: the exchange plan is computed on the device from the gathered counts, and the
    // step has no host synchronisation. TMT_MOE_EP_HOST_PLAN=1 keeps the host plan (measurement; the NCCL transport and
    // expert waves always use it: their message sizes and tile ranges are host values).
    bool device_plan = false;
};

namespace tmt {
namespace {

#define CKE(call)                                                                                              \
    do {                                                                                                       \
        cudaError_t e__ = (call);                                                                              \
        if (e__ != cudaSuccess) throw std::runtime_error(std::string(#call) + " failed: " + cudaGetErrorString(e__)); \
    } while (0)

#define NC(ep, call)                                                                                           \
    do {                                                                                                       \
        ncclResult_t r__ = (call);                                                                             \
        if (r__ != ncclSuccess)                                                                                \
            throw std::runtime_error(std::string(#call) + " failed: " + ((ep)->GetErrorString ? (ep)->GetErrorString(r__) : "?")); \
    } while (0)

template <class F>
void bind(void* lib, const char* name, F& fn) {
    fn = reinterpret_cast<F>(dlsym(lib, name));
    if (!fn) throw std::runtime_error(std::string("NCCL symbol missing: ") + name);
}

void load_nccl(tmt_ep_state* ep) {
    if (ep->lib) return;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    for (const char* n : names) {
        ep->lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (ep->lib) break;
    }
    if (!ep->lib) throw std::runtime_error("libnccl.so.2 not found (expert parallelism needs NCCL in the process)");
    bind(ep->lib, "ncclGetUniqueId", ep->GetUniqueId);
    bind(ep->lib, "ncclCommInitRank", ep->CommInitRank);
    bind(ep->lib, "ncclCommDestroy", ep->CommDestroy);
    bind(ep->lib, "ncclGroupStart", ep->GroupStart);
    bind(ep->lib, "ncclGroupEnd", ep->GroupEnd);
    bind(ep->lib, "ncclSend", ep->Send);
    bind(ep->lib, "ncclRecv", ep->Recv);
    bind(ep->lib, "ncclAllGather", ep->AllGather);
    bind(ep->lib, "ncclAllReduce", ep->AllReduce);
    bind(ep->lib, "ncclGetErrorString", ep->GetErrorString);
}

template <class T>
T* ep_alloc(tmt_moe* h, size_t n) {
    void* p = nullptr;
    CKE(cudaMalloc(&p, std::max<size_t>(n, 1) * sizeof(T)));
    h->allocs.push_back(p);
    h->bytes += n * sizeof(T);
    return static_cast<T*>(p);
}

}  // namespace
}  // namespace tmt

using namespace tmt;

extern "C" {

// Pure host arithmetic of one exchange plan (testable without a GPU). cnt_all[g*E + e] = rows
// rank g routes to global expert e. Outputs for rank r: tok_poff[E+1] (token-side group starts,
// padded to `pad`), x_counts[EL] / x_poff[EL+1] (expert-side groups of the local experts, rows
// of all sources concatenated in source order, padded), src_off[s*EL + le] (start of source s's
// rows inside local group le). Returns the expert-side row count x_poff[EL], or -1.
long long tmt_moe_ep_plan(int G, int r, int E, int pad, const int* cnt_all, int* tok_poff, int* x_counts,
                          int* x_poff, int* src_off) {
    if (G < 1 || r < 0 || r >= G || E < 1 || E % G || pad < 1 || !cnt_all) return -1;
    const int EL = E / G;
    long long p = 0;
    for (int e = 0; e < E; ++e) {
        tok_poff[e] = (int)p;
        p += (cnt_all[(size_t)r * E + e] + pad - 1) / pad * pad;
    }
    tok_poff[E] = (int)p;
    long long xp = 0;
    for (int le = 0; le < EL; ++le) {
        int n = 0;
        for (int s = 0; s < G; ++s) {
            src_off[(size_t)s * EL + le] = n;
            n += cnt_all[(size_t)s * E + r * EL + le];
        }
        x_counts[le] = n;
        x_poff[le] = (int)xp;
        xp += (n + pad - 1) / pad * pad;
        if (xp > 0x7fffffffLL) return -1;
    }
    x_poff[EL] = (int)xp;
    return xp;
}

// Every rank's expert-side row count against the capacity, from the all-gathered counts that every rank holds:
// all ranks reach the same verdict for a step, so an overloaded rank never leaves its peers waiting in an exchange.
// Returns -1 when every rank fits, otherwise the lowest rank that does not (its row count in *rows_out); -2 on bad arguments.
int tmt_moe_ep_check_capacity(int G, int E, int pad, const int* cnt_all, long long x_cap, long long* rows_out) {
    if (G < 1 || E < 1 || E % G || pad < 1 || !cnt_all) return -2;
    const int EL = E / G;
    for (int g = 0; g < G; ++g) {
        long long rows = 0;
        for (int le = 0; le < EL; ++le) {
            long long n = 0;
            for (int s = 0; s < G; ++s) n += cnt_all[(size_t)s * E + g * EL + le];
            rows += (n + pad - 1) / pad * pad;
        }
        if (rows > x_cap || rows > 0x7fffffffLL) {
            if (rows_out) *rows_out = rows;
            return g;
        }
    }
    return -1;
}

int tmt_moe_ep_unique_id(void* id128) {
    try {
        if (!id128) throw std::runtime_error("null argument");
        tmt_ep_state tmp;
        load_nccl(&tmp);
        ncclUniqueId id;
        NC(&tmp, tmp.GetUniqueId(&id));
        static_assert(sizeof(id) == 128, "ncclUniqueId is 128 bytes");
        memcpy(id128, &id, sizeof id);
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

int tmt_moe_ep_init(tmt_moe* h, const void* id128) {
    if (!h || !id128) { set_error("null argument"); return -1; }
    try {
        if (h->d.ep_world < 2) throw std::runtime_error("handle was created with ep_world = 1");
        if (h->ep) throw std::runtime_error("expert parallelism is already initialised");
        if (h->d.hidden == 0) throw std::runtime_error("expert parallelism needs the two-matrix mode (hidden > 0)");
        CKE(cudaSetDevice(h->d.device));
        std::unique_ptr<tmt_ep_state> ep(new tmt_ep_state());
        load_nccl(ep.get());
        ep->G = h->d.ep_world; ep->r = h->d.ep_rank; ep->EL = h->local_experts;
        ncclUniqueId id;
        memcpy(&id, id128, sizeof id);
        NC(ep.get(), ep->CommInitRank(&ep->comm, ep->G, id, ep->r));
        const int E = h->d.experts, D = h->d.dim;
        const size_t cap = h->dims.cap;
        ep->peer = h->d.ep_transport == TMT_MOE_EP_PEER;
        ep->dma = h->d.ep_transport == TMT_MOE_EP_DMA;
        if (h->d.ep_transport < 0 || h->d.ep_transport > TMT_MOE_EP_DMA) throw std::runtime_error("unknown ep_transport");
        const bool maps = ep->peer || ep->dma;         // both address the owners' buffers through CUDA IPC mappings
        if (maps) {
            if (const char* ov = getenv("TMT_MOE_EP_OVERLAP")) ep->overlap = atoi(ov) != 0;
            if (const char* th = getenv("TMT_MOE_EP_THIN")) ep->thin = atoi(th) != 0;
            if (const char* fw = getenv("TMT_MOE_EP_FETCH")) ep->fetch_waves = atoi(fw);
            if (const char* sm = getenv("TMT_MOE_EP_SMS")) ep->side_sms = std::max(0, std::min(atoi(sm), h->num_sms / 2));
            if (ep->dma) ep->waves = tmt_ep_state::kMaxWaves;     // copy-engine transfers overlap the GEMMs cleanly: waves by default
            if (ep->peer && ep->G >= 4 && h->two_cta) ep->waves = tmt_ep_state::kMaxWaves;   // the later waves' row kernels fit beside the CTA-pair GEMM only
            if (const char* wv = getenv("TMT_MOE_EP_WAVES")) ep->waves = std::max(1, std::min(atoi(wv), (int)tmt_ep_state::kMaxWaves));
            ep->waves = std::min(ep->waves, ep->EL);
            const char* hp = getenv("TMT_MOE_EP_HOST_PLAN");
            ep->device_plan = ep->peer && ep->waves < 2 && E <= 256 && ep->G <= 256 && !(hp && atoi(hp) != 0);
            for (int w = 0; w < tmt_ep_state::kMaxWaves; ++w) {
                CKE(cudaEventCreateWithFlags(&ep->ev_sent[w], cudaEventDisableTiming));
                CKE(cudaEventCreateWithFlags(&ep->ev_done[w], cudaEventDisableTiming));
            }
            CKE(cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking));
            CKE(cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming));
            CKE(cudaEventCreateWithFlags(&ep->ev_join, cudaEventDisableTiming));
        }
        ep->Yr = ep_alloc<uint16_t>(h, cap * D);
        ep->bar_word = ep_alloc<int>(h, 1);
        CKE(cudaMemsetAsync(ep->bar_word, 0, sizeof(int), h->stream));
        if (maps) {
            if (ep->peer) {
                const size_t tpad = (size_t)(h->d.tokens + h->pad - 1) / h->pad * h->pad;
                ep->Xc = ep_alloc<uint16_t>(h, tpad * D);
                CKE(cudaMemsetAsync(ep->Xc, 0, tpad * D * 2, h->stream));
            }
            ep->dest_row0 = ep_alloc<int>(h, E);
            ep->dest_row0_host.assign(E, 0);
            // exchange CUDA IPC handles of the four buffers peers write to or read from
            const int nbuf = h->d.training ? 4 : 2;
            void* mine[4] = {h->Xg, h->Yg, h->dYg, h->dXg};
            std::vector<cudaIpcMemHandle_t> local(4), all((size_t)4 * ep->G);
            for (int i = 0; i < nbuf; ++i) CKE(cudaIpcGetMemHandle(&local[i], mine[i]));
            unsigned char* dev_handles = ep_alloc<unsigned char>(h, sizeof(cudaIpcMemHandle_t) * 4 * (ep->G + 1));
            CKE(cudaMemcpyAsync(dev_handles, local.data(), sizeof(cudaIpcMemHandle_t) * 4, cudaMemcpyHostToDevice, h->stream));
            NC(ep.get(), ep->AllGather(dev_handles, dev_handles + sizeof(cudaIpcMemHandle_t) * 4, sizeof(cudaIpcMemHandle_t) * 4,
                                       ncclUint8, ep->comm, h->stream));
            CKE(cudaMemcpyAsync(all.data(), dev_handles + sizeof(cudaIpcMemHandle_t) * 4, sizeof(cudaIpcMemHandle_t) * 4 * ep->G,
                                cudaMemcpyDeviceToHost, h->stream));
            CKE(cudaStreamSynchronize(h->stream));
            std::vector<uint16_t*> tab((size_t)4 * ep->G, nullptr);
            for (int g = 0; g < ep->G; ++g)
                for (int i = 0; i < nbuf; ++i) {
                    if (g == ep->r) { tab[(size_t)i * ep->G + g] = static_cast<uint16_t*>(mine[i]); continue; }
                    void* p = nullptr;
                    CKE(cudaIpcOpenMemHandle(&p, all[(size_t)g * 4 + i], cudaIpcMemLazyEnablePeerAccess));
                    ep->opened.push_back(p);
                    tab[(size_t)i * ep->G + g] = static_cast<uint16_t*>(p);
                }
            uint16_t** dev_tab = ep_alloc<uint16_t*>(h, tab.size());
            CKE(cudaMemcpyAsync(dev_tab, tab.data(), tab.size() * sizeof(uint16_t*), cudaMemcpyHostToDevice, h->stream));
            CKE(cudaStreamSynchronize(h->stream));
            ep->peer_Xg = dev_tab; ep->peer_Yg = dev_tab + ep->G; ep->peer_dYg = dev_tab + 2 * ep->G; ep->peer_dXg = dev_tab + 3 * ep->G;
            ep->peer_tab_host = tab;
            if (ep->dma) {
                ep->copy_streams.assign(ep->G, nullptr);
                ep->copy_done.assign(ep->G, nullptr);
                for (int g = 0; g < ep->G; ++g) {
                    CKE(cudaStreamCreateWithFlags(&ep->copy_streams[g], cudaStreamNonBlocking));
                    CKE(cudaEventCreateWithFlags(&ep->copy_done[g], cudaEventDisableTiming));
                }
                CKE(cudaEventCreateWithFlags(&ep->copy_go, cudaEventDisableTiming));
                // X in token order for the router weight gradient, kept by the local dispatch kernel as on one GPU
                const size_t tpad = (size_t)(h->d.tokens + h->pad - 1) / h->pad * h->pad;
                ep->Xc = ep_alloc<uint16_t>(h, tpad * D);
                CKE(cudaMemsetAsync(ep->Xc, 0, tpad * D * 2, h->stream));
                if (h->d.training) h->Xc = ep->Xc;
            }
        }
        if (!ep->peer) {
            ep->Xs = ep_alloc<uint16_t>(h, cap * D);
            if (h->d.training) {
                ep->dYs = ep_alloc<uint16_t>(h, cap * D);
                ep->dXr = ep_alloc<uint16_t>(h, cap * D);
            }
        }
        ep->x_cap = h->x_cap;
        ep->x_max_tiles = ep->x_cap / kPad;
        ep->x_tables_host.assign((size_t)2 * ep->EL + 2 + ep->x_max_tiles, 0);
        ep->x_tables = ep_alloc<int>(h, ep->x_tables_host.size());
        ep->cnt_all_dev = ep_alloc<int>(h, (size_t)ep->G * E);
        ep->cnt_all.assign((size_t)ep->G * E, 0);
        ep->tok_poff.assign(E + 1, 0);
        ep->x_counts.assign(ep->EL, 0);
        ep->x_poff.assign(ep->EL + 1, 0);
        ep->src_off.assign((size_t)ep->G * ep->EL, 0);
        ep->stat_global = ep_alloc<float>(h, E + 1);
        h->ep_world_counts = ep_alloc<int>(h, E);
        h->ep = ep.release();
        const bool tok_order = h->ep->peer || (h->ep->dma && h->d.training);
        build_ep_maps(h, tok_order ? h->ep->Xc : h->ep->Xs, tok_order);
        return 0;
    } catch (const std::exception& e) { set_error("%s", e.what()); return -1; }
}

}  // extern "C"

namespace tmt {

void ep_teardown(tmt_moe* h) {
    if (!h->ep) return;
    for (void* p : h->ep->opened) cudaIpcCloseMemHandle(p);
    for (cudaStream_t st : h->ep->copy_streams) if (st) { cudaStreamSynchronize(st); cudaStreamDestroy(st); }
    for (cudaEvent_t e : h->ep->copy_done) if (e) cudaEventDestroy(e);
    if (h->ep->copy_go) cudaEventDestroy(h->ep->copy_go);
    if (h->ep->side) cudaStreamDestroy(h->ep->side);
    if (h->ep->ev_fork) cudaEventDestroy(h->ep->ev_fork);
    if (h->ep->ev_join) cudaEventDestroy(h->ep->ev_join);
    for (cudaEvent_t e : h->ep->ev_sent) if (e) cudaEventDestroy(e);
    for (cudaEvent_t e : h->ep->ev_done) if (e) cudaEventDestroy(e);
    if (h->ep->comm && h->ep->CommDestroy) h->ep->CommDestroy(h->ep->comm);
    delete h->ep;
    h->ep = nullptr;
}

namespace {

// The exchange plan on the device, one block: what plan_step computes on the host (tmt_moe_ep_plan for every owner,
// the capacity check, the tile table) from cnt_all[g][e] = rows rank g routes to expert e. tables = [EL+1] padded group
// starts | [EL] counts | [1] number of 128-row tiles | [max_tiles] tile -> local expert (-1 past the end).
__global__ void __launch_bounds__(256) ep_plan_kernel(int G, int r, int E, int EL, int pad, int x_cap, int max_tiles,
                                                      const int* __restrict__ cnt_all, int* __restrict__ tables,
                                                      int* __restrict__ dest_row0, int* __restrict__ world, int* status) {
    __shared__ int tot[256], padded[256], before_me[256], opoff[257];
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int n = 0, mine = 0;
        for (int g = 0; g < G; ++g) {
            const int c = cnt_all[g * E + e];
            if (g < r) mine += c;            // rows of lower ranks come first inside the owner's group (source order)
            n += c;
        }
        tot[e] = n; before_me[e] = mine;
        padded[e] = (n + pad - 1) / pad * pad;
        world[e] = n;
    }
    __syncthreads();
    if (threadIdx.x < G) {                   // one thread per owner: padded starts of its EL groups, capacity check
        const int g = threadIdx.x;
        long long p = 0;
        for (int le = 0; le < EL; ++le) { opoff[g * EL + le] = (int)p; p += padded[g * EL + le]; }
        if (p > x_cap) report(status, kErrCapacity);
        if (g == r) opoff[256] = (int)(p > x_cap ? x_cap / pad * pad : p);
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) dest_row0[e] = opoff[e] + before_me[e];
    const int rows = opoff[256];
    for (int le = threadIdx.x; le < EL; le += blockDim.x) {
        tables[le] = min(opoff[r * EL + le], rows);
        tables[EL + 1 + le] = tot[r * EL + le];
    }
    if (threadIdx.x == 0) { tables[EL] = rows; tables[2 * EL + 1] = rows / kPad; }
    int* te = tables + 2 * EL + 2;
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) {
        const int row = i * kPad;
        int le = -1;
        if (row < rows)
            for (int q = 0; q < EL; ++q)
                if (row >= opoff[r * EL + q] && row < opoff[r * EL + q] + padded[r * EL + q]) le = q;
        te[i] = le;
    }
}

// Pad rows of the expert-side groups read as zero (they feed the weight-gradient GEMMs): block = one local expert,
// rows from the device tables.
__global__ void __launch_bounds__(256) ep_zero_pads_kernel(const int* __restrict__ tables, int EL, uint16_t* __restrict__ buf, int width,
                                                           int x_cap) {
    const int le = blockIdx.x;
    const long r0 = (long)tables[le] + tables[EL + 1 + le], r1 = min(tables[le + 1], x_cap);
    const long n = (r1 - r0) * (width / 8);
    uint4* dst = reinterpret_cast<uint4*>(buf + r0 * width);
    for (long i = threadIdx.x; i < n; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
}

void plan_step_device(tmt_moe* h) {
    tmt_ep_state* ep = h->ep;
    const int E = h->d.experts;
    NC(ep, ep->AllGather(h->rb.counts, ep->cnt_all_dev, E, ncclInt32, ep->comm, h->stream));
    ep_plan_kernel<<<1, 256, 0, h->stream>>>(ep->G, ep->r, E, ep->EL, h->pad, ep->x_cap, ep->x_max_tiles, ep->cnt_all_dev, ep->x_tables,
                                             ep->dest_row0, h->ep_world_counts, h->rb.status);
    CKE(cudaGetLastError());
    h->launches += 2;
}

// Counts of every rank -> host, exchange plan, expert-side tables -> device. One stream sync.
void plan_step(tmt_moe* h) {
    if (h->ep->device_plan) { plan_step_device(h); return; }
    tmt_ep_state* ep = h->ep;
    const int E = h->d.experts, G = ep->G, EL = ep->EL;
    NC(ep, ep->AllGather(h->rb.counts, ep->cnt_all_dev, E, ncclInt32, ep->comm, h->stream));
    CKE(cudaMemcpyAsync(ep->cnt_all.data(), ep->cnt_all_dev, (size_t)G * E * sizeof(int), cudaMemcpyDeviceToHost, h->stream));
    CKE(cudaStreamSynchronize(h->stream));
    // Both transports: the verdict is the same on every rank (same cnt_all), so all of them refuse the step together,
    // before any row moves; no rank is left waiting for a partner that threw.
    long long over_rows = 0;
    const int over = tmt_moe_ep_check_capacity(G, E, h->pad, ep->cnt_all.data(), ep->x_cap, &over_rows);
    if (over != -1)
        throw std::runtime_error("expert-side capacity exceeded on rank " + std::to_string(over) + ": " + std::to_string(over_rows) +
                                 " rows routed to it, room for " + std::to_string(ep->x_cap) + " (raise desc.ep_capacity_factor)");
    const long long rows = tmt_moe_ep_plan(G, ep->r, E, h->pad, ep->cnt_all.data(), ep->tok_poff.data(), ep->x_counts.data(),
                                           ep->x_poff.data(), ep->src_off.data());
    if (rows < 0) throw std::runtime_error("exchange plan failed");
    int* t = ep->x_tables_host.data();
    memcpy(t, ep->x_poff.data(), (EL + 1) * sizeof(int));
    memcpy(t + EL + 1, ep->x_counts.data(), EL * sizeof(int));
    t[2 * EL + 1] = (int)(rows / kPad);
    int* te = t + 2 * EL + 2;
    std::fill(te, te + ep->x_max_tiles, -1);
    for (int le = 0; le < EL; ++le)
        for (int i = ep->x_poff[le] / kPad; i < ep->x_poff[le + 1] / kPad; ++i) te[i] = le;
    CKE(cudaMemcpyAsync(ep->x_tables, t, ep->x_tables_host.size() * sizeof(int), cudaMemcpyHostToDevice, h->stream));
    if (ep->peer || ep->dma) {
        // where this rank's rows start inside the owner's group: the owner's plan, computed here as well
        std::vector<int> o_tok(E + 1), o_cnt(EL), o_poff(EL + 1), o_src((size_t)G * EL);
        for (int g = 0; g < G; ++g) {
            tmt_moe_ep_plan(G, g, E, h->pad, ep->cnt_all.data(), o_tok.data(), o_cnt.data(), o_poff.data(), o_src.data());
            for (int le = 0; le < EL; ++le) ep->dest_row0_host[g * EL + le] = o_poff[le] + o_src[(size_t)ep->r * EL + le];
        }
        CKE(cudaMemcpyAsync(ep->dest_row0, ep->dest_row0_host.data(), E * sizeof(int), cudaMemcpyHostToDevice, h->stream));
    }
    std::vector<int> world(E, 0);
    for (int g = 0; g < G; ++g)
        for (int e = 0; e < E; ++e) world[e] += ep->cnt_all[(size_t)g * E + e];
    CKE(cudaMemcpyAsync(h->ep_world_counts, world.data(), E * sizeof(int), cudaMemcpyHostToDevice, h->stream));
    h->launches += 1;
}

// Pad rows of the expert-side groups must read as zero (they feed the weight-gradient GEMMs).
void zero_pads(tmt_moe* h, uint16_t* buf, int width) {
    tmt_ep_state* ep = h->ep;
    if (ep->device_plan) {
        ep_zero_pads_kernel<<<ep->EL, 256, 0, h->stream>>>(ep->x_tables, ep->EL, buf, width, ep->x_cap);
        CKE(cudaGetLastError());
        h->launches += 1;
        return;
    }
    for (int le = 0; le < ep->EL; ++le) {
        const size_t r0 = (size_t)ep->x_poff[le] + ep->x_counts[le], r1 = ep->x_poff[le + 1];
        if (r1 > r0) CKE(cudaMemsetAsync(buf + r0 * width, 0, (r1 - r0) * width * 2, h->stream));
    }
}

// to_experts: token-side groups -> owning ranks' expert-side groups; otherwise the way back.
void exchange(tmt_moe* h, bool to_experts, const uint16_t* src, uint16_t* dst, int width) {
    tmt_ep_state* ep = h->ep;
    const int E = h->d.experts, G = ep->G, EL = ep->EL, r = ep->r;
    prof_mark(h, kPhExchange);
    NC(ep, ep->GroupStart());
    for (int g = 0; g < G; ++g)
        for (int le = 0; le < EL; ++le) {
            const int e = g * EL + le;
            const size_t n_tok = (size_t)ep->cnt_all[(size_t)r * E + e];                 // my rows for expert e (owner g)
            const size_t n_exp = (size_t)ep->cnt_all[(size_t)g * E + r * EL + le];       // rank g's rows for my expert le
            const size_t tok_row = ep->tok_poff[e];
            const size_t exp_row = (size_t)ep->x_poff[le] + ep->src_off[(size_t)g * EL + le];
            if (to_experts) {
                if (n_tok) NC(ep, ep->Send(src + tok_row * width, n_tok * width, ncclBfloat16, g, ep->comm, h->stream));
                if (n_exp) NC(ep, ep->Recv(dst + exp_row * width, n_exp * width, ncclBfloat16, g, ep->comm, h->stream));
            } else {
                if (n_exp) NC(ep, ep->Send(src + exp_row * width, n_exp * width, ncclBfloat16, g, ep->comm, h->stream));
                if (n_tok) NC(ep, ep->Recv(dst + tok_row * width, n_tok * width, ncclBfloat16, g, ep->comm, h->stream));
            }
        }
    NC(ep, ep->GroupEnd());
    h->launches += 1;
}

// The DMA transport's row movement: one peer-to-peer copy (copy engine, no SM) per (owner, expert) segment of this rank's
// token-side groups, for the local experts [le_lo, le_hi) of every owner. push: local rows -> the owner's group (buffer
// `which` of the mapped tables); otherwise the owner's rows -> the local buffer. Owners are visited starting after this
// rank, so that at any moment the ranks target different owners.
void dma_rows(tmt_moe* h, bool push, int which, uint16_t* local, int le_lo, int le_hi, int width, cudaStream_t stream) {
    tmt_ep_state* ep = h->ep;
    const int E = h->d.experts, G = ep->G, EL = ep->EL, r = ep->r;
    // every owner's copies run on a stream of their own (fork from `stream`, join back into it)
    CKE(cudaEventRecord(ep->copy_go, stream));
    for (int i = 0; i < G; ++i) {
        const int g = (r + 1 + i) % G;
        cudaStream_t cs = ep->copy_streams[g];
        CKE(cudaStreamWaitEvent(cs, ep->copy_go, 0));
        uint16_t* owner = ep->peer_tab_host[(size_t)which * G + g];
        for (int le = le_lo; le < le_hi; ++le) {
            const int e = g * EL + le;
            const size_t n = (size_t)ep->cnt_all[(size_t)r * E + e];
            if (!n) continue;
            uint16_t* mine = local + (size_t)ep->tok_poff[e] * width;
            uint16_t* theirs = owner + (size_t)ep->dest_row0_host[e] * width;
            CKE(cudaMemcpyAsync(push ? theirs : mine, push ? mine : theirs, n * width * 2, cudaMemcpyDeviceToDevice, cs));
        }
        CKE(cudaEventRecord(ep->copy_done[g], cs));
        CKE(cudaStreamWaitEvent(stream, ep->copy_done[g], 0));
    }
    h->launches += 1;
}

// Stream-ordered meeting point of all ranks: when it completes here, every rank's stream has reached it.
void rank_barrier(tmt_moe* h, cudaStream_t stream = nullptr) {
    tmt_ep_state* ep = h->ep;
    NC(ep, ep->AllReduce(ep->bar_word, ep->bar_word, 1, ncclInt32, ncclSum, ep->comm, stream ? stream : h->stream));
    h->launches += 1;
}

PeerMap peer_map(tmt_moe* h, uint16_t** table, bool beside_gemm = false) {
    PeerMap pm;
    pm.base = table; pm.dest_row0 = h->ep->dest_row0; pm.experts_per_rank = h->ep->EL;
    pm.row_limit = h->ep->x_cap; pm.status = h->rb.status;
    if (beside_gemm && h->ep->side_sms > 0) pm.pad_smem = 4096;
    return pm;
}
int gemm_sms_beside_rows(tmt_moe* h) { return h->num_sms - std::max(2, h->ep->side_sms); }

void use_expert_layout(tmt_moe* h) {
    tmt_ep_state* ep = h->ep;
    h->g_poff = ep->x_tables;
    h->g_num_m_tiles = ep->x_tables + 2 * ep->EL + 1;
    h->g_tile_expert = ep->x_tables + 2 * ep->EL + 2;
    h->g_max_tiles = ep->x_max_tiles;
}

}  // namespace

void ep_forward(tmt_moe* h, const void* X, const void* Wr, const void* const* Wup, const void* const* Wdown, void* Y,
                float beta, int tokens) {
    tmt_ep_state* ep = h->ep;
    if (!ep) throw std::runtime_error("expert parallelism is not initialised on this handle (tmt_moe_ep_init)");
    if (tokens != h->d.tokens) throw std::runtime_error("expert-parallel steps carry exactly desc.tokens rows");
    if (!X || !Wr || !Wup || !Wdown || !Y) throw std::runtime_error("null argument");
    CKE(cudaSetDevice(h->d.device));
    use_expert_layout(h);
    h->dims.T = tokens;
    h->last_tokens = tokens;
    const int D = h->d.dim, E = h->d.experts;
    if (ep->peer) {
        route_only(h, static_cast<const uint16_t*>(X), Wr);
        plan_step(h);                       // all-gather of counts: also separates this step from the previous one
        zero_pads(h, h->Xg, D);
        if (!ep->overlap || ep->waves < 2) {
            prof_mark(h, kPhDispatch);
            CKE(launch_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(X), h->Xg, h->stream, peer_map(h, ep->peer_Xg),
                                h->d.training ? ep->Xc : nullptr));
            h->launches += 1;
            if (h->host_hooks) CKE(cudaEventRecord(h->host_ev[tmt_moe::kEvXFree], h->stream));     // X has been read for the last time
            prof_mark(h, kPhExchange);
            rank_barrier(h);                    // every rank's rows have landed
            expert_forward(h, Wup, Wdown, /*gate_in_epilogue=*/false);
            prof_mark(h, kPhExchange);
            rank_barrier(h);                    // every rank's expert outputs are complete
            prof_mark(h, kPhCombine);
            CKE(launch_combine(h->dims, h->rb, h->Yg, static_cast<uint16_t*>(Y), beta, /*mode=*/2, h->stream,
                               peer_map(h, ep->peer_Yg), h->d.training ? ep->Yr : nullptr));
            h->launches += 1;
        } else {
            // Expert waves: wave w = the local experts [w*EL/W, (w+1)*EL/W) of EVERY rank. The side stream sends wave after
            // wave (row kernel + rank barrier) and fetches the finished waves' output rows; the main stream runs a wave's
            // two GEMMs as soon as its rows have landed everywhere. So the transfer of wave w+1 runs under the GEMMs of
            // wave w, and the fetch of wave w under the GEMMs of the waves after it. The GEMM launches leave two SMs free
            // for the barriers' kernels; the later waves' row kernels (launch_wave_rows) are shaped to fit beside the
            // resident CTAs of the CTA-pair GEMM, the full-size ones do not.
            const int W = ep->waves, EL = ep->EL;
            CKE(cudaEventRecord(ep->ev_fork, h->stream));
            CKE(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
            auto wave_map = [&](uint16_t** table, int w) {
                PeerMap pm = peer_map(h, table, true);
                pm.wave_lo = (int)((long)EL * w / W); pm.wave_hi = (int)((long)EL * (w + 1) / W);
                return pm;
            };
            prof_mark(h, kPhDispatch);
            // The first wave fixes every assignment's slot and has the machine to itself; the later ones only move rows,
            // beside the GEMM CTAs of the waves before (launch_wave_rows).
            auto send = [&](int w) {
                if (w == 0 || !ep->thin)
                    CKE(launch_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(X), h->Xg, ep->side, wave_map(ep->peer_Xg, w),
                                        (h->d.training && w == 0) ? ep->Xc : nullptr));
                else
                    CKE(launch_wave_rows(h->dims, h->rb, 0, static_cast<const uint16_t*>(X), nullptr, nullptr, h->num_sms, ep->side,
                                         wave_map(ep->peer_Xg, w)));
                if (w == W - 1 && h->host_hooks) CKE(cudaEventRecord(h->host_ev[tmt_moe::kEvXFree], ep->side));   // last read of X
                rank_barrier(h, ep->side);      // every rank's rows of this wave have landed
                CKE(cudaEventRecord(ep->ev_sent[w], ep->side));
                h->launches += 1;
            };
            // Order on the second stream: the sends run two waves ahead of the GEMMs, a finished wave's fetch comes before
            // the send after next (W = 4: send 0, 1, 2, fetch 0, send 3, fetch 1, 2, 3).
            int sent = 0;
            for (; sent < std::min(W, 3); ++sent) send(sent);
            const int F = ep->fetch_waves < 0 ? W : std::min(ep->fetch_waves, W);      // waves fetched on the second stream
            struct Limit { tmt_moe* h; ~Limit() { h->sm_limit = 0; } } limit{h};
            for (int w = 0; w < W; ++w) {
                const int lo = (int)((long)EL * w / W), hi = (int)((long)EL * (w + 1) / W);
                CKE(cudaStreamWaitEvent(h->stream, ep->ev_sent[w], 0));
                h->sm_limit = gemm_sms_beside_rows(h);
                expert_forward(h, Wup, Wdown, /*gate_in_epilogue=*/false, ep->x_poff[lo] / kPad, (ep->x_poff[hi] - ep->x_poff[lo]) / kPad);
                h->sm_limit = 0;
                if (w < F) {
                    CKE(cudaEventRecord(ep->ev_done[w], h->stream));
                    CKE(cudaStreamWaitEvent(ep->side, ep->ev_done[w], 0));
                    rank_barrier(h, ep->side);      // every rank's outputs of this wave are complete
                    // a fetch that has GEMMs left to hide under runs beside them; the last wave's has none: full-size kernel
                    if (w == W - 1 || !ep->thin)
                        CKE(launch_combine(h->dims, h->rb, h->Yg, nullptr, 0.0f, /*mode=*/3, ep->side, wave_map(ep->peer_Yg, w), ep->Yr));
                    else
                        CKE(launch_wave_rows(h->dims, h->rb, 2, nullptr, ep->Yr, nullptr, h->num_sms, ep->side, wave_map(ep->peer_Yg, w)));
                    h->launches += 1;
                }
                if (sent < W) send(sent++);
            }
            CKE(cudaEventRecord(ep->ev_join, ep->side));
            CKE(cudaStreamWaitEvent(h->stream, ep->ev_join, 0));
            if (F == W) {
                prof_mark(h, kPhCombine);       // every row is in Yr (token-side slots): a local weighted sum remains
                CKE(launch_combine(h->dims, h->rb, ep->Yr, static_cast<uint16_t*>(Y), beta, /*mode=*/2, h->stream));
            } else {
                prof_mark(h, kPhExchange);
                rank_barrier(h);                // every rank's outputs of the waves not fetched yet are complete
                prof_mark(h, kPhCombine);       // the fetched waves' rows from Yr, the others straight from their owners
                PeerMap pm = peer_map(h, ep->peer_Yg);
                pm.fetched = ep->Yr; pm.fetched_hi = (int)((long)EL * F / W);
                CKE(launch_combine(h->dims, h->rb, h->Yg, static_cast<uint16_t*>(Y), beta, /*mode=*/2, h->stream, pm,
                                   h->d.training ? ep->Yr : nullptr));
            }
            h->launches += 1;
        }
    } else if (ep->dma) {
        // Rows are grouped locally (token-side layout), cross NVLink as copy-engine copies on the second stream, wave by
        // wave, and are summed locally at the end. The copies occupy no SM, so a wave's transfer really runs under the
        // previous wave's GEMMs whatever GEMM kernel runs there.
        route_and_dispatch(h, static_cast<const uint16_t*>(X), Wr, ep->Xs);
        plan_step(h);
        zero_pads(h, h->Xg, D);
        const int W = ep->waves, EL = ep->EL;
        CKE(cudaEventRecord(ep->ev_fork, h->stream));
        CKE(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
        prof_mark(h, kPhExchange);
        for (int w = 0; w < W; ++w) {
            dma_rows(h, true, 0, ep->Xs, (int)((long)EL * w / W), (int)((long)EL * (w + 1) / W), D, ep->side);
            rank_barrier(h, ep->side);          // every rank's rows of this wave have landed
            CKE(cudaEventRecord(ep->ev_sent[w], ep->side));
        }
        {
            struct Limit { tmt_moe* h; ~Limit() { h->sm_limit = 0; } } limit{h};
            h->sm_limit = h->num_sms - 2;       // room for the barriers' kernels beside the persistent GEMM CTAs
            for (int w = 0; w < W; ++w) {
                const int lo = (int)((long)EL * w / W), hi = (int)((long)EL * (w + 1) / W);
                CKE(cudaStreamWaitEvent(h->stream, ep->ev_sent[w], 0));
                expert_forward(h, Wup, Wdown, /*gate_in_epilogue=*/false, ep->x_poff[lo] / kPad, (ep->x_poff[hi] - ep->x_poff[lo]) / kPad);
                CKE(cudaEventRecord(ep->ev_done[w], h->stream));
            }
        }
        for (int w = 0; w < W; ++w) {
            CKE(cudaStreamWaitEvent(ep->side, ep->ev_done[w], 0));
            rank_barrier(h, ep->side);          // every rank's outputs of this wave are complete
            dma_rows(h, false, 1, ep->Yr, (int)((long)EL * w / W), (int)((long)EL * (w + 1) / W), D, ep->side);
        }
        CKE(cudaEventRecord(ep->ev_join, ep->side));
        CKE(cudaStreamWaitEvent(h->stream, ep->ev_join, 0));
        prof_mark(h, kPhCombine);
        CKE(launch_combine(h->dims, h->rb, ep->Yr, static_cast<uint16_t*>(Y), beta, /*mode=*/2, h->stream));
        h->launches += 1;
    } else {
        route_and_dispatch(h, static_cast<const uint16_t*>(X), Wr, ep->Xs);
        plan_step(h);
        zero_pads(h, h->Xg, D);
        exchange(h, true, ep->Xs, h->Xg, D);
        expert_forward(h, Wup, Wdown, /*gate_in_epilogue=*/false);
        exchange(h, false, h->Yg, ep->Yr, D);
        prof_mark(h, kPhCombine);
        CKE(launch_combine(h->dims, h->rb, ep->Yr, static_cast<uint16_t*>(Y), beta, /*mode=*/2, h->stream));
        h->launches += 1;
    }
    // statistics over all ranks' tokens: sum of probabilities and of lse^2 / T
    NC(ep, ep->AllReduce(h->rb.stat, ep->stat_global, E + 1, ncclFloat32, ncclSum, ep->comm, h->stream));
    prof_mark(h, -1);
    h->have_forward = true;
}

void ep_backward(tmt_moe* h, const void* dY, const void* Wr, const void* const* Wup, const void* const* Wdown,
                 float* dWr, float* const* dWup, float* const* dWdown, void* dX, float aux, float zcoef) {
    tmt_ep_state* ep = h->ep;
    if (!ep) throw std::runtime_error("expert parallelism is not initialised on this handle (tmt_moe_ep_init)");
    if (!h->d.training || !h->have_forward) throw std::runtime_error("backward needs training = 1 and a preceding forward");
    if (!dY || !Wr || !Wup || !Wdown || !dWr || !dWup || !dWdown || !dX) throw std::runtime_error("null argument");
    CKE(cudaSetDevice(h->d.device));
    use_expert_layout(h);
    const int D = h->d.dim, E = h->d.experts;
    prof_mark(h, kPhGradDispatch);
    // token side: w * dY[token] goes to the owner's gradient rows; s_j = <dY[token], Yr[slot]> (the expert output
    // came back unscaled and was kept)
    if (ep->peer) {
        zero_pads(h, h->dYg, D);             // own pad rows; peers store into data rows only
        const bool waved = ep->overlap && ep->waves >= 2;
        if (!waved) {
            CKE(launch_grad_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(dY), ep->Yr, h->dYg, h->s_j, /*mode=*/2, h->stream,
                                     peer_map(h, ep->peer_dYg)));
            h->launches += 1;
            if (h->host_hooks) CKE(cudaEventRecord(h->host_ev[tmt_moe::kEvDyFree], h->stream));    // dY has been read for the last time
            prof_mark(h, kPhExchange);
            rank_barrier(h);
        } else {
            CKE(cudaEventRecord(ep->ev_fork, h->stream));
            CKE(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
            for (int w = 0; w < ep->waves; ++w) {
                PeerMap pm = peer_map(h, ep->peer_dYg, true);
                pm.wave_lo = (int)((long)ep->EL * w / ep->waves); pm.wave_hi = (int)((long)ep->EL * (w + 1) / ep->waves);
                if (w == 0 || !ep->thin)
                    CKE(launch_grad_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(dY), ep->Yr, h->dYg, h->s_j, /*mode=*/2, ep->side, pm));
                else
                    CKE(launch_wave_rows(h->dims, h->rb, 1, static_cast<const uint16_t*>(dY), ep->Yr, h->s_j, h->num_sms, ep->side, pm));
                if (w == ep->waves - 1 && h->host_hooks) CKE(cudaEventRecord(h->host_ev[tmt_moe::kEvDyFree], ep->side));
                rank_barrier(h, ep->side);      // every rank's gradient rows of this wave have landed
                CKE(cudaEventRecord(ep->ev_sent[w], ep->side));
                h->launches += 1;
            }
        }
        // Input-gradient products first; then the rows of dXg travel back (rank barrier + scatter on the side stream)
        // while the main stream computes the weight gradients, which need nothing from other ranks. Those two GEMM
        // launches leave two SMs free so that the barrier's kernel can start while they run.
        if (!ep->overlap) {                 // measurement switch: everything on one stream, in dependency order
            expert_backward(h, Wup, Wdown, dWup, dWdown);
            prof_mark(h, kPhExchange);
            rank_barrier(h);
            router_backward(h, Wr, nullptr, ep->Xc, true, h->dXg, dWr, static_cast<uint16_t*>(dX), aux, zcoef, h->ep_world_counts,
                            (long)h->d.tokens * ep->G, peer_map(h, ep->peer_dXg));
        } else {
            if (waved) {
                // the same expert waves as in the forward pass: the gradient rows of wave w+1 travel (side stream) under the
                // dH / dXg products of wave w (main stream)
                struct Limit { tmt_moe* h; ~Limit() { h->sm_limit = 0; } } limit{h};
                h->sm_limit = gemm_sms_beside_rows(h);
                const int W = ep->waves, EL = ep->EL;
                for (int w = 0; w < W; ++w) {
                    const int lo = (int)((long)EL * w / W), hi = (int)((long)EL * (w + 1) / W);
                    CKE(cudaStreamWaitEvent(h->stream, ep->ev_sent[w], 0));
                    expert_backward(h, Wup, Wdown, dWup, dWdown, 1, ep->x_poff[lo] / kPad, (ep->x_poff[hi] - ep->x_poff[lo]) / kPad);
                }
                h->sm_limit = 0;
            } else {
                expert_backward(h, Wup, Wdown, dWup, dWdown, 1);
            }
            router_backward(h, Wr, nullptr, ep->Xc, true, h->dXg, dWr, static_cast<uint16_t*>(dX), aux, zcoef, h->ep_world_counts,
                            (long)h->d.tokens * ep->G, peer_map(h, ep->peer_dXg), /*defer_scatter=*/true);
            CKE(cudaEventRecord(ep->ev_fork, h->stream));
            CKE(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
            rank_barrier(h, ep->side);          // every rank's dXg is complete
            scatter_rows(h, Wr, h->dXg, static_cast<uint16_t*>(dX), ep->side, peer_map(h, ep->peer_dXg, true));
            CKE(cudaEventRecord(ep->ev_join, ep->side));
            struct Limit { tmt_moe* h; ~Limit() { h->sm_limit = 0; } } limit{h};
            h->sm_limit = gemm_sms_beside_rows(h);
            expert_backward(h, Wup, Wdown, dWup, dWdown, 2);
            h->sm_limit = 0;
            prof_mark(h, kPhScatter);
            CKE(cudaStreamWaitEvent(h->stream, ep->ev_join, 0));
        }
    } else if (ep->dma) {
        CKE(launch_grad_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(dY), ep->Yr, ep->dYs, h->s_j, /*mode=*/2, h->stream));
        h->launches += 1;
        if (h->host_hooks) CKE(cudaEventRecord(h->host_ev[tmt_moe::kEvDyFree], h->stream));
        zero_pads(h, h->dYg, D);
        const int W = ep->waves, EL = ep->EL;
        CKE(cudaEventRecord(ep->ev_fork, h->stream));
        CKE(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
        prof_mark(h, kPhExchange);
        for (int w = 0; w < W; ++w) {
            dma_rows(h, true, 2, ep->dYs, (int)((long)EL * w / W), (int)((long)EL * (w + 1) / W), D, ep->side);
            rank_barrier(h, ep->side);          // every rank's gradient rows of this wave have landed
            CKE(cudaEventRecord(ep->ev_sent[w], ep->side));
        }
        {
            struct Limit { tmt_moe* h; ~Limit() { h->sm_limit = 0; } } limit{h};
            h->sm_limit = h->num_sms - 2;
            for (int w = 0; w < W; ++w) {
                const int lo = (int)((long)EL * w / W), hi = (int)((long)EL * (w + 1) / W);
                CKE(cudaStreamWaitEvent(h->stream, ep->ev_sent[w], 0));
                expert_backward(h, Wup, Wdown, dWup, dWdown, 1, ep->x_poff[lo] / kPad, (ep->x_poff[hi] - ep->x_poff[lo]) / kPad);
                CKE(cudaEventRecord(ep->ev_done[w], h->stream));
            }
            // the input-gradient rows travel back (second stream) while the weight gradients are computed here
            for (int w = 0; w < W; ++w) {
                CKE(cudaStreamWaitEvent(ep->side, ep->ev_done[w], 0));
                rank_barrier(h, ep->side);      // every rank's dXg rows of this wave are complete
                dma_rows(h, false, 3, ep->dXr, (int)((long)EL * w / W), (int)((long)EL * (w + 1) / W), D, ep->side);
            }
            CKE(cudaEventRecord(ep->ev_join, ep->side));
            expert_backward(h, Wup, Wdown, dWup, dWdown, 2);
        }
        CKE(cudaStreamWaitEvent(h->stream, ep->ev_join, 0));
        router_backward(h, Wr, nullptr, ep->Xc, true, ep->dXr, dWr, static_cast<uint16_t*>(dX), aux, zcoef, h->ep_world_counts,
                        (long)h->d.tokens * ep->G);
    } else {
        CKE(launch_grad_dispatch(h->dims, h->rb, static_cast<const uint16_t*>(dY), ep->Yr, ep->dYs, h->s_j, /*mode=*/2, h->stream));
        h->launches += 1;
        if (h->host_hooks) CKE(cudaEventRecord(h->host_ev[tmt_moe::kEvDyFree], h->stream));
        zero_pads(h, h->dYg, D);
        exchange(h, true, ep->dYs, h->dYg, D);
        expert_backward(h, Wup, Wdown, dWup, dWdown);
        exchange(h, false, h->dXg, ep->dXr, D);
        // the router weight gradient of the local tokens, then summed over the ranks (the router is replicated)
        router_backward(h, Wr, nullptr, ep->Xs, true, ep->dXr, dWr, static_cast<uint16_t*>(dX), aux, zcoef, h->ep_world_counts,
                        (long)h->d.tokens * ep->G);
    }
    NC(ep, ep->AllReduce(dWr, dWr, (size_t)E * D, ncclFloat32, ncclSum, ep->comm, h->stream));
    prof_mark(h, -1);
    h->launches += 1;
}

const float* ep_stat(tmt_moe* h) { return h->ep ? h->ep->stat_global : h->rb.stat; }
int ep_waves(tmt_moe* h) { return h->ep ? h->ep->waves : 1; }

}  // namespace tmt

// The device-side plan kernel run alone on the current device, on counts given by the caller: what an expert-parallel
// step of rank r computes after its all-gather, without any communicator. Exported so that one GPU can check the
// kernel against the host plan (tmt_moe_ep_plan / tmt_moe_ep_check_capacity) for any number of ranks.
extern "C" int tmt_moe_ep_plan_device(int G, int r, int E, int pad, int x_cap, const int* cnt_all_host, int* tables_host,
                                      int* dest_row0_host, int* world_host, int* status_host) {
    using namespace tmt;
    try {
        if (G < 1 || G > 256 || r < 0 || r >= G || E < 1 || E > 256 || E % G || pad < 1 || pad % kPad || x_cap < pad || !cnt_all_host ||
            !tables_host || !dest_row0_host || !world_host || !status_host)
            throw std::runtime_error("ep_plan_device: bad arguments");
        const int EL = E / G, max_tiles = x_cap / kPad;
        const size_t nt = (size_t)2 * EL + 2 + max_tiles;
        int *cnt = nullptr, *tab = nullptr, *dst = nullptr, *wor = nullptr, *st = nullptr;
        CKE(cudaMalloc(&cnt, (size_t)G * E * 4)); CKE(cudaMalloc(&tab, nt * 4)); CKE(cudaMalloc(&dst, E * 4));
        CKE(cudaMalloc(&wor, E * 4)); CKE(cudaMalloc(&st, 4));
        CKE(cudaMemcpy(cnt, cnt_all_host, (size_t)G * E * 4, cudaMemcpyHostToDevice));
        CKE(cudaMemset(st, 0, 4));
        ep_plan_kernel<<<1, 256>>>(G, r, E, EL, pad, x_cap, max_tiles, cnt, tab, dst, wor, st);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaDeviceSynchronize();
        if (e == cudaSuccess) e = cudaMemcpy(tables_host, tab, nt * 4, cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(dest_row0_host, dst, E * 4, cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(world_host, wor, E * 4, cudaMemcpyDeviceToHost);
        if (e == cudaSuccess) e = cudaMemcpy(status_host, st, 4, cudaMemcpyDeviceToHost);
        for (int* q : {cnt, tab, dst, wor, st}) cudaFree(q);
        CKE(e);
        return 0;
    } catch (const std::exception& ex) { set_error("%s", ex.what()); return -1; }
}
