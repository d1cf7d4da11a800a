/* C ABI of the B200 (sm_100a) Mixture-of-Experts feed-forward block.
 *
 * Drop-in replacement for the MoE block of TMT (tmt-cuda/src/moe.cu): the functions
 * below take over what moe_keep_alloc / moe_ws_alloc / moe_forward / moe_aux_from /
 * moe_backward do there. Conventions follow the reference's existing C ABI
 * (tmt-cuda/src/capi.h, capi.cu:9-24): opaque handle, 0 on success and -1 on failure,
 * the message of the last failure of the calling thread from tmt_moe_last_error(),
 * C++ exceptions never cross, the library never calls exit().
 *
 * All tensor arguments are DEVICE pointers unless a function name ends in _host.
 * bf16 tensors are raw 16-bit patterns. Weight layout is the reference's [out,in]
 * row-major (tmt-cuda/src/linalg.cu:3-4).
 *
 * Two expert modes:
 *   hidden == 0  "reference mode": one dim x dim matrix per expert, SiLU applied in
 *                combine (moe.cu:142-158). Wup[e] is that matrix, Wdown is NULL.
 *   hidden  > 0  two-matrix FFN: h = silu(x Wup[e]^T), y = gate * (h Wdown[e]^T).
 *                Wup[e] is hidden x dim, Wdown[e] is dim x hidden.
 */
#ifndef TMT_MOE_H
#define TMT_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tmt_moe tmt_moe;

enum { TMT_MOE_BF16 = 0, TMT_MOE_F32 = 1 };
/* Grouped GEMM kernel. AUTO (what a zero-initialised descriptor selects) is the fastest one: CTA pairs on 256x256
 * tiles, expert groups padded to 256 rows. TCGEN05 = one CTA per 128x256 tile (groups padded to 128 rows). SIMT = slow
 * independent kernel the tests cross-check the tensor-core products with; nothing switches to it at run time. */
enum { TMT_MOE_GEMM_AUTO = 0, TMT_MOE_GEMM_SIMT = 1, TMT_MOE_GEMM_TCGEN05_2CTA = 2, TMT_MOE_GEMM_TCGEN05 = 3 };
enum { TMT_MOE_EP_PEER = 0, TMT_MOE_EP_NCCL = 1, TMT_MOE_EP_DMA = 2 };

/* Replaces the (N,E,K,D) arguments of moe_keep_alloc / moe_ws_alloc (moe.cu:330-362) and
 * the config knobs experts=, topk= (tmt-cuda/src/config.h:12). */
typedef struct tmt_moe_desc {
    int tokens;        /* capacity: most rows (batch*seqlen) one call may carry            */
    int dim;           /* model width D, multiple of 64 (one TMA box of bf16)              */
    int hidden;        /* expert hidden width H (multiple of 64); 0 = reference mode       */
    int experts;       /* E >= 1 (no upper bound of 16 as in config.h:51-52; E <= 256)      */
    int topk;          /* 1 <= K <= min(E, 8)                                               */
    int router_dtype;  /* TMT_MOE_BF16 (the reference's work copy, model.cu:513) or _F32    */
    int training;      /* 1: keep what backward needs; 0: forward only                     */
    int gemm_impl;     /* TMT_MOE_GEMM_AUTO (= _TCGEN05_2CTA: CTA pairs on 256x256 tiles, groups padded to 256
                          rows), _TCGEN05 (one CTA per tile) or _SIMT (slow cross-check kernel)               */
    int device;        /* CUDA device ordinal                                              */
    int host_io;       /* 1: also allocate staging for the *_host entry points             */
    void* stream;      /* cudaStream_t all work is queued on; NULL = legacy default stream  */
    int ep_world;      /* expert-parallel ranks (1 = all experts local)                    */
    int ep_rank;       /* this rank; it owns experts [rank*E/world, (rank+1)*E/world)        */
    float ep_capacity_factor; /* expert-parallel only: rows other ranks may route to this rank's
                          experts, as a multiple of tokens*topk (0 = 1.5); a step that needs more fails on every rank:
                          with -1 from the call where the exchange plan is made on the host (NCCL transport, expert
                          waves), through tmt_moe_device_status (code 4) where it is made on the device (peer transport:
                          the step then has no host synchronisation; rows past the capacity are not touched)        */
    int ep_transport;  /* TMT_MOE_EP_PEER: gather / scatter kernels address the owners' buffers over NVLink
                          (CUDA IPC peer memory); TMT_MOE_EP_NCCL: NCCL send / recv exchanges; TMT_MOE_EP_DMA: rows are
                          grouped locally and cross NVLink as peer-to-peer copies of the copy engines over the same
                          mappings, on a second stream, in expert waves (TMT_MOE_EP_WAVES) under the GEMMs          */
} tmt_moe_desc;

/* moe_keep_alloc + moe_ws_alloc (moe.cu:330-362): every buffer is allocated here, none later. */
int tmt_moe_create(const tmt_moe_desc* desc, tmt_moe** out);
/* moe_keep_free + moe_ws_free (moe.cu:342-348, 363-370). Never frees caller memory. */
void tmt_moe_destroy(tmt_moe* h);
/* capi.cu:24 tmt_last_error. */
const char* tmt_moe_last_error(void);

/* Optional per-expert additive bias on the router logits (host pointer, E floats, copied;
 * NULL removes it). The reference has no such term; the skewed-routing benchmark uses it. */
int tmt_moe_set_router_bias(tmt_moe* h, const float* bias_host);

/* moe_forward (moe.cu:374-466). X (tokens,D) bf16; Wrouter (E,D) in router_dtype; Wup / Wdown
 * HOST arrays of E device pointers (the reference's bf16** Wexp, model.cu:500); Y (tokens,D)
 * bf16, in/out when beta != 0 (Y = beta*Y + moe(X), the fused residual of model.cu:513-515).
 * tokens <= desc.tokens. Statistics stay on the device until tmt_moe_stats. */
int tmt_moe_forward(tmt_moe* h, const void* X, const void* Wrouter, const void* const* Wup,
                    const void* const* Wdown, void* Y, float beta, int tokens);

/* moe_aux_from + the hcnt read (moe.cu:470-475, capi.cu:131-136). Synchronises the stream.
 * stat[0..E) = sum over tokens of the router probabilities, stat[E] = mean lse^2 (z-loss);
 * counts[e] = tokens routed to expert e (global over expert-parallel ranks);
 * *aux = E * sum_e (stat[e]/N) * (counts[e]/(N*K)). Any pointer may be NULL. */
int tmt_moe_stats(tmt_moe* h, float* stat, int64_t* counts, float* aux);

/* The deferred statistics path of moe_forward (moe.cu:448-452): queues a device-to-device copy of
 * the E+1 statistics into a caller-owned DEVICE slot on the handle's stream; no synchronisation. */
int tmt_moe_copy_stats(tmt_moe* h, float* stat_device);

/* moe_backward (moe.cu:479-545); must follow the forward call on the same handle.
 * dY (tokens,D) bf16. Outputs: dX (tokens,D) bf16 (written, not accumulated), dWrouter (E,D)
 * fp32 (written), dWup[e] / dWdown[e] fp32 with the shape of the weight (written; zero for an
 * expert that received no token). aux and zcoef are the loss coefficients already divided by
 * the layer count (model.cu:676-677). */
int tmt_moe_backward(tmt_moe* h, const void* dY, const void* Wrouter, const void* const* Wup,
                     const void* const* Wdown, float* dWrouter, float* const* dWup,
                     float* const* dWdown, void* dX, float aux, float zcoef);

/* Host-buffer step used for end-to-end timing: copies X (and dY) from host memory, runs
 * forward (and backward when dY_host != NULL), copies Y (and dX) and the E+1 statistics back
 * and synchronises. Needs desc.host_io = 1. Weight and gradient pointers are device memory.
 * Works under expert parallelism too (every rank calls it with its own tokens); stat_host[E] is then the SUM over
 * the ranks of each rank's mean lse^2 (tmt_moe_stats divides it by the rank count). */
int tmt_moe_step_host(tmt_moe* h, const void* X_host, const void* dY_host, const void* Wrouter,
                      const void* const* Wup, const void* const* Wdown, float* dWrouter,
                      float* const* dWup, float* const* dWdown, void* Y_host, void* dX_host,
                      float* stat_host, float beta, float aux, float zcoef, int tokens);
/* The same step without the final synchronisation: the call returns once everything is queued. Uploads of
 * the next step start as soon as this step has consumed the staging buffers (under its GEMMs) and downloads
 * run under the following compute, so back-to-back calls keep PCIe busy in both directions while the GPU
 * computes. The host buffers must stay valid (and Y_host / dX_host / stat_host unread) until
 * tmt_moe_host_wait returns. No counterpart in the reference (its trainer keeps all data on the device). */
int tmt_moe_step_host_async(tmt_moe* h, const void* X_host, const void* dY_host, const void* Wrouter,
                      const void* const* Wup, const void* const* Wdown, float* dWrouter,
                      float* const* dWup, float* const* dWdown, void* Y_host, void* dX_host,
                      float* stat_host, float beta, float aux, float zcoef, int tokens);
/* Waits for every host step queued so far (uploads, compute, downloads). */
int tmt_moe_host_wait(tmt_moe* h);

/* Copies saved routing state to HOST memory (synchronises). The reference exposes the same
 * tensors as MoeKeep fields (moe.cu:294-315). name is one of
 *   "logits" "probs" (tokens*E f32)  "idx" "slot_of" (tokens*K i32)  "w" (tokens*K f32)
 *   "counts" (E i32)  "poff" (E+1 i32, 128-row padded group starts)  "lse" (tokens f32)
 *   "dlogits" (tokens*E f32, after backward)  "s_j" (tokens*K f32, after backward)
 *   "ep_waves" (1 i32: expert waves an expert-parallel step of this handle runs in, 1 = one exchange per pass;
 *   known after tmt_moe_ep_init)
 * Returns the number of bytes written, or -1. */
long long tmt_moe_read(tmt_moe* h, const char* name, void* dst_host, size_t dst_bytes);

/* Per-phase device timing, the counterpart of the reference's TMT_PROFILE switch
 * (moe.cu:380-394, 459-464) without its per-phase cudaDeviceSynchronize: while on, every
 * kernel of a step is bracketed by CUDA events on the handle's stream. tmt_moe_profile
 * synchronises, then returns accumulated milliseconds and launch counts per phase (arrays of
 * tmt_moe_num_phases() entries, names from tmt_moe_phase_name) and optionally resets them. */
int tmt_moe_set_profile(tmt_moe* h, int on);
int tmt_moe_profile(tmt_moe* h, float* ms, long long* count, int reset);
int tmt_moe_num_phases(void);
const char* tmt_moe_phase_name(int i);

/* Number of kernel launches the handle has queued since creation (the reference counts
 * nothing; used by the benchmark to report its launch count). */
long long tmt_moe_launch_count(const tmt_moe* h);
/* Router-balance telemetry (train_main.cu:204-209, 232-248; capi.cu:131-136 tmt_model_expert_counts): tokens routed
 * to each expert, accumulated ON THE DEVICE over every forward pass since the last reset (the reference adds the
 * host-side hcnt of every window). Returns the reference's summary: min_share / max_share = smallest / largest
 * expert share with 1.0 = uniform, dead = experts with a share below 0.01, passes = forward passes counted, totals
 * (may be NULL) = the E accumulated counts. reset != 0 clears the accumulators. Synchronises. Under expert parallelism
 * the counts are those of this rank's tokens (over all experts). */
int tmt_moe_usage(tmt_moe* h, double* min_share, double* max_share, long long* dead, long long* passes,
                  long long* totals, int reset);
/* Measurement only (no counterpart in the reference). With TMT_MOE_GEMM_CYCLES=1 in the environment at
 * tmt_moe_create, every tcgen05 GEMM launch records, per CTA, the clock cycles its TMA, MMA and
 * epilogue threads spent waiting and working. Copies the ring of the last *launches launches
 * ([launch % *launches][cta < *ctas][slot < *slots] long long) to `out` (may be NULL to query the
 * sizes) and returns the number of GEMM launches so far, -1 when the counters are off. Synchronises. */
int tmt_moe_debug_gemm_cycles(tmt_moe* h, long long* out, int* launches, int* ctas, int* slots);
/* Device-side status word: 0 when no kernel reported a problem; otherwise the first code recorded: 1 an index left its
 * range, 2 a bounded wait ran out, 3 tensor memory could not be allocated, 4 an expert-parallel step routed more rows
 * to a rank than its capacity. Synchronises. */
int tmt_moe_device_status(tmt_moe* h);

/* Failure-detection self-test (no counterpart in the reference): launches one block that waits on a
 * barrier nothing arrives on, with the given limit in clock cycles, through the same bounded-wait
 * routine the GEMM kernels use. Returns 2 (the time-out status code) when the wait ran out, the status
 * word was set and the kernel returned in order; the context stays usable. -1 on a host error. */
int tmt_moe_selftest_bounded_wait(tmt_moe* h, long long limit_cycles);

/* ---- NVFP4 expert weights for sampling (no counterpart in the reference) ---------------
 * e2m1 values, one e4m3 scale per 16 consecutive input elements, one fp32 scale per tensor. */
typedef struct tmt_nvfp4_weight {
    const void* packed;   /* rows*cols/2 bytes, element 2i in the low nibble            */
    const void* scales;   /* rows*cols/16 e4m3 bytes, row-major                         */
    float tensor_scale;
    int rows, cols;
} tmt_nvfp4_weight;

/* Quantises a bf16 (rows,cols) device matrix, cols % 16 == 0. packed/scales are device
 * buffers of the sizes above; the per-tensor scale is returned through a HOST pointer. */
int tmt_moe_quantize_nvfp4(const void* W_bf16, int rows, int cols, void* packed, void* scales,
                           float* tensor_scale_host, void* stream);

/* Forward with NVFP4 expert weights (hidden > 0 only, training = 0). Wup / Wdown are HOST
 * arrays of E descriptors. Router as in tmt_moe_forward.
 * Steps of at most 256 tokens with tokens * topk <= 1024 (the sampler's case), 16-byte aligned
 * packed / scales pointers, dim and hidden multiples of 256: the expert products read the packed
 * weights in place, so these must stay valid while the handle uses them. Larger steps expand the
 * weights once into scratch owned by the handle. Same numerics on both routes; the environment
 * variable TMT_MOE_DECODE_MAX_TOKENS moves the switch point (0: always expand).
 * The expansion is reused while the descriptors name the same pointers and tensor scales. A caller that
 * re-quantises INTO THE SAME BUFFERS (after an optimizer step or a checkpoint load) must call
 * tmt_moe_nvfp4_weights_changed before the next forward, or large steps keep using the old expansion. */
int tmt_moe_forward_nvfp4(tmt_moe* h, const void* X, const void* Wrouter,
                          const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown, void* Y,
                          float beta, int tokens);
/* The same forward with the LayerNorm in front of the block (layernorm_fwd, tmt-cuda/src/norm.cu:8-50; call site
 * model.cu:509-514) taken in: X holds the rows BEFORE the normalisation, gamma / beta_ln (dim fp32, device) are its
 * parameters, eps = 1e-5. For sampler-sized steps (the per-token router, tokens x experts <= 16384, on the packed-weight
 * route) the router's first kernel normalises each row itself, with the arithmetic of tmt_ln_forward (include/tmt_norm.h),
 * so a decode step stays at five launches and the result has the bits of tmt_ln_forward followed by
 * tmt_moe_forward_nvfp4; larger steps run that kernel and then the block. The residual (beta != 0) adds to Y as given:
 * the reference's residual stream is the un-normalised one (model.cu:513-515). */
int tmt_moe_forward_nvfp4_ln(tmt_moe* h, const void* X, const float* gamma, const float* beta_ln, const void* Wrouter,
                             const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown, void* Y, float beta, int tokens);

/* Drops everything the handle derived from NVFP4 weights (the bf16 expansion, the pointer table of the small-batch
 * route): the next tmt_moe_forward_nvfp4 builds it again from the descriptors it is given. */
int tmt_moe_nvfp4_weights_changed(tmt_moe* h);

/* ---- expert parallelism over NCCL (no counterpart in the reference) -------------------
 * One process per GPU. Rank 0 creates an id, the host program ships the 128 bytes to all
 * ranks, every rank calls tmt_moe_ep_init. Dispatch and combine then run as all-to-all
 * exchanges of grouped rows; Wup/Wdown hold only the E/world local experts. */
int tmt_moe_ep_unique_id(void* id128);
int tmt_moe_ep_init(tmt_moe* h, const void* id128);
/* Host arithmetic of one exchange (no GPU needed; exported so that it can be tested on CPU ranks).
 * cnt_all[g*E + e] = rows rank g routes to global expert e. For rank r: tok_poff[E+1] token-side
 * group starts padded to `pad` rows; x_counts[E/G], x_poff[E/G+1] the expert-side groups of r's
 * experts (rows of all source ranks in rank order, padded); src_off[s*(E/G) + le] where source
 * s's rows start inside local group le. Returns the expert-side row count, -1 on bad arguments. */
long long tmt_moe_ep_plan(int G, int r, int E, int pad, const int* cnt_all, int* tok_poff, int* x_counts,
                          int* x_poff, int* src_off);
/* The capacity check every rank runs on the all-gathered counts before any row moves (host arithmetic, exported
 * for CPU tests): -1 when the padded expert-side rows of every rank fit into x_cap rows, otherwise the lowest rank
 * that overflows (its row count in *rows_out, may be NULL); -2 on bad arguments. Same input on every rank, hence
 * the same verdict: a step that overflows one rank fails on all ranks together, with both transports. */
int tmt_moe_ep_check_capacity(int G, int E, int pad, const int* cnt_all, long long x_cap, long long* rows_out);
/* The same plan computed by the library's device kernel (what a peer-transport step without expert waves runs after its
 * all-gather), on host-given counts and on the current device, without a communicator: lets one GPU check the kernel
 * against the two functions above for any rank count. tables_host: [EL+1] padded group starts of rank r's experts |
 * [EL] their row counts | [1] number of 128-row tiles | [x_cap / 128] tile -> local expert (-1 past the end);
 * dest_row0_host[E]: where rank r's rows start inside the owner's group of each expert; world_host[E]: rows per expert
 * over all ranks; *status_host: 0, or 4 when some rank's rows exceed x_cap. HOST pointers. */
int tmt_moe_ep_plan_device(int G, int r, int E, int pad, int x_cap, const int* cnt_all_host, int* tables_host,
                           int* dest_row0_host, int* world_host, int* status_host);

/* ---- entry point that allocates nothing (no counterpart in the reference) ---------------
 * dWrouter[e, d] = sum_t bf16(dlogits[t, e]) * X[t, d], the router_dw phase of
 * tmt_moe_backward, for callers that cannot call cudaMalloc when they need it (the device is
 * owned by another allocator, a latency budget forbids the driver's allocation lock, ...).
 * No handle, no cudaMalloc / cudaFree: the partial sums live in a fixed 8 MiB array inside the
 * library image, so experts * dim <= 131072 (larger sizes are refused with a message).
 * dlogits (tokens, experts) fp32, X (tokens, dim) bf16, dWrouter (experts, dim) fp32: device
 * pointers; runs on `stream` of the current device. All calls on a GPU share the array: calls
 * that overlap on the GPU race, order them. The first call on a device looks up the array's
 * address; make it outside any stream capture. */
int tmt_moe_router_dw_noalloc(const float* dlogits, const void* X, int tokens, int dim, int experts,
                              float* dWrouter, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TMT_MOE_H */
