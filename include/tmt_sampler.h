/* C ABI of the batched multi-stream sampler session around the NVFP4 MoE block on B200 (sm_100a).
 *
 * The reference samples one stream at a time: Generator (tmt-cuda/src/generate.h:9-60) builds a batch-1, one-position
 * model, and every byte costs three blocking host-to-device copies, one forward_window and two blocking copies back
 * (generate.h:31-44); sample.cu:28-38 is the loop. This session advances `streams` independent byte streams together
 * and keeps a decode step free of host round trips:
 *   * the expert weights are NVFP4, quantised once by the caller (tmt_moe_quantize_nvfp4) and handed over once;
 *   * the block's input and output rows of a step live in device-resident ring slots (streams x dim bf16 each);
 *   * one decode step (router, the two expert products on the packed weights, combine) is recorded once per slot as a
 *     CUDA graph and replayed: tmt_sampler_step queues it and returns, with no copy and no synchronisation;
 *   * Generator::sample (generate.h:47-58) runs on the device for all streams at once, so the chosen bytes need not
 *     travel to the host before the next step is queued.
 * The rest of the model (embedding, recurrence, LayerNorm, decoder head) stays with the caller: it writes the block's
 * input rows into a slot and reads the output rows from it, on the session's stream.
 *
 * Conventions as in tmt_moe.h: opaque handle, 0 / -1, message from tmt_moe_last_error(), nothing calls exit(). */
#ifndef TMT_SAMPLER_H
#define TMT_SAMPLER_H

#include <stddef.h>
#include <stdint.h>

#include "tmt_moe.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct tmt_sampler tmt_sampler;

typedef struct tmt_sampler_desc {
    int streams;        /* independent byte streams advanced together (the reference: 1, generate.h:21)            */
    int dim, hidden;    /* block width and expert hidden width (hidden > 0)                                        */
    int experts, topk;  /* the config knobs experts=, topk=                                                        */
    int router_dtype;   /* TMT_MOE_BF16 or TMT_MOE_F32                                                             */
    int ring;           /* device-resident input / output slots, >= 1                                              */
    int device;         /* CUDA device ordinal                                                                     */
    void* stream;       /* cudaStream_t every step is queued on; NULL: the session creates its own (a legacy
                           default stream cannot be recorded into a graph)                                         */
    uint64_t seed;      /* key of the per-stream random draws (the reference's seed= option, sample.cu:17)         */
} tmt_sampler_desc;

/* Generator's constructor (generate.h:19-27): allocates the ring and the block's handle; nothing is allocated later
 * except one graph per slot at its first step. */
int tmt_sampler_create(const tmt_sampler_desc* desc, tmt_sampler** out);
void tmt_sampler_destroy(tmt_sampler* s);

/* load_weights_only (generate.h:26) for the block: router (experts x dim, router_dtype, device memory) and the
 * NVFP4 descriptors of every expert (host arrays of `experts` entries, copied; the packed bytes and scales they point
 * to must stay valid). Runs one warm-up step, synchronises, and drops the recorded graphs. Call it again after the
 * weights changed (new pointers or re-quantised in place). */
int tmt_sampler_set_weights(tmt_sampler* s, const void* Wrouter, const tmt_nvfp4_weight* Wup, const tmt_nvfp4_weight* Wdown);

/* Optional: the LayerNorm in front of the block (layernorm_fwd, norm.cu:8-50; model.cu:509-514) becomes part of the
 * step: the X rows of a slot are then the rows BEFORE the normalisation, and the router's first kernel normalises them
 * (tmt_moe_forward_nvfp4_ln), so the step has no separate LayerNorm launch. gamma / beta: dim fp32 each, device memory,
 * must stay valid; NULL, NULL switches it off again. Drops the recorded graphs. */
int tmt_sampler_set_layernorm(tmt_sampler* s, const float* gamma, const float* beta);

/* Device addresses of a slot's rows (streams x dim bf16): the caller's kernels write X and read Y there, ordered on
 * the session's stream. NULL for a slot outside [0, ring). */
void* tmt_sampler_x(tmt_sampler* s, int slot);
void* tmt_sampler_y(tmt_sampler* s, int slot);
/* The stream the session queues on (the caller's, or its own). */
void* tmt_sampler_stream(tmt_sampler* s);

/* The block's part of Generator::feed (generate.h:31-44 -> forward_window -> moe_forward with one row per stream):
 * Y[slot] = beta * Y[slot] + moe(X[slot]). Replays the slot's graph (recorded at the first call for that slot and
 * beta); queues and returns. */
int tmt_sampler_step(tmt_sampler* s, int slot, float beta);

/* Host convenience for callers whose rows start in host memory: asynchronous copies of a slot's X rows from, and Y
 * rows to, (pinned) host memory, and a wait for everything queued so far. The copies run on two streams of the
 * session's own and are ordered against the slot's steps by events (an upload waits until the slot's last step has read
 * its rows, a step waits for the slot's upload and for the download of its previous result, a download waits for the
 * slot's last step), so with several ring slots the copies of neighbouring decode steps overlap a step's kernels. A
 * caller that reads Y or writes X with kernels of its own on the session's stream, after a download or before an
 * upload of the same slot, orders those itself (tmt_sampler_sync, or events on tmt_sampler_stream). */
int tmt_sampler_upload(tmt_sampler* s, int slot, const void* X_host);
int tmt_sampler_download(tmt_sampler* s, int slot, void* Y_host);
int tmt_sampler_sync(tmt_sampler* s);

/* Generator::sample (generate.h:47-58) for all streams at once: logits (streams x 256 bf16, device) -> next byte of
 * every stream (streams int32, device). temp <= 0: the first maximum. Otherwise p[i] = exp((l[i] - max) / temp)
 * (quotient in fp32, exponential and sums in double, in index order), r = u * sum, the first i with (r -= p[i]) <= 0.
 * u is the draw of (seed, stream, position): splitmix64 of a key built from the three, top 53 bits / 2^53. The
 * reference draws from one std::mt19937 per generator (generate.h:13, 55); a batch needs draws that do not depend on
 * which streams share a step, so the generator here is counter-based: same seed, stream and position, same byte,
 * whatever the batch. Queues on the session's stream and returns. */
int tmt_sampler_sample(tmt_sampler* s, const void* logits, float temp, long long position, int* next_device);

/* Steps queued so far and graphs recorded so far (a replayed step adds no graph). */
long long tmt_sampler_steps(const tmt_sampler* s);
int tmt_sampler_graphs(const tmt_sampler* s);

#ifdef __cplusplus
}
#endif
#endif
