/* C ABI of the checkpoint pass-through for the MoE block's parameters on B200 (sm_100a).
 *
 * In the reference's V3 checkpoint the router and every expert matrix are ordinary parameters: the payload holds, per
 * parameter, `u64 n | master[n] | m[n] | v[n]` (fp32, little endian; tmt-cuda/src/checkpoint.h:142-148), written from
 * and read into DEVICE memory through a bounded host staging buffer (Checkpoint::device, checkpoint.h:36-46), and on
 * load the bf16 working copy the GEMMs read is re-materialised from the master (copy_bf16_kernel, checkpoint.h:149,
 * model.cu:54-57). The whole file is covered by a streaming FNV-1a checksum (hash_bytes, checkpoint.h:11-16).
 *
 * These functions move ONE parameter record between device memory and a host buffer in exactly that layout, so a host
 * program that owns the file (header, progress, the other parameters, stream state, trailer) can keep its format while
 * the block's parameters live behind this library. NVFP4 copies are derived data as well: after a load the caller
 * re-quantises from the bf16 copy (tmt_moe_quantize_nvfp4) and, when it quantises into the buffers a handle already
 * uses, calls tmt_moe_nvfp4_weights_changed.
 *
 * Conventions as in tmt_moe.h: 0 / -1, message from tmt_moe_last_error(), nothing calls exit(). */
#ifndef TMT_CKPT_H
#define TMT_CKPT_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* HASH_INIT of checkpoint.h:17. */
#define TMT_CKPT_HASH_INIT UINT64_C(14695981039346656037)

/* hash_bytes (checkpoint.h:11-16): h = (h ^ byte) * 1099511628211 over the bytes in order. */
uint64_t tmt_ckpt_hash(uint64_t h, const void* data, size_t size);

/* Bytes of one parameter record: 8 + 12 * n. */
size_t tmt_ckpt_record_bytes(long long n);

/* Save direction of checkpoint.h:144-148: writes `u64 n | master | m | v` of a parameter that lives in device memory
 * into record_host (record_bytes >= tmt_ckpt_record_bytes(n)). Synchronises `stream`. */
int tmt_ckpt_save_param(const float* master, const float* m, const float* v, long long n, void* record_host,
                        size_t record_bytes, void* stream);

/* Load direction: checks the stored n against the expected one ("checkpoint parameter shape mismatch",
 * checkpoint.h:146), copies master / m / v into device memory (m and v may be NULL: weights only, as
 * load_weights_only does for the sampler) and writes the bf16 working copy work_bf16[i] = bf16(master[i]), round to
 * nearest even (may be NULL). Synchronises `stream`. */
int tmt_ckpt_load_param(const void* record_host, size_t record_bytes, long long n, float* master, float* m, float* v,
                        void* work_bf16, void* stream);

#ifdef __cplusplus
}
#endif
#endif
