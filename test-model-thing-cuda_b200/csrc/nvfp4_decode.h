// Launchers of the small-batch NVFP4 kernels (nvfp4_decode.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace tmt {

constexpr int kDecodeMaxAsg = 1024;     // tokens * topk the small-batch route accepts

struct Fp4RowsArgs {
    const uint8_t* const* packed;       // [experts] e2m1 codes, rows x kdim / 2 bytes, 16-byte aligned
    const uint8_t* const* scales;       // [experts] e4m3 block scales, rows x kdim / 16 bytes
    const float* es;                    // [experts] tensor scale * 2^14
    const uint16_t* src; int src_ld;    // bf16 input rows; assignment a reads row a / src_div
    int src_div;
    uint16_t* out; int out_ld;          // bf16 output, one row per assignment
    const int* idx;                     // [n_asg] expert of each assignment
    const float* gate;                  // [n_asg] gate weights (mode 1)
    int n_asg, rows, kdim;
    int red_in_stage;                   // set by the launcher: the k-half exchange buffer lives in the staged rows
    int kphases;                        // set by the launcher: the token rows are staged in this many column slices
    int* status;                        // device status word (a bounded wait that ran out is reported there)
    int dbg;                            // measurement only (TMT_MOE_FP4_DEBUG): 1 stop after the list, 2 no products, 4 no staging
};

// out = expert rows x the assignments routed to the expert; grid = (rows / 128 or 256, experts).
cudaError_t launch_fp4_rows(const Fp4RowsArgs& a, int experts, int mode, cudaStream_t s);
cudaError_t launch_decode_combine(const uint16_t* Ya, uint16_t* Y, float beta, int T, int D, int K, cudaStream_t s);
bool fp4_rows_shape_ok(int rows, int kdim);

}  // namespace tmt
