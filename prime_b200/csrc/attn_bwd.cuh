// Parameter block shared by the flash-attention backward kernels (attn_bwd_sm100.cu, attn_bwd_t_sm100.cu).
#pragma once
#include "common.cuh"

namespace pb {

struct AttnBwdParams {
    int M, H, KV, n_tiles;
    const int* seq_start;
    const float* lse2;     // [H, M]
    const float* D;        // [H, M]
    float* dq_acc;         // [M, H*HD] fp32, zero-initialised by the caller
    __nv_bfloat16* dqkv;   // [M, (H+2KV)*HD]; the backward kernel writes the k and v column blocks
    long long dqkv_stride;
    float scale, scale_log2;
    int* status;
    // persistent (head size 64) kernel only: query-tile count per kv tile and the global work counter (both set
    // by a pre-pass of the launch), work-item count (= n_tiles * KV)
    const int* nq;
    int* counter;
    int n_items;
};

// Head size 64, transposed-score form (attn_bwd_t_sm100.cu).
// nq_scratch: >= n_tiles + 1 ints of device scratch (filled by a pre-pass of the launch).
int launch_attn_bwd_t64(const CUtensorMap& tq, const CUtensorMap& tdo, const CUtensorMap& tdq, const AttnBwdParams& p,
                        int* nq_scratch, cudaStream_t st);

}  // namespace pb
