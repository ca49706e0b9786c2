// Parameters shared by the attention kernels (CUDA-core and tensor-core forms).
#pragma once

#include "common.cuh"

namespace fd {

struct AttnParams {
    const void* q;             // [T, n_q * d]
    const void* k_pool;        // [num_blocks, n_kv, block_size, d]
    const void* v_pool;        // [num_blocks, n_kv, block_size, dv]
    void* out;                 // [T, n_q * dv]
    float* part_m;             // [T, n_q, n_splits]
    float* part_l;
    float* part_acc;           // [T, n_q, n_splits, dv]
    const int* block_table;    // [slots, max_blocks]
    const int* row_slot;       // per batch row: cache slot, or -1 for a padding row
    const int* row_q_start;    // first token of the row in the flat token arrays
    const int* row_q_len;      // new tokens of the row in this step
    const int* row_ctx_len;    // tokens of the row cached before this step
    int* status;
    int* counters;             // [rows, n_kv] arrival counts for the in-kernel merge of the splits (all zero between launches), or null
    int max_blocks, num_blocks, block_size;
    int n_q, n_kv, G, d;
    // The tensor-core decode kernel only: a group of more query heads than it takes is cut into kv_div smaller groups,
    // each a key/value head of its own as far as the kernel's grid, rows and counters go (n_kv and G are then the
    // numbers after the cut); the pool still has n_kv_pool heads per block and head kvh reads pool head kvh / kv_div.
    int n_kv_pool, kv_div;
    int dv;                    // size of a value head (= d in the tensor-core kernels)
    int QT, n_splits, split_len, window;
    int chunk;                 // > 0: a query at position i sees key j <= i only if i / chunk == j / chunk
    float scale;
    // The CUDA-core kernel and the extended prompt kernel only (the launchers of the others are not called when any of these is set):
    float softcap;             // > 0: score <- softcap * tanh(score / softcap) after scaling
    int keep_first;            // with a window: keys at positions below this stay visible however far back they lie
    const float* sink;         // [n_q] or null: exp(sink[h]) is one more term of head h's softmax denominator
    int v_rep;                 // > 1: every query head's weights are applied to each of v_rep value heads (the pool's
                               // n_kv heads); out is then [T, n_q, v_rep, dv]
    int v_all;                 // set by the CUDA-core launcher: a CTA takes a key head and all v_rep value heads, not one
    int out_f32;               // out is float whatever the type of q and the pools
    // decode steps on the tensor cores only: memory that a later kernel streams (the next part's first weights), or
    // null; every CTA asks L2 for its share once its own keys and values are through
    const unsigned char* pf_ptr;
    unsigned long long pf_bytes;
};

// decode steps (one new token per row) on the tensor cores; returns 1 if it
// does not take the sizes (the caller then uses the CUDA-core kernel)
int launch_attn_decode_mma(const AttnParams& p, int n_rows, cudaStream_t stream);
// prompt steps (several new tokens per row) on the tensor cores; same return convention
int launch_attn_prefill_mma(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream);
// prompt steps with capped scores, kept first keys, a keyless softmax term or repeated value heads (head sizes 64 and 128)
int launch_attn_prefill_mma_ext(const AttnParams& p, int n_rows, int max_q_len, cudaStream_t stream);
// the same on the tcgen05 tensor cores (head size 128, block sizes 8..128 that divide 128)
int launch_attn_prefill_tcgen05(const AttnParams& p, int n_rows, int T, int max_q_len, cudaStream_t stream);

}  // namespace fd
