// Argument block shared by the attention launchers (attention.cu, attention_mma.cu); mirrors
// titan_b200.kernels.AttnArgs.
#pragma once
#include "common.cuh"
#include "qk_args.h"

// Where the tensor-core prompt kernels take keys and values from.
#define TB_KV_FROM_STEP 1      // the step's own rows: every sequence of the step starts at position 0
#define TB_KV_FROM_CACHE 2     // the cache's pages, where the step's own keys have been appended already

struct AttnArgs {
    const void* q; int q_stride;            // [T][q_stride], head h at h*hd
    const void* kv_new; int kv_stride;      // [T][kv_stride]: K heads then V heads of this step (may be null)
    void* out; int out_stride;              // [T][out_stride]
    TbKvView cache;                         // storage may be null when every key is in kv_new
    TbBatch batch;
    int nh; int nkv; int hd;
    int window;                             // 0: all keys
    float scale;
    int chunk;                              // decode: fewest keys per split (see tb_split_keys)
    int n_splits;                           // decode: grid.z, the most splits a sequence is cut into
    float* scratch;                         // decode: [B][nh][n_splits][hd + 2]
    // decode, optional: lengths that were final before the step's first kernel ran, so that a kernel may read
    // them without waiting for its predecessors.  early_mode 1: early_len[b] = batch.kv_len[b] (the same numbers,
    // put there by a copy, not by a kernel); 2: early_len[slot] + 1 = batch.kv_len[b] (the cache's committed
    // length of the slot, for steps whose kv_len a kernel of the step computes); 0 or a null pointer: none.
    const int* early_len; int early_mode;
    // decode on tensor cores, optional: the head norm / rotary / append step folded into the attention kernel.  The
    // queries and the new token's key and value then come as the projection's float32 sums (fused_qk->in, rows of
    // fused_qk->in_stride: Q heads, K heads, V heads), with the norm weights, the rotary block, the row scales and the
    // cache of *fused_qk; ``q`` is not read.  Null: queries are bfloat16 rows at ``q`` and the cache holds every key.
    const QkArgs* fused_qk;
    // Keys and values of unequal width (the any-size kernels only; zero: both are ``hd`` wide).  hd_v: width of a
    // value row, of a head's output row and of the scratch partials.  v_alias: a value row is the first hd_v
    // elements of its key row (one stored row per token serves as both: attention in a shared latent space, where
    // the key is [latent | rotated part] and the value the latent alone), so no V plane or V columns are read.
    int hd_v; int v_alias;
    // Decode, the any-size kernel: how many blocks share the query heads of a launch (grid.y).  Zero: one block per kv
    // head, whose warps take that head's query heads in turn.  A model with many query heads on one kv head (all heads
    // over one shared latent) asks for more blocks: block y then takes heads [y * nh / head_blocks, (y + 1) * nh / head_blocks)
    // and reads kv head y * nkv / head_blocks.  Must divide nh and be a multiple of nkv.
    int head_blocks;
    // A sink in the softmax: sink[h] (float32, one per query head; null: none) joins the denominator of head h as one more
    // term exp(sink[h] - max), unscaled, without a key and without a value, once per query however the keys are split.
    const float* sink;
    // With a window: the first keep_first positions of a sequence stay visible to every later query, at their true
    // positions, beside the window's keys (0: the window alone).
    int keep_first;
    // Scores shaped before the softmax (the mixed-heads kernels, attention_mixed.cu; all zero / null: none of it).
    // softcap > 0: s <- softcap * tanh(s / softcap) after the scale.  rel_bias: a table [rel_far + 1][nh] (float32) of
    // which row min(query position - key position, rel_far) is added to the capped scores of the nh heads.  head_mix:
    // [nh][nh] (float32); the score of head h becomes sum_g head_mix[h][g] * score_g, all heads of one (query, key) pair
    // together, before the softmax.
    float softcap; const float* rel_bias; int rel_far; const float* head_mix;
    // One gate a (token, head): head_gate[t * head_gate_stride + h] (float32 logits; null: none) multiplies head h's
    // output row by its sigmoid where the softmax is finished (the any-size merge and the mixed-heads kernels).
    const float* head_gate; int head_gate_stride;
};

// How decode attention cuts the keys of ONE sequence into splits: ``chunk`` keys each while ``n_splits`` of
// them cover the sequence, else ``n_splits`` equal parts of whole 64-key pages.  Split s takes keys
// [s * keys, (s + 1) * keys) below the length; splits that start at or beyond the length are empty.  The
// borders depend on the sequence's own length and on the launch's two numbers, never on the other sequences
// of the batch, on the longest context the engine allows or on where the sequence lies in the cache.
// (berniehans/titan: num_splits = min(32, ceil(S / 256)), engine/engine-cuda/src/paged_attention.rs:368-370.)
__host__ __device__ __forceinline__ int tb_split_keys(int len, int chunk, int n_splits) {
    if ((long long)chunk * n_splits >= len) return chunk;
    return (((len + n_splits - 1) / n_splits) + 63) & ~63;
}
