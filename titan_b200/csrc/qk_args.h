// Argument block of the Q/K head norm + rotary (+ cache append) kernel (elementwise.cu); mirrors
// titan_b200.kernels.QkArgs.
#pragma once
#include "common.cuh"

// What a position encoding hands to the kernels (titan_b200.kernels.RotaryArgs): the mixer passes it on
// without looking inside.  angle_k(position) = (position + offset) * inv_freq[k]; the pair
// (k, k + rot/2) of a head is rotated by that angle and scaled by ``magnitude``.
struct TbRotary {
    const float* inv_freq;                  // [rot/2] or null (no rotation)
    int rot;                                // leading dims of a head that are rotated
    float offset;                           // added to every position (0 for plain rotary)
    float magnitude;                        // factor on cosines and sines (1 for plain rotary)
    int adjacent;                           // 0: dimension k is paired with k + rot/2; 1: dimension 2k with 2k + 1 (both turn by angle_k)
};

// Element e (< rot) of a rotated row: x[e] cos(angle_k) -/+ x[partner] sin(angle_k), where the first member of a pair
// takes the minus.  Gives the pair's index k, the partner's index and the sign for either pairing.
__host__ __device__ __forceinline__ void tb_rotary_pair(const TbRotary& r, int e, int* k, int* partner, float* sign) {
    const int half = r.rot >> 1;
    if (r.adjacent) { *k = e >> 1; *partner = e ^ 1; *sign = (e & 1) ? 1.f : -1.f; }
    else { *k = e < half ? e : e - half; *partner = e < half ? e + half : e - half; *sign = e < half ? -1.f : 1.f; }
}

struct QkArgs {
    const void* in; int in_stride;          // [T][in_stride]: Q | K | V
    void* q_out; int q_stride;              // [T][q_stride]
    void* k_out; int k_stride;              // [T][k_stride] (null: K goes to the cache only)
    const float* q_w; const float* k_w;     // [hd] or null
    TbRotary rope;
    float eps; int nh; int nkv; int hd;
    const int* pos_of; const int* seq_of; const int* slot_of_seq;
    TbKvView cache; int append; int T;
    int zero_in;                            // after reading a head, write zeros over it (an accumulation buffer is left clean)
    const int* kv_len;                      // [B] lengths after the step: in a ring, a row that a later token of the step reuses is not written
    // The input rows are products of UNSCALED activations (the RMS norm before the projection was folded into the
    // product): row t is first multiplied by 1/sqrt(sum_z row_sumsq[z][t] / row_width + row_eps), the row_parts partial
    // sums [part][32] added in the order of the parts.  Null: the rows are as they should be.
    const float* row_sumsq; int row_parts; int row_width; float row_eps;
    // A unit norm of every Q and K head, with or without a weight: norm_dims > 0 divides a head by the root mean square over
    // its first norm_dims elements (heads padded with zeros beyond them keep their mean), multiplied by q_w / k_w where given.
    // norm_after: the mean is taken over the rotated head (after the rotation) instead of before it.
    int norm_dims; int norm_after;
    // Values blended across layers: V head rows become (1 - *v_mix) v + *v_mix v_first[t] before they go anywhere
    // (v_first: rows [T][v_first_stride] of the output dtype, the kv heads side by side, each v_first_head wide; null: no blending).  v_keep
    // (null: nowhere) receives the V rows as they go to the cache, [T][v_keep_stride] in the output dtype: the place a later
    // layer blends with, or the step's own V columns, which the prompt kernels read.
    const void* v_first; int v_first_stride; const float* v_mix;
    void* v_keep; int v_keep_stride;
    // Width of a head in the rows of v_first (0: hd): the layer that kept them may pad its heads to another width than this
    // one; elements beyond the narrower of the two are padding (zero) on both sides.
    int v_first_head;
    // A unit norm of every V head without a weight: v_norm_dims > 0 divides a value head by the root mean square over its
    // first v_norm_dims elements (eps v_eps inside the root) before it goes to the cache, to v_keep or into a blend.
    int v_norm_dims; float v_eps;
};
