// Attention over a shared latent: what comes between the input projection and the attention kernel.
//
// A token's projection row (float32) holds, for each of H heads, ``dn`` unrotated and ``rd`` rotated query
// dimensions, and, in a layer that owns its keys, ``r`` latent dimensions and ``rd`` dimensions of one rotated key
// part that all heads share.  Per token this kernel
//   * copies the heads' unrotated query parts out in the compute dtype (the input of the per-head product with
//     the key expansion, which moves the query into the latent space),
//   * rotates the heads' rotated parts and writes them behind the place of that product's result, so that a
//     head's query row is [latent r | rotated rd | zero padding] of ``dk`` elements,
//   * RMS-norms the latent (float32, plain weight), rotates the shared key part, and writes the token's cache
//     row [latent r | rotated rd | zero padding] to the step's own rows and, where nothing of the step still
//     reads the row it replaces, into the cache's page.
// A row is padded to a multiple of 8 elements; the padding is zero in queries and keys, so scores ignore it.
// Keys and values are never expanded per head: the attention kernels score a head's [latent | rotated] query
// against the cached row and take the row's latent part as the value (AttnArgs.v_alias), and a per-head product
// with the value expansion follows.
#include "common.cuh"
#include "qk_args.h"

struct LatentArgs {
    const float* in; int in_stride;         // [T][in_stride] float32: H * (dn + rd) query columns, then r + rd
    void* q_nope; int qn_stride;            // [T][qn_stride]: head h at h * dn
    void* q_abs; int qa_stride;             // [T][qa_stride]: head h at h * dk; this kernel writes [r, dk) of each
    void* kv_rows; int kv_stride;           // [T][kv_stride] rows of dk (owner only; may be null)
    const float* latent_w; float eps;       // norm of the latent: weight [r]
    TbRotary rope;
    int H; int dn; int rd; int r; int dk;
    int owner;                              // the projection row holds a latent and a key part
    const int* pos_of; const int* seq_of; const int* slot_of_seq; const int* kv_len;
    TbKvView cache; int append; int T;
    void* q_full; int qf_stride;            // if set: [T][qf_stride], head h at h * (dn + rd) as [unrotated dn | rotated rd]; q_nope and q_abs are not written
    const float* kv_in;                     // where the first row's r + rd latent and key columns start, if not right behind the query columns (rows in_stride apart)
};

namespace {

// Element e of the rotated form of ``x`` (rd elements, the first rope.rot of them rotated), cs/sn by pair index.
__device__ __forceinline__ float rotated(const float* x, int e, const TbRotary& rope, const float* cs, const float* sn) {
    if (!rope.inv_freq || e >= rope.rot) return x[e];
    int k, partner; float sign;
    tb_rotary_pair(rope, e, &k, &partner, &sign);
    return x[e] * cs[k] + sign * x[partner] * sn[k];
}

template <typename T>
__global__ void __launch_bounds__(128) latent_prep_kernel(LatentArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int half = a.rope.rot >> 1;
    float* cs = sm;                         // [half]
    float* sn = cs + half;                  // [half]
    const float* row = a.in + (size_t)t * a.in_stride;
    const int pos = a.pos_of[t];
    if (a.rope.inv_freq) {
        const float p = (float)pos + a.rope.offset;
        for (int k = threadIdx.x; k < half; k += blockDim.x) {
            float sv, cv;
            sincosf(p * a.rope.inv_freq[k], &sv, &cv);
            sn[k] = sv * a.rope.magnitude; cs[k] = cv * a.rope.magnitude;
        }
    }
    __syncthreads();
    const int qw = a.dn + a.rd;
    if (a.q_full) {                          // whole heads for a kernel that scores expanded keys: [unrotated | rotated]
        T* qf = (T*)a.q_full + (size_t)t * a.qf_stride;
        for (int i = threadIdx.x; i < a.H * qw; i += blockDim.x) {
            const int h = i / qw, d = i % qw;
            stf(qf + i, d < a.dn ? row[i] : rotated(row + h * qw + a.dn, d - a.dn, a.rope, cs, sn));
        }
    } else {
        T* qn = (T*)a.q_nope + (size_t)t * a.qn_stride;
        T* qa = (T*)a.q_abs + (size_t)t * a.qa_stride;
        for (int i = threadIdx.x; i < a.H * a.dn; i += blockDim.x) {
            const int h = i / a.dn, d = i % a.dn;
            stf(qn + i, row[h * qw + d]);
        }
        const int tail = a.dk - a.r;        // rotated part and padding
        for (int i = threadIdx.x; i < a.H * tail; i += blockDim.x) {
            const int h = i / tail, e = i % tail;
            stf(qa + (size_t)h * a.dk + a.r + e, e < a.rd ? rotated(row + h * qw + a.dn, e, a.rope, cs, sn) : 0.f);
        }
    }
    if (!a.owner) return;
    const float* lat = a.kv_in ? a.kv_in + (size_t)t * a.in_stride : row + a.H * qw;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.r; i += blockDim.x) ss += lat[i] * lat[i];
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)a.r + a.eps);
    const int seq = a.seq_of[t];
    const bool to_cache = a.append && !(a.cache.ring_rows && a.kv_len && pos < a.kv_len[seq] - a.cache.ring_rows);
    T* own = a.kv_rows ? (T*)a.kv_rows + (size_t)t * a.kv_stride : nullptr;
    T* page = to_cache ? (T*)a.cache.storage + kv_row_offset(a.cache, a.slot_of_seq[seq], pos, 0) : nullptr;
    for (int i = threadIdx.x; i < a.dk; i += blockDim.x) {
        float v;
        if (i < a.r) v = lat[i] * scale * a.latent_w[i];
        else if (i < a.r + a.rd) v = rotated(lat + a.r, i - a.r, a.rope, cs, sn);
        else v = 0.f;
        if (own) stf(own + i, v);
        if (page) stf(page + i, v);
    }
}

// Rows of the step into the cache, after the last layer that still reads what they replace has run.
template <typename T>
__global__ void latent_append_kernel(const T* __restrict__ rows, int stride, TbKvView c, const int* pos_of,
                                     const int* seq_of, const int* slot_of_seq, const int* kv_len) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int seq = seq_of[t], pos = pos_of[t];
    if (c.ring_rows && pos < kv_len[seq] - c.ring_rows) return;
    const T* src = rows + (size_t)t * stride;
    T* dst = (T*)c.storage + kv_row_offset(c, slot_of_seq[seq], pos, 0);
    for (int e = threadIdx.x; e < c.head_dim; e += blockDim.x) dst[e] = src[e];
}

}  // namespace

extern "C" int tb_latent_prep(const LatentArgs* args, int out_dtype, cudaStream_t stream) {
    LatentArgs a = *args;
    TB_REQUIRE(a.T > 0 && a.H > 0 && a.dn > 0 && a.rd >= 0 && a.r > 0, "latent_prep: sizes must be positive");
    TB_REQUIRE(a.dk >= a.r + a.rd && a.dk % 8 == 0, "latent_prep: a row of %d elements for %d + %d (a multiple of 8 that holds both)", a.dk, a.r, a.rd);
    TB_REQUIRE(a.rope.rot >= 0 && a.rope.rot % 2 == 0 && a.rope.rot <= a.rd, "latent_prep: %d rotated dimensions of %d", a.rope.rot, a.rd);
    TB_REQUIRE(a.in && (a.q_full || (a.q_nope && a.q_abs)), "latent_prep: missing buffers");
    TB_REQUIRE(a.in_stride >= a.H * (a.dn + a.rd) + ((a.owner && !a.kv_in) ? a.r + a.rd : 0), "latent_prep: the projection row is too short");
    TB_REQUIRE(!a.owner || a.latent_w, "latent_prep: the latent's norm weight is missing");
    TB_REQUIRE(!a.append || (a.owner && a.cache.storage && a.cache.head_dim == a.dk && a.cache.kv_heads == 1), "latent_prep: the cache view does not match the rows");
    const size_t smem = (size_t)(a.rope.rot + 2) * sizeof(float);
    if (out_dtype == TB_F32) tb_launch(latent_prep_kernel<float>, a.T, 128, smem, stream, a);
    else if (out_dtype == TB_BF16) tb_launch(latent_prep_kernel<__nv_bfloat16>, a.T, 128, smem, stream, a);
    else TB_REQUIRE(false, "latent_prep: unknown dtype %d", out_dtype);
    TB_CHECK_LAUNCH("latent_prep");
    return 0;
}

extern "C" int tb_latent_append(const void* rows, int stride, int dtype, const TbKvView* cache, const TbBatch* b, cudaStream_t stream) {
    TB_REQUIRE(rows && cache && cache->storage && b && b->T > 0, "latent_append: nothing to append");
    TB_REQUIRE(cache->kv_heads == 1 && stride >= cache->head_dim, "latent_append: rows of %d for a cache of %d", stride, cache->head_dim);
    if (dtype == TB_F32) tb_launch(latent_append_kernel<float>, b->T, 128, 0, stream, (const float*)rows, stride, *cache, b->pos_of, b->seq_of, b->slot_of_seq, b->kv_len);
    else if (dtype == TB_BF16) tb_launch(latent_append_kernel<__nv_bfloat16>, b->T, 128, 0, stream, (const __nv_bfloat16*)rows, stride, *cache, b->pos_of, b->seq_of, b->slot_of_seq, b->kv_len);
    else TB_REQUIRE(false, "latent_append: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("latent_append");
    return 0;
}
