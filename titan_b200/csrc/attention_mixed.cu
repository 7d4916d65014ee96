// Softmax attention whose scores are shaped before the softmax and blended across heads, and the step before it.
//
//   tb_qkv_whole_norm       between the fused Q | K | V (| gate) projection and the attention: adds the projections' biases,
//                           divides ALL of a token's query elements by one root mean square (all heads together) and all of
//                           its key elements by another, times a weight as wide as the projection; writes the queries, the
//                           step's own K | V rows and the cache rows; adds the output projection's bias into the rows that
//                           the output projection will add into.  float32 in, compute dtype out.
//   tb_attn_mixed_prefill   queries of a ragged step over cache + step rows.  Where the tiles fit shared memory, a block takes
//                           TILE_Q neighbouring queries of one sequence and stages every round's 32 keys and values of all kv
//                           heads in shared memory once, for all the heads that read them and for both queries (what bounds the
//                           one-query kernel is the L2 traffic of every head of every query fetching its own rows)
//   tb_attn_mixed_decode    one query a sequence over its cached keys, cut into splits (tb_split_keys); partials in the
//                           layout of tb_attn_merge, which finishes
//
// For one (query i, key j) pair the nh heads' scores are made together:
//   s_g = q_g . k_kv(g) * scale;  s_g <- cap * tanh(s_g / cap);  s_g += rel[min(i - j, far)][g];  m_h = sum_g mix[h][g] s_g
// and head h's softmax runs over m_h.  A block takes one query (or one split of a sequence's keys) with one warp a head:
// in a round of 32 keys lane l of warp g scores key l for head g and leaves the shaped score in shared memory; after the
// block's barrier lane l of warp h blends the nh numbers of key l and folds them into head h's running softmax, then
// every lane adds its output dims over the 32 values.  The rounds' score buffers alternate, so a round costs one barrier.
// Scores, softmax and sums are float32 with precise expf and tanhf.
#include <float.h>

#include "attention_args.h"
#include "common.cuh"

struct WholeNormArgs {
    const float* in; int in_stride;         // [T][in_stride] float32: Q (nh * hd) | K (nkv * hd) | V (nkv * hd) | ...
    const float* bias;                      // [(nh + 2 nkv) * hd] added to the row first (null: none)
    const float* q_w; const float* k_w;     // [nh * hd], [nkv * hd] (null: no norm of that part)
    float eps;
    int q_count; int k_count;               // elements the means run over (heads padded with zeros count only their true width)
    void* q_out; int q_stride;              // [T][q_stride] compute dtype
    void* kv_out; int kv_stride;            // [T][kv_stride]: K | V rows of the step (null: to the cache only)
    int nh; int nkv; int hd;
    const int* pos_of; const int* seq_of; const int* slot_of_seq; const int* kv_len;
    TbKvView cache; int append; int T;
    const float* o_bias; float* o_out; int o_stride; int o_width;      // o_out[t][0..o_width) += o_bias (null: nothing)
};

namespace {

#define MIX_MAXE 8          // value rows of up to 256 elements

template <typename T> __device__ __forceinline__ void row8(const T* p, float* o);
template <> __device__ __forceinline__ void row8<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
template <> __device__ __forceinline__ void row8<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        o[2 * i] = __uint_as_float(w[i] << 16);
        o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
}

template <typename T>
__global__ void __launch_bounds__(128) qkv_whole_norm_kernel(WholeNormArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int Q = a.nh * a.hd, KV = a.nkv * a.hd;
    const float* row = a.in + (size_t)t * a.in_stride;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < Q + KV; i += blockDim.x) {
        const float v = row[i] + (a.bias ? a.bias[i] : 0.f);
        if (i < Q) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
    }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = a.q_w ? 1.0f / sqrtf(sq / (float)a.q_count + a.eps) : 1.f;
    const float rk = a.k_w ? 1.0f / sqrtf(sk / (float)a.k_count + a.eps) : 1.f;
    T* q = (T*)a.q_out + (size_t)t * a.q_stride;
    for (int i = threadIdx.x; i < Q; i += blockDim.x) {
        const float v = row[i] + (a.bias ? a.bias[i] : 0.f);
        stf(q + i, a.q_w ? v * rq * a.q_w[i] : v);
    }
    if (a.nkv > 0) {
        const int seq = a.seq_of[t], pos = a.pos_of[t];
        const bool to_cache = a.append && !(a.cache.ring_rows && a.kv_len && pos < a.kv_len[seq] - a.cache.ring_rows);
        T* own = a.kv_out ? (T*)a.kv_out + (size_t)t * a.kv_stride : nullptr;
        T* store = (T*)a.cache.storage;
        const size_t vhalf = to_cache ? kv_half_elems(a.cache) : 0;
        const int slot = a.slot_of_seq[seq];
        for (int i = threadIdx.x; i < 2 * KV; i += blockDim.x) {
            float v = row[Q + i] + (a.bias ? a.bias[Q + i] : 0.f);
            if (i < KV && a.k_w) v = v * rk * a.k_w[i];
            if (own) stf(own + i, v);
            if (to_cache) {
                const int j = i < KV ? i : i - KV, head = j / a.hd, e = j % a.hd;
                stf(store + (i < KV ? 0 : vhalf) + kv_row_offset(a.cache, slot, pos, head) + e, v);
            }
        }
    }
    if (a.o_bias)
        for (int i = threadIdx.x; i < a.o_width; i += blockDim.x) a.o_out[(size_t)t * a.o_stride + i] += a.o_bias[i];
}

// Running softmax of one head (a warp): every lane holds the same m and l, and acc for value dims lane + 32 j.
struct Running {
    float m, l;
    float acc[MIX_MAXE];
};

// Folds keys [lo, hi) of one sequence into ``st``, for the query at position ``qpos``; all warps of the block call it with
// the same range.  Keys at positions >= first_new come from the step's own rows, earlier ones from the cache.  ``round``
// counts the rounds the block has run (it chooses the score buffer).
template <typename T>
__device__ __forceinline__ void attend_mixed(Running& st, const float* qs, float* raw, const float mix_w, const AttnArgs& a,
                                             int lo, int hi, int qpos, int first_new, int first_new_row, int slot, int h,
                                             int lane, int& round) {
    const int hd = a.hd, hdv = a.hd_v > 0 ? a.hd_v : a.hd, nh = a.nh, kh = h / (nh / a.nkv);
    const T* knew = (const T*)a.kv_new;
    const T* cache = (const T*)a.cache.storage;
    const size_t vhalf = cache ? kv_half_elems(a.cache) : 0;
    const int vnew = a.nkv * hd;
    for (int base = lo; base < hi; base += 32, ++round) {
        const int kpos = base + lane;
        const bool valid = kpos < hi;
        const T* kp = nullptr;
        const T* vp = nullptr;
        float s = 0.f;
        if (valid) {
            if (kpos >= first_new) {
                kp = knew + (size_t)(first_new_row + kpos - first_new) * a.kv_stride + kh * hd;
                vp = kp + vnew;
            } else {
                kp = cache + kv_row_offset(a.cache, slot, kpos, kh);
                vp = kp + vhalf;
            }
            float dot = 0.f;
            for (int e = 0; e < hd; e += 8) {
                float kv[8];
                row8<T>(kp + e, kv);
#pragma unroll
                for (int i = 0; i < 8; ++i) dot = fmaf(qs[e + i], kv[i], dot);
            }
            s = dot * a.scale;
            if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
            if (a.rel_bias) s += a.rel_bias[(size_t)min(qpos - kpos, a.rel_far) * nh + h];
        }
        if (a.head_mix) {
            float* buf = raw + (round & 1) * nh * 32;
            buf[h * 32 + lane] = s;
            __syncthreads();
            float m = 0.f;
            for (int g = 0; g < nh; ++g) m = fmaf(__shfl_sync(0xffffffffu, mix_w, g), buf[g * 32 + lane], m);
            s = m;
        }
        if (!valid) s = -FLT_MAX;
        const float m_new = fmaxf(st.m, warp_max(s));
        const float alpha = expf(st.m - m_new);           // st.m = -FLT_MAX at the start: exp(-huge) = 0
        const float p = valid ? expf(s - m_new) : 0.f;
        st.l = st.l * alpha + warp_sum(p);
        st.m = m_new;
#pragma unroll
        for (int j = 0; j < MIX_MAXE; ++j) st.acc[j] *= alpha;
        // Values: four keys at a time, all their loads issued before the sums (a key's loads alone would wait out a round
        // trip to L2 each).  Lanes beyond the range hold p = 0 and the address of the round's first row, so a group of four
        // needs no tail.
        const unsigned long long v_first = __shfl_sync(0xffffffffu, (unsigned long long)vp, 0);
        const unsigned long long v_mine = valid ? (unsigned long long)vp : v_first;
        const int n_valid = min(32, hi - base);
        for (int kk = 0; kk < n_valid; kk += 4) {
            float pk[4];
            const T* v[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                pk[u] = __shfl_sync(0xffffffffu, p, kk + u);
                v[u] = (const T*)__shfl_sync(0xffffffffu, v_mine, kk + u);
            }
            float x[4][MIX_MAXE];
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int j = 0; j < MIX_MAXE; ++j) {
                    const int d = lane + 32 * j;
                    x[u][j] = d < hdv ? ldf(v[u] + d) : 0.f;
                }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int j = 0; j < MIX_MAXE; ++j) st.acc[j] = fmaf(pk[u], x[u][j], st.acc[j]);
        }
    }
}

// shared memory: nh * hd query floats, then 2 * nh * 32 scores
template <typename T>
__device__ __forceinline__ void load_heads(float* qs, const T* q, int n, int tid, int threads) {
    for (int e = tid; e < n; e += threads) qs[e] = ldf(q + e);
    __syncthreads();
}

// grid (T); block of nh warps.
template <typename T>
__global__ void __launch_bounds__(1024) attn_mixed_prefill_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    const int t = blockIdx.x, hd = a.hd, nh = a.nh;
    float* raw = sm + nh * hd;
    load_heads<T>(sm, (const T*)a.q + (size_t)t * a.q_stride, nh * hd, threadIdx.x, blockDim.x);
    const float mix_w = (a.head_mix && lane < nh) ? a.head_mix[h * nh + lane] : 0.f;
    const int seq = a.batch.seq_of[t], pos = a.batch.pos_of[t];
    const int slot = a.batch.slot_of_seq[seq];
    const int first_new = a.kv_new ? a.batch.start_pos[seq] : 0x7fffffff;
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    Running st;
    st.m = -FLT_MAX; st.l = 0.f;
#pragma unroll
    for (int j = 0; j < MIX_MAXE; ++j) st.acc[j] = 0.f;
    int round = 0;
    attend_mixed<T>(st, sm + h * hd, raw, mix_w, a, lo, pos + 1, pos, first_new, a.batch.q_start[seq], slot, h, lane, round);
    float inv = 1.0f / st.l;
    if (a.head_gate) inv *= 1.0f / (1.0f + expf(-a.head_gate[(size_t)t * a.head_gate_stride + h]));
    const int hdv = a.hd_v > 0 ? a.hd_v : a.hd;
    T* o = (T*)a.out + (size_t)t * a.out_stride + h * hdv;
#pragma unroll
    for (int j = 0; j < MIX_MAXE; ++j) {
        const int d = lane + 32 * j;
        if (d < hdv) stf(o + d, st.acc[j] * inv);
    }
}

// grid (B, n_splits); block of nh warps.  Partial of (sequence b, head h, split s) at
// scratch[((b * nh + h) * n_splits + s) * (hdv + 2)]: hdv unnormalised outputs, then m, then l (0: the split saw no key).
template <typename T>
__global__ void __launch_bounds__(1024) attn_mixed_decode_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    const int b = blockIdx.x, split = blockIdx.y, hd = a.hd, nh = a.nh;
    const int hdv = a.hd_v > 0 ? a.hd_v : a.hd;
    const int len = a.batch.kv_len[b];
    const int keys = tb_split_keys(len, a.chunk, a.n_splits);
    if ((long long)split * keys >= len) return;     // the merge reads ceil(len / keys) splits only
    const int pos = len - 1;
    const int slot = a.batch.slot_of_seq[b];
    const int wlo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    const int lo = max(wlo, split * keys), hi = min(len, (split + 1) * keys);
    float* raw = sm + nh * hd;
    Running st;
    st.m = -FLT_MAX; st.l = 0.f;
#pragma unroll
    for (int j = 0; j < MIX_MAXE; ++j) st.acc[j] = 0.f;
    if (lo < hi) {
        load_heads<T>(sm, (const T*)a.q + (size_t)b * a.q_stride, nh * hd, threadIdx.x, blockDim.x);
        const float mix_w = (a.head_mix && lane < nh) ? a.head_mix[h * nh + lane] : 0.f;
        int round = 0;
        attend_mixed<T>(st, sm + h * hd, raw, mix_w, a, lo, hi, pos, 0x7fffffff, 0, slot, h, lane, round);
    }
    float* part = a.scratch + ((size_t)(b * nh + h) * a.n_splits + split) * (hdv + 2);
#pragma unroll
    for (int j = 0; j < MIX_MAXE; ++j) {
        const int d = lane + 32 * j;
        if (d < hdv) part[d] = st.acc[j];
    }
    if (lane == 0) { part[hdv] = st.m; part[hdv + 1] = st.l; }
}

template <typename T> __device__ __forceinline__ float2 pair2(const T* p);
template <> __device__ __forceinline__ float2 pair2<float>(const float* p) { return *reinterpret_cast<const float2*>(p); }
template <> __device__ __forceinline__ float2 pair2<__nv_bfloat16>(const __nv_bfloat16* p) {
    const uint32_t w = *reinterpret_cast<const uint32_t*>(p);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xffff0000u));
}
template <typename T> struct Chunk8;
template <> struct Chunk8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = reinterpret_cast<const float4*>(p)[0]; b = reinterpret_cast<const float4*>(p)[1]; }
    __device__ __forceinline__ void store(float* p) const { reinterpret_cast<float4*>(p)[0] = a; reinterpret_cast<float4*>(p)[1] = b; }
};
template <> struct Chunk8<__nv_bfloat16> {
    uint4 a;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { a = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void store(__nv_bfloat16* p) const { *reinterpret_cast<uint4*>(p) = a; }
};
template <typename T> __device__ __forceinline__ void zero8(T* dst);
template <> __device__ __forceinline__ void zero8<float>(float* dst) {
    reinterpret_cast<float4*>(dst)[0] = make_float4(0.f, 0.f, 0.f, 0.f);
    reinterpret_cast<float4*>(dst)[1] = make_float4(0.f, 0.f, 0.f, 0.f);
}
template <> __device__ __forceinline__ void zero8<__nv_bfloat16>(__nv_bfloat16* dst) { *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0); }

#define TILE_Q 2            // queries a block of the tiled kernel takes
#define TILE_MAXJ 4         // a lane holds value dims 2 * lane + 64 j and the next one: rows of up to 256

// Shared memory of the tiled kernel, in this order: TILE_Q * nh * hd query floats; TILE_Q * 2 * nh * 32 scores; then the
// K tile and the V tile, each nkv * 32 rows of hd + 8 elements of T (the 8 spare elements keep a lane's 16-byte reads of
// its own row off its neighbours' banks); then one address a row of the tiles.
template <typename T>
size_t tile_smem(const AttnArgs& a) {
    return ((size_t)TILE_Q * a.nh * a.hd + (size_t)TILE_Q * 2 * a.nh * 32) * sizeof(float) + 2 * (size_t)a.nkv * 32 * (a.hd + 8) * sizeof(T)
           + 2 * (size_t)a.nkv * 32 * sizeof(void*);           // and where each row of the tiles comes from
}

// grid (ceil(max_new / TILE_Q), B); block of nh warps.  Block (i, b) takes queries i * TILE_Q .. of sequence b.
template <typename T>
__global__ void __launch_bounds__(1024) attn_mixed_prefill_tile_kernel(AttnArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
    const int b = blockIdx.y, hd = a.hd, nh = a.nh, nkv = a.nkv, row = hd + 8;
    const int hdv = a.hd_v > 0 ? a.hd_v : a.hd;
    const int t0 = a.batch.q_start[b] + blockIdx.x * TILE_Q, t_end = a.batch.q_start[b + 1];
    if (t0 >= t_end) return;
    const int nq = min(TILE_Q, t_end - t0);
    float* qs = sm;
    float* raw = qs + TILE_Q * nh * hd;
    T* kt = reinterpret_cast<T*>(raw + TILE_Q * 2 * nh * 32);
    T* vt = kt + (size_t)nkv * 32 * row;
    for (int e = threadIdx.x; e < TILE_Q * nh * hd; e += blockDim.x) {
        const int q = e / (nh * hd), i = e % (nh * hd);
        qs[e] = q < nq ? ldf((const T*)a.q + (size_t)(t0 + q) * a.q_stride + i) : 0.f;
    }
    const float mix_w = (a.head_mix && lane < nh) ? a.head_mix[h * nh + lane] : 0.f;
    const int slot = a.batch.slot_of_seq[b];
    const int pos0 = a.batch.pos_of[t0], pos_last = pos0 + nq - 1;
    const int first_new = a.kv_new ? a.batch.start_pos[b] : 0x7fffffff, first_new_row = a.batch.q_start[b];
    const int lo = a.window > 0 ? max(0, pos0 - a.window + 1) : 0, hi = pos_last + 1;
    const int kh = h / (nh / nkv);
    const T* knew = (const T*)a.kv_new;
    const T* cache = (const T*)a.cache.storage;
    const size_t vhalf = cache ? kv_half_elems(a.cache) : 0;
    const int chunks = hd >> 3;
    float m_run[TILE_Q], l_run[TILE_Q], acc[TILE_Q][2 * TILE_MAXJ];
#pragma unroll
    for (int q = 0; q < TILE_Q; ++q) {
        m_run[q] = -FLT_MAX; l_run[q] = 0.f;
#pragma unroll
        for (int j = 0; j < 2 * TILE_MAXJ; ++j) acc[q][j] = 0.f;
    }
    // Row id (v * nkv + g) * 32 + r is key base + r of kv head g, in the K tile (v = 0) or the V tile (v = 1); src_of[id] is where
    // its hd elements lie (in the step's own rows or in the cache's page), null past the range.
    const int n_rows = 2 * nkv * 32;
    const T** src_of = reinterpret_cast<const T**>(vt + (size_t)nkv * 32 * row);
    const int cshift = (chunks & (chunks - 1)) == 0 ? __ffs(chunks) - 1 : -1;
    auto locate_rows = [&](int base) {
        for (int id = threadIdx.x; id < n_rows; id += blockDim.x) {
            const int r = id & 31, gv = id >> 5, is_v = gv >= nkv, g = gv - is_v * nkv, kpos = base + r;
            const T* src = nullptr;
            if (kpos < hi)
                src = kpos >= first_new
                    ? knew + (size_t)(first_new_row + kpos - first_new) * a.kv_stride + (is_v ? nkv * hd : 0) + g * hd
                    : cache + (is_v ? vhalf : 0) + kv_row_offset(a.cache, slot, kpos, g);
            src_of[id] = src;
        }
    };
    locate_rows(lo);
    int round = 0;
    for (int base = lo; base < hi; base += 32, ++round) {
        __syncthreads();                                    // the tiles of the round before have been read (and the queries and the rows' places are there)
        // Eight elements a copy, two copies a thread in flight (both loads are issued before the first store).  Where a row comes
        // from was worked out once a row, by the threads that had the round before's scores to wait for (``src_of``); a row past
        // the range is stored as zeros.  Copy c is part c % chunks of row c / chunks: a shift where the head's width allows.
        const int total = n_rows * chunks;
        for (int c0 = threadIdx.x; c0 < total; c0 += 2 * blockDim.x) {
            Chunk8<T> held[2];
            T* dst[2];
            bool real[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int c = min(c0 + u * (int)blockDim.x, total - 1);
                const int rid = cshift >= 0 ? c >> cshift : c / chunks, part = c - rid * chunks;
                const T* src = src_of[rid];
                real[u] = src != nullptr;
                dst[u] = kt + (size_t)rid * row + part * 8;          // the V tile lies right behind the K tile: row ids run through both
                held[u].load((real[u] ? src : src_of[0]) + part * 8);
            }
#pragma unroll
            for (int u = 0; u < 2; ++u)
                if (c0 + u * (int)blockDim.x < total) { if (real[u]) held[u].store(dst[u]); else zero8<T>(dst[u]); }
        }
        __syncthreads();
        if (base + 32 < hi) locate_rows(base + 32);          // for the next round; nothing reads the list before that round's first barrier
        const int kpos = base + lane;
        float s[TILE_Q];
#pragma unroll
        for (int q = 0; q < TILE_Q; ++q) s[q] = 0.f;
        {
            const T* kp = kt + ((size_t)kh * 32 + lane) * row;
            for (int e = 0; e < hd; e += 8) {
                float kv[8];
                row8<T>(kp + e, kv);
#pragma unroll
                for (int q = 0; q < TILE_Q; ++q) {
                    const float* qv = qs + (q * nh + h) * hd + e;
#pragma unroll
                    for (int i = 0; i < 8; ++i) s[q] = fmaf(qv[i], kv[i], s[q]);
                }
            }
        }
        bool seen[TILE_Q];
#pragma unroll
        for (int q = 0; q < TILE_Q; ++q) {
            const int qpos = pos0 + q;
            seen[q] = q < nq && kpos <= qpos && (a.window <= 0 || kpos > qpos - a.window);
            float v = 0.f;
            if (seen[q]) {
                v = s[q] * a.scale;
                if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
                if (a.rel_bias) v += a.rel_bias[(size_t)min(qpos - kpos, a.rel_far) * nh + h];
            }
            s[q] = v;
        }
        if (a.head_mix) {
            float* buf = raw + (round & 1) * TILE_Q * nh * 32;
#pragma unroll
            for (int q = 0; q < TILE_Q; ++q) buf[(q * nh + h) * 32 + lane] = s[q];
            __syncthreads();
#pragma unroll
            for (int q = 0; q < TILE_Q; ++q) s[q] = 0.f;
            for (int g = 0; g < nh; ++g) {
                const float w = __shfl_sync(0xffffffffu, mix_w, g);
#pragma unroll
                for (int q = 0; q < TILE_Q; ++q) s[q] = fmaf(w, buf[(q * nh + g) * 32 + lane], s[q]);
            }
        }
        float p[TILE_Q];
#pragma unroll
        for (int q = 0; q < TILE_Q; ++q) {
            const float sv = seen[q] ? s[q] : -FLT_MAX;
            const float m_new = fmaxf(m_run[q], warp_max(sv));
            const float alpha = expf(m_run[q] - m_new);
            p[q] = seen[q] ? expf(sv - m_new) : 0.f;
            l_run[q] = l_run[q] * alpha + warp_sum(p[q]);
            m_run[q] = m_new;
#pragma unroll
            for (int j = 0; j < 2 * TILE_MAXJ; ++j) acc[q][j] *= alpha;
        }
        const T* vbase = vt + (size_t)kh * 32 * row + 2 * lane;
        const int n_valid = min(32, hi - base);
        for (int kk = 0; kk < n_valid; ++kk) {
            float pk[TILE_Q];
#pragma unroll
            for (int q = 0; q < TILE_Q; ++q) pk[q] = __shfl_sync(0xffffffffu, p[q], kk);
            const T* v = vbase + (size_t)kk * row;
#pragma unroll
            for (int j = 0; j < TILE_MAXJ; ++j) {
                if (2 * lane + 64 * j < hdv) {
                    const float2 x = pair2<T>(v + 64 * j);
#pragma unroll
                    for (int q = 0; q < TILE_Q; ++q) {
                        acc[q][2 * j] = fmaf(pk[q], x.x, acc[q][2 * j]);
                        acc[q][2 * j + 1] = fmaf(pk[q], x.y, acc[q][2 * j + 1]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int q = 0; q < TILE_Q; ++q) {
        if (q >= nq) break;
        float inv = 1.0f / l_run[q];
        if (a.head_gate) inv *= 1.0f / (1.0f + expf(-a.head_gate[(size_t)(t0 + q) * a.head_gate_stride + h]));
        T* o = (T*)a.out + (size_t)(t0 + q) * a.out_stride + h * hdv;
#pragma unroll
        for (int j = 0; j < TILE_MAXJ; ++j) {
            const int d = 2 * lane + 64 * j;
            if (d < hdv) { stf(o + d, acc[q][2 * j] * inv); stf(o + d + 1, acc[q][2 * j + 1] * inv); }
        }
    }
}

int check_mixed(const AttnArgs& a, const char* who) {
    TB_REQUIRE(a.nh > 0 && a.nkv > 0 && a.nh % a.nkv == 0, "%s: %d query heads are not a multiple of %d kv heads", who, a.nh, a.nkv);
    TB_REQUIRE(a.nh <= 32, "%s: %d heads (one warp a head, at most 32)", who, a.nh);
    TB_REQUIRE(a.hd >= 8 && a.hd % 8 == 0 && a.hd <= 32 * MIX_MAXE, "%s: head_dim %d must be a multiple of 8 up to %d", who, a.hd, 32 * MIX_MAXE);
    TB_REQUIRE(a.hd_v >= 0 && a.hd_v <= 32 * MIX_MAXE && !a.v_alias, "%s: a value row of %d elements (at most %d, stored apart from the key)", who, a.hd_v, 32 * MIX_MAXE);
    TB_REQUIRE(a.q_stride % 8 == 0 && a.kv_stride % 8 == 0, "%s: row strides must be multiples of 8 elements", who);
    TB_REQUIRE(a.window >= 0 && a.keep_first == 0 && !a.sink, "%s: no kept first tokens and no sink here", who);
    TB_REQUIRE(!a.cache.storage || (a.cache.head_dim == a.hd && a.cache.kv_heads == a.nkv), "%s: the cache view does not match the heads", who);
    TB_REQUIRE(!a.rel_bias || a.rel_far >= 0, "%s: the distance table needs its last row's distance", who);
    TB_REQUIRE(!a.head_gate || a.head_gate_stride >= a.nh, "%s: the heads' gates need a row of at least %d", who, a.nh);
    return 0;
}

size_t mixed_smem(const AttnArgs& a) { return ((size_t)a.nh * a.hd + 2 * (size_t)a.nh * 32) * sizeof(float); }

}  // namespace

extern "C" int tb_attn_merge(const AttnArgs* args, int dtype, cudaStream_t stream);

static int g_mixed_tile = 1;
extern "C" int tb_set_attn_mixed_tile(int on) { g_mixed_tile = on ? 1 : 0; return 0; }

extern "C" int tb_qkv_whole_norm(const WholeNormArgs* args, int out_dtype, cudaStream_t stream) {
    WholeNormArgs a = *args;
    TB_REQUIRE(a.T > 0 && a.nh > 0 && a.nkv >= 0 && a.hd > 0, "qkv_whole_norm: sizes must be positive");
    TB_REQUIRE(a.in && a.q_out && a.in_stride >= (a.nh + 2 * a.nkv) * a.hd, "qkv_whole_norm: the projection row is too short");
    TB_REQUIRE((!a.q_w || a.q_count > 0) && (!a.k_w || a.k_count > 0), "qkv_whole_norm: a norm needs the number of elements its mean runs over");
    TB_REQUIRE(a.nkv == 0 || (a.pos_of && a.seq_of && a.slot_of_seq), "qkv_whole_norm: the layout arrays are missing");
    TB_REQUIRE(!a.append || (a.nkv > 0 && a.cache.storage && a.cache.head_dim == a.hd && a.cache.kv_heads == a.nkv), "qkv_whole_norm: the cache view does not match the heads");
    TB_REQUIRE(!a.o_bias || (a.o_out && a.o_stride >= a.o_width && a.o_width > 0), "qkv_whole_norm: a bias of the output needs the rows it is added to");
    if (out_dtype == TB_F32) tb_launch(qkv_whole_norm_kernel<float>, a.T, 128, 0, stream, a);
    else if (out_dtype == TB_BF16) tb_launch(qkv_whole_norm_kernel<__nv_bfloat16>, a.T, 128, 0, stream, a);
    else TB_REQUIRE(false, "qkv_whole_norm: unknown dtype %d", out_dtype);
    TB_CHECK_LAUNCH("qkv_whole_norm");
    return 0;
}

extern "C" int tb_attn_mixed_prefill(const AttnArgs* args, int dtype, cudaStream_t stream) {
    AttnArgs a = *args;
    if (check_mixed(a, "attn_mixed_prefill")) return 1;
    TB_REQUIRE(a.batch.T > 0 && (a.kv_new || a.cache.storage), "attn_mixed_prefill: no tokens, or neither new keys nor a cache");
    TB_REQUIRE(dtype == TB_F32 || dtype == TB_BF16, "attn_mixed_prefill: unknown dtype %d", dtype);
    // The tiled kernel where a round's keys and values of every kv head fit shared memory beside the queries (value rows of an
    // even width, so that a lane's pair of dims is whole); g_mixed_tile 0 keeps the one-query kernel (tests compare the two).
    const size_t tsmem = dtype == TB_F32 ? tile_smem<float>(a) : tile_smem<__nv_bfloat16>(a);
    const int hdv = a.hd_v > 0 ? a.hd_v : a.hd;
    if (g_mixed_tile && tsmem <= 200 * 1024 && hdv % 2 == 0 && a.batch.max_new > 1 && a.batch.B <= 65535) {
        void (*kernel)(AttnArgs) = dtype == TB_F32 ? attn_mixed_prefill_tile_kernel<float> : attn_mixed_prefill_tile_kernel<__nv_bfloat16>;
        static bool configured[2] = {false, false};
        const int which = dtype == TB_BF16 ? 1 : 0;
        if (!configured[which]) {
            const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            TB_REQUIRE(e == cudaSuccess, "attn_mixed_prefill: cannot reserve shared memory: %s", cudaGetErrorString(e));
            configured[which] = true;
        }
        dim3 grid((a.batch.max_new + TILE_Q - 1) / TILE_Q, a.batch.B);
        tb_launch(kernel, grid, a.nh * 32, tsmem, stream, a);
        TB_CHECK_LAUNCH("attn_mixed_prefill");
        return 0;
    }
    const size_t smem = mixed_smem(a);
    TB_REQUIRE(smem <= 48 * 1024, "attn_mixed_prefill: %d heads of %d need %zu bytes of shared memory (at most 48 KB)", a.nh, a.hd, smem);
    if (dtype == TB_F32) tb_launch(attn_mixed_prefill_kernel<float>, a.batch.T, a.nh * 32, smem, stream, a);
    else if (dtype == TB_BF16) tb_launch(attn_mixed_prefill_kernel<__nv_bfloat16>, a.batch.T, a.nh * 32, smem, stream, a);
    else TB_REQUIRE(false, "attn_mixed_prefill: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("attn_mixed_prefill");
    return 0;
}

extern "C" int tb_attn_mixed_decode(const AttnArgs* args, int dtype, cudaStream_t stream) {
    AttnArgs a = *args;
    if (check_mixed(a, "attn_mixed_decode")) return 1;
    TB_REQUIRE(a.batch.B > 0 && a.cache.storage && a.scratch, "attn_mixed_decode: needs sequences, a cache and scratch");
    TB_REQUIRE(a.chunk > 0 && a.n_splits > 0 && a.n_splits <= 65535, "attn_mixed_decode: bad split (chunk=%d splits=%d)", a.chunk, a.n_splits);
    const size_t smem = mixed_smem(a);
    TB_REQUIRE(smem <= 48 * 1024, "attn_mixed_decode: %d heads of %d need %zu bytes of shared memory (at most 48 KB)", a.nh, a.hd, smem);
    dim3 grid(a.batch.B, a.n_splits);
    if (dtype == TB_F32) tb_launch(attn_mixed_decode_kernel<float>, grid, a.nh * 32, smem, stream, a);
    else if (dtype == TB_BF16) tb_launch(attn_mixed_decode_kernel<__nv_bfloat16>, grid, a.nh * 32, smem, stream, a);
    else TB_REQUIRE(false, "attn_mixed_decode: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("attn_mixed_decode");
    return tb_attn_merge(args, dtype, stream);
}
