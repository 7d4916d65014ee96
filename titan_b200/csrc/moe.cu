// Mixture of experts: routing, the experts' products, and the weighted sum.
//
//   tb_moe_route     one warp a token: the ``top`` largest of its E router logits (float32; the lowest index wins a
//                    tie), their weights = softmax over the chosen logits only, and, if the router's row has one more
//                    column, the sigmoid of that column (the gate of an expert that every token uses).
//                    Token t's k-th choice is *pair* t * top + k.
//   tb_moe_plan      one block: pairs grouped by expert (``perm``: sorted place -> pair), and the list of row tiles
//                    (expert, first sorted row, rows) that the grouped product's blocks work through.
//   tb_moe_grouped   out = epilogue(X . W_e^T) on the CUDA cores for every tile of the plan, any size, either dtype:
//                    rows gathered from the tokens (gate-and-up, SwiGLU epilogue) or scattered back to pair order
//                    (down, float32).  The plain path and the true 32-bit path.
//   tb_moe_rows      the same two products for a handful of pairs (decode steps): a warp per output column (or
//                    gate/up pair) of one pair, lanes along K, weights read once per pair through L2; no plan.
//   tb_moe_combine   out[t] += sum_k weight[t][k] * y[t * top + k] (+ gate[t] * shared[t]), float32, in pair order.
#include <float.h>

#include "common.cuh"
#include "gemm.h"

#define MOE_BM 64
#define MOE_BN 64
#define MOE_BK 16

namespace {

// 16 bytes of a row as floats: 4 float32 or 8 bfloat16.
template <typename T> __device__ __forceinline__ void load_vec(const T* p, float* o);
template <> __device__ __forceinline__ void load_vec<float>(const float* p, float* o) {
    const float4 a = *reinterpret_cast<const float4*>(p);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w;
}
template <> __device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float* o) {
    const uint4 r = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

// ------------------------------------------------------------------ route
// One warp, the row's E logits in shared memory (``mine``; destroyed): the ``top`` largest, their softmax, the gate's sigmoid.
__device__ __forceinline__ void route_row(float* mine, int E, int top, int has_gate, float gate_logit, int* __restrict__ ids,
                                          float* __restrict__ wts, float* __restrict__ gate, int t, int lane) {
    float first = 0.f, total = 0.f;
    for (int k = 0; k < top; ++k) {
        float best = -FLT_MAX; int at = 0x7fffffff;
        for (int e = lane; e < E; e += 32) {
            const float v = mine[e];
            if (v > best) { best = v; at = e; }          // ascending e: the lowest index of equal values stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (k == 0) first = best;
        const float p = expf(best - first);               // the first chosen is the largest
        total += p;
        if (lane == 0) { ids[(size_t)t * top + k] = at; wts[(size_t)t * top + k] = p; mine[at] = -FLT_MAX; }
        __syncwarp();
    }
    const float inv = 1.0f / total;
    __syncwarp();
    for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= inv;
    if (has_gate && lane == 0) gate[t] = 1.0f / (1.0f + expf(-gate_logit));
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ z, int ldz, int E, int top, int has_gate,
                                                        int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ gate, int T_) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];           // per warp: E logits
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T_) return;
    float* mine = sm + (size_t)warp * E;
    const float* row = z + (size_t)t * ldz;
    for (int e = lane; e < E; e += 32) mine[e] = row[e];
    __syncwarp();
    route_row(mine, E, top, has_gate, has_gate ? row[E] : 0.f, ids, wts, gate, t, lane);
}

// Routing by scores over ALL experts: s = softmax(z) over the row's n_all logits; an expert is chosen by s + correction,
// and only inside the ``keep`` groups (of n_all / groups neighbours each) whose best such score is largest; the weights
// are the chosen experts' s over their sum (+ 1e-20).  One warp a token; the lowest index wins a tie.  ``score`` and
// ``choice`` are the warp's rows in shared memory.
// ``sigmoid``: the scores are sigmoids of the router's outputs, each on its own, instead of a softmax over the row.
// ``group_best``: a group's score is the sum of its ``group_best`` largest choice scores (1: its best one).  ``renorm`` 0:
// the weights are the chosen experts' scores as they are, not divided by their sum.
__global__ void __launch_bounds__(128) moe_route_all_kernel(const float* __restrict__ z, int ldz, int n_all, int top,
                                                            const float* __restrict__ correction, int groups, int keep,
                                                            int* __restrict__ ids, float* __restrict__ wts, int T_,
                                                            int sigmoid, int group_best, int renorm) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float sm[];           // per warp: n_all scores, n_all choice scores, ``groups`` group scores and as many marks
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int t = blockIdx.x * 4 + warp;
    if (t >= T_) return;
    float* score = sm + (size_t)warp * (2 * n_all + 2 * groups);
    float* choice = score + n_all;
    float* best_of = choice + n_all;
    float* kept = best_of + groups;
    const float* row = z + (size_t)t * ldz;
    if (sigmoid) {
        for (int e = lane; e < n_all; e += 32) {
            score[e] = 1.0f / (1.0f + expf(-row[e]));
            choice[e] = score[e] + (correction ? correction[e] : 0.f);
        }
    } else {
        float m = -FLT_MAX;
        for (int e = lane; e < n_all; e += 32) m = fmaxf(m, row[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < n_all; e += 32) { const float p = expf(row[e] - m); score[e] = p; sum += p; }
        sum = warp_sum(sum);
        const float inv = 1.0f / sum;
        for (int e = lane; e < n_all; e += 32) { score[e] *= inv; choice[e] = score[e] + (correction ? correction[e] : 0.f); }
    }
    __syncwarp();
    auto arg_max = [&](const float* v, int n, float* best_out) -> int {
        float best = -INFINITY; int at = 0x7fffffff;
        for (int e = lane; e < n; e += 32)
            if (v[e] > best) { best = v[e]; at = e; }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        *best_out = best;
        return at;
    };
    if (groups > 1 && keep < groups) {
        const int per = n_all / groups;
        for (int g = lane; g < groups; g += 32) {
            if (group_best <= 1) {
                float b = -INFINITY;
                for (int e = g * per; e < (g + 1) * per; ++e) b = fmaxf(b, choice[e]);
                best_of[g] = b;
            } else {                        // the sum of the group's largest few: one pass a rank, below the one before (ties by index)
                float total = 0.f, last = INFINITY;
                int last_at = -1;
                for (int k = 0; k < group_best && k < per; ++k) {
                    float b = -INFINITY;
                    int at = -1;
                    for (int e = g * per; e < (g + 1) * per; ++e) {
                        const float c = choice[e];
                        const bool below = c < last || (c == last && e > last_at);
                        if (below && c > b) { b = c; at = e; }
                    }
                    if (at < 0) break;
                    total += b; last = b; last_at = at;
                }
                best_of[g] = total;
            }
        }
        __syncwarp();
        for (int g = lane; g < groups; g += 32) kept[g] = 0.f;
        __syncwarp();
        for (int k = 0; k < keep; ++k) {
            float b;
            const int g = arg_max(best_of, groups, &b);
            __syncwarp();
            if (lane == 0 && g < groups) { best_of[g] = -INFINITY; kept[g] = 1.f; }
            __syncwarp();
        }
        for (int e = lane; e < n_all; e += 32)
            if (kept[e / per] == 0.f) choice[e] = -INFINITY;      // minus infinity, not zero: choice scores may be negative
        __syncwarp();
    }
    float total = 0.f;
    for (int k = 0; k < top; ++k) {
        float b;
        const int at = arg_max(choice, n_all, &b);
        const int e = at < n_all ? at : 0;
        const float w = score[e];
        total += w;
        __syncwarp();
        if (lane == 0) { ids[(size_t)t * top + k] = e; wts[(size_t)t * top + k] = w; choice[e] = -INFINITY; }
        __syncwarp();
    }
    if (!renorm) return;
    const float norm = 1.0f / (total + 1e-20f);
    for (int k = lane; k < top; k += 32) wts[(size_t)t * top + k] *= norm;
}

// ------------------------------------------------------------------ plan
// counts [E], rank [P] are scratch; perm [P]; tiles: tile_e, tile_row0, tile_rows [max_tiles]; n_tiles [1].
__global__ void __launch_bounds__(1024) moe_plan_kernel(const int* __restrict__ ids, int P, int E, int* __restrict__ rank,
                                                        int* __restrict__ perm, int* __restrict__ tile_e, int* __restrict__ tile_row0,
                                                        int* __restrict__ tile_rows, int* __restrict__ n_tiles, int max_tiles,
                                                        int* __restrict__ offsets, int* __restrict__ inverse) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ int smi[];            // count [E], offset [E]
    int* count = smi;
    int* offset = smi + E;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < P; i += blockDim.x) rank[i] = atomicAdd(&count[ids[i]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            offset[e] = at;
            for (int r0 = 0; r0 < count[e]; r0 += MOE_BM) {
                if (tiles < max_tiles) { tile_e[tiles] = e; tile_row0[tiles] = at + r0; tile_rows[tiles] = min(MOE_BM, count[e] - r0); }
                ++tiles;
            }
            at += count[e];
        }
        *n_tiles = min(tiles, max_tiles);
    }
    __syncthreads();
    for (int e = threadIdx.x; e <= E; e += blockDim.x) offsets[e] = e < E ? offset[e] : P;     // first sorted row of every expert, then P
    for (int i = threadIdx.x; i < P; i += blockDim.x) {
        const int at = offset[ids[i]] + rank[i];
        perm[at] = i;
        inverse[i] = at;
    }
}

// out[r] = x[perm[r] / top]: the tokens' rows in the plan's order, for products that want an expert's rows side by side.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ x, int ldx, const int* __restrict__ perm, int top, T* __restrict__ out, int K) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t r = blockIdx.x;
    const T* src = x + (size_t)(perm[r] / top) * ldx;
    T* dst = out + r * K;
    constexpr int PER = 16 / sizeof(T);
    if (K % PER == 0 && ((uintptr_t)src % 16 == 0) && ((uintptr_t)dst % 16 == 0)) {
        for (int e = threadIdx.x; e < K / PER; e += blockDim.x) reinterpret_cast<uint4*>(dst)[e] = reinterpret_cast<const uint4*>(src)[e];
    } else {
        for (int e = threadIdx.x; e < K; e += blockDim.x) dst[e] = src[e];
    }
}

// ------------------------------------------------------------------ grouped product on the CUDA cores
// MODE 0: rows of X are tokens, gathered as perm[row] / top; W [E][N][K] with gate and up rows interleaved; output row
//         = sorted row, SwiGLU epilogue in the compute dtype [P][N/2].
// MODE 1: rows of X are sorted rows; output (float32) goes to row perm[row] (pair order) [P][N].
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ X, int ldx, const T* __restrict__ W, void* __restrict__ out, int ldo,
                   const int* __restrict__ perm, const int* __restrict__ tile_e, const int* __restrict__ tile_row0,
                   const int* __restrict__ tile_rows, const int* __restrict__ n_tiles, int N, int K, int top, int n_real, int act, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    if ((int)blockIdx.y >= *n_tiles) return;
    if (tile_e[blockIdx.y] >= n_real) return;         // an expert without matrices (its output is its input): nothing to multiply
    __shared__ float xs[MOE_BK][MOE_BM + 4];
    __shared__ float ws[MOE_BK][MOE_BN + 4];
    __shared__ int src[MOE_BM];
    const int tid = threadIdx.x;
    const int e = tile_e[blockIdx.y], row0 = tile_row0[blockIdx.y], rows = tile_rows[blockIdx.y];
    const int n0 = blockIdx.x * MOE_BN;
    const T* We = W + (size_t)e * N * K;
    if (tid < MOE_BM) src[tid] = tid < rows ? perm[row0 + tid] : -1;
    __syncthreads();
    const int tx = tid % 16, ty = tid / 16;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int idx = tid + i * 256;
            const int r = idx / MOE_BK, kk = idx % MOE_BK;
            const int k = k0 + kk;
            float xv = 0.f;
            if (r < rows && k < K) {
                const size_t xr = MODE == 0 ? (size_t)(src[r] / top) : (size_t)(row0 + r);
                xv = ldf(X + xr * ldx + k);
            }
            xs[kk][r] = xv;
            ws[kk][r] = (n0 + r < N && k < K) ? ldf(We + (size_t)(n0 + r) * K + k) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MOE_BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = xs[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (r >= rows) continue;
        if (MODE == 0) {
            T* o = (T*)out + (size_t)(row0 + r) * ldo;
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int n = n0 + tx * 4 + j;
                if (n + 1 < N) {
                    const float g = acc[i][j], u = acc[i][j + 1];
                    stf(o + n / 2, tb_gated(act, limit, g, u));
                }
            }
        } else {
            float* o = (float*)out + (size_t)src[r] * ldo;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + tx * 4 + j;
                if (n < N) o[n] = acc[i][j];
            }
        }
    }
}

// ------------------------------------------------------------------ a few pairs: a warp per output
// MODE 0: act[p][n] = silu(W_e[2n] . x[p / top]) * (W_e[2n + 1] . x[p / top]); MODE 1: y[p][n] = W_e[n] . act[p].
template <typename T, int MODE>
__global__ void __launch_bounds__(256)
moe_rows_kernel(const T* __restrict__ X, int ldx, const T* __restrict__ W, void* __restrict__ out, int ldo,
                const int* __restrict__ ids, int N_out, int K, int top, int n_real, int act, float limit) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int p = blockIdx.x;
    const int n = blockIdx.y * 8 + warp;
    if (n >= N_out) return;
    const int e = ids[p];
    if (e >= n_real) return;                          // an expert without matrices: the combine kernel adds the input itself
    const T* x = X + (size_t)(MODE == 0 ? p / top : p) * ldx;
    constexpr int PER = 16 / sizeof(T);                 // elements of a 16-byte load
    const bool wide = K % PER == 0 && ldx % PER == 0 && ((uintptr_t)X % 16 == 0) && ((uintptr_t)W % 16 == 0);
    if (MODE == 0) {
        const T* wg = W + ((size_t)e * 2 * N_out + 2 * n) * K;
        const T* wu = wg + K;
        float g = 0.f, u = 0.f;
        if (wide) {
            for (int k = lane * PER; k < K; k += 32 * PER) {
                float xv[PER], a[PER], b[PER];
                load_vec<T>(x + k, xv); load_vec<T>(wg + k, a); load_vec<T>(wu + k, b);
#pragma unroll
                for (int i = 0; i < PER; ++i) { g = fmaf(a[i], xv[i], g); u = fmaf(b[i], xv[i], u); }
            }
        } else
        for (int k = lane; k < K; k += 32) {
            const float xv = ldf(x + k);
            g = fmaf(ldf(wg + k), xv, g);
            u = fmaf(ldf(wu + k), xv, u);
        }
        g = warp_sum(g); u = warp_sum(u);
        if (lane == 0) stf((T*)out + (size_t)p * ldo + n, tb_gated(act, limit, g, u));
    } else {
        const T* w = W + ((size_t)e * N_out + n) * K;
        float s = 0.f;
        if (wide) {
            for (int k = lane * PER; k < K; k += 32 * PER) {
                float xv[PER], a[PER];
                load_vec<T>(x + k, xv); load_vec<T>(w + k, a);
#pragma unroll
                for (int i = 0; i < PER; ++i) s = fmaf(a[i], xv[i], s);
            }
        } else
        for (int k = lane; k < K; k += 32) s = fmaf(ldf(w + k), ldf(x + k), s);
        s = warp_sum(s);
        if (lane == 0) ((float*)out)[(size_t)p * ldo + n] = s;
    }
}

// ------------------------------------------------------------------ combine
// ``ids`` with ``n_real`` and ``x``: a pair whose expert is n_real or beyond has no matrices and no row in y; its output
// is the token's own input row x[t].
template <typename T>
__global__ void moe_combine_kernel(const float* __restrict__ y, const float* __restrict__ wts, const float* __restrict__ shared_y,
                                   const float* __restrict__ gate, float* __restrict__ out, int H, int top, const int* __restrict__ where,
                                   const int* __restrict__ ids, int n_real, const T* __restrict__ x, int ldx) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.x;
    const int per = (H + gridDim.y - 1) / gridDim.y, i0 = blockIdx.y * per, i1 = min(H, i0 + per);      // gridDim.y blocks share a row (steps of few rows)
    for (int i = i0 + threadIdx.x; i < i1; i += blockDim.x) {
        float s = 0.f;
        for (int k = 0; k < top; ++k) {
            if (ids && ids[t * top + k] >= n_real) { s = fmaf(wts[t * top + k], ldf(x + t * ldx + i), s); continue; }
            const size_t row = where ? (size_t)where[t * top + k] : t * top + k;       // pair order, or where the plan put the pair
            s = fmaf(wts[t * top + k], y[row * H + i], s);
        }
        if (shared_y) s = fmaf(gate ? gate[t] : 1.f, shared_y[t * H + i], s);
        out[t * H + i] += s;
    }
}

}  // namespace

extern "C" int tb_moe_route(const float* z, int ldz, int E, int top, int has_gate, int* ids, float* wts, float* gate,
                            int T_, cudaStream_t stream) {
    TB_REQUIRE(T_ > 0 && E > 0 && top > 0 && top <= E, "moe_route: %d of %d experts", top, E);
    TB_REQUIRE(E <= 2048, "moe_route: %d experts (at most 2048)", E);
    TB_REQUIRE(ldz >= E + (has_gate ? 1 : 0) && z && ids && wts && (!has_gate || gate), "moe_route: missing buffers");
    tb_launch(moe_route_kernel, (T_ + 3) / 4, 128, (size_t)4 * E * sizeof(float), stream, z, ldz, E, top, has_gate, ids, wts, gate, T_);
    TB_CHECK_LAUNCH("moe_route");
    return 0;
}

extern "C" int tb_moe_route_scored(const float* z, int ldz, int n_all, int top, const float* correction, int groups, int keep,
                                   int* ids, float* wts, int T_, int sigmoid, int group_best, int renorm, cudaStream_t stream);

extern "C" int tb_moe_route_all(const float* z, int ldz, int n_all, int top, const float* correction, int groups, int keep,
                                int* ids, float* wts, int T_, cudaStream_t stream) {
    return tb_moe_route_scored(z, ldz, n_all, top, correction, groups, keep, ids, wts, T_, 0, 1, 1, stream);
}

// The same choice with the scores' kind (softmax over the row, or a sigmoid an output), the number of a group's best choice
// scores that make the group's score, and whether the chosen weights are divided by their sum, as arguments.
extern "C" int tb_moe_route_scored(const float* z, int ldz, int n_all, int top, const float* correction, int groups, int keep,
                                   int* ids, float* wts, int T_, int sigmoid, int group_best, int renorm, cudaStream_t stream) {
    TB_REQUIRE(group_best >= 1, "moe_route_all: a group's score is the sum of at least one of its experts' scores");
    TB_REQUIRE(T_ > 0 && n_all > 0 && top > 0 && top <= n_all && n_all <= 2048, "moe_route_all: %d of %d experts (at most 2048)", top, n_all);
    TB_REQUIRE(groups > 0 && keep > 0 && keep <= groups && n_all % groups == 0, "moe_route_all: %d groups of which %d are kept, over %d experts", groups, keep, n_all);
    TB_REQUIRE(top <= keep * (n_all / groups), "moe_route_all: %d experts a token out of %d groups of %d", top, keep, n_all / groups);
    TB_REQUIRE(ldz >= n_all && z && ids && wts, "moe_route_all: missing buffers");
    tb_launch(moe_route_all_kernel, (T_ + 3) / 4, 128, (size_t)4 * (2 * n_all + 2 * groups) * sizeof(float), stream, z, ldz, n_all, top, correction,
              groups, keep, ids, wts, T_, sigmoid, group_best, renorm);
    TB_CHECK_LAUNCH("moe_route_all");
    return 0;
}

extern "C" int tb_moe_plan_tiles(int pairs, int E) { return (pairs + MOE_BM - 1) / MOE_BM + E; }

extern "C" int tb_moe_plan(const int* ids, int P, int E, int* rank, int* perm, int* tile_e, int* tile_row0, int* tile_rows,
                           int* n_tiles, int max_tiles, int* offsets, int* inverse, cudaStream_t stream) {
    TB_REQUIRE(P > 0 && E > 0 && E <= 4096, "moe_plan: %d pairs, %d experts (at most 4096)", P, E);
    TB_REQUIRE(max_tiles >= tb_moe_plan_tiles(P, E), "moe_plan: room for %d tiles, %d may be needed", max_tiles, tb_moe_plan_tiles(P, E));
    tb_launch(moe_plan_kernel, 1, 1024, (size_t)2 * E * sizeof(int), stream, ids, P, E, rank, perm, tile_e, tile_row0, tile_rows, n_tiles, max_tiles, offsets, inverse);
    TB_CHECK_LAUNCH("moe_plan");
    return 0;
}

// mode 0: gate-and-up with SwiGLU (N = 2 * ff rows a expert, output [P][ff]); mode 1: down (output float32 [P][N], pair order).
extern "C" int tb_moe_grouped(const void* X, int ldx, const void* W, void* out, int ldo, int dtype, int mode, const int* perm,
                              const int* tile_e, const int* tile_row0, const int* tile_rows, const int* n_tiles, int max_tiles,
                              int N, int K, int top, int n_real, int act, float limit, cudaStream_t stream) {
    TB_REQUIRE(N > 0 && K > 0 && top > 0 && max_tiles > 0 && max_tiles <= 65535, "moe_grouped: sizes (N=%d K=%d tiles=%d)", N, K, max_tiles);
    TB_REQUIRE(act >= 0 && act < TB_ACT_KINDS && n_real > 0, "moe_grouped: unknown gate %d or no expert", act);
    TB_REQUIRE(mode == 1 || N % 2 == 0, "moe_grouped: gate and up rows come in pairs");
    dim3 grid((N + MOE_BN - 1) / MOE_BN, max_tiles);
#define MOE_G(TT, MM) tb_launch(moe_grouped_kernel<TT, MM>, grid, 256, 0, stream, (const TT*)X, ldx, (const TT*)W, out, ldo, perm, tile_e, tile_row0, tile_rows, n_tiles, N, K, top, n_real, act, limit)
    if (dtype == TB_F32) { if (mode == 0) MOE_G(float, 0); else MOE_G(float, 1); }
    else if (dtype == TB_BF16) { if (mode == 0) MOE_G(__nv_bfloat16, 0); else MOE_G(__nv_bfloat16, 1); }
    else TB_REQUIRE(false, "moe_grouped: unknown dtype %d", dtype);
#undef MOE_G
    TB_CHECK_LAUNCH("moe_grouped");
    return 0;
}

// mode 0: N_out = ff (W holds 2 * ff interleaved rows an expert); mode 1: N_out = rows of the down matrix.
extern "C" int tb_moe_rows(const void* X, int ldx, const void* W, void* out, int ldo, int dtype, int mode, const int* ids,
                           int P, int N_out, int K, int top, int n_real, int act, float limit, cudaStream_t stream) {
    TB_REQUIRE(P > 0 && N_out > 0 && K > 0 && top > 0 && (N_out + 7) / 8 <= 65535, "moe_rows: sizes (P=%d N=%d K=%d)", P, N_out, K);
    TB_REQUIRE(act >= 0 && act < TB_ACT_KINDS && n_real > 0, "moe_rows: unknown gate %d or no expert", act);
    dim3 grid(P, (N_out + 7) / 8);
#define MOE_R(TT, MM) tb_launch(moe_rows_kernel<TT, MM>, grid, 256, 0, stream, (const TT*)X, ldx, (const TT*)W, out, ldo, ids, N_out, K, top, n_real, act, limit)
    if (dtype == TB_F32) { if (mode == 0) MOE_R(float, 0); else MOE_R(float, 1); }
    else if (dtype == TB_BF16) { if (mode == 0) MOE_R(__nv_bfloat16, 0); else MOE_R(__nv_bfloat16, 1); }
    else TB_REQUIRE(false, "moe_rows: unknown dtype %d", dtype);
#undef MOE_R
    TB_CHECK_LAUNCH("moe_rows");
    return 0;
}

extern "C" int tb_moe_gather(const void* x, int ldx, const int* perm, int top, void* out, int dtype, int P, int K, cudaStream_t stream) {
    TB_REQUIRE(P > 0 && K > 0 && top > 0 && x && perm && out, "moe_gather: sizes must be positive");
    if (dtype == TB_F32) tb_launch(moe_gather_kernel<float>, P, 128, 0, stream, (const float*)x, ldx, perm, top, (float*)out, K);
    else if (dtype == TB_BF16) tb_launch(moe_gather_kernel<__nv_bfloat16>, P, 128, 0, stream, (const __nv_bfloat16*)x, ldx, perm, top, (__nv_bfloat16*)out, K);
    else TB_REQUIRE(false, "moe_gather: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("moe_gather");
    return 0;
}

// ``where`` (may be null): row of y that holds pair p, if y is not in pair order.
// ids, n_real, x (rows of ``x_dtype``, stride ldx): pairs of experts from n_real on add the token's input row instead of a
// row of y (all null / zero: every pair has a row).
extern "C" int tb_moe_combine(const float* y, const float* wts, const float* shared_y, const float* gate, float* out, int T_,
                              int H, int top, const int* where, const int* ids, int n_real, const void* x, int ldx, int x_dtype,
                              cudaStream_t stream) {
    TB_REQUIRE(T_ > 0 && H > 0 && top > 0 && y && wts && out, "moe_combine: sizes must be positive");
    TB_REQUIRE(!ids || (x && ldx >= H && n_real > 0), "moe_combine: experts without matrices need the tokens' input rows");
    const int threads = H >= 1024 ? 256 : 128;
    const dim3 grid(T_, T_ >= 256 ? 1 : (H + threads - 1) / threads);
    if (ids && x_dtype == TB_BF16)
        tb_launch(moe_combine_kernel<__nv_bfloat16>, grid, threads, 0, stream, y, wts, shared_y, gate, out, H, top, where, ids, n_real, (const __nv_bfloat16*)x, ldx);
    else
        tb_launch(moe_combine_kernel<float>, grid, threads, 0, stream, y, wts, shared_y, gate, out, H, top, where, ids, n_real, (const float*)x, ldx);
    TB_CHECK_LAUNCH("moe_combine");
    return 0;
}
