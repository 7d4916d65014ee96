// Several residual streams instead of one ("hyper-connections"): the kernel between two sublayers.
//
// A model with S streams keeps rows [S][W] per token.  A sublayer reads one blend of them, u = sum_s in[s] x_s, normed;
// its result y then goes into every stream while the streams are mixed among themselves:
//
//     x'_r = sum_s mix[s][r] x_s + out[r] * y          (all r at once, from the old streams)
//
// tb_hyper does, per token and in this order, whichever of the two halves it is given: the write of the sublayer that
// has just run (y, mix, out; y may be left zeroed for the next sublayer's products to add into) and the read of the
// sublayer that runs next (in, then an RMS norm with a weight into the compute dtype, or, without a norm, the plain
// blend in float32: with in = 1 that is the sum of the streams, which is what leaves the last layer).  Everything is
// float32; one block a token, the blend of the row kept in shared memory between the sum of squares and the scaling.
#include "common.cuh"

#define HYPER_MAX_STREAMS 8

struct HyperArgs {
    float* xs; int S; int W; int rows;      // [rows][S][W]
    float* y;                               // [rows][W] or null: nothing to write
    const float* mix;                       // [S][S], indexed [from][to]
    const float* out_w;                     // [S]
    int zero_y;
    const float* in_w;                      // [S] or null: nothing to read
    const float* norm_w;                    // [W] or null: h receives the blend itself, in float32
    float eps;
    void* h;                                // [rows][W]
};

namespace {

// V: neighbouring elements of a row that a thread takes at a time (4 where the row's width allows 16-byte accesses).
// NS: the number of streams.
template <typename T, int V, int NS>
__global__ void __launch_bounds__(256) hyper_kernel(HyperArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float blend[];        // [W]
    __shared__ float mix[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], out_w[HYPER_MAX_STREAMS], in_w[HYPER_MAX_STREAMS], red[33];
    struct alignas(4 * V) Vec { float v[V]; };
    constexpr int S = NS;
    const int W = a.W;
    if (threadIdx.x < S * S) mix[threadIdx.x] = a.y ? a.mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        out_w[threadIdx.x] = a.y ? a.out_w[threadIdx.x] : 0.f;
        in_w[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const size_t t = blockIdx.x;
    float* x = a.xs + t * S * W;
    float ss = 0.f;
    for (int w = threadIdx.x * V; w < W; w += blockDim.x * V) {
        Vec old[S];
        float u[V];                                       // the next sublayer's blend, gathered as the new rows are made
#pragma unroll
        for (int e = 0; e < V; ++e) u[e] = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) {
            if (s < S) old[s] = *reinterpret_cast<const Vec*>(x + (size_t)s * W + w);
            else
#pragma unroll
                for (int e = 0; e < V; ++e) old[s].v[e] = 0.f;
        }
        if (a.y) {
            const Vec yv = *reinterpret_cast<const Vec*>(a.y + t * W + w);
            if (a.zero_y) {
                Vec z;
#pragma unroll
                for (int e = 0; e < V; ++e) z.v[e] = 0.f;
                *reinterpret_cast<Vec*>(a.y + t * W + w) = z;
            }
#pragma unroll
            for (int r = 0; r < S; ++r) {
                if (r >= S) break;
                Vec now;
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float v = out_w[r] * yv.v[e];
#pragma unroll
                    for (int s = 0; s < S; ++s)
                        if (s < S) v = fmaf(mix[s * S + r], old[s].v[e], v);
                    now.v[e] = v;
                    u[e] = fmaf(in_w[r], v, u[e]);
                }
                *reinterpret_cast<Vec*>(x + (size_t)r * W + w) = now;
            }
        } else {
#pragma unroll
            for (int r = 0; r < S; ++r)
                if (r < S)
#pragma unroll
                    for (int e = 0; e < V; ++e) u[e] = fmaf(in_w[r], old[r].v[e], u[e]);
        }
        if (a.in_w) {
#pragma unroll
            for (int e = 0; e < V; ++e) {
                blend[w + e] = u[e];
                ss = fmaf(u[e], u[e], ss);
            }
        }
    }
    if (!a.in_w) return;
    if (!a.norm_w) {
        float* h = (float*)a.h + t * W;
        for (int w = threadIdx.x * V; w < W; w += blockDim.x * V)           // every thread reads what it wrote itself
#pragma unroll
            for (int e = 0; e < V; ++e) h[w + e] = blend[w + e];
        return;
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)W + a.eps);
    T* h = (T*)a.h + t * W;
    for (int w = threadIdx.x * V; w < W; w += blockDim.x * V)
#pragma unroll
        for (int e = 0; e < V; ++e) stf(h + w + e, blend[w + e] * scale * a.norm_w[w + e]);
}

template <typename T>
void launch_hyper(const HyperArgs& a, size_t smem, cudaStream_t stream) {
    const bool wide = a.W % 4 == 0 && ((uintptr_t)a.xs | (uintptr_t)a.y) % 16 == 0;
    switch (a.S) {
#define HYPER_CASE(N) case N: \
        if (wide) tb_launch(hyper_kernel<T, 4, N>, dim3(a.rows), dim3(256), smem, stream, a); \
        else tb_launch(hyper_kernel<T, 1, N>, dim3(a.rows), dim3(256), smem, stream, a); \
        break;
        HYPER_CASE(1) HYPER_CASE(2) HYPER_CASE(3) HYPER_CASE(4) HYPER_CASE(5) HYPER_CASE(6) HYPER_CASE(7) HYPER_CASE(8)
#undef HYPER_CASE
        default: break;
    }
}

}  // namespace

extern "C" int tb_hyper(const HyperArgs* args, int h_dtype, cudaStream_t stream) {
    HyperArgs a = *args;
    TB_REQUIRE(a.xs && a.rows > 0 && a.W > 0, "hyper: rows of streams are wanted");
    TB_REQUIRE(a.S >= 1 && a.S <= HYPER_MAX_STREAMS, "hyper: %d streams (1 to %d)", a.S, HYPER_MAX_STREAMS);
    TB_REQUIRE(!a.y || (a.mix && a.out_w), "hyper: a sublayer's result needs the mixing matrix and the output weights");
    TB_REQUIRE(a.y || a.in_w, "hyper: nothing to do");
    TB_REQUIRE(!a.in_w || a.h, "hyper: the blend needs a place");
    TB_REQUIRE(h_dtype == TB_F32 || h_dtype == TB_BF16, "hyper: unknown dtype %d", h_dtype);
    TB_REQUIRE(a.norm_w || !a.in_w || h_dtype == TB_F32, "hyper: a blend without a norm is float32");
    const size_t smem = (size_t)a.W * sizeof(float);
    TB_REQUIRE(smem <= 48 * 1024, "hyper: rows of %d elements (at most 12,288)", a.W);
    if (h_dtype == TB_F32) launch_hyper<float>(a, smem, stream);
    else launch_hyper<__nv_bfloat16>(a, smem, stream);
    TB_CHECK_LAUNCH("hyper");
    return 0;
}
