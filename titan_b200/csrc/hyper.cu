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

template <typename T>
__global__ void __launch_bounds__(256) hyper_kernel(HyperArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float blend[];        // [W]
    __shared__ float mix[HYPER_MAX_STREAMS * HYPER_MAX_STREAMS], out_w[HYPER_MAX_STREAMS], in_w[HYPER_MAX_STREAMS], red[33];
    const int S = a.S, W = a.W;
    if (threadIdx.x < S * S) mix[threadIdx.x] = a.y ? a.mix[threadIdx.x] : 0.f;
    if (threadIdx.x < S) {
        out_w[threadIdx.x] = a.y ? a.out_w[threadIdx.x] : 0.f;
        in_w[threadIdx.x] = a.in_w ? a.in_w[threadIdx.x] : 0.f;
    }
    __syncthreads();
    const size_t t = blockIdx.x;
    float* x = a.xs + t * S * W;
    float ss = 0.f;
    for (int w = threadIdx.x; w < W; w += blockDim.x) {
        float old[HYPER_MAX_STREAMS], now[HYPER_MAX_STREAMS];
#pragma unroll
        for (int s = 0; s < HYPER_MAX_STREAMS; ++s) old[s] = s < S ? x[(size_t)s * W + w] : 0.f;
        if (a.y) {
            const float yv = a.y[t * W + w];
            if (a.zero_y) a.y[t * W + w] = 0.f;
#pragma unroll
            for (int r = 0; r < HYPER_MAX_STREAMS; ++r) {
                if (r >= S) break;
                float v = out_w[r] * yv;
#pragma unroll
                for (int s = 0; s < HYPER_MAX_STREAMS; ++s)
                    if (s < S) v = fmaf(mix[s * S + r], old[s], v);
                now[r] = v;
                x[(size_t)r * W + w] = v;
            }
        } else {
#pragma unroll
            for (int r = 0; r < HYPER_MAX_STREAMS; ++r) now[r] = old[r];
        }
        if (a.in_w) {
            float u = 0.f;
#pragma unroll
            for (int r = 0; r < HYPER_MAX_STREAMS; ++r)
                if (r < S) u = fmaf(in_w[r], now[r], u);
            blend[w] = u;
            ss = fmaf(u, u, ss);
        }
    }
    if (!a.in_w) return;
    if (!a.norm_w) {
        float* h = (float*)a.h + t * W;
        for (int w = threadIdx.x; w < W; w += blockDim.x) h[w] = blend[w];      // every thread reads what it wrote itself
        return;
    }
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)W + a.eps);
    T* h = (T*)a.h + t * W;
    for (int w = threadIdx.x; w < W; w += blockDim.x) stf(h + w, blend[w] * scale * a.norm_w[w]);
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
    if (h_dtype == TB_F32) tb_launch(hyper_kernel<float>, dim3(a.rows), dim3(256), smem, stream, a);
    else tb_launch(hyper_kernel<__nv_bfloat16>, dim3(a.rows), dim3(256), smem, stream, a);
    TB_CHECK_LAUNCH("hyper");
    return 0;
}
