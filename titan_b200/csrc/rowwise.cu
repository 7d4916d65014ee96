// Activations that need a whole row, and gates between a mixer's heads and its output projection.
//
//   tb_polynorm    y = a N(z) + b N(z^2) + c N(z^3) + e over a row z of F elements, where powers are taken element by
//                  element and N divides its row by the row's root mean square, 1 / sqrt(mean(.^2) + eps): the
//                  activation of a feed-forward without a gate.  The three sums of squares and the result are float32;
//                  z is read in the compute dtype and y written in it.  One block a row.
//   tb_gate_rows   y = x * act(g) * scale, element by element over rows (act: sigmoid or silu in float32): the output gate
//                  of an attention mixer, with the factor of a mixer that runs beside another.  In place if y == x.
//   tb_head_norm_gate   per head of dv elements: y = o / sqrt(mean(o^2) + eps) * w * act(g) * scale, o float32, the weight
//                  one row of dv for all heads or a row per head.  One warp a (token, head).
#include "common.cuh"

namespace {

__device__ __forceinline__ float act_gate(float g, int act) {
    const float sg = 1.0f / (1.0f + expf(-g));
    return act == 1 ? g * sg : sg;
}

template <typename T>
__global__ void __launch_bounds__(256) polynorm_kernel(const T* z, int ldz, const float* __restrict__ coef, float eps,
                                                       T* y, int ldy, int F) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t t = blockIdx.x;
    const T* row = z + t * ldz;
    float s1 = 0.f, s2 = 0.f, s3 = 0.f;
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = ldf(row + i), v2 = v * v, v3 = v2 * v;
        s1 = fmaf(v, v, s1); s2 = fmaf(v2, v2, s2); s3 = fmaf(v3, v3, s3);
    }
    s1 = block_sum(s1, red); s2 = block_sum(s2, red); s3 = block_sum(s3, red);
    const float n = (float)F;
    const float r1 = coef[0] / sqrtf(s1 / n + eps), r2 = coef[1] / sqrtf(s2 / n + eps), r3 = coef[2] / sqrtf(s3 / n + eps), e = coef[3];
    for (int i = threadIdx.x; i < F; i += blockDim.x) {
        const float v = ldf(row + i), v2 = v * v;
        stf(y + t * ldy + i, fmaf(r1, v, fmaf(r2, v2, fmaf(r3, v2 * v, e))));
    }
}

template <typename T>
__global__ void __launch_bounds__(256) gate_rows_kernel(const T* x, int ldx, const T* __restrict__ g, int ldg,
                                                        T* y, int ldy, int n, int act, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t t = blockIdx.y;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) stf(y + t * ldy + i, ldf(x + t * ldx + i) * act_gate(ldf(g + t * ldg + i), act) * scale);
}

template <typename T, typename G>
__global__ void __launch_bounds__(128) head_norm_gate_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, int w_head,
                                                             const G* __restrict__ g, int ldg, T* __restrict__ y, int ldy,
                                                             int H, int dv, int act, float scale, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, h = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (h >= H) return;
    const size_t t = blockIdx.x;
    const float* row = o + t * ldo + (size_t)h * dv;
    float ss = 0.f;
    for (int i = lane; i < dv; i += 32) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    const float r = scale / sqrtf(ss / (float)dv + eps);
    for (int i = lane; i < dv; i += 32)
        stf(y + t * ldy + (size_t)h * dv + i, row[i] * r * w[(size_t)h * w_head + i] * act_gate(ldf(g + t * ldg + (size_t)h * dv + i), act));
}

}  // namespace

extern "C" int tb_polynorm(const void* z, int ldz, const float* coef, float eps, void* y, int ldy, int dtype, int rows, int F, cudaStream_t stream) {
    TB_REQUIRE(z && y && coef && rows > 0 && F > 0, "polynorm: rows are wanted (rows=%d F=%d)", rows, F);
    if (dtype == TB_F32) tb_launch(polynorm_kernel<float>, dim3(rows), dim3(256), 0, stream, (const float*)z, ldz, coef, eps, (float*)y, ldy, F);
    else if (dtype == TB_BF16) tb_launch(polynorm_kernel<__nv_bfloat16>, dim3(rows), dim3(256), 0, stream, (const __nv_bfloat16*)z, ldz, coef, eps, (__nv_bfloat16*)y, ldy, F);
    else TB_REQUIRE(false, "polynorm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("polynorm");
    return 0;
}

extern "C" int tb_gate_rows(const void* x, int ldx, const void* g, int ldg, void* y, int ldy, int dtype, int rows, int n, int act, float scale,
                            cudaStream_t stream) {
    TB_REQUIRE(x && g && y && rows > 0 && n > 0 && rows <= 65535 * 32, "gate_rows: rows are wanted (rows=%d n=%d)", rows, n);
    TB_REQUIRE(act == 0 || act == 1, "gate_rows: the gate is a sigmoid (0) or silu (1)");
    for (int r0 = 0; r0 < rows; r0 += 65535) {
        const int nr = rows - r0 < 65535 ? rows - r0 : 65535;
        dim3 grid((n + 255) / 256, nr);
        if (dtype == TB_F32)
            tb_launch(gate_rows_kernel<float>, grid, dim3(256), 0, stream, (const float*)x + (size_t)r0 * ldx, ldx, (const float*)g + (size_t)r0 * ldg, ldg,
                      (float*)y + (size_t)r0 * ldy, ldy, n, act, scale);
        else if (dtype == TB_BF16)
            tb_launch(gate_rows_kernel<__nv_bfloat16>, grid, dim3(256), 0, stream, (const __nv_bfloat16*)x + (size_t)r0 * ldx, ldx,
                      (const __nv_bfloat16*)g + (size_t)r0 * ldg, ldg, (__nv_bfloat16*)y + (size_t)r0 * ldy, ldy, n, act, scale);
        else TB_REQUIRE(false, "gate_rows: unknown dtype %d", dtype);
    }
    TB_CHECK_LAUNCH("gate_rows");
    return 0;
}

extern "C" int tb_head_norm_gate_from(const float* o, int ldo, const float* w, int w_head, const void* g, int ldg, int g_dtype, void* y, int ldy,
                                      int dtype, int rows, int H, int dv, int act, float scale, float eps, cudaStream_t stream);

extern "C" int tb_head_norm_gate(const float* o, int ldo, const float* w, int w_head, const void* g, int ldg, void* y, int ldy, int dtype,
                                 int rows, int H, int dv, int act, float scale, float eps, cudaStream_t stream) {
    return tb_head_norm_gate_from(o, ldo, w, w_head, g, ldg, dtype, y, ldy, dtype, rows, H, dv, act, scale, eps, stream);
}

// The same with the gate's rows in a dtype of their own (g_dtype): float32 gate logits that came out of one product with the
// recurrence's inputs, beside an output in bfloat16.
extern "C" int tb_head_norm_gate_from(const float* o, int ldo, const float* w, int w_head, const void* g, int ldg, int g_dtype, void* y, int ldy,
                                      int dtype, int rows, int H, int dv, int act, float scale, float eps, cudaStream_t stream) {
    TB_REQUIRE(o && w && g && y && rows > 0 && H > 0 && dv > 0, "head_norm_gate: rows of heads are wanted");
    TB_REQUIRE(act == 0 || act == 1, "head_norm_gate: the gate is a sigmoid (0) or silu (1)");
    TB_REQUIRE((H + 3) / 4 <= 65535, "head_norm_gate: too many heads");
    dim3 grid(rows, (H + 3) / 4);
    if (dtype == TB_F32 && g_dtype == TB_F32) tb_launch(head_norm_gate_kernel<float, float>, grid, dim3(128), 0, stream, o, ldo, w, w_head, (const float*)g, ldg, (float*)y, ldy, H, dv, act, scale, eps);
    else if (dtype == TB_BF16 && g_dtype == TB_BF16) tb_launch(head_norm_gate_kernel<__nv_bfloat16, __nv_bfloat16>, grid, dim3(128), 0, stream, o, ldo, w, w_head, (const __nv_bfloat16*)g, ldg, (__nv_bfloat16*)y, ldy, H, dv, act, scale, eps);
    else if (dtype == TB_BF16 && g_dtype == TB_F32) tb_launch(head_norm_gate_kernel<__nv_bfloat16, float>, grid, dim3(128), 0, stream, o, ldo, w, w_head, (const float*)g, ldg, (__nv_bfloat16*)y, ldy, H, dv, act, scale, eps);
    else TB_REQUIRE(false, "head_norm_gate: unsupported dtypes (output %d, gate %d)", dtype, g_dtype);
    TB_CHECK_LAUNCH("head_norm_gate");
    return 0;
}
