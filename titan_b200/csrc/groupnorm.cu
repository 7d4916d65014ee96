// RMS norm in groups, alone and behind the residual sum of a block whose sublayers share one norm.
//
// A row of H elements is cut into ``groups`` equal runs; every run is divided by its own sqrt(mean(run^2) + eps) and the
// whole row is multiplied by one weight of H elements.  groups = 1 is the plain RMS norm.  float32 inside.
//
//   tb_group_rmsnorm        y = norm(x[rows[r]] or x[r]) in the compute dtype (the row gather serves the final norm, which
//                           runs on the wanted rows only)
//   tb_residual_group_norm  x += mult * y;  y <- 0 (the buffer the next block's sublayers add into);  and, if asked,
//                           h = norm(new x) with the weight of the norm that reads x next.  One pass over the row for the
//                           sum and the statistics, a second one (from registers or L1) for h.
//
// One block a row, one warp a group at a time: a group's sum is a warp's sum in a fixed order, so the same row gives
// the same bits in any batch.
#include "common.cuh"

namespace {

template <typename T>
__device__ __forceinline__ void norm_groups(const float* __restrict__ xr, const float* __restrict__ w, T* __restrict__ yr, int H,
                                            int groups, float eps) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int per = H / groups;
    for (int g = warp; g < groups; g += warps) {
        const float* run = xr + (size_t)g * per;
        float ss = 0.f;
        for (int i = lane; i < per; i += 32) ss = fmaf(run[i], run[i], ss);
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)per + eps);
        for (int i = lane; i < per; i += 32) stf(yr + (size_t)g * per + i, run[i] * scale * w[(size_t)g * per + i]);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) group_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                                                            const int* __restrict__ rows, int H, int groups, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    norm_groups<T>(x + (size_t)(rows ? rows[r] : r) * H, w, y + (size_t)r * H, H, groups, eps);
}

template <typename T>
__global__ void __launch_bounds__(256) residual_group_norm_kernel(float* __restrict__ y, float mult, float* __restrict__ x,
                                                                  const float* __restrict__ w, T* __restrict__ h, int H, int groups,
                                                                  float eps) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const size_t r = blockIdx.x;
    float* xr = x + r * H;
    float* yr = y + r * H;
    const int per = H / groups;
    for (int g = warp; g < groups; g += warps) {
        float* run = xr + (size_t)g * per;
        float ss = 0.f;
        for (int i = lane; i < per; i += 32) {
            const float v = fmaf(mult, yr[(size_t)g * per + i], run[i]);
            run[i] = v;
            yr[(size_t)g * per + i] = 0.f;
            ss = fmaf(v, v, ss);
        }
        if (!h) continue;
        ss = warp_sum(ss);
        const float scale = 1.0f / sqrtf(ss / (float)per + eps);
        __syncwarp();
        for (int i = lane; i < per; i += 32) stf(h + r * H + (size_t)g * per + i, run[i] * scale * w[(size_t)g * per + i]);
    }
}

int threads_for(int groups) { return 32 * (groups >= 8 ? 8 : groups); }

}  // namespace

extern "C" int tb_group_rmsnorm(const float* x, const float* w, void* y, int dtype, const int* rows, int n_rows, int H, int groups,
                                float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && H > 0 && x && w && y, "group_rmsnorm: sizes must be positive (rows=%d H=%d)", n_rows, H);
    TB_REQUIRE(groups > 0 && H % groups == 0, "group_rmsnorm: %d groups do not divide a row of %d", groups, H);
    if (dtype == TB_F32) tb_launch(group_rmsnorm_kernel<float>, n_rows, threads_for(groups), 0, stream, x, w, (float*)y, rows, H, groups, eps);
    else if (dtype == TB_BF16) tb_launch(group_rmsnorm_kernel<__nv_bfloat16>, n_rows, threads_for(groups), 0, stream, x, w, (__nv_bfloat16*)y, rows, H, groups, eps);
    else TB_REQUIRE(false, "group_rmsnorm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("group_rmsnorm");
    return 0;
}

extern "C" int tb_residual_group_norm(float* y, float mult, float* x, const float* w, void* h, int dtype, int n_rows, int H, int groups,
                                      float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && H > 0 && x && y, "residual_group_norm: sizes must be positive (rows=%d H=%d)", n_rows, H);
    TB_REQUIRE(groups > 0 && H % groups == 0, "residual_group_norm: %d groups do not divide a row of %d", groups, H);
    TB_REQUIRE(!h || w, "residual_group_norm: normed rows are wanted without the norm's weight");
    if (dtype == TB_F32) tb_launch(residual_group_norm_kernel<float>, n_rows, threads_for(groups), 0, stream, y, mult, x, w, (float*)h, H, groups, eps);
    else if (dtype == TB_BF16) tb_launch(residual_group_norm_kernel<__nv_bfloat16>, n_rows, threads_for(groups), 0, stream, y, mult, x, w, (__nv_bfloat16*)h, H, groups, eps);
    else TB_REQUIRE(false, "residual_group_norm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("residual_group_norm");
    return 0;
}
