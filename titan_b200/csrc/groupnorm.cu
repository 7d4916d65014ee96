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
// One block a (row, group), so that the few rows of a decode step still spread over the machine.
#include "common.cuh"

namespace {

// A block takes one run (group) of one row: grid (rows, groups).  The run's sum of squares is a block's sum in a fixed order
// (lanes, then warps), so the same row gives the same bits in any batch.
template <typename T>
__global__ void __launch_bounds__(256) group_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                                                            const int* __restrict__ rows, int H, int per, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const int r = blockIdx.x, g = blockIdx.y;
    const float* run = x + (size_t)(rows ? rows[r] : r) * H + (size_t)g * per;
    const float* wr = w + (size_t)g * per;
    T* yr = y + (size_t)r * H + (size_t)g * per;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) ss = fmaf(run[i], run[i], ss);
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)per + eps);
    for (int i = threadIdx.x; i < per; i += blockDim.x) stf(yr + i, run[i] * scale * wr[i]);
}

template <typename T>
__global__ void __launch_bounds__(256) residual_group_norm_kernel(float* __restrict__ y, float mult, float* __restrict__ x,
                                                                  const float* __restrict__ w, T* __restrict__ h, int H, int per,
                                                                  float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t at = (size_t)blockIdx.x * H + (size_t)blockIdx.y * per;
    float* run = x + at;
    float* yr = y + at;
    float ss = 0.f;
    for (int i = threadIdx.x; i < per; i += blockDim.x) {
        const float v = fmaf(mult, yr[i], run[i]);
        run[i] = v;
        yr[i] = 0.f;
        ss = fmaf(v, v, ss);
    }
    if (!h) return;
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)per + eps);
    const float* wr = w + (size_t)blockIdx.y * per;
    for (int i = threadIdx.x; i < per; i += blockDim.x) stf(h + at + i, run[i] * scale * wr[i]);      // a thread reads back what it wrote itself
}

// Threads of a block for a run of ``per`` elements: a warp for each 128 of them, at most eight.
int threads_for(int per) { const int warps = (per + 127) / 128; return 32 * (warps < 1 ? 1 : (warps > 8 ? 8 : warps)); }

}  // namespace

extern "C" int tb_group_rmsnorm(const float* x, const float* w, void* y, int dtype, const int* rows, int n_rows, int H, int groups,
                                float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && H > 0 && x && w && y, "group_rmsnorm: sizes must be positive (rows=%d H=%d)", n_rows, H);
    TB_REQUIRE(groups > 0 && H % groups == 0, "group_rmsnorm: %d groups do not divide a row of %d", groups, H);
    TB_REQUIRE(groups <= 65535, "group_rmsnorm: %d groups (at most 65535)", groups);
    const int per = H / groups;
    const dim3 grid(n_rows, groups);
    if (dtype == TB_F32) tb_launch(group_rmsnorm_kernel<float>, grid, threads_for(per), 0, stream, x, w, (float*)y, rows, H, per, eps);
    else if (dtype == TB_BF16) tb_launch(group_rmsnorm_kernel<__nv_bfloat16>, grid, threads_for(per), 0, stream, x, w, (__nv_bfloat16*)y, rows, H, per, eps);
    else TB_REQUIRE(false, "group_rmsnorm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("group_rmsnorm");
    return 0;
}

extern "C" int tb_residual_group_norm(float* y, float mult, float* x, const float* w, void* h, int dtype, int n_rows, int H, int groups,
                                      float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && H > 0 && x && y, "residual_group_norm: sizes must be positive (rows=%d H=%d)", n_rows, H);
    TB_REQUIRE(groups > 0 && H % groups == 0, "residual_group_norm: %d groups do not divide a row of %d", groups, H);
    TB_REQUIRE(!h || w, "residual_group_norm: normed rows are wanted without the norm's weight");
    TB_REQUIRE(groups <= 65535, "residual_group_norm: %d groups (at most 65535)", groups);
    const int per = H / groups;
    const dim3 grid(n_rows, groups);
    if (dtype == TB_F32) tb_launch(residual_group_norm_kernel<float>, grid, threads_for(per), 0, stream, y, mult, x, w, (float*)h, H, per, eps);
    else if (dtype == TB_BF16) tb_launch(residual_group_norm_kernel<__nv_bfloat16>, grid, threads_for(per), 0, stream, y, mult, x, w, (__nv_bfloat16*)h, H, per, eps);
    else TB_REQUIRE(false, "residual_group_norm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("residual_group_norm");
    return 0;
}
