// Linear attention with a per-head decay ("lightning" mixer): the recurrence and the gated norm after it.
//
//   S_t = decay_h S_{t-1} + k_t v_t^T        S: [dk][dv] float32 per (sequence, head), kept in the cache's state group
//   o_t = S_t^T q_t
// with q = silu(.), k = silu(.), v = silu(.) of the projection's columns (the projection may be in the compute
// dtype; the activation, the state and the sums are float32).  A sequence's tokens are taken in order, so a prompt
// run whole, in pieces or token by token leaves the same state up to the order of float32 sums (which is the same
// here: one token after the other in every case).
//
// tb_lightning_scan   grid (sequences, heads, ceil(dv / 32)): a block owns 32 value columns of one head's state;
//                     four neighbouring lanes share a column (each keeps a quarter of its rows in registers) and
//                     add their parts of o with two shuffles.  Tokens are staged in shared memory sixteen at a time,
//                     the next sixteen requested while these are worked through.
// tb_gated_rmsnorm    y = o / sqrt(mean(o^2) + eps) * w * sigmoid(g) over the concatenated heads, one block a token.
// tb_rotary_rows      rotates heads that lie side by side in float32 rows, in place, and scales some of them: what the
//                     retention mixer does to q and k between its projection and this recurrence (LightningArgs.plain).
#include "common.cuh"
#include "qk_args.h"

struct LightningArgs {
    const void* proj; int stride;           // [T][stride]: q (H*dk) | k (H*dk) | v (H*dv) | g (H*dv), compute dtype
    float* out; int out_stride;             // [T][out_stride] float32: head h at h * dv
    float* state;                           // [slots][H][dk][dv] float32
    const float* decay;                     // [H]
    const int* q_start; const int* slot_of_seq;
    int B; int H; int dk; int dv;
    int max_new;                            // most tokens a sequence brings in this step (1: a step of single tokens)
    int plain;                              // 1: q, k and v enter the recurrence as they stand in the rows (no silu): the retention mixer, whose rows are float32
};

namespace {

__device__ __forceinline__ float silu_f(float z) { return z / (1.0f + expf(-z)); }

// CH tokens of a sequence are staged in shared memory at a time (q and k of the head with the activation applied, and the
// block's 32 value columns), requested into registers while the chunk before is worked through, so that the latency of
// the loads is paid once a chunk and not once a token.  Within a chunk the tokens are taken one after the other from
// shared memory: a thread keeps rows [s * R, (s + 1) * R) of its column of the state in registers (s = lane & 3), reads
// the matching q and k as 16-byte loads (rows of the four s are 16 bytes apart in the banks), and the four partial sums
// of o meet by two shuffles.
template <typename T, int R, int CH>
__global__ void __launch_bounds__(128) lightning_scan_kernel(LightningArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int DKP = 4 * (R + 4);                    // a q or k row in shared memory: four runs of R, each padded by 4
    constexpr int ROW = 2 * DKP + 32;                   // q | k | 32 values
    constexpr int PER = (CH * ROW + 127) / 128;         // staged elements a thread
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, s = tid & 3, col = tid >> 2, j = blockIdx.z * 32 + col;
    const int dk = a.dk, dv = a.dv;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const bool live = j < dv;
    float* S_g = a.state + (((size_t)a.slot_of_seq[b] * a.H + h) * dk) * dv + j;
    float S[R];
#pragma unroll
    for (int ii = 0; ii < R; ++ii) {
        const int i = s * R + ii;
        S[ii] = (live && i < dk) ? S_g[(size_t)i * dv] : 0.f;
    }
    const float decay = a.decay[h];
    const T* base = (const T*)a.proj;
    const int kq = h * dk, kk = a.H * dk + h * dk, kvv = 2 * a.H * dk + h * dv + blockIdx.z * 32;
    float stage[PER];
    // Element e of a chunk's staging area: token e / ROW, and within the row q (padded), k (padded) or a value.  Gives
    // the address to read (always a valid one: indices are clamped, so that the load needs no condition and nothing
    // waits for it before the chunk is due) and whether the element is real or padding.
    auto source = [&](int u, int first, bool* real) -> const T* {
        const int e = tid + 128 * u, ec = min(e, CH * ROW - 1), tok = ec / ROW, x = ec % ROW;
        bool ok = e < CH * ROW && first + tok < t1;
        const T* row = base + (size_t)min(first + tok, t1 - 1) * a.stride;
        if (x < 2 * DKP) {
            const int y = x < DKP ? x : x - DKP, run = y / (R + 4), within = y % (R + 4), i = run * R + within;
            ok = ok && within < R && i < dk;
            *real = ok;
            return row + (x < DKP ? kq : kk) + (ok ? i : 0);
        }
        const int c = x - 2 * DKP;
        ok = ok && blockIdx.z * 32 + c < dv;
        *real = ok;
        return row + kvv + (ok ? c : 0);
    };
    auto request = [&](int first) {
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            bool real;
            stage[u] = ldf(source(u, first, &real));
        }
    };
    if (t0 < t1) request(t0);
    for (int c0 = t0; c0 < t1; c0 += CH) {
        __syncthreads();                                // the chunk before has been read from shared memory
#pragma unroll
        for (int u = 0; u < PER; ++u) {
            const int e = tid + 128 * u;
            bool real;
            source(u, c0, &real);
            if (e < CH * ROW) sm[e] = real ? (a.plain ? stage[u] : silu_f(stage[u])) : 0.f;
        }
        __syncthreads();
        if (c0 + CH < t1) request(c0 + CH);
        const int n = min(CH, t1 - c0);
        for (int tt = 0; tt < n; ++tt) {
            const float* qs = sm + tt * ROW + s * (R + 4);
            const float* ks = qs + DKP;
            const float vj = sm[tt * ROW + 2 * DKP + col];
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < R; ii += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + ii), q4 = *reinterpret_cast<const float4*>(qs + ii);
                S[ii] = fmaf(decay, S[ii], k4.x * vj);         acc = fmaf(S[ii], q4.x, acc);
                S[ii + 1] = fmaf(decay, S[ii + 1], k4.y * vj); acc = fmaf(S[ii + 1], q4.y, acc);
                S[ii + 2] = fmaf(decay, S[ii + 2], k4.z * vj); acc = fmaf(S[ii + 2], q4.z, acc);
                S[ii + 3] = fmaf(decay, S[ii + 3], k4.w * vj); acc = fmaf(S[ii + 3], q4.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            if (s == 0 && live) a.out[(size_t)(c0 + tt) * a.out_stride + h * dv + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s * R + ii;
            if (i < dk) S_g[(size_t)i * dv] = S[ii];
        }
    }
}

// Eight consecutive elements of a row, as they come from one (bfloat16) or two (float32) 16-byte loads.
template <typename T> struct Pack8;
template <> struct Pack8<__nv_bfloat16> {
    uint4 a;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { a = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void get(float* o) const {
        const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) { o[2 * i] = __uint_as_float(w[i] << 16); o[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
    }
};
template <> struct Pack8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4); }
    __device__ __forceinline__ void get(float* o) const { o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w; }
};

// The same recurrence for sizes in multiples of 8 (dk, dv, the projection's row stride): a block owns 16 value columns,
// eight neighbouring lanes share a column (R rows of it each, dk <= 8 R), and a chunk of tokens is staged by 16-byte
// loads of eight elements, a few a thread.  Twice the blocks of the kernel above, half the arithmetic a thread and
// token, and an eighth of the load instructions.
template <typename T, int R, int CH>
__global__ void __launch_bounds__(128) lightning_scan_vec_kernel(LightningArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int DKP = 8 * (R + 4);                    // a q or k row in shared memory: eight runs of R, each padded by 4
    constexpr int ROW = 2 * DKP + 16;                   // q | k | 16 values
    const int b = blockIdx.x, h = blockIdx.y;
    const int tid = threadIdx.x, s = tid & 7, col = tid >> 3, j = blockIdx.z * 16 + col;
    const int dk = a.dk, dv = a.dv;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const bool live = j < dv;
    float* S_g = a.state + (((size_t)a.slot_of_seq[b] * a.H + h) * dk) * dv + j;
    float S[R];
#pragma unroll
    for (int ii = 0; ii < R; ++ii) {
        const int i = s * R + ii;
        S[ii] = (live && i < dk) ? S_g[(size_t)i * dv] : 0.f;
    }
    const float decay = a.decay[h];
    const T* base = (const T*)a.proj;
    const int kq = h * dk, kk = a.H * dk + h * dk, kvv = 2 * a.H * dk + h * dv + blockIdx.z * 16;
    const int qk_units = dk >> 3, units = 2 * qk_units + 2, total = CH * units;       // units of eight elements a token, a chunk
    constexpr int PERU = (CH * (2 * R + 2) + 127) / 128;                              // at most 8 R / 8 = R units of q and of k a token
    Pack8<T> stage[PERU];
    // unit n of a chunk: token n / units; then q (qk_units of them), k, and two units of values.  Gives a valid address
    // (clamped, so the load carries no condition), where the eight floats go in shared memory, and whether they are real.
    auto source = [&](int u, int first, bool* real, int* to) -> const T* {
        const int n = tid + 128 * u, nc = min(n, total - 1), tok = nc / units, x = nc % units;
        bool ok = n < total && first + tok < t1;
        const T* row = base + (size_t)min(first + tok, t1 - 1) * a.stride;
        if (x < 2 * qk_units) {
            const int g = x < qk_units ? x : x - qk_units, i = g * 8;
            *to = tok * ROW + (x < qk_units ? 0 : DKP) + (i / R) * (R + 4) + (i % R);
            *real = ok;
            return row + (x < qk_units ? kq : kk) + i;
        }
        const int c = (x - 2 * qk_units) * 8;
        ok = ok && blockIdx.z * 16 + c < dv;
        *to = tok * ROW + 2 * DKP + c;
        *real = ok;
        return row + kvv + (ok ? c : 0);
    };
    auto request = [&](int first) {
#pragma unroll
        for (int u = 0; u < PERU; ++u) {
            bool real; int to;
            stage[u].load(source(u, first, &real, &to));
        }
    };
    // rows of the padded q and k areas beyond dk are never written by a unit: zero them once (they are read as factors)
    for (int e = tid; e < CH * ROW; e += 128) sm[e] = 0.f;
    if (t0 < t1) request(t0);
    for (int c0 = t0; c0 < t1; c0 += CH) {
        __syncthreads();                                // the chunk before has been read from shared memory (or the zeros are in place)
#pragma unroll
        for (int u = 0; u < PERU; ++u) {
            bool real; int to;
            source(u, c0, &real, &to);
            if (tid + 128 * u < total) {
                float v[8];
                stage[u].get(v);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = real ? (a.plain ? v[i] : silu_f(v[i])) : 0.f;
                *reinterpret_cast<float4*>(sm + to) = make_float4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<float4*>(sm + to + 4) = make_float4(v[4], v[5], v[6], v[7]);
            }
        }
        __syncthreads();
        if (c0 + CH < t1) request(c0 + CH);
        const int n = min(CH, t1 - c0);
        for (int tt = 0; tt < n; ++tt) {
            const float* qs = sm + tt * ROW + s * (R + 4);
            const float* ks = qs + DKP;
            const float vj = sm[tt * ROW + 2 * DKP + col];
            float acc = 0.f;
#pragma unroll
            for (int ii = 0; ii < R; ii += 4) {
                const float4 k4 = *reinterpret_cast<const float4*>(ks + ii), q4 = *reinterpret_cast<const float4*>(qs + ii);
                S[ii] = fmaf(decay, S[ii], k4.x * vj);         acc = fmaf(S[ii], q4.x, acc);
                S[ii + 1] = fmaf(decay, S[ii + 1], k4.y * vj); acc = fmaf(S[ii + 1], q4.y, acc);
                S[ii + 2] = fmaf(decay, S[ii + 2], k4.z * vj); acc = fmaf(S[ii + 2], q4.z, acc);
                S[ii + 3] = fmaf(decay, S[ii + 3], k4.w * vj); acc = fmaf(S[ii + 3], q4.w, acc);
            }
            acc += __shfl_xor_sync(0xffffffffu, acc, 1);
            acc += __shfl_xor_sync(0xffffffffu, acc, 2);
            acc += __shfl_xor_sync(0xffffffffu, acc, 4);
            if (s == 0 && live) a.out[(size_t)(c0 + tt) * a.out_stride + h * dv + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s * R + ii;
            if (i < dk) S_g[(size_t)i * dv] = S[ii];
        }
    }
}

template <typename T>
__global__ void gated_rmsnorm_kernel(const float* __restrict__ o, int ldo, const float* __restrict__ w, const T* __restrict__ gate,
                                     int ldg, T* __restrict__ y, int ldy, int N, float eps) {
    pdl_launch_dependents();
    pdl_wait();
    __shared__ float red[33];
    const size_t t = blockIdx.x;
    const float* row = o + t * ldo;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss += row[i] * row[i];
    ss = block_sum(ss, red);
    const float scale = 1.0f / sqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        const float g = ldf(gate + t * ldg + i);
        stf(y + t * ldy + i, row[i] * scale * w[i] * (1.0f / (1.0f + expf(-g))));
    }
}

// One block a token; a thread takes pairs of one head's rotated dimensions (both members, so the rotation is in place),
// then the elements that pass unrotated.  Heads from ``scale_from`` on are multiplied by ``scale`` after the rotation.
__global__ void __launch_bounds__(128) rotary_rows_kernel(float* x, int stride, const int* __restrict__ pos_of, int heads, int hd,
                                                          TbRotary rope, int scale_from, float scale) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float cs[];           // [half] cosines, [half] sines
    const int t = blockIdx.x, half = rope.rot >> 1;
    float* sn = cs + half;
    const float p = (float)pos_of[t] + rope.offset;
    for (int k = threadIdx.x; k < half; k += blockDim.x) {
        float sv, cv;
        sincosf(p * rope.inv_freq[k], &sv, &cv);
        sn[k] = sv * rope.magnitude; cs[k] = cv * rope.magnitude;
    }
    __syncthreads();
    float* row = x + (size_t)t * stride;
    const int per = half + (hd - rope.rot);          // work items a head: pairs, then single elements
    for (int i = threadIdx.x; i < heads * per; i += blockDim.x) {
        const int h = i / per, w = i % per;
        float* head = row + (size_t)h * hd;
        const float f = h >= scale_from ? scale : 1.f;
        if (w < half) {
            const int ia = rope.adjacent ? 2 * w : w, ib = rope.adjacent ? 2 * w + 1 : w + half;
            const float u = head[ia], v = head[ib];
            head[ia] = (u * cs[w] - v * sn[w]) * f;
            head[ib] = (v * cs[w] + u * sn[w]) * f;
        } else {
            head[rope.rot + (w - half)] *= f;
        }
    }
}

template <typename T, int R, int CH>
int launch_one(const LightningArgs& a, dim3 grid, cudaStream_t stream) {
    constexpr size_t smem = (size_t)CH * (2 * 4 * (R + 4) + 32) * sizeof(float);
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(lightning_scan_kernel<T, R, CH>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        TB_REQUIRE(e == cudaSuccess, "lightning_scan: cannot reserve %zu bytes of shared memory: %s", smem, cudaGetErrorString(e));
        configured = true;
    }
    tb_launch(lightning_scan_kernel<T, R, CH>, grid, 128, smem, stream, a);
    return 0;
}

// Rows of the state a thread keeps (a quarter of dk, rounded up to 8, 16, 32 or 64) and tokens staged at a time: sixteen for
// prompts, one for steps of single tokens (nothing to amortise, and less to request).
template <typename T, int R, int CH>
int launch_vec(const LightningArgs& a, cudaStream_t stream) {
    constexpr size_t smem = (size_t)CH * (2 * 8 * (R + 4) + 16) * sizeof(float);
    static_assert(smem <= 48 * 1024, "the staging area fits the default shared memory");
    dim3 grid(a.B, a.H, (a.dv + 15) / 16);
    tb_launch(lightning_scan_vec_kernel<T, R, CH>, grid, 128, smem, stream, a);
    return 0;
}

template <typename T>
int launch_scan(const LightningArgs& a, bool single, cudaStream_t stream) {
    // sizes in multiples of 8 and rows that 16-byte loads can take: the kernel of eight lanes a column
    if (a.dk % 8 == 0 && a.dv % 8 == 0 && a.stride % 8 == 0 && ((uintptr_t)a.proj % 16 == 0) && a.dk >= 64 && (a.dv + 15) / 16 <= 65535) {
        const int rows = a.dk / 8;
        if (single) {
            if (rows <= 8) return launch_vec<T, 8, 1>(a, stream);
            if (rows <= 16) return launch_vec<T, 16, 1>(a, stream);
            return launch_vec<T, 32, 1>(a, stream);
        }
        if (rows <= 8) return launch_vec<T, 8, 16>(a, stream);
        if (rows <= 16) return launch_vec<T, 16, 16>(a, stream);
        return launch_vec<T, 32, 8>(a, stream);
    }
    dim3 grid(a.B, a.H, (a.dv + 31) / 32);
    const int rows = (a.dk + 3) / 4;
    if (single) {
        if (rows <= 8) return launch_one<T, 8, 1>(a, grid, stream);
        if (rows <= 16) return launch_one<T, 16, 1>(a, grid, stream);
        if (rows <= 32) return launch_one<T, 32, 1>(a, grid, stream);
        return launch_one<T, 64, 1>(a, grid, stream);
    }
    if (rows <= 8) return launch_one<T, 8, 16>(a, grid, stream);
    if (rows <= 16) return launch_one<T, 16, 16>(a, grid, stream);
    if (rows <= 32) return launch_one<T, 32, 16>(a, grid, stream);
    return launch_one<T, 64, 8>(a, grid, stream);
}

}  // namespace

extern "C" int tb_lightning_scan(const LightningArgs* args, int dtype, cudaStream_t stream) {
    LightningArgs a = *args;
    TB_REQUIRE(a.B > 0 && a.H > 0 && a.dk > 0 && a.dv > 0, "lightning_scan: sizes must be positive");
    TB_REQUIRE(a.dk <= 256, "lightning_scan: %d key dimensions a head (at most 256)", a.dk);
    TB_REQUIRE(a.H <= 65535 && (a.dv + 31) / 32 <= 65535, "lightning_scan: too many heads or value columns");
    TB_REQUIRE(a.proj && a.out && a.state && a.decay && a.q_start && a.slot_of_seq, "lightning_scan: missing buffers");
    TB_REQUIRE(a.stride >= 2 * a.H * a.dk + a.H * a.dv, "lightning_scan: the projection row is too short");
    TB_REQUIRE(dtype == TB_F32 || dtype == TB_BF16, "lightning_scan: unknown dtype %d", dtype);
    const bool single = a.max_new <= 1;
    if (dtype == TB_F32 ? launch_scan<float>(a, single, stream) : launch_scan<__nv_bfloat16>(a, single, stream)) return 1;
    TB_CHECK_LAUNCH("lightning_scan");
    return 0;
}

extern "C" int tb_gated_rmsnorm(const float* o, int ldo, const float* w, const void* gate, int ldg, void* y, int ldy,
                                int dtype, int n_rows, int N, float eps, cudaStream_t stream) {
    TB_REQUIRE(n_rows > 0 && N > 0 && o && w && gate && y, "gated_rmsnorm: sizes must be positive (rows=%d N=%d)", n_rows, N);
    const int threads = N >= 2048 ? 256 : (N >= 512 ? 128 : 64);
    if (dtype == TB_F32) tb_launch(gated_rmsnorm_kernel<float>, n_rows, threads, 0, stream, o, ldo, w, (const float*)gate, ldg, (float*)y, ldy, N, eps);
    else if (dtype == TB_BF16) tb_launch(gated_rmsnorm_kernel<__nv_bfloat16>, n_rows, threads, 0, stream, o, ldo, w, (const __nv_bfloat16*)gate, ldg, (__nv_bfloat16*)y, ldy, N, eps);
    else TB_REQUIRE(false, "gated_rmsnorm: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("gated_rmsnorm");
    return 0;
}

extern "C" int tb_rotary_rows(float* x, int stride, const int* pos_of, int n_rows, int heads, int hd, const TbRotary* rope, int scale_from,
                              float scale, cudaStream_t stream) {
    TB_REQUIRE(x && pos_of && rope && n_rows > 0 && heads > 0 && hd > 0 && stride >= heads * hd, "rotary_rows: rows of heads are wanted");
    TB_REQUIRE(rope->inv_freq && rope->rot > 0 && rope->rot % 2 == 0 && rope->rot <= hd, "rotary_rows: %d rotated dimensions of a head of %d", rope->rot, hd);
    tb_launch(rotary_rows_kernel, n_rows, 128, (size_t)rope->rot * sizeof(float), stream, x, stride, pos_of, heads, hd, *rope, scale_from, scale);
    TB_CHECK_LAUNCH("rotary_rows");
    return 0;
}
