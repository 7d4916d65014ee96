// Two recurrences over a matrix state S [dk][dv] per (sequence, head), float32, kept in the cache's state group:
//
//   the gated delta rule     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                            (one decay g and one write strength beta per head and token; q and k unit vectors)
//   the mLSTM matrix memory  m' = max(f + m, i);  S <- e^(f + m - m') S + e^(i - m') k v^T;  n likewise with k alone;
//                            o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)
//                            (i and f the logarithms of an input and a forget gate; m a running maximum that starts at 0)
//
// tb_delta_prep   what lies between the delta rule's projections and its recurrence, one block a token: a short causal
//                 convolution over time of every q, k and v channel (the inputs before the step come from the sequence's
//                 state, which starts as zeros) with silu; q and k heads made unit vectors, q times dk^(-1/2); beta =
//                 sigmoid(.) and g = exp(-exp(A_log) softplus(. + dt_bias)) per head.  All float32, results float32.
// tb_recurrent_scan   either recurrence, tokens of a sequence in order whatever the step brings (a prompt, a piece of it,
//                 one token): a block owns 8 value columns of one head's state, sixteen neighbouring lanes share a column
//                 (a sixteenth of its rows in registers each) and add their parts with four shuffles.  Sixteen tokens are
//                 staged in shared memory at a time, and the next sixteen are on their way from memory into registers
//                 while these are computed.  For the delta rule the sequence's blocks, a share of the channels each,
//                 also move the convolution's window on: the last taps - 1 inputs of the sequence become its state.
#include "common.cuh"

struct DeltaPrepArgs {
    const void* proj; int stride;           // [T][stride], compute dtype: q (G*dk) | k (G*dk) | v (H*dv) | ...
    const float* taps; int n_taps;          // [C][n_taps], C = 2 G dk + H dv; the last column is the current token's
    const float* state; long long state_stride; int conv_off;   // per slot: ... | at conv_off: [n_taps - 1][C] inputs, oldest first
    const float* ba; int ba_stride;         // [T][>= 2H] float32: the projections for beta (H), then for the decay (H)
    const float* a_log; const float* dt_bias;   // [H]
    float* qkv; int qkv_stride;             // [T][C] float32 out: q | k | v as the recurrence takes them
    float* gates; int gates_stride;         // [T][2H] float32 out: decay g (H), then beta (H)
    const int* seq_of; const int* q_start; const int* slot_of_seq;
    int T; int H; int G; int dk; int dv;
};

struct ScanArgs {
    const void* q; int q_stride;            // rows of q heads side by side (dk each); a value head h reads q head h / group
    const void* k; int k_stride;
    const void* v; int v_stride;            // rows of H value heads (dv each)
    int group;                              // value heads that share a q / k head
    const float* gates; int gates_stride;   // [T][2H] float32.  delta: g, then beta.  mLSTM: the input gate's, then the forget gate's projection
    const float* i_bias; const float* f_bias; float cap;      // mLSTM: [H] each; gates are capped as cap * tanh(. / cap)
    float q_scale;                          // q is multiplied by this on the way in
    float* out; int out_stride;             // [T][H * dv] float32
    float* state; long long state_stride;   // per slot: S [H][dk][dv]; mLSTM: then n [H][dk], then m [H]
    const int* q_start; const int* slot_of_seq;
    int B; int H; int dk; int dv;
    // delta rule: the convolution's window (see DeltaPrepArgs), moved on by this kernel
    const void* conv_in; int conv_stride; int conv_bf16; int conv_channels; int n_taps; int conv_off;
};

namespace {

__device__ __forceinline__ float as_float(float x) { return x; }
__device__ __forceinline__ float as_float(__nv_bfloat16 x) { return __bfloat162float(x); }
__device__ __forceinline__ float silu_r(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplus_r(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float logsigmoid_r(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

template <typename T>
__global__ void __launch_bounds__(256) delta_prep_kernel(DeltaPrepArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ float act[];          // [C]
    const int t = blockIdx.x, H = a.H, G = a.G, dk = a.dk, dv = a.dv, n = a.n_taps;
    const int C = 2 * G * dk + H * dv;
    const int seq = a.seq_of[t], first = a.q_start[seq], i = t - first;
    const float* old = a.state + (size_t)a.slot_of_seq[seq] * a.state_stride + a.conv_off;
    const T* proj = (const T*)a.proj;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        float acc = 0.f;
        for (int j = 0; j < n; ++j) {
            const int idx = i - (n - 1) + j;          // which token of the step (negative: before it)
            const float x = idx >= 0 ? ldf(proj + (size_t)(first + idx) * a.stride + c) : old[(size_t)(n - 1 + idx) * C + c];
            acc = fmaf(a.taps[(size_t)c * n + j], x, acc);
        }
        act[c] = silu_r(acc);
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    float* out = a.qkv + (size_t)t * a.qkv_stride;
    for (int head = warp; head < 2 * G; head += nwarp) {           // q heads, then k heads: unit vectors
        const float* x = act + head * dk;
        float ss = 0.f;
        for (int e = lane; e < dk; e += 32) ss = fmaf(x[e], x[e], ss);
        ss = warp_sum(ss);
        const float r = (head < G ? 1.0f / sqrtf((float)dk) : 1.0f) / sqrtf(ss + 1e-6f);
        for (int e = lane; e < dk; e += 32) out[head * dk + e] = x[e] * r;
    }
    for (int c = 2 * G * dk + threadIdx.x; c < C; c += blockDim.x) out[c] = act[c];
    if (threadIdx.x < H) {
        const int h = threadIdx.x;
        const float* ba = a.ba + (size_t)t * a.ba_stride;
        float* g = a.gates + (size_t)t * a.gates_stride;
        g[h] = expf(-expf(a.a_log[h]) * softplus_r(ba[H + h] + a.dt_bias[h]));
        g[H + h] = 1.0f / (1.0f + expf(-ba[h]));
    }
}

#define SCAN_DELTA 0
#define SCAN_MLSTM 1
#define SCAN_CH 16
#ifndef SCAN_LANES
#define SCAN_LANES 8
#endif                                   // lanes that share a state column
#ifndef SCAN_UNROLL
#define SCAN_UNROLL 4                                   // tokens of the inner loop laid out together, so that one's loads pass under another's sums
#endif
#define SCAN_COLS (128 / SCAN_LANES)                    // value columns of a block

// R: state rows a lane holds (a column's dk rows, rounded up, over the sixteen lanes).  NI: 128-element runs of a q or k row.
template <typename TIN, int MODE, int R, int NI>
__global__ void __launch_bounds__(128) recurrent_scan_kernel(ScanArgs a) {
    pdl_launch_dependents();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    constexpr int L = SCAN_LANES, COLS = SCAN_COLS, TOKENS_UNROLLED = SCAN_UNROLL;
    constexpr int DKP = L * (R + 4);                    // a q or k row in shared memory: sixteen runs of R, each padded by 4
    constexpr int NV = (SCAN_CH * COLS + 127) / 128;
    float* qs = sm;                                     // [SCAN_CH][DKP]
    float* ks = qs + SCAN_CH * DKP;                     // [SCAN_CH][DKP]
    float* vs = ks + SCAN_CH * DKP;                     // [SCAN_CH][COLS]
    float* g0 = vs + SCAN_CH * COLS;                    // [SCAN_CH]
    float* g1 = g0 + SCAN_CH;                           // [SCAN_CH]
    const int b = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, s = tid & (L - 1), col = tid / L, j = blockIdx.z * COLS + col;
    const int dk = a.dk, dv = a.dv, H = a.H;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const bool live = j < dv;
    float* slot_state = a.state + (size_t)a.slot_of_seq[b] * a.state_stride;
    float* S_g = slot_state + ((size_t)h * dk) * dv + j;
    float* n_g = slot_state + (size_t)H * dk * dv + (size_t)h * dk;
    float* m_g = slot_state + (size_t)H * dk * dv + (size_t)H * dk + h;
    float S[R], nn[MODE == SCAN_MLSTM ? R : 1];
    float m = 0.f;
#pragma unroll
    for (int ii = 0; ii < R; ++ii) {
        const int i = s * R + ii;
        S[ii] = (live && i < dk) ? S_g[(size_t)i * dv] : 0.f;
        if constexpr (MODE == SCAN_MLSTM) nn[ii] = i < dk ? n_g[i] : 0.f;
    }
    if constexpr (MODE == SCAN_MLSTM) m = *m_g;
    const int qh = h / a.group;
    const TIN* qb = (const TIN*)a.q + (size_t)qh * dk;
    const TIN* kb = (const TIN*)a.k + (size_t)qh * dk;
    const TIN* vb = (const TIN*)a.v + (size_t)h * dv + blockIdx.z * COLS;
    for (int e = tid; e < 2 * SCAN_CH * DKP; e += 128) sm[e] = 0.f;      // the padding is read as factors: zeros

    // A chunk's rows wait in registers while the chunk before is computed: element i of token tok's q and k rows
    // (i = tid, tid + 128), a value column and, in the first threads, a token's two gate numbers.
    TIN pq[SCAN_CH * NI], pk[SCAN_CH * NI], pv[NV];
    float pg0 = 0.f, pg1 = 0.f;
    auto fetch = [&](int c0, int n) {
#pragma unroll
        for (int tok = 0; tok < SCAN_CH; ++tok)
#pragma unroll
            for (int r = 0; r < NI; ++r) {
                const int i = tid + 128 * r;
                if (tok < n && i < dk) {
                    pq[tok * NI + r] = qb[(size_t)(c0 + tok) * a.q_stride + i];
                    pk[tok * NI + r] = kb[(size_t)(c0 + tok) * a.k_stride + i];
                }
            }
#pragma unroll
        for (int r = 0; r < NV; ++r) {
            const int e = tid + 128 * r, tok = e / COLS, c = e % COLS;
            if (tok < n && blockIdx.z * COLS + c < dv) pv[r] = vb[(size_t)(c0 + tok) * a.v_stride + c];
        }
        if (tid < n) {
            const float* g = a.gates + (size_t)(c0 + tid) * a.gates_stride;
            pg0 = g[h]; pg1 = g[H + h];
        }
    };
    auto stash = [&](int n) {
#pragma unroll
        for (int tok = 0; tok < SCAN_CH; ++tok)
#pragma unroll
            for (int r = 0; r < NI; ++r) {
                const int i = tid + 128 * r, at = tok * DKP + (i / R) * (R + 4) + (i % R);
                if (tok < n && i < dk) {
                    qs[at] = as_float(pq[tok * NI + r]) * a.q_scale;
                    ks[at] = as_float(pk[tok * NI + r]);
                }
            }
#pragma unroll
        for (int r = 0; r < NV; ++r) {
            const int e = tid + 128 * r, tok = e / COLS, c = e % COLS;
            if (tok < n) vs[e] = blockIdx.z * COLS + c < dv ? as_float(pv[r]) : 0.f;
        }
        if (tid < n) {
            if constexpr (MODE == SCAN_DELTA) {
                g0[tid] = pg0; g1[tid] = pg1;
            } else {                                    // logarithms of the input gate and of the forget gate, capped
                g1[tid] = a.cap * tanhf((pg0 + a.i_bias[h]) / a.cap);
                g0[tid] = logsigmoid_r(a.cap * tanhf((pg1 + a.f_bias[h]) / a.cap));
            }
        }
    };

    if (t0 < t1) fetch(t0, min(SCAN_CH, t1 - t0));
    for (int c0 = t0; c0 < t1; c0 += SCAN_CH) {
        const int n = min(SCAN_CH, t1 - c0);
        __syncthreads();                                // the chunk before has been read
        stash(n);
        __syncthreads();
        if (c0 + SCAN_CH < t1) fetch(c0 + SCAN_CH, min(SCAN_CH, t1 - c0 - SCAN_CH));
#pragma unroll TOKENS_UNROLLED
        for (int tt = 0; tt < n; ++tt) {
            const float4* qr = reinterpret_cast<const float4*>(qs + tt * DKP + s * (R + 4));
            const float4* kr = reinterpret_cast<const float4*>(ks + tt * DKP + s * (R + 4));
            const float vj = vs[tt * COLS + col];
            float acc;
            // sums over a lane's rows run as four chains each, so that one product does not wait for the one before
            if constexpr (MODE == SCAN_DELTA) {
                // Both read-outs of the state come from the state BEFORE this token's write, side by side: with
                // S' = g S + k u^T, the prediction is g (S^T k) and the output S'^T q = g (S^T q) + (k . q) u.  The two
                // sums and k . q cross the lanes together, and only u stands between a token's sums and the next one's.
                const float decay = g0[tt], beta = g1[tt];
                float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f, r0 = 0.f, r1 = 0.f, r2 = 0.f, r3 = 0.f, c0s = 0.f, c1s = 0.f, c2s = 0.f, c3s = 0.f;
                float4 kk[R / 4];
#pragma unroll
                for (int ii = 0; ii < R; ii += 4) {
                    const float4 k4 = kr[ii >> 2], q4 = qr[ii >> 2];
                    kk[ii >> 2] = k4;
                    p0 = fmaf(S[ii], k4.x, p0); p1 = fmaf(S[ii + 1], k4.y, p1);
                    p2 = fmaf(S[ii + 2], k4.z, p2); p3 = fmaf(S[ii + 3], k4.w, p3);
                    r0 = fmaf(S[ii], q4.x, r0); r1 = fmaf(S[ii + 1], q4.y, r1);
                    r2 = fmaf(S[ii + 2], q4.z, r2); r3 = fmaf(S[ii + 3], q4.w, r3);
                    c0s = fmaf(k4.x, q4.x, c0s); c1s = fmaf(k4.y, q4.y, c1s);
                    c2s = fmaf(k4.z, q4.z, c2s); c3s = fmaf(k4.w, q4.w, c3s);
                }
                float pred = (p0 + p1) + (p2 + p3), read = (r0 + r1) + (r2 + r3), kq = (c0s + c1s) + (c2s + c3s);
#pragma unroll
                for (int d = 1; d < L; d <<= 1) {
                    pred += __shfl_xor_sync(0xffffffffu, pred, d);
                    read += __shfl_xor_sync(0xffffffffu, read, d);
                    kq += __shfl_xor_sync(0xffffffffu, kq, d);
                }
                const float u = beta * (vj - decay * pred);
                acc = fmaf(kq, u, decay * read);
#pragma unroll
                for (int ii = 0; ii < R; ii += 4) {
                    const float4 k4 = kk[ii >> 2];
                    S[ii] = fmaf(decay, S[ii], k4.x * u); S[ii + 1] = fmaf(decay, S[ii + 1], k4.y * u);
                    S[ii + 2] = fmaf(decay, S[ii + 2], k4.z * u); S[ii + 3] = fmaf(decay, S[ii + 3], k4.w * u);
                }
            } else {
                const float f = g0[tt], i = g1[tt];
                const float m_new = fmaxf(f + m, i), keep = expf(f + m - m_new), add = expf(i - m_new);
                m = m_new;
                const float av = add * vj;
                float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f, n0 = 0.f, n1 = 0.f, n2 = 0.f, n3 = 0.f;
#pragma unroll
                for (int ii = 0; ii < R; ii += 4) {
                    const float4 k4 = kr[ii >> 2], q4 = qr[ii >> 2];
                    S[ii] = fmaf(keep, S[ii], k4.x * av); S[ii + 1] = fmaf(keep, S[ii + 1], k4.y * av);
                    S[ii + 2] = fmaf(keep, S[ii + 2], k4.z * av); S[ii + 3] = fmaf(keep, S[ii + 3], k4.w * av);
                    nn[ii] = fmaf(keep, nn[ii], add * k4.x); nn[ii + 1] = fmaf(keep, nn[ii + 1], add * k4.y);
                    nn[ii + 2] = fmaf(keep, nn[ii + 2], add * k4.z); nn[ii + 3] = fmaf(keep, nn[ii + 3], add * k4.w);
                    p0 = fmaf(S[ii], q4.x, p0); p1 = fmaf(S[ii + 1], q4.y, p1);
                    p2 = fmaf(S[ii + 2], q4.z, p2); p3 = fmaf(S[ii + 3], q4.w, p3);
                    n0 = fmaf(nn[ii], q4.x, n0); n1 = fmaf(nn[ii + 1], q4.y, n1);
                    n2 = fmaf(nn[ii + 2], q4.z, n2); n3 = fmaf(nn[ii + 3], q4.w, n3);
                }
                acc = (p0 + p1) + (p2 + p3);
                float nq = (n0 + n1) + (n2 + n3);
#pragma unroll
                for (int d = 1; d < L; d <<= 1) {
                    acc += __shfl_xor_sync(0xffffffffu, acc, d);
                    nq += __shfl_xor_sync(0xffffffffu, nq, d);
                }
                acc = acc / (fmaxf(fabsf(nq), expf(-m_new)) + 1e-6f);
            }
            if (s == 0 && live) a.out[(size_t)(c0 + tt) * a.out_stride + (size_t)h * dv + j] = acc;
        }
    }
    if (live) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s * R + ii;
            if (i < dk) S_g[(size_t)i * dv] = S[ii];
        }
    }
    if constexpr (MODE == SCAN_MLSTM) if (blockIdx.z == 0 && col == 0) {
#pragma unroll
        for (int ii = 0; ii < R; ++ii) {
            const int i = s * R + ii;
            if (i < dk) n_g[i] = nn[ii];
        }
        if (s == 0) *m_g = m;
    }
    if constexpr (MODE == SCAN_DELTA) if (a.conv_in && a.n_taps > 1) {
        // The sequence's last n_taps - 1 inputs become the convolution's state: from the step's rows, or, where the step
        // brought fewer, from the old state moved up.  The sequence's blocks share the channels; a thread owns a channel
        // and goes from the oldest row on, so that it reads every old row before it writes over it.
        const int C = a.conv_channels, rows = a.n_taps - 1, Ls = t1 - t0;
        const int block = h * gridDim.z + blockIdx.z, blocks = H * gridDim.z;
        float* st = slot_state + a.conv_off;
        for (int c = block * 128 + tid; c < C; c += blocks * 128) {
            for (int r = 0; r < rows; ++r) {
                const int idx = Ls - rows + r;
                float x;
                if (idx >= 0) {
                    const size_t at = (size_t)(t0 + idx) * a.conv_stride + c;
                    x = a.conv_bf16 ? __bfloat162float(((const __nv_bfloat16*)a.conv_in)[at]) : ((const float*)a.conv_in)[at];
                } else {
                    x = st[(size_t)(r + Ls) * C + c];
                }
                st[(size_t)r * C + c] = x;
            }
        }
    }
}

template <typename TIN, int MODE, int R, int NI>
int launch_scan_r(const ScanArgs& a, cudaStream_t stream) {
    constexpr size_t smem = (size_t)(2 * SCAN_CH * SCAN_LANES * (R + 4) + SCAN_CH * SCAN_COLS + 2 * SCAN_CH) * sizeof(float);
    static_assert(smem <= 48 * 1024, "the staging area fits the default shared memory");
    static_assert(128 * NI >= SCAN_LANES * R, "a q row is fetched in runs of 128 elements");
    dim3 grid(a.B, a.H, (a.dv + SCAN_COLS - 1) / SCAN_COLS);
    tb_launch(recurrent_scan_kernel<TIN, MODE, R, NI>, grid, dim3(128), smem, stream, a);
    return 0;
}

template <typename TIN, int MODE, int R>
int launch_scan_rows(const ScanArgs& a, cudaStream_t stream) {
    return launch_scan_r<TIN, MODE, R, (SCAN_LANES * R > 128 ? 2 : 1)>(a, stream);
}

template <typename TIN, int MODE>
int launch_scan(const ScanArgs& a, cudaStream_t stream) {
    constexpr int MOST = 256 / SCAN_LANES;              // rows a lane holds at 256 key dimensions
    const int rows = (a.dk + SCAN_LANES - 1) / SCAN_LANES;
    if (rows <= 4 || MOST <= 4) return launch_scan_rows<TIN, MODE, 4>(a, stream);
    if (rows <= 8 || MOST <= 8) return launch_scan_rows<TIN, MODE, (MOST < 8 ? MOST : 8)>(a, stream);
    if (rows <= 16 || MOST <= 16) return launch_scan_rows<TIN, MODE, (MOST < 16 ? MOST : 16)>(a, stream);
    if (rows <= 32 || MOST <= 32) return launch_scan_rows<TIN, MODE, (MOST < 32 ? MOST : 32)>(a, stream);
    return launch_scan_rows<TIN, MODE, MOST>(a, stream);
}

}  // namespace

extern "C" int tb_delta_prep(const DeltaPrepArgs* args, int dtype, cudaStream_t stream) {
    DeltaPrepArgs a = *args;
    TB_REQUIRE(a.T > 0 && a.H > 0 && a.G > 0 && a.H % a.G == 0 && a.dk > 0 && a.dv > 0, "delta_prep: sizes must be positive, heads a multiple of the key heads");
    TB_REQUIRE(a.n_taps >= 1 && a.n_taps <= 64, "delta_prep: %d taps (1 to 64)", a.n_taps);
    TB_REQUIRE(a.H <= 256, "delta_prep: %d heads (at most 256)", a.H);
    TB_REQUIRE(a.proj && a.taps && a.state && a.ba && a.a_log && a.dt_bias && a.qkv && a.gates && a.seq_of && a.q_start && a.slot_of_seq, "delta_prep: missing buffers");
    const int C = 2 * a.G * a.dk + a.H * a.dv;
    TB_REQUIRE(a.stride >= C && a.qkv_stride >= C && a.ba_stride >= 2 * a.H && a.gates_stride >= 2 * a.H, "delta_prep: rows too short");
    const size_t smem = (size_t)C * sizeof(float);
    TB_REQUIRE(smem <= 48 * 1024, "delta_prep: %d channels (at most 12,288)", C);
    if (dtype == TB_F32) tb_launch(delta_prep_kernel<float>, dim3(a.T), dim3(256), smem, stream, a);
    else if (dtype == TB_BF16) tb_launch(delta_prep_kernel<__nv_bfloat16>, dim3(a.T), dim3(256), smem, stream, a);
    else TB_REQUIRE(false, "delta_prep: unknown dtype %d", dtype);
    TB_CHECK_LAUNCH("delta_prep");
    return 0;
}

// mode 0: the gated delta rule (q, k, v float32); mode 1: the mLSTM memory (q, k, v in ``dtype``).
extern "C" int tb_recurrent_scan(const ScanArgs* args, int mode, int dtype, cudaStream_t stream) {
    ScanArgs a = *args;
    TB_REQUIRE(a.B > 0 && a.H > 0 && a.dk > 0 && a.dv > 0 && a.group > 0 && a.H % a.group == 0, "recurrent_scan: sizes must be positive");
    TB_REQUIRE(a.dk <= 256, "recurrent_scan: %d key dimensions a head (at most 256)", a.dk);
    TB_REQUIRE(a.H <= 65535 && (a.dv + 31) / 32 <= 65535, "recurrent_scan: too many heads or value columns");
    TB_REQUIRE(a.q && a.k && a.v && a.gates && a.out && a.state && a.q_start && a.slot_of_seq, "recurrent_scan: missing buffers");
    TB_REQUIRE(dtype == TB_F32 || dtype == TB_BF16, "recurrent_scan: unknown dtype %d", dtype);
    if (mode == SCAN_DELTA) {
        TB_REQUIRE(dtype == TB_F32, "recurrent_scan: the delta rule takes float32 q, k and v");
        TB_REQUIRE(!a.conv_in || (a.n_taps >= 1 && a.conv_channels > 0), "recurrent_scan: the convolution's window needs its sizes");
        if (launch_scan<float, SCAN_DELTA>(a, stream)) return 1;
    } else if (mode == SCAN_MLSTM) {
        TB_REQUIRE(a.i_bias && a.f_bias && a.cap > 0.f, "recurrent_scan: the mLSTM gates need their biases and a positive cap");
        if (dtype == TB_F32 ? launch_scan<float, SCAN_MLSTM>(a, stream) : launch_scan<__nv_bfloat16, SCAN_MLSTM>(a, stream)) return 1;
    } else {
        TB_REQUIRE(false, "recurrent_scan: unknown mode %d", mode);
    }
    TB_CHECK_LAUNCH("recurrent_scan");
    return 0;
}
