// The matrix memory with exponential gates (mLSTM) as a recurrent mixer.
//
// Per head, with a log input gate i_t and a log forget gate f_t (both capped: i = cap *
// tanh(z_i / cap), f = logsigmoid(cap * tanh(z_f / cap))) and a running maximum m that
// starts at 0:
//     m_t = max(f_t + m_(t-1), i_t)
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        [d, dv]
//     n_t = the same with k_t alone                                            [d]
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps)
// S, n and m of a sequence live in 32-bit in its slot of the cache's fixed-size state
// ([H, d, dv] | [H, d] | [H]), zero when the slot is taken, read at the start of a step and
// written at its end.  A prompt and a decoded token run the same kernels.
//
//  * agv_mlstm_prepare: from a token's row  q | k | v | g | i | f  of the stacked projection
//    (32-bit, or 32-bit partial sums over ranges of K): q times q_mult, k, v and the two log
//    gates, 32-bit.
//  * agv_mlstm_scan: the recurrence over the step's tokens, sequence by sequence.  A column
//    of S goes to L lanes that hold 16 rows each in registers (rows l, l + L, ...); a token
//    is one update of those rows, two dot products with q (for S and for n), one round of
//    L-wide shuffles.  Tokens come through shared memory, a chunk at a time.
//  * agv_mlstm_out: every head's o over its root mean square, times a weight per channel,
//    times sigmoid(g), rounded to the compute dtype for the output product.
#include "common.cuh"
#include "row_in.cuh"

namespace {

constexpr int ML_ROWS = 16;          // rows of S a lane holds
constexpr int ML_CHUNK = 16;         // tokens staged in shared memory at a time

__global__ void __launch_bounds__(256)
mlstm_prepare_kernel(RowIn<float> in, int n_tokens, int H, int d, int dv,
                     const float* __restrict__ bias_i, const float* __restrict__ bias_f,
                     float cap, float q_mult, float* __restrict__ qkv, float* __restrict__ gates) {
    pdl_wait();
    pdl_launch_next();
    const int t = blockIdx.x;
    const int nq = H * d, nv = H * dv;
    const int C = 2 * nq + nv;
    float* o = qkv + (size_t)t * C;
    for (int e = threadIdx.x; e < C; e += blockDim.x) {
        // (the gate logits g lie between v and the two recurrence gates and stay where they are)
        const float x = in.at(t, e);
        o[e] = e < nq ? x * q_mult : x;
    }
    for (int e = threadIdx.x; e < 2 * H; e += blockDim.x) {
        const bool forget = e >= H;
        const int h = forget ? e - H : e;
        float z = in.at(t, C + nv + e) + (forget ? bias_f[h] : bias_i[h]);
        z = cap * tanhf(z / cap);
        if (forget) z = fminf(z, 0.f) - log1pf(expf(-fabsf(z)));          // log sigmoid
        gates[(size_t)t * 2 * H + e] = z;
    }
}

// grid (column blocks, heads, sequences); thread = column * L + lane.
template <int L>
__global__ void __launch_bounds__(256)
mlstm_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ gates,
                  float* __restrict__ out, int H, int d, int dv, float den_eps,
                  float* __restrict__ state, long long state_stride,
                  const int* __restrict__ slots, const int* __restrict__ cu_seqlens, int cols) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float sm[];
    constexpr int DP = L * ML_ROWS;                   // rows, padded
    float* ks = sm;                                   // [CHUNK][DP]
    float* qs = ks + ML_CHUNK * DP;                   // [CHUNK][DP]
    float* vs = qs + ML_CHUNK * DP;                   // [CHUNK][cols]
    float* gs = vs + ML_CHUNK * cols;                 // [CHUNK][2]
    const int b = blockIdx.z, h = blockIdx.y;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int slot = slots[b];
    const int col = blockIdx.x * cols + threadIdx.x / L, lane = threadIdx.x % L;
    const bool live = col < dv && threadIdx.x / L < cols;
    const int nq = H * d, C = 2 * nq + H * dv;
    if (slot < 0) {
        // a padding entry: its rows are written, with zeros
        for (int t = t0; t < t1; ++t)
            if (live && lane == 0) out[(size_t)t * H * dv + (size_t)h * dv + col] = 0.f;
        return;
    }
    float* st = state + (size_t)slot * state_stride;
    float* S_g = st + (size_t)h * d * dv;
    float* n_g = st + (size_t)H * d * dv + (size_t)h * d;
    float* m_g = st + (size_t)H * d * dv + (size_t)H * d + h;
    float S[ML_ROWS], n[ML_ROWS];
#pragma unroll
    for (int i = 0; i < ML_ROWS; ++i) {
        const int r = lane + L * i;
        S[i] = live && r < d ? S_g[(size_t)r * dv + col] : 0.f;
        n[i] = r < d ? n_g[r] : 0.f;
    }
    float m = *m_g;
    for (int c0 = t0; c0 < t1; c0 += ML_CHUNK) {
        const int nt = min(ML_CHUNK, t1 - c0);
        __syncthreads();                              // everybody is past the chunk before
        for (int idx = threadIdx.x; idx < nt * DP; idx += blockDim.x) {
            const int tt = idx / DP, r = idx % DP;
            const float* row = qkv + (size_t)(c0 + tt) * C + (size_t)h * d;
            qs[idx] = r < d ? row[r] : 0.f;
            ks[idx] = r < d ? row[nq + r] : 0.f;
        }
        for (int idx = threadIdx.x; idx < nt * cols; idx += blockDim.x) {
            const int tt = idx / cols, c = blockIdx.x * cols + idx % cols;
            vs[idx] = c < dv ? qkv[(size_t)(c0 + tt) * C + 2 * nq + (size_t)h * dv + c] : 0.f;
        }
        for (int idx = threadIdx.x; idx < nt * 2; idx += blockDim.x) {
            const int tt = idx >> 1, which = idx & 1;
            gs[idx] = gates[(size_t)(c0 + tt) * 2 * H + which * H + h];
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            const float gi = gs[2 * tt], gf = gs[2 * tt + 1];
            const float m_new = fmaxf(gf + m, gi);
            const float a = expf(gf + m - m_new), w = expf(gi - m_new);
            m = m_new;
            const float wv = w * vs[tt * cols + threadIdx.x / L];
            const float* kr = ks + tt * DP + lane;
            const float* qr = qs + tt * DP + lane;
            float ds = 0.f, dn = 0.f;
#pragma unroll
            for (int i = 0; i < ML_ROWS; ++i) {
                const float kk = kr[L * i], qq = qr[L * i];
                S[i] = fmaf(a, S[i], wv * kk);
                n[i] = fmaf(a, n[i], w * kk);
                ds = fmaf(S[i], qq, ds);
                dn = fmaf(n[i], qq, dn);
            }
#pragma unroll
            for (int o = L >> 1; o > 0; o >>= 1) {
                ds += __shfl_xor_sync(0xffffffffu, ds, o);
                dn += __shfl_xor_sync(0xffffffffu, dn, o);
            }
            if (live && lane == 0) {
                const float den = fmaxf(fabsf(dn), expf(-m)) + den_eps;
                out[(size_t)(c0 + tt) * H * dv + (size_t)h * dv + col] = ds / den;
            }
        }
    }
    if (t1 > t0) {
#pragma unroll
        for (int i = 0; i < ML_ROWS; ++i) {
            const int r = lane + L * i;
            if (live && r < d) S_g[(size_t)r * dv + col] = S[i];
            if (blockIdx.x == 0 && threadIdx.x < L && r < d) n_g[r] = n[i];
        }
        if (blockIdx.x == 0 && threadIdx.x == 0) *m_g = m;
    }
}

// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ o, RowIn<float> in, int gate_off,
                 const float* __restrict__ weight, float eps, int n_tokens, int H, int dv,
                 T* __restrict__ y) {
    pdl_wait();
    pdl_launch_next();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const float* row = o + ((size_t)t * H + h) * dv;
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) ss = fmaf(row[e], row[e], ss);
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dv + eps);
    for (int e = lane; e < dv; e += 32) {
        const float g = in.at(t, gate_off + h * dv + e);
        y[((size_t)t * H + h) * dv + e] =
            from_f32<T>(row[e] * inv * weight[h * dv + e] / (1.0f + expf(-g)));
    }
}

int row_in(RowIn<float>& in, const float* row, long long ld, const float* part, int n_splits,
           int T, int W) {
    AGV_REQUIRE((row != nullptr) != (part != nullptr && n_splits > 0),
                "mlstm: the projection comes as rows or as partial sums");
    AGV_REQUIRE(part || ld >= W, "mlstm: row stride shorter than a row");
    in = RowIn<float>{row, ld, part, n_splits, (long long)T * W, W};
    return 0;
}

}  // namespace

AGV_API int agv_mlstm_prepare(const float* row, long long ld, const float* part, int n_splits,
                              int T, int H, int d, int dv, const float* bias_i,
                              const float* bias_f, float cap, float q_mult, float* qkv,
                              float* gates, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && H > 0 && d > 0 && dv > 0 && cap > 0.f, "mlstm_prepare: bad sizes");
    if (T == 0) return 0;
    RowIn<float> in;
    if (int rc = row_in(in, row, ld, part, n_splits, T, 2 * H * d + 2 * H * dv + 2 * H)) return rc;
    agv_launch(mlstm_prepare_kernel, (unsigned)T, 256, 0, stream, in, T, H, d, dv, bias_i, bias_f,
               cap, q_mult, qkv, gates);
    AGV_LAUNCH_OK("mlstm_prepare_kernel");
    return 0;
}

AGV_API int agv_mlstm_state_numel(int H, int d, int dv) { return H * d * dv + H * d + H; }

AGV_API int agv_mlstm_scan(const float* qkv, const float* gates, float* out, int T, int B, int H,
                           int d, int dv, float den_eps, float* state, long long state_stride,
                           const int* slots, const int* cu_seqlens, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && B > 0 && H > 0 && d > 0 && dv > 0, "mlstm_scan: bad sizes");
    AGV_REQUIRE(d <= 16 * ML_ROWS, "mlstm_scan: head size %d exceeds %d", d, 16 * ML_ROWS);
    AGV_REQUIRE(state_stride >= agv_mlstm_state_numel(H, d, dv), "mlstm_scan: state too small");
    if (T == 0) return 0;
    int L = 1;
    while (L * ML_ROWS < d) L *= 2;
    int cols = 256 / L;
    if (cols > dv) cols = dv;
    // (a warp holds whole columns: cols * L is rounded up to a warp by idle threads)
    const int threads = (cols * L + 31) / 32 * 32;
    const dim3 grid((unsigned)((dv + cols - 1) / cols), (unsigned)H, (unsigned)B);
    const size_t smem = ((size_t)2 * ML_CHUNK * L * ML_ROWS + (size_t)ML_CHUNK * cols +
                         2 * ML_CHUNK) * sizeof(float);
#define AGV_SCAN(LL)                                                                           \
    agv_launch_after(mlstm_scan_kernel<LL>, grid, threads, smem, stream, qkv, gates, out, H, d, \
                     dv, den_eps, state, state_stride, slots, cu_seqlens, cols)
    switch (L) {
        case 1: AGV_SCAN(1); break;
        case 2: AGV_SCAN(2); break;
        case 4: AGV_SCAN(4); break;
        case 8: AGV_SCAN(8); break;
        default: AGV_SCAN(16); break;
    }
#undef AGV_SCAN
    AGV_LAUNCH_OK("mlstm_scan_kernel");
    return 0;
}

AGV_API int agv_mlstm_out(const float* o, const float* row, long long ld, const float* part,
                          int n_splits, const float* weight, float eps, int T, int H, int d,
                          int dv, void* y, int dtype, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && H > 0 && dv > 0, "mlstm_out: bad sizes");
    if (T == 0) return 0;
    RowIn<float> in;
    if (int rc = row_in(in, row, ld, part, n_splits, T, 2 * H * d + 2 * H * dv + 2 * H)) return rc;
    const int gate_off = 2 * H * d + H * dv;
    const unsigned grid = (unsigned)(((long long)T * H + 3) / 4);
    if (dtype == AGV_F32)
        agv_launch(mlstm_out_kernel<float>, grid, 128, 0, stream, o, in, gate_off, weight, eps, T,
                   H, dv, (float*)y);
    else if (dtype == AGV_BF16)
        agv_launch(mlstm_out_kernel<__nv_bfloat16>, grid, 128, 0, stream, o, in, gate_off, weight,
                   eps, T, H, dv, (__nv_bfloat16*)y);
    else
        return agv_fail(-1, "mlstm_out: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("mlstm_out_kernel");
    return 0;
}
