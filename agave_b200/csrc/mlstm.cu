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
// ([H, d, dv] | [H, d] | [H, ceil(dv / 8)]), zero when the slot is taken, read at the start of a step and
// written at its end.  A prompt and a decoded token run the same kernels.
//
//  * agv_mlstm_prepare: from a token's row  q | k | v | g | i | f  of the stacked projection
//    (32-bit, or 32-bit partial sums over ranges of K): q times q_mult, k, v and the two log
//    gates, 32-bit.
//  * agv_mlstm_scan: the recurrence over the step's tokens, sequence by sequence.  A column
//    of S goes to L lanes that hold 16 rows each in registers; n is one more such column
//    (its value is 1).  A token is one update of those rows, one dot product with q, one round
//    of L-wide shuffles; it leaves S_t^T q_t, n_t . q_t and exp(-m_t).
//  * agv_mlstm_out: the division, every head's o over its root mean square, times a weight
//    per channel, times sigmoid(g), rounded to the compute dtype for the output product.
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

// How the columns of a head's S are dealt out: L lanes a column (L * 16 >= d), at most
// 256 / L columns a CTA.  The running maximum has a copy per ML_MCOLS columns in the state, so
// that the number of columns a CTA takes (a multiple of ML_MCOLS, or all of them) can follow
// the size of the launch.
constexpr int ML_MCOLS = 8;
__host__ __device__ inline int mlstm_lanes(int d) {
    int l = 1;
    while (l * ML_ROWS < d) l *= 2;
    return l;
}
__host__ __device__ inline int mlstm_m_copies(int dv) { return (dv + ML_MCOLS - 1) / ML_MCOLS; }

__device__ __forceinline__ void cp_async4(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                     (unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// grid (column blocks, heads, sequences).  Thread groups of L lanes: group g < cols holds
// column blockIdx.x * cols + g of S, group `cols` holds n (a column whose value is 1; live in
// the first column block only).  A lane's 16 rows are four quads, quad i = rows
// (i * L + lane) * 4 .. + 3, so that a group's lanes read consecutive 16-byte pieces of k and
// q in shared memory and all groups the same pieces.  Tokens come 16 at a time through two
// buffers filled by asynchronous copies while the lanes work on the other; the first warp
// turns the chunk's gate logarithms into the factors a_t = exp(f + m_(t-1) - m_t) and
// b_t = exp(i - m_t) with a scan over the chunk (m -> max(f + m, i) composes: (f2, i2) after
// (f1, i1) is (f1 + f2, max(f2 + i1, i2))).  The kernel leaves the read-out's numerator
// S_t^T q_t in `num` and n_t . q_t, exp(-m_t) in `den`; the division is the next kernel's.
// Every group of eight columns has a copy of the head's running maximum in the state; a CTA
// reads its first group's and writes all of its groups', so that no CTA reads what another
// writes.
template <int L>
__global__ void __launch_bounds__(288)
mlstm_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ gates,
                  float* __restrict__ num, float* __restrict__ den, int H, int d, int dv,
                  float* __restrict__ state, long long state_stride,
                  const int* __restrict__ slots, const int* __restrict__ cu_seqlens, int cols) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ __align__(16) float sm[];
    constexpr int DP = L * ML_ROWS;                   // rows, padded
    constexpr int CH = ML_CHUNK;
    const int CW = cols;                              // values staged per token
    const int buf_len = CH * (2 * DP + CW);
    float* coef = sm + 2 * buf_len;                   // [2][CH][2]: a, b
    const int b = blockIdx.z, h = blockIdx.y;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int slot = slots[b];
    const int grp = threadIdx.x / L, lane = threadIdx.x % L;
    const bool is_n = grp == cols;
    const int col = blockIdx.x * cols + grp;
    const bool live = is_n ? blockIdx.x == 0 : (grp < cols && col < dv);
    const int nq = H * d, C = 2 * nq + H * dv;
    if (slot < 0) {
        // a padding entry: its rows are written, with zeros
        for (int t = t0; t < t1; ++t) {
            if (live && lane == 0 && !is_n) num[(size_t)t * H * dv + (size_t)h * dv + col] = 0.f;
            if (live && lane == 0 && is_n) {
                den[((size_t)t * H + h) * 2] = 0.f;
                den[((size_t)t * H + h) * 2 + 1] = 1.f;
            }
        }
        return;
    }
    float* st = state + (size_t)slot * state_stride;
    float* S_g = st + (size_t)h * d * dv;
    float* n_g = st + (size_t)H * d * dv + (size_t)h * d;
    const int m_copies = mlstm_m_copies(dv);
    float* m_g = st + (size_t)H * d * dv + (size_t)H * d + (size_t)h * m_copies +
                 (blockIdx.x * cols) / ML_MCOLS;
    float S[ML_ROWS];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int r = (i * L + lane) * 4 + c;
            S[i * 4 + c] = !live || r >= d ? 0.f : is_n ? n_g[r] : S_g[(size_t)r * dv + col];
        }
    // the padding rows of both buffers stay zero
    for (int i = threadIdx.x; i < 2 * buf_len; i += blockDim.x) sm[i] = 0.f;
    __syncthreads();
    float m_in = *m_g;                                // (used by the first warp)
    const int n_chunks = (t1 - t0 + CH - 1) / CH;
    auto issue = [&](int c) {
        float* qs = sm + (c & 1) * buf_len;
        float* ks = qs + CH * DP;
        float* vs = ks + CH * DP;
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        // a warp a token, lanes along the row: no division in the walk
        const int warp = threadIdx.x >> 5, ln = threadIdx.x & 31, n_warps = blockDim.x >> 5;
        for (int tt = warp; tt < nt; tt += n_warps) {
            const float* row = qkv + (size_t)(c0 + tt) * C + (size_t)h * d;
            for (int r = ln; r < d; r += 32) {
                cp_async4(qs + tt * DP + r, row + r);
                cp_async4(ks + tt * DP + r, row + nq + r);
            }
            const float* vrow = qkv + (size_t)(c0 + tt) * C + 2 * nq + (size_t)h * dv +
                                (size_t)blockIdx.x * cols;
            const int nv = min(CW, dv - (int)blockIdx.x * cols);
            for (int g = ln; g < nv; g += 32) cp_async4(vs + tt * CW + g, vrow + g);
        }
        cp_async_commit();
    };
    // the first warp's lanes hold the gate logarithms of the chunk they turn into factors next
    float gi = -INFINITY, gf = 0.f;
    auto load_gates = [&](int c) {
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        gi = -INFINITY, gf = 0.f;                     // (beyond the chunk: m stays)
        if (threadIdx.x < nt) {
            gi = gates[(size_t)(c0 + threadIdx.x) * 2 * H + h];
            gf = gates[(size_t)(c0 + threadIdx.x) * 2 * H + H + h];
        }
    };
    if (n_chunks > 0) {
        issue(0);
        if (threadIdx.x < 32) load_gates(0);
    }
    for (int c = 0; c < n_chunks; ++c) {
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        float* cf = coef + (c & 1) * CH * 2;
        if (threadIdx.x < 32) {
            // scan of the chunk's gates: lane t ends with the map of tokens 0..t composed.  The
            // sums are 64-bit and every m_t is rounded to 32 bits once, so that the exponents
            // f + m_(t-1) - m_t carry the roundings of the m's they are formed from (a forget
            // gate next to one moves m by less than its last bit a token)
            double F = gf, I = gi;
#pragma unroll
            for (int o = 1; o < CH; o <<= 1) {
                const double Fp = __shfl_up_sync(0xffffffffu, F, o);
                const double Ip = __shfl_up_sync(0xffffffffu, I, o);
                if ((int)threadIdx.x >= o) {
                    I = fmax(F + Ip, I);
                    F += Fp;
                }
            }
            const float m_t = (float)fmax(F + (double)m_in, I);
            float m_p = __shfl_up_sync(0xffffffffu, m_t, 1);
            if (threadIdx.x == 0) m_p = m_in;
            if (threadIdx.x < nt) {
                cf[threadIdx.x * 2] = expf((float)((double)gf + (double)m_p - (double)m_t));
                cf[threadIdx.x * 2 + 1] = expf((float)((double)gi - (double)m_t));
                if (blockIdx.x == 0) den[((size_t)(c0 + threadIdx.x) * H + h) * 2 + 1] = expf(-m_t);
            }
            m_in = __shfl_sync(0xffffffffu, m_t, nt - 1);
        }
        if (c + 1 < n_chunks) {
            issue(c + 1);
            if (threadIdx.x < 32) load_gates(c + 1);
            cp_async_wait<1>();                       // chunk c has landed, c + 1 is under way
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float* qs = sm + (c & 1) * buf_len;
        const float* ks = qs + CH * DP;
        const float* vs = ks + CH * DP;
        // a token's sum over its lanes and its store run under the next token's loads
        float pend = 0.f;
        auto finish = [&](int tt, float ds) {
#pragma unroll
            for (int o = L >> 1; o > 0; o >>= 1) ds += __shfl_xor_sync(0xffffffffu, ds, o);
            if (live && lane == 0) {
                if (is_n) den[((size_t)(c0 + tt) * H + h) * 2] = ds;
                else num[(size_t)(c0 + tt) * H * dv + (size_t)h * dv + col] = ds;
            }
        };
        const int vcol = min(grp, CW - 1);
#pragma unroll 2
        for (int tt = 0; tt < nt; ++tt) {
            const float a = cf[tt * 2], w = cf[tt * 2 + 1];
            const float vj = vs[tt * CW + vcol];
            const float4* k4 = reinterpret_cast<const float4*>(ks + tt * DP) + lane;
            const float4* q4 = reinterpret_cast<const float4*>(qs + tt * DP) + lane;
            float4 kk[4], qq[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                kk[i] = k4[i * L];
                qq[i] = q4[i * L];
            }
            if (tt > 0) finish(tt - 1, pend);
            const float wv = is_n ? w : w * vj;
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                S[i * 4 + 0] = fmaf(wv, kk[i].x, a * S[i * 4 + 0]);
                S[i * 4 + 1] = fmaf(wv, kk[i].y, a * S[i * 4 + 1]);
                S[i * 4 + 2] = fmaf(wv, kk[i].z, a * S[i * 4 + 2]);
                S[i * 4 + 3] = fmaf(wv, kk[i].w, a * S[i * 4 + 3]);
                acc[0] = fmaf(S[i * 4 + 0], qq[i].x, acc[0]);
                acc[1] = fmaf(S[i * 4 + 1], qq[i].y, acc[1]);
                acc[2] = fmaf(S[i * 4 + 2], qq[i].z, acc[2]);
                acc[3] = fmaf(S[i * 4 + 3], qq[i].w, acc[3]);
            }
            pend = (acc[0] + acc[1]) + (acc[2] + acc[3]);
        }
        if (nt > 0) finish(nt - 1, pend);
        __syncthreads();                              // everybody is done with this buffer
    }
    if (t1 > t0 && live) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int r = (i * L + lane) * 4 + c;
                if (r < d) {
                    if (is_n) n_g[r] = S[i * 4 + c];
                    else S_g[(size_t)r * dv + col] = S[i * 4 + c];
                }
            }
    }
    if (t1 > t0 && threadIdx.x == 0) {
        const int mine = min(cols, dv - (int)blockIdx.x * cols);
        for (int i = 0; i * ML_MCOLS < mine; ++i) m_g[i] = m_in;
    }
}

// One warp per (token, head): the read-out o = num / (max(|n . q|, exp(-m)) + den_eps), over
// its root mean square, times the weight, times sigmoid(g).
template <typename T>
__global__ void __launch_bounds__(128)
mlstm_out_kernel(const float* __restrict__ num, const float* __restrict__ den, float den_eps,
                 RowIn<float> in, int gate_off, const float* __restrict__ weight, float eps,
                 int n_tokens, int H, int dv, T* __restrict__ y) {
    pdl_wait();
    pdl_launch_next();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)n_tokens * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const float* row = num + ((size_t)t * H + h) * dv;
    const float2 dn = *reinterpret_cast<const float2*>(den + ((size_t)t * H + h) * 2);
    const float inv_den = 1.0f / (fmaxf(fabsf(dn.x), dn.y) + den_eps);
    float ss = 0.f;
    for (int e = lane; e < dv; e += 32) {
        const float o = row[e] * inv_den;
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)dv + eps) * inv_den;
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

AGV_API int agv_mlstm_state_numel(int H, int d, int dv) {
    return H * d * dv + H * d + H * mlstm_m_copies(dv);
}

// qkv [T, 2 H d + H dv] and gates [T, 2 H] from agv_mlstm_prepare; num [T, H dv] receives
// S_t^T q_t and den [T, H, 2] receives n_t . q_t and exp(-m_t); state [n_slots, stride] holds
// S [H, d, dv], n [H, d] and a copy of m per eight columns [H, ceil(dv / 8)] of every sequence.
AGV_API int agv_mlstm_scan(const float* qkv, const float* gates, float* num, float* den, int T,
                           int B, int H, int d, int dv, float* state, long long state_stride,
                           const int* slots, const int* cu_seqlens, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && B > 0 && H > 0 && d > 0 && dv > 0, "mlstm_scan: bad sizes");
    AGV_REQUIRE(d <= 16 * ML_ROWS, "mlstm_scan: head size %d exceeds %d", d, 16 * ML_ROWS);
    AGV_REQUIRE(state_stride >= agv_mlstm_state_numel(H, d, dv), "mlstm_scan: state too small");
    AGV_REQUIRE(agv_aligned(den, 8), "mlstm_scan: den must be 8-byte aligned");
    if (T == 0) return 0;
    const int L = mlstm_lanes(d);
    // columns a CTA: as many as 256 threads hold, fewer (down to eight) while that still
    // leaves every CTA an SM of its own.  (Measured on one prompt of 2,048 tokens, 32 heads of
    // 128 x 128: 128 CTAs of 32 columns 851 us; 256 of 16, two to an SM, 941; 512 of 8, 1,027:
    // a token costs a warp about 800 cycles whatever its company.)
    int cols = 256 / L;
    if (cols > dv) cols = dv;
    static int sms = 0;
    if (!sms) {
        int dev = 0;
        AGV_CUDA_OK(cudaGetDevice(&dev));
        AGV_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    }
    while (cols % (2 * ML_MCOLS) == 0 && (long long)H * B * ((dv + cols - 1) / cols) * 2 <= sms)
        cols /= 2;
    const int blocks = (dv + cols - 1) / cols;
    // (a warp holds whole groups: (cols + 1) * L is rounded up to a warp by idle threads)
    const int threads = ((cols + 1) * L + 31) / 32 * 32;
    const dim3 grid((unsigned)blocks, (unsigned)H, (unsigned)B);
    const size_t smem = ((size_t)2 * ML_CHUNK * (2 * L * ML_ROWS + cols) + 4 * ML_CHUNK) *
                        sizeof(float);
#define AGV_SCAN(LL)                                                                          \
    do {                                                                                      \
        auto kern = mlstm_scan_kernel<LL>;                                                    \
        if (smem > 48 * 1024)                                                                 \
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem));                                     \
        agv_launch_after(kern, grid, threads, smem, stream, qkv, gates, num, den, H, d, dv,   \
                         state, state_stride, slots, cu_seqlens, cols);                       \
    } while (0)
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

AGV_API int agv_mlstm_out(const float* num, const float* den, float den_eps, const float* row,
                          long long ld, const float* part, int n_splits, const float* weight,
                          float eps, int T, int H, int d, int dv, void* y, int dtype,
                          cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && H > 0 && dv > 0, "mlstm_out: bad sizes");
    if (T == 0) return 0;
    RowIn<float> in;
    if (int rc = row_in(in, row, ld, part, n_splits, T, 2 * H * d + 2 * H * dv + 2 * H)) return rc;
    const int gate_off = 2 * H * d + H * dv;
    const unsigned grid = (unsigned)(((long long)T * H + 3) / 4);
    if (dtype == AGV_F32)
        agv_launch(mlstm_out_kernel<float>, grid, 128, 0, stream, num, den, den_eps, in, gate_off,
                   weight, eps, T, H, dv, (float*)y);
    else if (dtype == AGV_BF16)
        agv_launch(mlstm_out_kernel<__nv_bfloat16>, grid, 128, 0, stream, num, den, den_eps, in,
                   gate_off, weight, eps, T, H, dv, (__nv_bfloat16*)y);
    else
        return agv_fail(-1, "mlstm_out: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("mlstm_out_kernel");
    return 0;
}
