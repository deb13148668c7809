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
//  * agv_mlstm_scan: the recurrence over the step's tokens, sequence by sequence.  A thread
//    holds 16 rows of one column of S in registers, a warp 32 columns, so that k and q of a
//    token are read by a whole warp at once; the row blocks' parts of a column's dot product
//    with q meet in shared memory after a chunk of tokens.  It leaves S_t^T q_t, n_t . q_t
//    and exp(-m_t).
//  * agv_mlstm_out: the division, every head's o over its root mean square, times a weight
//    per channel, times sigmoid(g), rounded to the compute dtype for the output product.
#include "common.cuh"
#include "row_in.cuh"

namespace {

constexpr int ML_COLS = 32;          // columns of S a CTA holds, one a lane
constexpr int ML_ROWS = 16;          // rows of a column a thread holds
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

// The running maximum has a copy per ML_MCOLS columns in the state (see the scan).
constexpr int ML_MCOLS = 8;
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

// grid (column blocks of 32, heads, sequences); RW + 1 warps, RW * 16 >= d.  Thread (w, lane)
// of the first RW warps holds rows w * 16 .. + 15 of column blockIdx.x * 32 + lane of S in
// registers: all lanes of a warp read the same k and q of a token (one broadcast piece of
// shared memory at a time) and their own v; a token is one update of the thread's 16 values
// and its part of the column's dot product with q, which goes to shared memory; the parts
// of the RW warps are added, for all tokens of a chunk at once, after the chunk.  No shuffle
// and no other thread's result lies on a token's path.  The last warp has the rows of n dealt
// round its lanes (n . q by warp sums, a chunk's tokens side by side; written by the first
// column block only) and, while the
// others work on a chunk, turns the next chunk's gate logarithms into the factors
// a_t = exp(f + m_(t-1) - m_t) and b_t = exp(i - m_t) by a scan over the chunk (m -> max(f + m,
// i) composes: (f2, i2) after (f1, i1) is (f1 + f2, max(f2 + i1, i2))).  Tokens come 16 at a
// time through two buffers filled by asynchronous copies.  The kernel leaves the read-out's
// numerator S_t^T q_t in `num` and n_t . q_t, exp(-m_t) in `den`; the division is the next
// kernel's.  Every group of eight columns has a copy of the head's running maximum in the
// state; a CTA reads its first group's and writes all of its groups', so that no CTA reads
// what another writes.
template <int RW>
__global__ void __launch_bounds__((RW + 1) * 32)
mlstm_scan_kernel(const float* __restrict__ qkv, const float* __restrict__ gates,
                  float* __restrict__ num, float* __restrict__ den, int H, int d, int dv,
                  float* __restrict__ state, long long state_stride,
                  const int* __restrict__ slots, const int* __restrict__ cu_seqlens) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ __align__(16) float sm[];
    constexpr int DP = RW * ML_ROWS;                  // rows, padded
    constexpr int NR = RW >= 2 ? RW / 2 : 1;          // rows of n a lane of the last warp holds
    constexpr int CH = ML_CHUNK;
    constexpr int CW = ML_COLS;
    constexpr int BUF = CH * (2 * DP + CW);
    float* coef = sm + 2 * BUF;                       // [2][CH][2]: a, b
    float* psum = coef + 4 * CH;                      // [2][CH][RW][CW]
    const int b = blockIdx.z, h = blockIdx.y;
    const int t0 = cu_seqlens[b], t1 = cu_seqlens[b + 1];
    const int slot = slots[b];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool is_nw = warp == RW;
    const int col = blockIdx.x * CW + lane;
    const bool live = col < dv;
    const int nq = H * d, C = 2 * nq + H * dv;
    if (slot < 0) {
        // a padding entry: its rows are written, with zeros
        for (int t = t0; t < t1; ++t) {
            if (warp == 0 && live) num[(size_t)t * H * dv + (size_t)h * dv + col] = 0.f;
            if (is_nw && lane == 0 && blockIdx.x == 0) {
                den[((size_t)t * H + h) * 2] = 0.f;
                den[((size_t)t * H + h) * 2 + 1] = 1.f;
            }
        }
        return;
    }
    float* st = state + (size_t)slot * state_stride;
    float* S_g = st + (size_t)h * d * dv;
    float* n_g = st + (size_t)H * d * dv + (size_t)h * d;
    float* m_g = st + (size_t)H * d * dv + (size_t)H * d + (size_t)h * mlstm_m_copies(dv) +
                 (blockIdx.x * CW) / ML_MCOLS;
    // a row warp's thread: S[j] = row warp * 16 + j of its column; the last warp's: its rows
    // j * 32 + lane of n in S[0 .. NR)
    float S[ML_ROWS];
#pragma unroll
    for (int j = 0; j < ML_ROWS; ++j) {
        S[j] = 0.f;
        if (!is_nw) {
            const int r = warp * ML_ROWS + j;
            if (live && r < d) S[j] = S_g[(size_t)r * dv + col];
        } else if (j < NR) {
            const int r = j * 32 + lane;
            if (r < d) S[j] = n_g[r];
        }
    }
    // the padding rows of both buffers stay zero
    for (int i = threadIdx.x; i < 2 * BUF; i += blockDim.x) sm[i] = 0.f;
    __syncthreads();
    float m_in = *m_g;                                // (the last warp's)
    const int n_chunks = (t1 - t0 + CH - 1) / CH;
    auto issue = [&](int c) {
        float* qs = sm + (c & 1) * BUF;
        float* ks = qs + CH * DP;
        float* vs = ks + CH * DP;
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        // a warp a token, lanes along the row: no division in the walk
        for (int tt = warp; tt < nt; tt += RW + 1) {
            const float* row = qkv + (size_t)(c0 + tt) * C + (size_t)h * d;
            for (int r = lane; r < d; r += 32) {
                cp_async4(qs + tt * DP + r, row + r);
                cp_async4(ks + tt * DP + r, row + nq + r);
            }
            if (live)
                cp_async4(vs + tt * CW + lane,
                          qkv + (size_t)(c0 + tt) * C + 2 * nq + (size_t)h * dv + col);
        }
        cp_async_commit();
    };
    // the last warp's lanes hold the gate logarithms of the chunk they turn into factors next
    float gi = -INFINITY, gf = 0.f;
    auto load_gates = [&](int c) {
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        gi = -INFINITY, gf = 0.f;                     // (beyond the chunk: m stays)
        if (lane < nt) {
            gi = gates[(size_t)(c0 + lane) * 2 * H + h];
            gf = gates[(size_t)(c0 + lane) * 2 * H + H + h];
        }
    };
    // Scan of a chunk's gates (the last warp): lane t ends with the map of tokens 0..t
    // composed.  The sums are 64-bit and every m_t is rounded to 32 bits once, so that the
    // exponents f + m_(t-1) - m_t carry the roundings of the m's they are formed from (a
    // forget gate next to one moves m by less than its last bit a token).
    auto factors = [&](int c) {
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        float* cf = coef + (c & 1) * CH * 2;
        double F = gf, I = gi;
#pragma unroll
        for (int o = 1; o < CH; o <<= 1) {
            const double Fp = __shfl_up_sync(0xffffffffu, F, o);
            const double Ip = __shfl_up_sync(0xffffffffu, I, o);
            if (lane >= o) {
                I = fmax(F + Ip, I);
                F += Fp;
            }
        }
        const float m_t = (float)fmax(F + (double)m_in, I);
        float m_p = __shfl_up_sync(0xffffffffu, m_t, 1);
        if (lane == 0) m_p = m_in;
        if (lane < nt) {
            cf[lane * 2] = expf((float)((double)gf + (double)m_p - (double)m_t));
            cf[lane * 2 + 1] = expf((float)((double)gi - (double)m_t));
            if (blockIdx.x == 0) den[((size_t)(c0 + lane) * H + h) * 2 + 1] = expf(-m_t);
        }
        m_in = __shfl_sync(0xffffffffu, m_t, nt - 1);
    };
    if (n_chunks > 0) {
        issue(0);
        if (is_nw) {
            load_gates(0);
            factors(0);
        }
    }
    for (int c = 0; c < n_chunks; ++c) {
        const int c0 = t0 + c * CH, nt = min(CH, t1 - c0);
        const float* cf = coef + (c & 1) * CH * 2;
        float* ps = psum + (c & 1) * CH * RW * CW;
        if (c + 1 < n_chunks) {
            issue(c + 1);
            if (is_nw) load_gates(c + 1);
            cp_async_wait<1>();                       // chunk c has landed, c + 1 is under way
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();                              // chunk c and its factors are there
        const float* qs = sm + (c & 1) * BUF;
        const float* ks = qs + CH * DP;
        const float* vs = ks + CH * DP;
        if (!is_nw) {
            const float4* kbase = reinterpret_cast<const float4*>(ks + warp * ML_ROWS);
            const float4* qbase = reinterpret_cast<const float4*>(qs + warp * ML_ROWS);
#pragma unroll 2
            for (int tt = 0; tt < nt; ++tt) {
                const float a = cf[tt * 2];
                const float wv = cf[tt * 2 + 1] * vs[tt * CW + lane];
                const float4* k4 = kbase + tt * (DP / 4);
                const float4* q4 = qbase + tt * (DP / 4);
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (int j = 0; j < ML_ROWS / 4; ++j) {
                    const float4 kk = k4[j], qq = q4[j];
                    S[j * 4 + 0] = fmaf(wv, kk.x, a * S[j * 4 + 0]);
                    S[j * 4 + 1] = fmaf(wv, kk.y, a * S[j * 4 + 1]);
                    S[j * 4 + 2] = fmaf(wv, kk.z, a * S[j * 4 + 2]);
                    S[j * 4 + 3] = fmaf(wv, kk.w, a * S[j * 4 + 3]);
                    acc[0] = fmaf(S[j * 4 + 0], qq.x, acc[0]);
                    acc[1] = fmaf(S[j * 4 + 1], qq.y, acc[1]);
                    acc[2] = fmaf(S[j * 4 + 2], qq.z, acc[2]);
                    acc[3] = fmaf(S[j * 4 + 3], qq.w, acc[3]);
                }
                ps[(tt * RW + warp) * CW + lane] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
            }
        } else {
            // n over the chunk, each lane's part of every token's n . q kept; then the warp
            // sums of all the chunk's tokens side by side (their shuffles overlap)
            float dn[CH];
#pragma unroll
            for (int tt = 0; tt < CH; ++tt) {
                dn[tt] = 0.f;
                if (tt < nt) {
                    const float a = cf[tt * 2], w = cf[tt * 2 + 1];
#pragma unroll
                    for (int j = 0; j < NR; ++j) {
                        const int r = j * 32 + lane;
                        const float kk = r < DP ? ks[tt * DP + r] : 0.f;
                        const float qq = r < DP ? qs[tt * DP + r] : 0.f;
                        S[j] = fmaf(w, kk, a * S[j]);
                        dn[tt] = fmaf(S[j], qq, dn[tt]);
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1)
#pragma unroll
                for (int tt = 0; tt < CH; ++tt) dn[tt] += __shfl_xor_sync(0xffffffffu, dn[tt], o);
            if (blockIdx.x == 0) {
                float mine = 0.f;
#pragma unroll
                for (int tt = 0; tt < CH; ++tt)
                    if (lane == tt) mine = dn[tt];
                if (lane < nt) den[((size_t)(c0 + lane) * H + h) * 2] = mine;
            }
            if (c + 1 < n_chunks) factors(c + 1);
        }
        __syncthreads();                              // the chunk's parts are there
        for (int idx = threadIdx.x; idx < nt * CW; idx += blockDim.x) {
            const int tt = idx / CW, l = idx % CW;
            float sum = 0.f;
#pragma unroll
            for (int w = 0; w < RW; ++w) sum += ps[(tt * RW + w) * CW + l];
            if (blockIdx.x * CW + l < dv)
                num[(size_t)(c0 + tt) * H * dv + (size_t)h * dv + blockIdx.x * CW + l] = sum;
        }
    }
    if (t1 > t0) {
#pragma unroll
        for (int j = 0; j < ML_ROWS; ++j) {
            if (!is_nw) {
                const int r = warp * ML_ROWS + j;
                if (live && r < d) S_g[(size_t)r * dv + col] = S[j];
            } else if (j < NR && blockIdx.x == 0) {
                const int r = j * 32 + lane;
                if (r < d) n_g[r] = S[j];
            }
        }
        if (is_nw && lane == 0) {
            const int mine = min(CW, dv - (int)blockIdx.x * CW);
            for (int i = 0; i * ML_MCOLS < mine; ++i) m_g[i] = m_in;
        }
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
    AGV_REQUIRE(d <= 256, "mlstm_scan: head size %d exceeds 256", d);
    AGV_REQUIRE(state_stride >= agv_mlstm_state_numel(H, d, dv), "mlstm_scan: state too small");
    AGV_REQUIRE(agv_aligned(den, 8), "mlstm_scan: den must be 8-byte aligned");
    if (T == 0) return 0;
    int RW = 1;
    while (RW * ML_ROWS < d) RW *= 2;
    const dim3 grid((unsigned)((dv + ML_COLS - 1) / ML_COLS), (unsigned)H, (unsigned)B);
    const size_t smem = ((size_t)2 * ML_CHUNK * (2 * RW * ML_ROWS + ML_COLS) + 4 * ML_CHUNK +
                         (size_t)2 * ML_CHUNK * RW * ML_COLS) * sizeof(float);
#define AGV_SCAN(RR)                                                                          \
    do {                                                                                      \
        auto kern = mlstm_scan_kernel<RR>;                                                    \
        static bool configured = false;          /* (the size follows from RR alone) */       \
        if (smem > 48 * 1024 && !configured) {                                                \
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem));                                     \
            configured = true;                                                                \
        }                                                                                     \
        agv_launch_after(kern, grid, (RR + 1) * 32, smem, stream, qkv, gates, num, den, H, d, \
                         dv, state, state_stride, slots, cu_seqlens);                         \
    } while (0)
    switch (RW) {
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
