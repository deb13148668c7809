// The gated delta rule with a decay per key channel, as a recurrent mixer's kernels.
//
// A token's row of the stacked projection is  q | k | v | b | a1 | g1  (G*d, G*d, H*dv, H, ra
// and rg wide).  q, k and v pass a short causal convolution over time, channel by channel
// (``taps`` weights a channel, the last one the current token's; zeros before the start of a
// sequence), and silu.  Every q and k head becomes a unit vector (x / sqrt(sum x^2 + eps_unit)),
// q times a constant besides.  beta = sigmoid(b), one per head.  a1 and g1 are low-rank
// bottlenecks: a = W_a2 a1 and the gate W_g2 g1 are products of their own between the
// kernels here.  With the decay  g = exp(neg_a[h] * softplus(a + dt_bias))  per head and key
// channel, a head's state S [d, dv] goes
//
//      S <- diag(g) S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// token by token (the read-out sees the token's own write), query/key head h / (H / G)
// serving head h.  The head's o is divided by its root mean square (eps_out), multiplied by a
// weight [dv] and by sigmoid(gate), and rounded to the compute dtype for the output product.
//
// The columns of S are independent recurrences over d-vectors, so the scan gives every column
// to a group of L lanes that hold 16 rows of it each in registers; the two dot products of a
// token are finished with L-wide shuffles.  A sequence's tokens run in order; sequences,
// heads and groups of columns run side by side.  The state of a sequence (S of every head,
// and the last taps - 1 inputs of the convolution) lives in 32-bit in the sequence's slot of
// the fixed-size state and is read at the start of a step and written at its end, so a
// prompt and a decoded token run the same code.
//
// 32-bit throughout: sums over partial products, the convolution, silu, unit norms, beta, the
// decay, the state and the recurrence, the output norm and the gate's sigmoid.
#include "common.cuh"
#include "row_in.cuh"

namespace {

constexpr int DL_R = 16;           // rows of a column a lane holds
constexpr int DL_MAX_TAPS = 16;

struct DeltaDims {
    int G, H, d, dv, taps, ra, rg;
    __host__ __device__ int nq() const { return G * d; }
    __host__ __device__ int nv() const { return H * dv; }
    __host__ __device__ int C() const { return 2 * G * d + H * dv; }      // convolved channels
    __host__ __device__ int W() const { return C() + H + ra + rg; }
};

// Where a step's sequences keep their state.
struct DeltaState {
    float* state;              // [n_slots, stride]
    long long stride;
    long long conv_off;        // the convolution's inputs [taps - 1, C] start here; S [H, dv, d] at 0
    const int* slots;          // [B]; negative: padding entry
    const int* cu;             // [B + 1] first token of each entry
    const int* seq_index;      // [T]
    const int* positions;      // [T]
};

__device__ __forceinline__ float silu_f(float t) { return t / (1.0f + expf(-t)); }
__device__ __forceinline__ float sigmoid_f(float t) { return 1.0f / (1.0f + expf(-t)); }
__device__ __forceinline__ float softplus_f(float t) {
    return t > 20.0f ? t : log1pf(expf(t));
}

// ------------------------------------------------------------------ prepare
// One CTA per token.  fused_state: the CTA's token is the only one its sequence brings (a
// decode step), so it also shifts the convolution's inputs by one.
template <typename T>
__global__ void __launch_bounds__(256)
delta_prepare_kernel(RowIn<T> in, DeltaDims dm, DeltaState st, const float* __restrict__ conv_w,
                     float eps_unit, float q_mult, int fused_state, float* __restrict__ qkv,
                     float* __restrict__ beta, T* __restrict__ low_a, T* __restrict__ low_g) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float buf[];               // [C] convolved and activated channels
    const int t = blockIdx.x;
    const int b = st.seq_index[t];
    const int slot = st.slots[b];
    if (slot < 0) return;
    const int C = dm.C(), nq = dm.nq(), taps = dm.taps;
    const int p = st.positions[t];
    const int first = st.cu[b];                  // first token of the sequence in this step
    const int p0 = p - (t - first);              // its position
    float* cs = st.state + (size_t)slot * st.stride + st.conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        const float* w = conv_w + (size_t)c * taps;
        float acc = 0.f;
        // oldest input first; input p - k meets weight taps - 1 - k
        for (int k = taps - 1; k >= 0; --k) {
            const int pp = p - k;
            float x = 0.f;
            if (pp >= p0) x = in.at(t - k, c);
            else if (pp >= 0) x = cs[(size_t)(pp - p0 + taps - 1) * C + c];
            acc = fmaf(w[taps - 1 - k], x, acc);
        }
        buf[c] = silu_f(acc);
        if (fused_state && taps > 1) {
            for (int i = 0; i + 2 < taps; ++i) cs[(size_t)i * C + c] = cs[(size_t)(i + 1) * C + c];
            cs[(size_t)(taps - 2) * C + c] = in.at(t, c);
        }
    }
    __syncthreads();
    // unit vectors: q heads, then k heads (2 G groups of d), a warp a group
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float* orow = qkv + (size_t)t * C;
    for (int grp = warp; grp < 2 * dm.G; grp += nwarps) {
        const float* x = buf + (size_t)grp * dm.d;
        float ss = 0.f;
        for (int i = lane; i < dm.d; i += 32) ss = fmaf(x[i], x[i], ss);
        ss = warp_sum(ss);
        const float r = (1.0f / sqrtf(ss + eps_unit)) * (grp < dm.G ? q_mult : 1.0f);
        for (int i = lane; i < dm.d; i += 32) orow[(size_t)grp * dm.d + i] = x[i] * r;
    }
    for (int c = 2 * nq + threadIdx.x; c < C; c += blockDim.x) orow[c] = buf[c];
    for (int h = threadIdx.x; h < dm.H; h += blockDim.x)
        beta[(size_t)t * dm.H + h] = sigmoid_f(in.at(t, C + h));
    for (int i = threadIdx.x; i < dm.ra; i += blockDim.x)
        low_a[(size_t)t * dm.ra + i] = from_f32<T>(in.at(t, C + dm.H + i));
    for (int i = threadIdx.x; i < dm.rg; i += blockDim.x)
        low_g[(size_t)t * dm.rg + i] = from_f32<T>(in.at(t, C + dm.H + dm.ra + i));
}

// The convolution's inputs after a step of several tokens a sequence: the last taps - 1 of
// what the sequence has seen.  One CTA per sequence, a thread a channel; it runs after the
// prepare kernel, which reads the inputs of before the step.
template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(RowIn<T> in, DeltaDims dm, DeltaState st) {
    pdl_wait();
    pdl_launch_next();
    const int b = blockIdx.x;
    const int slot = st.slots[b];
    if (slot < 0) return;
    const int C = dm.C(), taps = dm.taps;
    const int first = st.cu[b], n = st.cu[b + 1] - first;
    if (n <= 0) return;
    const int p0 = st.positions[first], len = p0 + n;
    float* cs = st.state + (size_t)slot * st.stride + st.conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x) {
        for (int i = 0; i + 1 < taps; ++i) {
            const int pp = len - (taps - 1) + i;
            float x = 0.f;
            if (pp >= p0) x = in.at(first + pp - p0, c);
            else if (pp >= 0) x = cs[(size_t)(pp - p0 + taps - 1) * C + c];   // an entry after i
            cs[(size_t)i * C + c] = x;
        }
    }
}

// --------------------------------------------------------------------- scan
// grid (column groups, H, B); a CTA has CC columns of one head of one sequence, L lanes a
// column (L a power of two, L * 16 >= d), thread = column * L + lane.  The tokens of the
// sequence come through shared memory TCH at a time: k, q and the decay of the head's key
// channels (padded with zeros to L * 16 rows, which keeps the padded rows of S at zero), the
// CTA's columns of v, and beta.
struct ScanArgs {
    const float* qkv;          // [T, C]: q | k | v, prepared
    const float* beta;         // [T, H]
    const float* a;            // [T, H * d]: the decay's pre-activation, without its bias
    const float* dt_bias;      // [H * d]
    const float* neg_a;        // [H]: -exp(A_log)
    float* out;                // [T, H * dv]
    int L, CC, TCH;
};

__global__ void __launch_bounds__(256)
delta_scan_kernel(ScanArgs a, DeltaDims dm, DeltaState st) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float smem[];
    const int b = blockIdx.z;
    const int slot = st.slots[b];
    if (slot < 0) return;
    const int t0 = st.cu[b], n = st.cu[b + 1] - t0;
    if (n <= 0) return;
    const int h = blockIdx.y, g = h / (dm.H / dm.G);
    const int d = dm.d, dv = dm.dv, C = dm.C(), nq = dm.nq();
    const int L = a.L, CC = a.CC, TCH = a.TCH, Dp = L * DL_R;
    const int l = threadIdx.x & (L - 1);
    const int jc = threadIdx.x / L;
    const int j = blockIdx.x * CC + jc;
    const bool live = jc < CC && j < dv;
    float* sk = smem;                          // [TCH][Dp]
    float* sq = sk + (size_t)TCH * Dp;
    float* sg = sq + (size_t)TCH * Dp;
    float* sv = sg + (size_t)TCH * Dp;         // [TCH][CC]
    float* sb = sv + (size_t)TCH * CC;         // [TCH]

    float S[DL_R];
    float* srow = st.state + (size_t)slot * st.stride + ((size_t)h * dv + (live ? j : 0)) * d;
#pragma unroll
    for (int i = 0; i < DL_R; ++i) {
        const int r = l * DL_R + i;
        S[i] = live && r < d ? srow[r] : 0.f;
    }
    const float na = a.neg_a[h];
    for (int c0 = 0; c0 < n; c0 += TCH) {
        const int m = min(TCH, n - c0);
        __syncthreads();
        for (int idx = threadIdx.x; idx < m * Dp; idx += blockDim.x) {
            const int tt = idx / Dp, r = idx - tt * Dp;
            const size_t t = (size_t)(t0 + c0 + tt);
            float kv = 0.f, qv = 0.f, gv = 0.f;
            if (r < d) {
                qv = a.qkv[t * C + (size_t)g * d + r];
                kv = a.qkv[t * C + nq + (size_t)g * d + r];
                const float pre = a.a[t * dm.H * d + (size_t)h * d + r] + a.dt_bias[(size_t)h * d + r];
                gv = expf(na * softplus_f(pre));
            }
            sk[idx] = kv; sq[idx] = qv; sg[idx] = gv;
        }
        for (int idx = threadIdx.x; idx < m * CC; idx += blockDim.x) {
            const int tt = idx / CC, c = idx - tt * CC;
            const int col = blockIdx.x * CC + c;
            sv[idx] = col < dv ? a.qkv[(size_t)(t0 + c0 + tt) * C + 2 * nq + (size_t)h * dv + col] : 0.f;
        }
        for (int tt = threadIdx.x; tt < m; tt += blockDim.x)
            sb[tt] = a.beta[(size_t)(t0 + c0 + tt) * dm.H + h];
        __syncthreads();
        for (int tt = 0; tt < m; ++tt) {
            const float4* k4 = reinterpret_cast<const float4*>(sk + (size_t)tt * Dp + l * DL_R);
            const float4* q4 = reinterpret_cast<const float4*>(sq + (size_t)tt * Dp + l * DL_R);
            const float4* g4 = reinterpret_cast<const float4*>(sg + (size_t)tt * Dp + l * DL_R);
            float kk[DL_R];
            float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int i = 0; i < DL_R / 4; ++i) {
                const float4 kq = k4[i], gq = g4[i];
                kk[4 * i] = kq.x; kk[4 * i + 1] = kq.y; kk[4 * i + 2] = kq.z; kk[4 * i + 3] = kq.w;
                S[4 * i] *= gq.x; S[4 * i + 1] *= gq.y; S[4 * i + 2] *= gq.z; S[4 * i + 3] *= gq.w;
                acc0 = fmaf(S[4 * i], kq.x, acc0);
                acc1 = fmaf(S[4 * i + 1], kq.y, acc1);
                acc0 = fmaf(S[4 * i + 2], kq.z, acc0);
                acc1 = fmaf(S[4 * i + 3], kq.w, acc1);
            }
            float acc = acc0 + acc1;
            for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
            const float u = sb[tt] * (sv[(size_t)tt * CC + (jc < CC ? jc : 0)] - acc);
            float o0 = 0.f, o1 = 0.f;
#pragma unroll
            for (int i = 0; i < DL_R / 4; ++i) {
                const float4 qq = q4[i];
                S[4 * i] = fmaf(kk[4 * i], u, S[4 * i]);
                S[4 * i + 1] = fmaf(kk[4 * i + 1], u, S[4 * i + 1]);
                S[4 * i + 2] = fmaf(kk[4 * i + 2], u, S[4 * i + 2]);
                S[4 * i + 3] = fmaf(kk[4 * i + 3], u, S[4 * i + 3]);
                o0 = fmaf(S[4 * i], qq.x, o0);
                o1 = fmaf(S[4 * i + 1], qq.y, o1);
                o0 = fmaf(S[4 * i + 2], qq.z, o0);
                o1 = fmaf(S[4 * i + 3], qq.w, o1);
            }
            float ov = o0 + o1;
            for (int o = 1; o < L; o <<= 1) ov += __shfl_xor_sync(0xffffffffu, ov, o);
            if (live && l == 0)
                a.out[(size_t)(t0 + c0 + tt) * dm.H * dv + (size_t)h * dv + j] = ov;
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DL_R; ++i) {
            const int r = l * DL_R + i;
            if (r < d) srow[r] = S[i];
        }
    }
}

// ---------------------------------------------------------------- read-out
// y[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * sigmoid(gate[t, h, :]): one CTA a token,
// a warp a head.
template <typename T>
__global__ void __launch_bounds__(128)
delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                 const float* __restrict__ w, float eps, int n_tokens, int H, int dv,
                 const int* __restrict__ seq_index, const int* __restrict__ slots,
                 T* __restrict__ y) {
    pdl_wait();
    pdl_launch_next();
    const int t = blockIdx.x;
    const bool pad = slots[seq_index[t]] < 0;      // a padding entry's row is zeros
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int h = warp; h < H; h += nwarps) {
        const size_t base = ((size_t)t * H + h) * dv;
        if (pad) {
            for (int i = lane; i < dv; i += 32) y[base + i] = from_f32<T>(0.f);
            continue;
        }
        float ss = 0.f;
        for (int i = lane; i < dv; i += 32) ss = fmaf(o[base + i], o[base + i], ss);
        ss = warp_sum(ss);
        const float r = 1.0f / sqrtf(ss / (float)dv + eps);
        for (int i = lane; i < dv; i += 32)
            y[base + i] = from_f32<T>(o[base + i] * r * w[i] * sigmoid_f(gate[base + i]));
    }
}

}  // namespace

static int check_dims(const DeltaDims& dm) {
    AGV_REQUIRE(dm.G > 0 && dm.H > 0 && dm.d > 0 && dm.dv > 0 && dm.ra >= 0 && dm.rg >= 0,
                "delta: bad sizes");
    AGV_REQUIRE(dm.H % dm.G == 0, "delta: %d heads are not a multiple of %d query/key heads",
                dm.H, dm.G);
    AGV_REQUIRE(dm.taps >= 1 && dm.taps <= DL_MAX_TAPS, "delta: %d taps, at most %d", dm.taps,
                DL_MAX_TAPS);
    AGV_REQUIRE(dm.d <= 32 * DL_R, "delta: key heads of %d exceed %d", dm.d, 32 * DL_R);
    return 0;
}

// row: [T, W] with row stride ld (dtype), or part: [n_splits, T, W] 32-bit partial sums, W =
// 2 G d + H dv + H + ra + rg.  conv_w: [2 G d + H dv, taps] 32-bit.  state: [n_slots,
// state_stride] 32-bit, the convolution's inputs [taps - 1, 2 G d + H dv] at conv_off.
// several != 0: sequences may bring more than one token (a prompt step); the convolution's
// inputs are then renewed by a launch of its own.  Outputs: qkv [T, 2 G d + H dv] and beta
// [T, H] 32-bit, low_a [T, ra] and low_g [T, rg] in dtype.
AGV_API int agv_delta_prepare(const void* row, long long ld, const float* part, int n_splits,
                              int dtype, int T, int B, int G, int H, int d, int dv, int taps,
                              int ra, int rg, const float* conv_w, float eps_unit, float q_mult,
                              float* state, long long state_stride, long long conv_off,
                              const int* slots, const int* cu, const int* seq_index,
                              const int* positions, int several, float* qkv, float* beta,
                              void* low_a, void* low_g, cudaStream_t stream) {
    const DeltaDims dm{G, H, d, dv, taps, ra, rg};
    if (int rc = check_dims(dm)) return rc;
    AGV_REQUIRE(T >= 0 && B >= 0 && (row || part), "delta_prepare: no input");
    AGV_REQUIRE(state && conv_off >= (long long)H * dv * d &&
                state_stride >= conv_off + (long long)(taps - 1) * dm.C(),
                "delta_prepare: the state is too small");
    if (T == 0) return 0;
    const DeltaState st{state, state_stride, conv_off, slots, cu, seq_index, positions};
    const size_t smem = (size_t)dm.C() * sizeof(float);
#define AGV_DP(TT)                                                                              \
    do {                                                                                        \
        RowIn<TT> in{(const TT*)row, ld, part, n_splits, (long long)T * dm.W(), dm.W()};        \
        auto kern = delta_prepare_kernel<TT>;                                                   \
        if (smem > 48 * 1024)                                                                   \
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem));                                       \
        agv_launch(kern, (unsigned)T, 256, smem, stream, in, dm, st, conv_w, eps_unit, q_mult,  \
                   several ? 0 : 1, qkv, beta, (TT*)low_a, (TT*)low_g);                         \
        AGV_LAUNCH_OK("delta_prepare_kernel");                                                  \
        if (several && taps > 1) {                                                              \
            agv_launch(delta_conv_state_kernel<TT>, (unsigned)B, 256, 0, stream, in, dm, st);   \
            AGV_LAUNCH_OK("delta_conv_state_kernel");                                           \
        }                                                                                       \
    } while (0)
    AGV_REQUIRE(smem <= 200 * 1024, "delta_prepare: %d channels exceed shared memory", dm.C());
    if (dtype == AGV_F32) AGV_DP(float);
    else if (dtype == AGV_BF16) AGV_DP(__nv_bfloat16);
    else return agv_fail(-1, "delta_prepare: unknown dtype %d", dtype);
#undef AGV_DP
    return 0;
}

// The recurrence over the step's tokens, sequence by sequence; all tensors 32-bit.
AGV_API int agv_delta_scan(const float* qkv, const float* beta, const float* a,
                           const float* dt_bias, const float* neg_a, float* out, int T, int B,
                           int G, int H, int d, int dv, float* state, long long state_stride,
                           const int* slots, const int* cu, cudaStream_t stream) {
    const DeltaDims dm{G, H, d, dv, 1, 0, 0};
    if (int rc = check_dims(dm)) return rc;
    AGV_REQUIRE(state && state_stride >= (long long)H * dv * d, "delta_scan: the state is too small");
    AGV_REQUIRE(B <= 65535 && H <= 65535, "delta_scan: batch or head count exceeds the grid limit");
    if (T == 0 || B == 0) return 0;
    int L = 1;
    while (L * DL_R < d) L <<= 1;
    // 128 threads a CTA where the columns allow, whole warps always
    int CC = 128 / L;
    while (CC > 32 / L && CC / 2 >= dv) CC >>= 1;
    if (CC < 1) CC = 1;
    const int Dp = L * DL_R;
    int TCH = 16;
    while (TCH > 1 && (size_t)TCH * (3 * Dp + CC + 1) * sizeof(float) > 40 * 1024) TCH >>= 1;
    const size_t smem = (size_t)TCH * (3 * Dp + CC + 1) * sizeof(float);
    ScanArgs sa{qkv, beta, a, dt_bias, neg_a, out, L, CC, TCH};
    const DeltaState st{state, state_stride, 0, slots, cu, nullptr, nullptr};
    dim3 grid((unsigned)((dv + CC - 1) / CC), (unsigned)H, (unsigned)B);
    agv_launch(delta_scan_kernel, grid, (unsigned)(CC * L), smem, stream, sa, dm, st);
    AGV_LAUNCH_OK("delta_scan_kernel");
    return 0;
}

// o, gate: [T, H * dv] 32-bit; w: [dv] 32-bit; y: [T, H * dv] in dtype.
AGV_API int agv_delta_out(const float* o, const float* gate, const float* w, float eps, int T,
                          int H, int dv, const int* seq_index, const int* slots, void* y,
                          int dtype, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && H > 0 && dv > 0, "delta_out: bad sizes");
    if (T == 0) return 0;
    if (dtype == AGV_F32)
        agv_launch(delta_out_kernel<float>, (unsigned)T, 128, 0, stream, o, gate, w, eps, T, H, dv,
                   seq_index, slots, (float*)y);
    else if (dtype == AGV_BF16)
        agv_launch(delta_out_kernel<__nv_bfloat16>, (unsigned)T, 128, 0, stream, o, gate, w, eps, T,
                   H, dv, seq_index, slots, (__nv_bfloat16*)y);
    else
        return agv_fail(-1, "delta_out: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("delta_out_kernel");
    return 0;
}
