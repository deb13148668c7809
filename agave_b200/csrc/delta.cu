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
// The convolution's inputs of a sequence are a ring by position: the input of position pp is
// row pp % (taps - 1) of the slot's [taps - 1, C] block, so a step writes the rows of its own
// last taps - 1 positions and moves nothing.
//
// One CTA per token.  The token's row of the stacked product comes into shared memory first
// (all its loads in flight at once), earlier tokens of the same step are read in place.
// fused_state: the CTA's token is the only one its sequence brings (a decode step), so it
// also stores its inputs in the ring.
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
    const int C = dm.C(), nq = dm.nq(), taps = dm.taps, R = taps - 1;
    float* rowbuf = buf + C;                     // [W] the token's row, 32-bit
    const int p = st.positions[t];
    const int first = st.cu[b];                  // first token of the sequence in this step
    const int p0 = p - (t - first);              // its position
    in.load(t, rowbuf);
    {
        const float* __restrict__ cs = st.state + (size_t)slot * st.stride + st.conv_off;
#pragma unroll 4
        for (int c = threadIdx.x; c < C; c += blockDim.x) {
            const float* w = conv_w + (size_t)c * taps;
            float acc = 0.f;
            // oldest input first; input p - k meets weight taps - 1 - k
            for (int k = R; k >= 1; --k) {
                const int pp = p - k;
                float x = 0.f;
                if (pp >= p0) x = in.at(t - k, c);
                else if (pp >= 0) x = cs[(size_t)(pp % R) * C + c];
                acc = fmaf(w[R - k], x, acc);
            }
            buf[c] = silu_f(fmaf(w[R], rowbuf[c], acc));
        }
    }
    if (fused_state && R > 0) {
        // (the row of position p is the one position p - R had: read above by this thread)
        float* cs = st.state + (size_t)slot * st.stride + st.conv_off + (size_t)(p % R) * C;
        for (int c = threadIdx.x; c < C; c += blockDim.x) cs[c] = rowbuf[c];
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
        beta[(size_t)t * dm.H + h] = sigmoid_f(rowbuf[C + h]);
    for (int i = threadIdx.x; i < dm.ra; i += blockDim.x)
        low_a[(size_t)t * dm.ra + i] = from_f32<T>(rowbuf[C + dm.H + i]);
    for (int i = threadIdx.x; i < dm.rg; i += blockDim.x)
        low_g[(size_t)t * dm.rg + i] = from_f32<T>(rowbuf[C + dm.H + dm.ra + i]);
}

// The convolution's inputs after a step of several tokens a sequence: the step's last
// taps - 1 positions go to their rows of the ring (fewer, if the step is shorter: the rows of
// earlier positions stay).  One CTA per sequence, a thread a channel; it runs after the
// prepare kernel, which reads the inputs of before the step.
template <typename T>
__global__ void __launch_bounds__(256)
delta_conv_state_kernel(RowIn<T> in, DeltaDims dm, DeltaState st) {
    pdl_wait();
    pdl_launch_next();
    const int b = blockIdx.x;
    const int slot = st.slots[b];
    if (slot < 0) return;
    const int C = dm.C(), R = dm.taps - 1;
    const int first = st.cu[b], n = st.cu[b + 1] - first;
    if (n <= 0 || R <= 0) return;
    const int p0 = st.positions[first], len = p0 + n;
    const int from = len - R > p0 ? len - R : p0;
    float* cs = st.state + (size_t)slot * st.stride + st.conv_off;
    for (int c = threadIdx.x; c < C; c += blockDim.x)
        for (int pp = from; pp < len; ++pp)
            cs[(size_t)(pp % R) * C + c] = in.at(first + pp - p0, c);
}

// --------------------------------------------------------------------- scan
// grid (column groups, H, B); a CTA has CC columns of one head of one sequence, L lanes a
// column (L a power of two, L * 16 >= d), thread = column * L + lane.  The tokens of the
// sequence come through shared memory TCH at a time: k, q and the decay of the head's key
// channels (padded with zeros to L * 16 rows, which keeps the padded rows of S at zero), the
// CTA's columns of v, and beta.  L is a template parameter: the shuffle rounds are unrolled.
// A lane's 16 rows are four quads, quad i of lane l being rows (i * L + l) * 4 .. + 3: the
// lanes of a column then read consecutive 16 bytes of a token's row, free of bank conflicts
// (the columns of a warp read the same addresses).
struct ScanArgs {
    const float* qkv;          // [T, C]: q | k | v, prepared
    const float* beta;         // [T, H]
    const float* a;            // [T, H * d]: the decay's pre-activation, without its bias
    const float* dt_bias;      // [H * d]
    const float* neg_a;        // [H]: -exp(A_log)
    float* out;                // [T, H * dv]
    int L, CC, TCH;
    // what does not depend on the state, made by the launch before, [T, H, L * 16] each with
    // zeros in the padding, and k . q [T, H]
    float *wk, *wg, *wgk, *wgq, *wkq;
};

// What a token's step needs besides the state, for every head: k, the decay g = exp(neg_a *
// softplus(a + bias)), g * k, g * q and k . q.  A warp a (token, head); rows of Dp = L * 16
// floats, the padding zero, so that the scan copies them 16 bytes at a time.
__global__ void __launch_bounds__(256)
delta_decay_kernel(ScanArgs a, DeltaDims dm, int T, int Dp) {
    pdl_wait();
    pdl_launch_next();
    const int lane = threadIdx.x & 31;
    const long long w = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (w >= (long long)T * dm.H) return;
    const int t = (int)(w / dm.H), h = (int)(w - (long long)t * dm.H), g = h / (dm.H / dm.G);
    const int d = dm.d;
    const float* q = a.qkv + (size_t)t * dm.C() + (size_t)g * d;
    const float* k = q + dm.nq();
    const float* pre = a.a + ((size_t)t * dm.H + h) * d;
    const float* bias = a.dt_bias + (size_t)h * d;
    const float na = a.neg_a[h];
    const size_t o = (size_t)w * Dp;
    float s = 0.f;
    for (int r = lane; r < Dp; r += 32) {
        float kv = 0.f, gv = 0.f, qv = 0.f;
        if (r < d) {
            kv = k[r];
            qv = q[r];
            gv = expf(na * softplus_f(pre[r] + bias[r]));
        }
        a.wk[o + r] = kv;
        a.wg[o + r] = gv;
        a.wgk[o + r] = gv * kv;
        a.wgq[o + r] = gv * qv;
        s = fmaf(kv, qv, s);
    }
    s = warp_sum(s);
    if (lane == 0) a.wkq[w] = s;
}

// A 4-byte asynchronous copy into shared memory (the sources are rows of 32-bit tensors at
// offsets that need not be multiples of 16 bytes).
__device__ __forceinline__ void cp_async_f32(float* dst, const float* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;"
                 :: "r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_16(float* dst, const float* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;"
                 :: "r"((unsigned)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" :: "n"(N) : "memory"); }

// The tokens come through two buffers: while the lanes run the recurrence over one, the next
// TCH tokens' k, q, decay pre-activation, v and beta are on their way (asynchronous copies),
// so the trip to L2 or HBM is paid once a sequence, not once a buffer.  What does not depend
// on the state was made by the launch before for all tokens at once: the decay g, g * k,
// g * q and the token's k . q.  With them a token is one round of dot products,
//
//      a = (g S)^T k = sum_r S_r (g k)_r      r = (g S)^T q = sum_r S_r (g q)_r
//      u = beta (v - a);    o = r + (k . q) u;    S <- g S + k u
//
// the same sums as  S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q  with the
// read-out split into the part the state had and the token's own write: one round of
// shuffles a token instead of two, and the state's update off the output's path.
struct ScanBuf {
    float *k, *gk, *gq, *g, *v, *beta, *kq;
    __device__ ScanBuf(float* base, int TCH, int Dp, int CC) {
        k = base;
        gk = k + (size_t)TCH * Dp;       // (q arrives in gq's place, the pre-activation in g's)
        gq = gk + (size_t)TCH * Dp;
        g = gq + (size_t)TCH * Dp;
        v = g + (size_t)TCH * Dp;
        beta = v + (size_t)TCH * CC;
        kq = beta + TCH;
    }
};
__host__ __device__ inline size_t scan_buf_floats(int TCH, int Dp, int CC) {
    return ((size_t)TCH * (4 * Dp + CC + 2) + 3) / 4 * 4;      // (16-byte rows in the next buffer)
}

template <int L>
__global__ void __launch_bounds__(256)
delta_scan_kernel(ScanArgs a, DeltaDims dm, DeltaState st) {
    pdl_wait();
    extern __shared__ float smem[];
    const int b = blockIdx.z;
    const int slot = st.slots[b];
    if (slot < 0) return;
    const int t0 = st.cu[b], n = st.cu[b + 1] - t0;
    if (n <= 0) return;
    const int h = blockIdx.y;
    const int d = dm.d, dv = dm.dv, C = dm.C(), nq = dm.nq();
    constexpr int Dp = L * DL_R;
    const int CC = a.CC, TCH = a.TCH;
    const int l = threadIdx.x & (L - 1);
    const int jc = threadIdx.x / L;
    const int j = blockIdx.x * CC + jc;
    const bool live = jc < CC && j < dv;
    const size_t per = scan_buf_floats(TCH, Dp, CC);
    // (columns of v past dv are never copied: zero them once)
    for (size_t i = threadIdx.x; i < 2 * per; i += blockDim.x) smem[i] = 0.f;
    __syncthreads();

    auto fetch = [&](int c0, float* base) {
        const int m = min(TCH, n - c0);
        const ScanBuf sb(base, TCH, Dp, CC);
        // rows of Dp floats a token: tokens of a head lie H * Dp apart
        constexpr int Q = Dp / 4;
        for (int idx = threadIdx.x; idx < m * Q; idx += blockDim.x) {
            const int tt = idx / Q, c4 = (idx - tt * Q) * 4;
            const size_t src = ((size_t)(t0 + c0 + tt) * dm.H + h) * Dp + c4;
            const int dst = tt * Dp + c4;
            cp_async_16(sb.k + dst, a.wk + src);
            cp_async_16(sb.g + dst, a.wg + src);
            cp_async_16(sb.gk + dst, a.wgk + src);
            cp_async_16(sb.gq + dst, a.wgq + src);
        }
        for (int idx = threadIdx.x; idx < m * CC; idx += blockDim.x) {
            const int tt = idx / CC, c = idx - tt * CC;
            const int col = blockIdx.x * CC + c;
            if (col < dv)
                cp_async_f32(sb.v + idx, a.qkv + (size_t)(t0 + c0 + tt) * C + 2 * nq + (size_t)h * dv + col);
        }
        for (int tt = threadIdx.x; tt < m; tt += blockDim.x) {
            cp_async_f32(sb.beta + tt, a.beta + (size_t)(t0 + c0 + tt) * dm.H + h);
            cp_async_f32(sb.kq + tt, a.wkq + (size_t)(t0 + c0 + tt) * dm.H + h);
        }
        cp_async_commit();
    };

    float S[DL_R];
    float* srow = st.state + (size_t)slot * st.stride + ((size_t)h * dv + (live ? j : 0)) * d;
    fetch(0, smem);
#pragma unroll
    for (int i = 0; i < DL_R; ++i) {
        const int r = ((i >> 2) * L + l) * 4 + (i & 3);
        S[i] = live && r < d ? srow[r] : 0.f;
    }
    int cur = 0;
    for (int c0 = 0; c0 < n; c0 += TCH, cur ^= 1) {
        const int m = min(TCH, n - c0);
        const ScanBuf sb(smem + (size_t)cur * per, TCH, Dp, CC);
        // (the other buffer was read in the round before, which ended with a barrier)
        if (c0 + TCH < n) {
            fetch(c0 + TCH, smem + (size_t)(cur ^ 1) * per);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const float* pk = sb.k + l * 4;
        const float* pgk = sb.gk + l * 4;
        const float* pgq = sb.gq + l * 4;
        const float* pg = sb.g + l * 4;
        const float* pv = sb.v + (jc < CC ? jc : 0);
        float* po = a.out + (size_t)(t0 + c0) * dm.H * dv + (size_t)h * dv + (live ? j : 0);
#pragma unroll 2
        for (int tt = 0; tt < m; ++tt) {
            float gk[DL_R], gq[DL_R], kk[DL_R], gg[DL_R];
#pragma unroll
            for (int i = 0; i < DL_R / 4; ++i) {
                const float4 x = reinterpret_cast<const float4*>(pgk)[i * L];
                const float4 y = reinterpret_cast<const float4*>(pgq)[i * L];
                gk[4 * i] = x.x; gk[4 * i + 1] = x.y; gk[4 * i + 2] = x.z; gk[4 * i + 3] = x.w;
                gq[4 * i] = y.x; gq[4 * i + 1] = y.y; gq[4 * i + 2] = y.z; gq[4 * i + 3] = y.w;
            }
            float ac[4] = {0.f, 0.f, 0.f, 0.f}, rc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int i = 0; i < DL_R; ++i) {
                ac[i & 3] = fmaf(S[i], gk[i], ac[i & 3]);
                rc[i & 3] = fmaf(S[i], gq[i], rc[i & 3]);
            }
#pragma unroll
            for (int i = 0; i < DL_R / 4; ++i) {
                const float4 x = reinterpret_cast<const float4*>(pk)[i * L];
                const float4 y = reinterpret_cast<const float4*>(pg)[i * L];
                kk[4 * i] = x.x; kk[4 * i + 1] = x.y; kk[4 * i + 2] = x.z; kk[4 * i + 3] = x.w;
                gg[4 * i] = y.x; gg[4 * i + 1] = y.y; gg[4 * i + 2] = y.z; gg[4 * i + 3] = y.w;
            }
            float acc = (ac[0] + ac[1]) + (ac[2] + ac[3]);
            float rr = (rc[0] + rc[1]) + (rc[2] + rc[3]);
#pragma unroll
            for (int o = 1; o < L; o <<= 1) {
                acc += __shfl_xor_sync(0xffffffffu, acc, o);
                rr += __shfl_xor_sync(0xffffffffu, rr, o);
            }
#pragma unroll
            for (int i = 0; i < DL_R; ++i) gg[i] *= S[i];          // g S: needs no u
            const float u = sb.beta[tt] * (*pv - acc);
            if (live && l == 0) *po = fmaf(sb.kq[tt], u, rr);
#pragma unroll
            for (int i = 0; i < DL_R; ++i) S[i] = fmaf(kk[i], u, gg[i]);
            pk += Dp; pgk += Dp; pgq += Dp; pg += Dp; pv += CC;
            po += (size_t)dm.H * dv;
        }
        __syncthreads();
    }
    pdl_launch_next();
    if (live) {
#pragma unroll
        for (int i = 0; i < DL_R; ++i) {
            const int r = ((i >> 2) * L + l) * 4 + (i & 3);
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
// state_stride] 32-bit, the convolution's inputs [taps - 1, 2 G d + H dv] at conv_off (a ring:
// position pp in row pp % (taps - 1)).
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
    const size_t smem = (size_t)(dm.C() + dm.W()) * sizeof(float);
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
// work: scratch of agv_delta_scan_work(T, H, d) floats.
AGV_API long long agv_delta_scan_work(int T, int H, int d) {
    int L = 1;
    while (L * DL_R < d) L <<= 1;
    return (long long)T * H * (4LL * L * DL_R + 1);
}

AGV_API int agv_delta_scan(const float* qkv, const float* beta, const float* a,
                           const float* dt_bias, const float* neg_a, float* out, int T, int B,
                           int G, int H, int d, int dv, float* state, long long state_stride,
                           const int* slots, const int* cu, float* work, cudaStream_t stream) {
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
    // two buffers of TCH tokens and the decay's bias, within the 48 KB every launch may have
    int TCH = T <= B ? 1 : 16;             // (a decode step brings a token a sequence)
    while (TCH > 1 && 2 * scan_buf_floats(TCH, Dp, CC) * sizeof(float) > 46 * 1024) TCH >>= 1;
    const size_t smem = 2 * scan_buf_floats(TCH, Dp, CC) * sizeof(float);
    AGV_REQUIRE(smem <= 48 * 1024, "delta_scan: key heads of %d need too much shared memory", d);
    AGV_REQUIRE(work && ((size_t)work & 15) == 0, "delta_scan: no scratch, or not 16-byte aligned");
    const size_t row = (size_t)T * H * Dp;
    ScanArgs sa{qkv, beta, a, dt_bias, neg_a, out, L, CC, TCH,
                work, work + row, work + 2 * row, work + 3 * row, work + 4 * row};
    {
        const long long warps = (long long)T * H;
        agv_launch(delta_decay_kernel, (unsigned)((warps + 7) / 8), 256, 0, stream, sa, dm, T, Dp);
        AGV_LAUNCH_OK("delta_decay_kernel");
    }
    const DeltaState st{state, state_stride, 0, slots, cu, nullptr, nullptr};
    dim3 grid((unsigned)((dv + CC - 1) / CC), (unsigned)H, (unsigned)B);
    switch (L) {
#define AGV_SCAN(LL) case LL: agv_launch_after(delta_scan_kernel<LL>, grid, (unsigned)(CC * L), smem, \
                                               stream, sa, dm, st); break
        AGV_SCAN(1); AGV_SCAN(2); AGV_SCAN(4); AGV_SCAN(8); AGV_SCAN(16); AGV_SCAN(32);
#undef AGV_SCAN
        default: return agv_fail(-1, "delta_scan: %d lanes a column", L);
    }
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
