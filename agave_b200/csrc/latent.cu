// What a mixer does to a token's row of a stacked projection before it attends, for two
// kinds of mixer that the per-head q/k norm kernel does not cover, and the small products
// and element-wise steps of latent attention.
//
//  * whole-projection norm (agv_proj_norm_store): the row is q | k | v; q and k are each
//    RMS-normed over their WHOLE width (all heads at once, a weight of that width), v is
//    taken as it is or, with v_first [T, nv] and a weight m, as (1 - m) v + m v_first (the
//    values of an earlier layer for the same tokens, mixed in 32-bit before the one
//    rounding); k and v go to the paged cache.
//  * latent attention (agv_latent_prepare): the row is Q | c | kr | g.  c (the key/value
//    latent) is RMS-normed, kr (one rotated key part shared by all heads) is rotated by
//    position, and c | kr is the cache row of the position.  Q is either the queries
//    themselves, [heads, d + r] with the last r of every head rotated, or a query latent
//    that is RMS-normed (the queries then come from one more product and are rotated by
//    agv_rotate_heads).  g (gate logits) is passed through.
//  * agv_heads_linear: out[t, a, :] = W[a] x[t, a, :] for every head a (absorbing the
//    key up-projection into the query, and the value up-projection after the attention).
//  * agv_gate_sigmoid: out[t, i] *= sigmoid(g[t, i / per]).
//  * agv_relu2: z <- max(z, 0)^2.
//  * agv_rope_table_freqs: cos / sin tables from a list of frequencies and a multiplier.
//
// Rotation pairs are (i, i + r/2) or, interleaved, (2i, 2i + 1); the pair (u, v) becomes
// (u cos - v sin, v cos + u sin).  Norm statistics, sums over partial products, angles and
// the sigmoid are 32-bit whatever the row's dtype.
#include "common.cuh"
#include "cache_write.cuh"
#include "row_in.cuh"

namespace {

// Cache row of token t, or null when nothing is stored for it (padding, or a ring row that
// a later token of the same step overwrites).
template <typename T>
__device__ __forceinline__ T* cache_row(void* pool, const CacheWrite& cw, int t, int p,
                                        int row_width) {
    if (!pool) return nullptr;
    const int b = cw.seq_index[t];
    const int slot = cw.slots[b];
    if (slot < 0) return nullptr;
    if (p < cw.lens[b] - cw.cap) return nullptr;
    const int r = p % cw.cap;
    const int page = cw.page_table[(size_t)slot * cw.max_pages + r / cw.page];
    return (T*)pool + ((size_t)page * cw.page + r % cw.page) * row_width;
}

__device__ __forceinline__ void rotate_pair(float u, float v, float c, float s, float& ou,
                                            float& ov) {
    ou = u * c - v * s;
    ov = v * c + u * s;
}

// ------------------------------------------------------- whole-projection norm
template <typename T>
__global__ void __launch_bounds__(1024)
proj_norm_store_kernel(RowIn<T> in, T* __restrict__ out, long long ldo, int n_tokens, int nq,
                       int nk, int nv, const float* __restrict__ wq, const float* __restrict__ wk,
                       float eps, const int* __restrict__ positions, CacheWrite cw,
                       const T* __restrict__ v_first, long long ldvf, float v_mix) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float buf[];           // the row, 32-bit
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int W = nq + nk + nv;
    float sq = 0.f, sk = 0.f;
    in.load(t, buf);
    for (int e = threadIdx.x; e < nq + nk; e += blockDim.x) {
        const float v = buf[e];
        if (e < nq) sq += v * v;
        else sk += v * v;
    }
    const float rq = 1.0f / sqrtf(block_sum(sq, red) / (float)nq + eps);
    const float rk = 1.0f / sqrtf(block_sum(sk, red) / (float)nk + eps);
    const int p = positions[t];
    T* kc = cache_row<T>(cw.k_pool, cw, t, p, nk);
    T* vc = cache_row<T>(cw.v_pool, cw, t, p, nv);
    T* o = out + (size_t)t * ldo;
    for (int e = threadIdx.x; e < W; e += blockDim.x) {
        float v = buf[e];
        if (e < nq) v = v * rq * wq[e];
        else if (e < nq + nk) v = v * rk * wk[e - nq];
        else if (v_first)      // the values lean towards an earlier layer's of the same token
            v = (1.0f - v_mix) * v + v_mix * to_f32(v_first[(size_t)t * ldvf + e - nq - nk]);
        const T r = from_f32<T>(v);
        o[e] = r;
        if (e >= nq + nk) { if (vc) vc[e - nq - nk] = r; }
        else if (e >= nq) { if (kc) kc[e - nq] = r; }
    }
}

// ------------------------------------------------------------ latent prepare
template <typename T>
__global__ void __launch_bounds__(1024)
latent_prepare_kernel(RowIn<T> in, T* __restrict__ out, long long ldo, int n_tokens, int q_width,
                      int q_latent, int heads, int d, int r, int R, int G,
                      const float* __restrict__ w_q, const float* __restrict__ w_c, float eps,
                      const float* __restrict__ cosv, const float* __restrict__ sinv,
                      int interleaved, const int* __restrict__ positions, CacheWrite cw) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float buf[];
    __shared__ float red[33];
    const int t = blockIdx.x;
    const int c_at = q_width, kr_at = q_width + R, g_at = q_width + R + r;
    float sq = 0.f, sc = 0.f;
    in.load(t, buf);
    for (int e = threadIdx.x; e < kr_at; e += blockDim.x) {
        const float v = buf[e];
        if (e < q_width) sq += v * v;
        else sc += v * v;
    }
    float rq = 1.f;
    if (q_latent) rq = 1.0f / sqrtf(block_sum(sq, red) / (float)q_width + eps);
    const float rc = 1.0f / sqrtf(block_sum(sc, red) / (float)R + eps);
    const int p = positions[t];
    const int half = r / 2;
    const float* cs = cosv + (size_t)t * half;
    const float* sn = sinv + (size_t)t * half;
    T* kc = cache_row<T>(cw.k_pool, cw, t, p, R + r);
    T* o = out + (size_t)t * ldo;
    // queries
    if (q_latent) {
        for (int e = threadIdx.x; e < q_width; e += blockDim.x)
            o[e] = from_f32<T>(buf[e] * rq * w_q[e]);
    } else {
        const int hw = d + r;
        for (int e = threadIdx.x; e < heads * d; e += blockDim.x) {
            const int a = e / d, i = e % d;
            o[a * hw + i] = from_f32<T>(buf[a * hw + i]);
        }
        for (int e = threadIdx.x; e < heads * half; e += blockDim.x) {
            const int a = e / half, i = e % half;
            const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
            float u, v;
            rotate_pair(buf[a * hw + d + iu], buf[a * hw + d + iv], cs[i], sn[i], u, v);
            o[a * hw + d + iu] = from_f32<T>(u);
            o[a * hw + d + iv] = from_f32<T>(v);
        }
    }
    // the latent and the shared rotated key part; together they are the cache row
    for (int e = threadIdx.x; e < R; e += blockDim.x) {
        const T v = from_f32<T>(buf[c_at + e] * rc * w_c[e]);
        o[c_at + e] = v;
        if (kc) kc[e] = v;
    }
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
        float u, v;
        rotate_pair(buf[kr_at + iu], buf[kr_at + iv], cs[i], sn[i], u, v);
        const T tu = from_f32<T>(u), tv = from_f32<T>(v);
        o[kr_at + iu] = tu;
        o[kr_at + iv] = tv;
        if (kc) { kc[R + iu] = tu; kc[R + iv] = tv; }
    }
    for (int e = threadIdx.x; e < G; e += blockDim.x) o[g_at + e] = from_f32<T>(buf[g_at + e]);
}

// x [T, heads, hw] (row stride ld): the last r of every head rotated in place.
template <typename T>
__global__ void rotate_heads_kernel(T* __restrict__ x, long long ld, int n_tokens, int heads,
                                    int hw, int r, const float* __restrict__ cosv,
                                    const float* __restrict__ sinv, int interleaved) {
    pdl_wait();
    pdl_launch_next();
    const int half = r / 2;
    const long long n = (long long)n_tokens * heads * half;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % half);
        const int a = (int)((idx / half) % heads);
        const int t = (int)(idx / ((long long)half * heads));
        T* h = x + (size_t)t * ld + (size_t)a * hw + (hw - r);
        const int iu = interleaved ? 2 * i : i, iv = interleaved ? 2 * i + 1 : i + half;
        float u, v;
        rotate_pair(to_f32(h[iu]), to_f32(h[iv]), cosv[(size_t)t * half + i],
                    sinv[(size_t)t * half + i], u, v);
        h[iu] = from_f32<T>(u);
        h[iv] = from_f32<T>(v);
    }
}

// k_out [T, heads, d + r]: head a is k_plain[t, a, :d] followed by kr[t, :r] (the rotated part
// every head shares); k_plain has row stride ldp, kr row stride ldr.
template <typename T>
__global__ void assemble_keys_kernel(const T* __restrict__ k_plain, long long ldp,
                                     const T* __restrict__ kr, long long ldr,
                                     T* __restrict__ k_out, int n_tokens, int heads, int d, int r) {
    pdl_wait();
    pdl_launch_next();
    const int hw = d + r;
    const long long n = (long long)n_tokens * heads * hw;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % hw);
        const int a = (int)((idx / hw) % heads);
        const long long t = idx / ((long long)hw * heads);
        k_out[idx] = i < d ? k_plain[t * ldp + (size_t)a * d + i] : kr[t * ldr + (i - d)];
    }
}

// --------------------------------------------------------- per-head products
constexpr int HL_TOK = 8;      // tokens a CTA keeps in shared memory
constexpr int HL_WARPS = 8;

// out[t, a, n] = sum_k W[a, n, k] x[t, a, k].  One warp per output row n of a head, lanes
// over k (coalesced weight reads), HL_TOK tokens at a time from shared memory.
template <typename T, typename TO>
__global__ void __launch_bounds__(HL_WARPS * 32)
heads_linear_kernel(const T* __restrict__ x, long long ldx, long long xs, const T* __restrict__ W,
                    TO* __restrict__ out, long long ldo, long long os, int n_tokens, int N, int K,
                    int rows_per_cta, int tail, const T* __restrict__ gate, long long ldg,
                    int gate_per_head) {
    extern __shared__ float xsh[];           // [HL_TOK, K]
    const int a = blockIdx.y;
    const int t0 = blockIdx.z * HL_TOK;
    const int nt = min(HL_TOK, n_tokens - t0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_wait();
    pdl_launch_next();
    for (int e = threadIdx.x; e < nt * K; e += blockDim.x) {
        const int tt = e / K, k = e % K;
        xsh[e] = to_f32(x[(size_t)(t0 + tt) * ldx + (size_t)a * xs + k]);
    }
    __syncthreads();
    // the values that follow a head's K inputs pass through to behind its N outputs
    if (tail > 0 && blockIdx.x == 0)
        for (int e = threadIdx.x; e < nt * tail; e += blockDim.x) {
            const int tt = e / tail, i = e % tail;
            out[(size_t)(t0 + tt) * ldo + (size_t)a * os + N + i] =
                from_f32<TO>(to_f32(x[(size_t)(t0 + tt) * ldx + (size_t)a * xs + K + i]));
        }
    const int n_lo = blockIdx.x * rows_per_cta;
    const int n_hi = min(N, n_lo + rows_per_cta);
    for (int n = n_lo + warp; n < n_hi; n += HL_WARPS) {
        const T* w = W + ((size_t)a * N + n) * K;
        float acc[HL_TOK];
#pragma unroll
        for (int tt = 0; tt < HL_TOK; ++tt) acc[tt] = 0.f;
        for (int k = lane; k < K; k += 32) {
            const float wv = to_f32(w[k]);
#pragma unroll
            for (int tt = 0; tt < HL_TOK; ++tt)
                if (tt < nt) acc[tt] = fmaf(wv, xsh[tt * K + k], acc[tt]);
        }
#pragma unroll
        for (int tt = 0; tt < HL_TOK; ++tt) {
            if (tt < nt) {
                float s = warp_sum(acc[tt]);
                if (lane == 0) {
                    if (gate) {
                        // an output gate: sigmoid of one logit per head, or per output value
                        const float z = to_f32(gate[(size_t)(t0 + tt) * ldg +
                                                    (gate_per_head ? a : a * N + n)]);
                        s /= 1.0f + expf(-z);
                    }
                    out[(size_t)(t0 + tt) * ldo + (size_t)a * os + n] = from_f32<TO>(s);
                }
            }
        }
    }
}

template <typename T>
__global__ void gate_sigmoid_kernel(T* __restrict__ out, long long ldo, const T* __restrict__ g,
                                    long long ldg, int n_tokens, int width, int per) {
    pdl_wait();
    pdl_launch_next();
    const long long n = (long long)n_tokens * width;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const int i = (int)(idx % width);
        const long long t = idx / width;
        const float z = to_f32(g[t * ldg + i / per]);
        T* o = out + t * ldo + i;
        *o = from_f32<T>(to_f32(*o) / (1.0f + expf(-z)));
    }
}

// The same in 16-byte pieces of eight bfloat16 values: a logit per value (per == 1) or per
// `per` values with per a multiple of 8; width and both strides multiples of 8.
__global__ void gate_sigmoid_bf16x8_kernel(__nv_bfloat16* __restrict__ out, long long ldo,
                                           const __nv_bfloat16* __restrict__ g, long long ldg,
                                           int n_tokens, int width, int per) {
    pdl_wait();
    pdl_launch_next();
    const int cpr = width / 8;
    const long long n = (long long)n_tokens * cpr;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / cpr;
        const int c = (int)(idx - t * cpr) * 8;
        uint4 ov = *reinterpret_cast<const uint4*>(out + t * ldo + c);
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
        float z[8];
        if (per == 1) {
            const uint4 gv = *reinterpret_cast<const uint4*>(g + t * ldg + c);
            const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float2 f = __bfloat1622float2(g2[i]);
                z[2 * i] = f.x;
                z[2 * i + 1] = f.y;
            }
        } else {
            const float zz = __bfloat162float(g[t * ldg + c / per]);
#pragma unroll
            for (int i = 0; i < 8; ++i) z[i] = zz;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(o2[i]);
            f.x = f.x / (1.0f + __expf(-z[2 * i]));
            f.y = f.y / (1.0f + __expf(-z[2 * i + 1]));
            o2[i] = __floats2bfloat162_rn(f.x, f.y);
        }
        *reinterpret_cast<uint4*>(out + t * ldo + c) = ov;
    }
}

// Key assembly in 16-byte pieces: d, r and both strides multiples of 8 (bfloat16).
__global__ void assemble_keys_bf16x8_kernel(const __nv_bfloat16* __restrict__ k_plain,
                                            long long ldp, const __nv_bfloat16* __restrict__ kr,
                                            long long ldr, __nv_bfloat16* __restrict__ k_out,
                                            int n_tokens, int heads, int d, int r) {
    pdl_wait();
    pdl_launch_next();
    const int cph = (d + r) / 8, cpr = heads * cph;
    const long long n = (long long)n_tokens * cpr;
    for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long t = idx / cpr;
        const int rem = (int)(idx - t * cpr);
        const int a = rem / cph, i = (rem - a * cph) * 8;
        const __nv_bfloat16* src = i < d ? k_plain + t * ldp + (size_t)a * d + i
                                         : kr + t * ldr + (i - d);
        *reinterpret_cast<uint4*>(k_out + idx * 8) = *reinterpret_cast<const uint4*>(src);
    }
}

template <typename T>
__global__ void relu2_kernel(T* __restrict__ z, long long n) {
    pdl_wait();
    pdl_launch_next();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float v = fmaxf(to_f32(z[i]), 0.f);
        z[i] = from_f32<T>(v * v);
    }
}

__global__ void rope_table_freqs_kernel(const int* __restrict__ positions,
                                        const double* __restrict__ freqs, float* __restrict__ cosv,
                                        float* __restrict__ sinv, int T, int half, double mult) {
    pdl_wait();
    pdl_launch_next();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= T * half) return;
    const int t = idx / half, i = idx % half;
    double s, c;
    sincos((double)positions[t] * freqs[i], &s, &c);
    cosv[idx] = (float)(c * mult);
    sinv[idx] = (float)(s * mult);
}

// Threads of a one-CTA-per-token kernel: a decode step has few tokens, and what hides a
// load's latency there is more threads per row; a prompt has rows enough.
int row_threads(int T) { return T <= 64 ? 1024 : 256; }

unsigned flat_grid(long long n, int threads) {
    long long b = (n + threads - 1) / threads;
    if (b > 148 * 32) b = 148 * 32;
    return (unsigned)(b < 1 ? 1 : b);
}

}  // namespace

// cos, sin [T, half] = mult * cos / sin(position * freqs[i]); freqs: 64-bit, on the device.
AGV_API int agv_rope_table_freqs(const int* positions, const double* freqs, float* cosv,
                                 float* sinv, int T, int half, double mult, cudaStream_t stream) {
    AGV_REQUIRE(half > 0 && freqs, "rope_table_freqs: needs frequencies");
    if (T == 0) return 0;
    const int n = T * half;
    agv_launch(rope_table_freqs_kernel, (n + 127) / 128, 128, 0, stream, positions, freqs, cosv,
               sinv, T, half, mult);
    AGV_LAUNCH_OK("rope_table_freqs_kernel");
    return 0;
}

// row: [T, W] with row stride ld (dtype), or part: [n_splits, T, W] 32-bit partial sums
// (row may then be null).  out: [T, W] with row stride ldo (may be row itself).  W = nq + nk
// + nv.  wq [nq], wk [nk]: 32-bit.  Pools (may be null): rows of nk and nv elements.
// v_first (may be null): [T, nv] with row stride ldvf, in the row's dtype; v_mix its weight.
AGV_API int agv_proj_norm_store(const void* row, long long ld, const float* part, int n_splits,
                                void* out, long long ldo, int dtype, int T, int nq, int nk, int nv,
                                const float* wq, const float* wk, float eps, const int* positions,
                                void* k_pool, void* v_pool, const int* page_table,
                                const int* slots, const int* lens, const int* seq_index,
                                int max_pages, int page, int cap, const void* v_first,
                                long long ldvf, float v_mix, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && nq > 0 && nk >= 0 && nv >= 0, "proj_norm: bad sizes");
    AGV_REQUIRE(!v_first || (ldvf >= nv && v_first != out), "proj_norm: the values to mix in need "
                "rows of their own, at least as wide as the values");
    AGV_REQUIRE(row || part, "proj_norm: no input");
    AGV_REQUIRE(wq && (nk == 0 || wk), "proj_norm: norm weights are missing");
    AGV_REQUIRE(!k_pool || (page_table && slots && lens && seq_index && page > 0 && cap > 0),
                "proj_norm: a cache store needs the page table and the step arrays");
    const int W = nq + nk + nv;
    AGV_REQUIRE(ld >= W || !row, "proj_norm: row stride shorter than the row");
    AGV_REQUIRE((size_t)W * 4 <= 200 * 1024, "proj_norm: rows of %d values do not fit", W);
    if (T == 0) return 0;
    CacheWrite cw{k_pool, v_pool, page_table, slots, lens, seq_index, max_pages, page, cap};
    const size_t smem = (size_t)W * 4;
#define AGV_PN(TT)                                                                              \
    do {                                                                                        \
        RowIn<TT> in{(const TT*)row, ld, part, n_splits, (long long)T * W, W};                  \
        auto kern = proj_norm_store_kernel<TT>;                                                 \
        if (smem > 48 * 1024)                                                                   \
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem));                                       \
        agv_launch(kern, (unsigned)T, row_threads(T), smem, stream, in, (TT*)out, ldo, T, nq,   \
                   nk, nv, wq, wk, eps, positions, cw, (const TT*)v_first, ldvf, v_mix);        \
    } while (0)
    if (dtype == AGV_F32) AGV_PN(float);
    else if (dtype == AGV_BF16) AGV_PN(__nv_bfloat16);
    else return agv_fail(-1, "proj_norm: unknown dtype %d", dtype);
#undef AGV_PN
    AGV_LAUNCH_OK("proj_norm_store_kernel");
    return 0;
}

// The row is Q (q_width) | c (R) | kr (r) | g (G); see the head of this file.  q_latent != 0:
// Q is a latent normed with w_q [q_width]; else Q is [heads, d + r] and q_width = heads * (d + r).
// k_pool (may be null): cache rows of R + r elements.
AGV_API int agv_latent_prepare(const void* row, long long ld, const float* part, int n_splits,
                               void* out, long long ldo, int dtype, int T, int q_width,
                               int q_latent, int heads, int d, int r, int R, int G,
                               const float* w_q, const float* w_c, float eps, const float* cosv,
                               const float* sinv, int interleaved, const int* positions,
                               void* k_pool, const int* page_table, const int* slots,
                               const int* lens, const int* seq_index, int max_pages, int page,
                               int cap, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && q_width > 0 && R > 0 && r >= 0 && G >= 0 && r % 2 == 0,
                "latent_prepare: bad sizes");
    AGV_REQUIRE(row || part, "latent_prepare: no input");
    AGV_REQUIRE(q_latent ? w_q != nullptr : q_width == heads * (d + r),
                "latent_prepare: the query part does not fit its description");
    AGV_REQUIRE(w_c && (r == 0 || (cosv && sinv)), "latent_prepare: weights or tables missing");
    AGV_REQUIRE(!k_pool || (page_table && slots && lens && seq_index && page > 0 && cap > 0),
                "latent_prepare: a cache store needs the page table and the step arrays");
    const int W = q_width + R + r + G;
    AGV_REQUIRE(ld >= W || !row, "latent_prepare: row stride shorter than the row");
    AGV_REQUIRE((size_t)W * 4 <= 200 * 1024, "latent_prepare: rows of %d values do not fit", W);
    if (T == 0) return 0;
    CacheWrite cw{k_pool, nullptr, page_table, slots, lens, seq_index, max_pages, page, cap};
    const size_t smem = (size_t)W * 4;
#define AGV_LP(TT)                                                                              \
    do {                                                                                        \
        RowIn<TT> in{(const TT*)row, ld, part, n_splits, (long long)T * W, W};                  \
        auto kern = latent_prepare_kernel<TT>;                                                  \
        if (smem > 48 * 1024)                                                                   \
            AGV_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                             (int)smem));                                       \
        agv_launch(kern, (unsigned)T, row_threads(T), smem, stream, in, (TT*)out, ldo, T,       \
                   q_width, q_latent, heads, d, r, R, G, w_q, w_c, eps, cosv, sinv,             \
                   interleaved, positions, cw);                                                 \
    } while (0)
    if (dtype == AGV_F32) AGV_LP(float);
    else if (dtype == AGV_BF16) AGV_LP(__nv_bfloat16);
    else return agv_fail(-1, "latent_prepare: unknown dtype %d", dtype);
#undef AGV_LP
    AGV_LAUNCH_OK("latent_prepare_kernel");
    return 0;
}

AGV_API int agv_rotate_heads(void* x, long long ld, int dtype, int T, int heads, int hw, int r,
                             const float* cosv, const float* sinv, int interleaved,
                             cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && heads > 0 && r >= 0 && r % 2 == 0 && r <= hw, "rotate_heads: bad sizes");
    if (T == 0 || r == 0) return 0;
    const long long n = (long long)T * heads * (r / 2);
    if (dtype == AGV_F32)
        agv_launch(rotate_heads_kernel<float>, flat_grid(n, 256), 256, 0, stream, (float*)x, ld, T,
                   heads, hw, r, cosv, sinv, interleaved);
    else if (dtype == AGV_BF16)
        agv_launch(rotate_heads_kernel<__nv_bfloat16>, flat_grid(n, 256), 256, 0, stream,
                   (__nv_bfloat16*)x, ld, T, heads, hw, r, cosv, sinv, interleaved);
    else return agv_fail(-1, "rotate_heads: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("rotate_heads_kernel");
    return 0;
}

AGV_API int agv_assemble_keys(const void* k_plain, long long ldp, const void* kr, long long ldr,
                              void* k_out, int dtype, int T, int heads, int d, int r,
                              cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && heads > 0 && d > 0 && r >= 0, "assemble_keys: bad sizes");
    if (T == 0) return 0;
    const long long n = (long long)T * heads * (d + r);
    if (dtype == AGV_F32)
        agv_launch(assemble_keys_kernel<float>, flat_grid(n, 256), 256, 0, stream,
                   (const float*)k_plain, ldp, (const float*)kr, ldr, (float*)k_out, T, heads, d, r);
    else if (dtype == AGV_BF16 && d % 8 == 0 && r % 8 == 0 && ldp % 8 == 0 && ldr % 8 == 0 &&
             agv_aligned(k_plain, 16) && agv_aligned(kr, 16) && agv_aligned(k_out, 16))
        agv_launch(assemble_keys_bf16x8_kernel, flat_grid(n / 8, 256), 256, 0, stream,
                   (const __nv_bfloat16*)k_plain, ldp, (const __nv_bfloat16*)kr, ldr,
                   (__nv_bfloat16*)k_out, T, heads, d, r);
    else if (dtype == AGV_BF16)
        agv_launch(assemble_keys_kernel<__nv_bfloat16>, flat_grid(n, 256), 256, 0, stream,
                   (const __nv_bfloat16*)k_plain, ldp, (const __nv_bfloat16*)kr, ldr,
                   (__nv_bfloat16*)k_out, T, heads, d, r);
    else return agv_fail(-1, "assemble_keys: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("assemble_keys_kernel");
    return 0;
}

// x: [T, heads, K] (row stride ldx, head stride xs); W: [heads, N, K] dense; out: [T, heads, N]
// (row stride ldo, head stride os), in dtype or, with out_f32, 32-bit.  tail > 0: the tail
// values x[t, a, K .. K + tail) are copied to out[t, a, N .. N + tail).  gate (may be null):
// logits [T, heads] (gate_per_head) or [T, heads * N] with row stride ldg; an output is
// multiplied by the sigmoid of its logit.
AGV_API int agv_heads_linear(const void* x, long long ldx, long long xs, const void* W, void* out,
                             long long ldo, long long os, int dtype, int out_f32, int T,
                             int heads, int N, int K, int tail, const void* gate, long long ldg,
                             int gate_per_head, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && heads > 0 && N > 0 && K > 0 && tail >= 0, "heads_linear: bad sizes");
    AGV_REQUIRE(xs >= K + tail && os >= N + tail, "heads_linear: heads overlap");
    AGV_REQUIRE(heads <= 65535, "heads_linear: too many heads");
    AGV_REQUIRE((size_t)HL_TOK * K * 4 <= 48 * 1024, "heads_linear: K = %d too long", K);
    if (T == 0) return 0;
    // enough CTAs to fill the device when heads and tokens are few
    int rows_per_cta = 64;
    while (rows_per_cta > HL_WARPS &&
           (long long)((N + rows_per_cta - 1) / rows_per_cta) * heads * ((T + HL_TOK - 1) / HL_TOK) < 296)
        rows_per_cta /= 2;
    dim3 grid((N + rows_per_cta - 1) / rows_per_cta, heads, (T + HL_TOK - 1) / HL_TOK);
    const size_t smem = (size_t)HL_TOK * K * 4;
    if (dtype == AGV_F32)
        agv_launch(heads_linear_kernel<float, float>, grid, HL_WARPS * 32, smem, stream,
                   (const float*)x, ldx, xs, (const float*)W, (float*)out, ldo, os, T, N, K,
                   rows_per_cta, tail, (const float*)gate, ldg, gate_per_head);
    else if (dtype == AGV_BF16 && out_f32)
        agv_launch(heads_linear_kernel<__nv_bfloat16, float>, grid, HL_WARPS * 32, smem, stream,
                   (const __nv_bfloat16*)x, ldx, xs, (const __nv_bfloat16*)W, (float*)out, ldo, os,
                   T, N, K, rows_per_cta, tail, (const __nv_bfloat16*)gate, ldg, gate_per_head);
    else if (dtype == AGV_BF16)
        agv_launch(heads_linear_kernel<__nv_bfloat16, __nv_bfloat16>, grid, HL_WARPS * 32, smem,
                   stream, (const __nv_bfloat16*)x, ldx, xs, (const __nv_bfloat16*)W,
                   (__nv_bfloat16*)out, ldo, os, T, N, K, rows_per_cta, tail,
                   (const __nv_bfloat16*)gate, ldg, gate_per_head);
    else return agv_fail(-1, "heads_linear: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("heads_linear_kernel");
    return 0;
}

// out [T, width] (row stride ldo) *= sigmoid(g [T, width / per] (row stride ldg)).
AGV_API int agv_gate_sigmoid(void* out, long long ldo, const void* g, long long ldg, int dtype,
                             int T, int width, int per, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && width > 0 && per > 0 && width % per == 0, "gate_sigmoid: bad sizes");
    if (T == 0) return 0;
    const long long n = (long long)T * width;
    if (dtype == AGV_F32)
        agv_launch(gate_sigmoid_kernel<float>, flat_grid(n, 256), 256, 0, stream, (float*)out, ldo,
                   (const float*)g, ldg, T, width, per);
    else if (dtype == AGV_BF16 && width % 8 == 0 && (per == 1 || per % 8 == 0) && ldo % 8 == 0 &&
             (per != 1 || ldg % 8 == 0) && agv_aligned(out, 16) && (per != 1 || agv_aligned(g, 16)))
        agv_launch(gate_sigmoid_bf16x8_kernel, flat_grid(n / 8, 256), 256, 0, stream,
                   (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)g, ldg, T, width, per);
    else if (dtype == AGV_BF16)
        agv_launch(gate_sigmoid_kernel<__nv_bfloat16>, flat_grid(n, 256), 256, 0, stream,
                   (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)g, ldg, T, width, per);
    else return agv_fail(-1, "gate_sigmoid: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("gate_sigmoid_kernel");
    return 0;
}

AGV_API int agv_relu2(void* z, long long n, int dtype, cudaStream_t stream) {
    AGV_REQUIRE(n >= 0, "relu2: bad size");
    if (n == 0) return 0;
    if (dtype == AGV_F32)
        agv_launch(relu2_kernel<float>, flat_grid(n, 256), 256, 0, stream, (float*)z, n);
    else if (dtype == AGV_BF16)
        agv_launch(relu2_kernel<__nv_bfloat16>, flat_grid(n, 256), 256, 0, stream,
                   (__nv_bfloat16*)z, n);
    else return agv_fail(-1, "relu2: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("relu2_kernel");
    return 0;
}
