// Routed feed-forward (mixture of experts): router, the plan that sorts (token, choice)
// pairs by expert, and the experts' products run as grouped products over that plan.
//
// Router (32-bit): z = W_r x, s = sigmoid(z), choice score c = s + correction.  The experts
// lie in n_groups equal groups of neighbours; a group's score is the sum of its two largest
// c; the choice is made among the experts of the `keep` best groups alone (every other
// expert is masked out before the top-k, whatever the sign of the scores); the `top`
// largest c among them win, and their weights are their s, unchanged.  n_groups = keep = 1
// is plain top-k routing; correction null adds nothing.  Ties go to the lower index.
// Two options: a bias [E] added to the logits (z = W_r x + b), and weights that are the
// softmax over the chosen experts' logits alone (the logits then also make the choice)
// instead of their sigmoids.
//
// Plan: the P = T * top pairs are laid out by expert, every expert's run padded to a
// multiple of the row tile, so that a tile of the grouped products belongs to one expert.
// Everything is sized on the host from upper bounds (P + E * tile rows, P / tile + E tiles)
// and decided on the device: nothing is read back, so a step records into a CUDA graph.
//
// Grouped products: out[pos, :] = a[src(pos), :] * W[e(tile)]^T, plain, or the gated pair
// act(a Wg^T) * (a Wu^T); a row of the result can be scaled and scattered (the down
// product leaves w_pair * y at [choice, token, :], which the join that follows adds over
// the choices in order).  Each output element is one dot product accumulated in ascending
// k in 32-bit: a token's result does not depend on its company.
#include "common.cuh"

namespace {

enum { MOE_ACT_GELU_TANH = 0, MOE_ACT_SILU = 1 };

__device__ __forceinline__ float moe_act(float t, int act) {
    if (act == MOE_ACT_SILU) return t / (1.0f + expf(-t));
    const float u = 0.7978845608028654f * (t + 0.044715f * t * t * t);
    return 0.5f * t * (1.0f + tanhf(u));
}

constexpr int RT_WARPS = 4;
constexpr int RT_MAX_E = 512;

// How a logit becomes a score: bias [E] (or null) is added to it first.  mode 0: the score,
// and the weight, is the logit's sigmoid.  mode 1 (softmax over the chosen): the score is the
// logit itself and the chosen experts' weights are the softmax over their logits.  mode 2
// (softmax over all): the scores are the softmax over all the logits, score + correction
// chooses, and the chosen experts' scores, divided by their sum (+ 1e-20) and multiplied by
// `scale`, weigh.
struct RouteScore {
    const float* bias;
    int mode;
    float scale;
    __device__ __forceinline__ float score(float z, int e) const {
        if (bias) z += bias[e];
        return mode ? z : 1.0f / (1.0f + expf(-z));
    }
    // mode 2, by one thread: s [E] logits become their softmax, c = s + correction
    __device__ __forceinline__ void spread(float* s, float* c, const float* correction,
                                           int E) const {
        if (mode != 2) return;
        float m = s[0];
        for (int e = 1; e < E; ++e) m = fmaxf(m, s[e]);
        float sum = 0.f;
        for (int e = 0; e < E; ++e) { s[e] = expf(s[e] - m); sum += s[e]; }
        for (int e = 0; e < E; ++e) {
            s[e] /= sum;
            c[e] = s[e] + (correction ? correction[e] : 0.f);
        }
    }
    // the same by a warp
    __device__ __forceinline__ void spread_warp(float* s, float* c, const float* correction,
                                                int E, int lane) const {
        if (mode != 2) return;
        float m = -INFINITY;
        for (int e = lane; e < E; e += 32) m = fmaxf(m, s[e]);
        m = warp_max(m);
        float sum = 0.f;
        for (int e = lane; e < E; e += 32) { const float x = expf(s[e] - m); s[e] = x; sum += x; }
        sum = warp_sum(sum);
        for (int e = lane; e < E; e += 32) {
            const float x = s[e] / sum;
            s[e] = x;
            c[e] = x + (correction ? correction[e] : 0.f);
        }
        __syncwarp();
    }
    // the chosen experts' scores become their weights, by one thread
    __device__ __forceinline__ void weigh(float* w, int top) const {
        if (mode == 1) {
            float m = w[0];
            for (int k = 1; k < top; ++k) m = fmaxf(m, w[k]);
            float sum = 0.f;
            for (int k = 0; k < top; ++k) { w[k] = expf(w[k] - m); sum += w[k]; }
            for (int k = 0; k < top; ++k) w[k] /= sum;
        } else if (mode == 2) {
            float sum = 0.f;
            for (int k = 0; k < top; ++k) sum += w[k];
            for (int k = 0; k < top; ++k) w[k] = w[k] / (sum + 1e-20f) * scale;
        }
    }
};

// The choice of one token from its scores (one thread): s [E] sigmoid scores, c [E] choice
// scores (consumed).
__device__ void moe_choose(float* s, float* c, int E, int n_groups, int keep, int top,
                           int* __restrict__ ids, float* __restrict__ wts, RouteScore rs) {
    const int per = E / n_groups;
    if (keep < n_groups) {
        // group scores: the two largest choice scores of each group, summed
        unsigned long long kept[RT_MAX_E / 64] = {};
        for (int k = 0; k < keep; ++k) {
            int best = -1;
            float best_v = -INFINITY;
            for (int g = 0; g < n_groups; ++g) {
                if (kept[g >> 6] >> (g & 63) & 1ull) continue;
                float a = -INFINITY, b = -INFINITY;          // largest, second largest
                for (int i = 0; i < per; ++i) {
                    const float v = c[g * per + i];
                    if (v > a) { b = a; a = v; }
                    else if (v > b) b = v;
                }
                const float sc = per > 1 ? a + b : a;
                if (best < 0 || sc > best_v) { best = g; best_v = sc; }
            }
            kept[best >> 6] |= 1ull << (best & 63);
        }
        for (int g = 0; g < n_groups; ++g)
            if (!(kept[g >> 6] >> (g & 63) & 1ull))
                for (int i = 0; i < per; ++i) c[g * per + i] = -INFINITY;
    }
    for (int k = 0; k < top; ++k) {
        int best = -1;
        float best_v = -INFINITY;
        for (int e = 0; e < E; ++e) {
            const float v = c[e];
            if (v > best_v) { best = e; best_v = v; }
        }
        if (best < 0) best = 0;                 // (no finite score left: cannot happen with finite inputs)
        ids[k] = best;
        wts[k] = s[best];
        c[best] = -INFINITY;
    }
    rs.weigh(wts, top);
}

// Index of the greatest of v[0..n) over a warp (the lowest index among equals; -1 if all are
// minus infinity); every lane gets the result.
__device__ __forceinline__ int warp_argmax(const float* v, int n, int lane) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
        const float x = v[i];
        if (x > bv) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    return bi == 0x7fffffff ? -1 : bi;
}

// The same choice made by a whole warp: gs [n_groups] is scratch for the group scores.
__device__ void moe_choose_warp(float* s, float* c, float* gs, int E, int n_groups, int keep,
                                int top, int* __restrict__ ids, float* __restrict__ wts,
                                int lane, RouteScore rs) {
    const int per = E / n_groups;
    if (keep < n_groups) {
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;              // largest, second largest
            for (int i = 0; i < per; ++i) {
                const float v = c[g * per + i];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        // a kept group's score becomes "not a number", which is never the greatest again;
        // the groups that still hold a number afterwards are dropped
        for (int k = 0; k < keep; ++k) {
            int best = warp_argmax(gs, n_groups, lane);
            if (best < 0) {
                // (only groups of minus infinity left: take the first not yet kept)
                best = 0;
                while (best < n_groups - 1 && gs[best] != gs[best]) ++best;
            }
            __syncwarp();
            if (lane == 0) gs[best] = NAN;
            __syncwarp();
        }
        for (int e = lane; e < E; e += 32)
            if (gs[e / per] == gs[e / per]) c[e] = -INFINITY;    // not marked: dropped
        __syncwarp();
    }
    for (int k = 0; k < top; ++k) {
        int best = warp_argmax(c, E, lane);
        if (best < 0) best = 0;                 // (no finite score left: cannot happen with finite inputs)
        __syncwarp();
        if (lane == 0) {
            ids[k] = best;
            wts[k] = s[best];
            c[best] = -INFINITY;
        }
        __syncwarp();
    }
    if (lane == 0) rs.weigh(wts, top);
}

// One warp per token: logits by lanes over H, then lane 0 chooses.  The general form (any
// H, any alignment).
template <typename T>
__global__ void __launch_bounds__(RT_WARPS * 32)
moe_route_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ wr,
                 const float* __restrict__ correction, int n_tokens, int H, int E, int n_groups,
                 int keep, int top, int* __restrict__ ids, float* __restrict__ wts,
                 RouteScore rs) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * RT_WARPS + warp;
    if (t >= n_tokens) return;
    float* s = smem + (size_t)warp * 2 * E;      // sigmoid scores
    float* c = s + E;                            // choice scores (consumed by the choice)
    const T* xr = x + (size_t)t * ldx;
    for (int e = 0; e < E; ++e) {
        const T* w = wr + (size_t)e * H;
        float z = 0.f;
        for (int i = lane; i < H; i += 32) z = fmaf(to_f32(xr[i]), to_f32(w[i]), z);
        z = warp_sum(z);
        if (lane == 0) {
            const float sg = rs.score(z, e);
            s[e] = sg;
            c[e] = sg + (correction ? correction[e] : 0.f);
        }
    }
    __syncwarp();
    if (lane == 0) {
        rs.spread(s, c, correction, E);
        moe_choose(s, c, E, n_groups, keep, top, ids + (size_t)t * top, wts + (size_t)t * top, rs);
    }
}

// 16 bytes of a row as 32-bit values.
template <typename T> struct Row16;
template <> struct Row16<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[4]) {
        const float4 t = *reinterpret_cast<const float4*>(p);
        v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
    }
};
template <> struct Row16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void load(const __nv_bfloat16* p, float (&v)[8]) {
        const uint4 t = *reinterpret_cast<const uint4*>(p);
        const unsigned u[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(u[i] << 16);
            v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};

// The same for rows that move in 16-byte pieces: a CTA of RT_VW warps takes RT_TOK tokens,
// warp w the experts w, w + RT_VW, ...; a lane's piece of a router row meets the same piece
// of every token of the CTA, so the router's matrix is read once per RT_TOK tokens, and the
// loads of a row are independent of one another.  Then warp t chooses for token t.  Few
// tokens (decoding) take a CTA of sixteen warps each, many (prompts) share CTAs of eight by
// fours.
template <typename T, int RT_TOK, int RT_VW>
__global__ void __launch_bounds__(RT_VW * 32)
moe_route_tiled_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ wr,
                       const float* __restrict__ correction, int n_tokens, int H, int E,
                       int n_groups, int keep, int top, int* __restrict__ ids,
                       float* __restrict__ wts, RouteScore rs) {
    pdl_wait();
    pdl_launch_next();
    extern __shared__ float smem[];              // [RT_TOK][3][E]
    constexpr int N = Row16<T>::N;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * RT_TOK;
    const int pieces = H / N;
    const T* xr[RT_TOK];
#pragma unroll
    for (int k = 0; k < RT_TOK; ++k) xr[k] = x + (size_t)min(t0 + k, n_tokens - 1) * ldx;
    for (int e = warp; e < E; e += RT_VW) {
        const T* w = wr + (size_t)e * H;
        float z[RT_TOK] = {};
#pragma unroll 4
        for (int i = lane; i < pieces; i += 32) {
            float wv[N], xv[N];
            Row16<T>::load(w + i * N, wv);
#pragma unroll
            for (int k = 0; k < RT_TOK; ++k) {
                Row16<T>::load(xr[k] + i * N, xv);
#pragma unroll
                for (int j = 0; j < N; ++j) z[k] = fmaf(xv[j], wv[j], z[k]);
            }
        }
#pragma unroll
        for (int k = 0; k < RT_TOK; ++k) {
            const float zz = warp_sum(z[k]);
            if (lane == 0) {
                const float sg = rs.score(zz, e);
                smem[(k * 3) * E + e] = sg;
                smem[(k * 3 + 1) * E + e] = sg + (correction ? correction[e] : 0.f);
            }
        }
    }
    __syncthreads();
    if (warp < RT_TOK && t0 + warp < n_tokens) {
        const int t = t0 + warp;
        rs.spread_warp(smem + (warp * 3) * E, smem + (warp * 3 + 1) * E, correction, E, lane);
        moe_choose_warp(smem + (warp * 3) * E, smem + (warp * 3 + 1) * E,
                        smem + (warp * 3 + 2) * E, E, n_groups, keep, top, ids + (size_t)t * top,
                        wts + (size_t)t * top, lane, rs);
    }
}

// One CTA lays the pairs out by expert.  tile: rows per tile of the grouped products.
//   tok[pos]    token of the pair at sorted position pos, -1 for padding
//   dst[pos]    choice * T + token: the row the down product writes
//   wpos[pos]   the pair's weight
//   pos_of[p]   where pair p went (for consumers that walk pairs)
//   tile_e[i]   expert of tile i, -1 for tiles beyond the last
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, const float* __restrict__ wts, int n_tokens, int top,
                int E, int tile, int* __restrict__ tok, int* __restrict__ dst,
                float* __restrict__ wpos, int* __restrict__ pos_of, int* __restrict__ tile_e,
                int max_rows, int max_tiles) {
    pdl_launch_next();
    extern __shared__ int sm[];
    int* count = sm;              // [E]
    int* start = sm + E;          // [E + 1] first row of each expert's run
    const int P = n_tokens * top;
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    pdl_wait();
    for (int i = threadIdx.x; i < max_rows; i += blockDim.x) tok[i] = -1;
    for (int p = threadIdx.x; p < P; p += blockDim.x)
        if (ids[p] < E) atomicAdd(&count[ids[p]], 1);     // (an id beyond the experts: a pair no expert runs)
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            start[e] = at;
            at += (count[e] + tile - 1) / tile * tile;
        }
        start[E] = at;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) {
        const int row0 = i * tile;
        int e = -1;
        if (row0 < start[E]) {
            // the expert whose run holds row0 (runs are in expert order; E is small)
            int lo = 0, hi = E - 1;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (start[mid] <= row0) lo = mid; else hi = mid - 1;
            }
            e = lo;          // (the last of the experts that start here: the others' runs are empty)
        }
        tile_e[i] = e;
    }
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;     // now the cursors
    __syncthreads();
    // a pair takes the next free row of its expert's run; the order inside a run is
    // whatever the atomics make it, which no result depends on (rows are independent)
    for (int p = threadIdx.x; p < P; p += blockDim.x) {
        const int e = ids[p];
        if (e >= E) { pos_of[p] = -1; continue; }
        const int pos = start[e] + atomicAdd(&count[e], 1);
        tok[pos] = p / top;
        dst[pos] = (p % top) * n_tokens + p / top;
        wpos[pos] = wts[p];
        pos_of[p] = pos;
    }
}

constexpr int GM = 64, GN = 64, GK = 16;

// 64 sorted rows x 64 output features of one expert (sub of these to a tile of the plan).  A rows are gathered through
// a_index (null: row = pos, live where tok[pos] >= 0); C rows go to c_index[pos] (null:
// pos) times c_scale[pos] (null: 1).
template <typename TA, typename TW, typename TO, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const TA* __restrict__ A, long long lda, const int* __restrict__ a_index,
                   const int* __restrict__ tok, const TW* __restrict__ W,
                   const TW* __restrict__ W2, TO* __restrict__ C, long long ldc,
                   const int* __restrict__ c_index, const float* __restrict__ c_scale,
                   const int* __restrict__ tile_e, int N, int K, int act, int sub) {
    pdl_wait();
    pdl_launch_next();
    const int e = tile_e[blockIdx.y / sub];
    if (e < 0) return;
    __shared__ float As[GK][GM + 4];
    __shared__ float Ws[GK][GN + 4];
    __shared__ float Us[GATED ? GK : 1][GATED ? GN + 4 : 1];
    __shared__ int arow[GM];
    const int tid = threadIdx.x;
    const int tx = tid % 16, ty = tid / 16;
    const int m0 = blockIdx.y * GM, n0 = blockIdx.x * GN;
    if (tid < GM) {
        const int pos = m0 + tid;
        const int t = tok[pos];
        arow[tid] = t < 0 ? -1 : (a_index ? a_index[pos] : pos);
    }
    __syncthreads();
    const TW* We = W + (size_t)e * N * K;
    const TW* We2 = GATED ? W2 + (size_t)e * N * K : nullptr;
    float acc[4][4] = {};
    float acc2[GATED ? 4 : 1][GATED ? 4 : 1] = {};
    const int lr = tid / 4, lk = (tid % 4) * 4;
    const int ar = arow[lr];
    for (int k0 = 0; k0 < K; k0 += GK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k = k0 + lk + i;
            const int n = n0 + lr;
            As[lk + i][lr] = (ar >= 0 && k < K) ? to_f32(A[(size_t)ar * lda + k]) : 0.f;
            Ws[lk + i][lr] = (n < N && k < K) ? to_f32(We[(size_t)n * K + k]) : 0.f;
            if (GATED) Us[lk + i][lr] = (n < N && k < K) ? to_f32(We2[(size_t)n * K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < GK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            if (GATED) {
#pragma unroll
                for (int j = 0; j < 4; ++j) b[j] = Us[k][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc2[i][j] = fmaf(a[i], b[j], acc2[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = ty * 4 + i;
        if (arow[r] < 0) continue;
        const int pos = m0 + r;
        const size_t crow = c_index ? (size_t)c_index[pos] : (size_t)pos;
        const float sc = c_scale ? c_scale[pos] : 1.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n >= N) continue;
            float v = acc[i][j];
            if (GATED) v = moe_act(v, act) * acc2[i][j];
            C[crow * ldc + n] = from_f32<TO>(v * sc);
        }
    }
}

}  // namespace

// x: [T, H] rows of stride ldx, wr: [E, H] (both `dtype`); correction: [E] 32-bit or null;
// ids, wts: [T, top] outputs.
// bias: [E] 32-bit or null, added to the logits; softmax_top != 0: the logits choose and the
// weights are the softmax over the chosen logits (else sigmoids, see the head of this file).
AGV_API int agv_moe_route_mode(const void* x, long long ldx, const void* wr,
                               const float* correction, const float* bias, int mode, float scale,
                               int dtype, int T, int H, int E, int n_groups, int keep, int top,
                               int* ids, float* wts, cudaStream_t stream);

AGV_API int agv_moe_route_ex(const void* x, long long ldx, const void* wr,
                             const float* correction, const float* bias, int softmax_top,
                             int dtype, int T, int H, int E, int n_groups, int keep, int top,
                             int* ids, float* wts, cudaStream_t stream) {
    return agv_moe_route_mode(x, ldx, wr, correction, bias, softmax_top ? 1 : 0, 1.0f, dtype, T, H,
                              E, n_groups, keep, top, ids, wts, stream);
}

// mode: 0 sigmoid scores, 1 softmax over the chosen logits, 2 softmax over all logits with
// the chosen scores renormalised and multiplied by `scale` (see RouteScore).
AGV_API int agv_moe_route_mode(const void* x, long long ldx, const void* wr,
                               const float* correction, const float* bias, int mode, float scale,
                               int dtype, int T, int H, int E, int n_groups, int keep, int top,
                               int* ids, float* wts, cudaStream_t stream) {
    const RouteScore rs{bias, mode, scale};
    AGV_REQUIRE(mode >= 0 && mode <= 2, "moe_route: unknown mode %d", mode);
    AGV_REQUIRE(T >= 0 && H > 0 && E > 0 && top > 0, "moe_route: bad sizes");
    AGV_REQUIRE(E <= RT_MAX_E, "moe_route: %d experts exceed %d", E, RT_MAX_E);
    AGV_REQUIRE(n_groups >= 1 && E % n_groups == 0, "moe_route: %d experts do not form %d equal "
                "groups", E, n_groups);
    AGV_REQUIRE(keep >= 1 && keep <= n_groups, "moe_route: keep %d outside 1..%d", keep, n_groups);
    AGV_REQUIRE(top <= keep * (E / n_groups), "moe_route: top %d exceeds the %d experts of the "
                "groups kept", top, keep * (E / n_groups));
    AGV_REQUIRE(ldx >= H, "moe_route: row stride shorter than a row");
    if (T == 0) return 0;
    const int piece = dtype == AGV_F32 ? 4 : 8;
    if (H % piece == 0 && ldx % piece == 0 && agv_aligned(x, 16) && agv_aligned(wr, 16)) {
        AGV_REQUIRE(dtype == AGV_F32 || dtype == AGV_BF16, "moe_route: unknown dtype %d", dtype);
#define AGV_ROUTE(TT, TOK, VW)                                                                  \
    agv_launch(moe_route_tiled_kernel<TT, TOK, VW>, (unsigned)((T + TOK - 1) / TOK), VW * 32,   \
               (size_t)TOK * 3 * E * sizeof(float), stream, (const TT*)x, ldx, (const TT*)wr,   \
               correction, T, H, E, n_groups, keep, top, ids, wts, rs)
        if (T <= 64) {
            if (dtype == AGV_F32) AGV_ROUTE(float, 1, 16);
            else AGV_ROUTE(__nv_bfloat16, 1, 16);
        } else {
            if (dtype == AGV_F32) AGV_ROUTE(float, 4, 8);
            else AGV_ROUTE(__nv_bfloat16, 4, 8);
        }
#undef AGV_ROUTE
        AGV_LAUNCH_OK("moe_route_tiled_kernel");
        return 0;
    }
    const unsigned grid = (unsigned)((T + RT_WARPS - 1) / RT_WARPS);
    const size_t smem = (size_t)RT_WARPS * 2 * E * sizeof(float);
    if (dtype == AGV_F32)
        agv_launch(moe_route_kernel<float>, grid, RT_WARPS * 32, smem, stream, (const float*)x, ldx,
                   (const float*)wr, correction, T, H, E, n_groups, keep, top, ids, wts, rs);
    else if (dtype == AGV_BF16)
        agv_launch(moe_route_kernel<__nv_bfloat16>, grid, RT_WARPS * 32, smem, stream,
                   (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)wr, correction, T, H, E,
                   n_groups, keep, top, ids, wts, rs);
    else
        return agv_fail(-1, "moe_route: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("moe_route_kernel");
    return 0;
}

AGV_API int agv_moe_route(const void* x, long long ldx, const void* wr, const float* correction,
                          int dtype, int T, int H, int E, int n_groups, int keep, int top,
                          int* ids, float* wts, cudaStream_t stream) {
    return agv_moe_route_ex(x, ldx, wr, correction, nullptr, 0, dtype, T, H, E, n_groups, keep,
                            top, ids, wts, stream);
}

// y [T, H] (32-bit) *= sigmoid(x[t, :] . w) per row t: one gate value per token for a branch
// that runs for every token.  x: [T, K] rows of stride ldx, w: [K] (both `dtype`); the dot
// product and the sigmoid are 32-bit.
namespace {
template <typename T>
__global__ void __launch_bounds__(128)
row_gate_kernel(const T* __restrict__ x, long long ldx, const T* __restrict__ w,
                float* __restrict__ y, int K, int H) {
    pdl_wait();
    pdl_launch_next();
    __shared__ float red[33];
    const int t = blockIdx.x;
    const T* xr = x + (size_t)t * ldx;
    float z = 0.f;
    for (int i = threadIdx.x; i < K; i += blockDim.x) z = fmaf(to_f32(xr[i]), to_f32(w[i]), z);
    z = block_sum(z, red);
    const float g = 1.0f / (1.0f + expf(-z));
    float* yr = y + (size_t)t * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] *= g;
}
}  // namespace

AGV_API int agv_row_gate(const void* x, long long ldx, const void* w, int dtype, float* y, int T,
                         int K, int H, cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && K > 0 && H > 0 && ldx >= K, "row_gate: bad sizes");
    if (T == 0) return 0;
    if (dtype == AGV_F32)
        agv_launch(row_gate_kernel<float>, (unsigned)T, 128, 0, stream, (const float*)x, ldx,
                   (const float*)w, y, K, H);
    else if (dtype == AGV_BF16)
        agv_launch(row_gate_kernel<__nv_bfloat16>, (unsigned)T, 128, 0, stream,
                   (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)w, y, K, H);
    else
        return agv_fail(-1, "row_gate: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("row_gate_kernel");
    return 0;
}

// Upper bounds the caller sizes the plan's arrays with; tile: rows per tile (a multiple of 64).
AGV_API int agv_moe_plan_tiles(int T, int top, int E, int tile) {
    return (T * top + tile - 1) / tile + E;
}
AGV_API int agv_moe_plan_rows(int T, int top, int E, int tile) {
    return agv_moe_plan_tiles(T, top, E, tile) * tile;
}

// See moe_plan_kernel; tok, dst, wpos: [agv_moe_plan_rows], pos_of: [T * top],
// tile_e: [agv_moe_plan_tiles].
AGV_API int agv_moe_plan(const int* ids, const float* wts, int T, int top, int E, int tile,
                         int* tok, int* dst, float* wpos, int* pos_of, int* tile_e,
                         cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && top > 0 && E > 0, "moe_plan: bad sizes");
    AGV_REQUIRE(tile >= GM && tile % GM == 0, "moe_plan: tiles of %d rows (a multiple of %d)", tile, GM);
    AGV_REQUIRE(E <= 4096, "moe_plan: %d experts exceed 4096", E);
    if (T == 0) return 0;
    const size_t smem = (size_t)(2 * E + 1) * sizeof(int);
    agv_launch(moe_plan_kernel, 1u, 1024, smem, stream, ids, wts, T, top, E, tile, tok, dst, wpos,
               pos_of, tile_e, agv_moe_plan_rows(T, top, E, tile),
               agv_moe_plan_tiles(T, top, E, tile));
    AGV_LAUNCH_OK("moe_plan_kernel");
    return 0;
}

// The grouped product over a plan.  a: rows of stride lda (a_index null: row = sorted
// position); tile: the plan's rows per tile; w (and w2 for the gated form): [E, N, K] dense; c: rows of stride ldc at
// c_index[pos] (null: pos), times c_scale[pos] (null: 1).  in_dtype: a and the weights;
// out_dtype: c.
AGV_API int agv_moe_grouped(const void* a, long long lda, const int* a_index, const int* tok,
                            const void* w, const void* w2, void* c, long long ldc,
                            const int* c_index, const float* c_scale, const int* tile_e,
                            int n_tiles, int tile, int N, int K, int in_dtype, int out_dtype,
                            int act, cudaStream_t stream) {
    AGV_REQUIRE(n_tiles >= 0 && N > 0 && K > 0, "moe_grouped: bad sizes");
    AGV_REQUIRE(tile >= GM && tile % GM == 0, "moe_grouped: tiles of %d rows (a multiple of %d)",
                tile, GM);
    const int sub = tile / GM;
    n_tiles *= sub;
    AGV_REQUIRE(lda >= K && ldc >= N, "moe_grouped: row strides shorter than rows");
    AGV_REQUIRE(n_tiles <= 65535, "moe_grouped: %d tiles exceed the grid limit", n_tiles);
    if (n_tiles == 0) return 0;
    dim3 grid((N + GN - 1) / GN, n_tiles);
#define AGV_MOE(TA, TO)                                                                          \
    do {                                                                                         \
        if (w2)                                                                                  \
            agv_launch(moe_grouped_kernel<TA, TA, TO, true>, grid, 256, 0, stream, (const TA*)a, \
                       lda, a_index, tok, (const TA*)w, (const TA*)w2, (TO*)c, ldc, c_index,     \
                       c_scale, tile_e, N, K, act, sub);                                         \
        else                                                                                     \
            agv_launch(moe_grouped_kernel<TA, TA, TO, false>, grid, 256, 0, stream,              \
                       (const TA*)a, lda, a_index, tok, (const TA*)w, (const TA*)nullptr,        \
                       (TO*)c, ldc, c_index, c_scale, tile_e, N, K, act, sub);                   \
    } while (0)
    if (in_dtype == AGV_F32 && out_dtype == AGV_F32) AGV_MOE(float, float);
    else if (in_dtype == AGV_BF16 && out_dtype == AGV_BF16) AGV_MOE(__nv_bfloat16, __nv_bfloat16);
    else if (in_dtype == AGV_BF16 && out_dtype == AGV_F32) AGV_MOE(__nv_bfloat16, float);
    else return agv_fail(-1, "moe_grouped: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef AGV_MOE
    AGV_LAUNCH_OK("moe_grouped_kernel");
    return 0;
}

// Pairs whose id lies at or beyond the experts are identities: the pair's output is the
// token's own input times the pair's weight.  y [top, T, H] (32-bit) receives it in the rows
// the experts' scatter leaves out.
namespace {
template <typename T>
__global__ void __launch_bounds__(256)
moe_identity_kernel(const T* __restrict__ x, long long ldx, const int* __restrict__ ids,
                    const float* __restrict__ wts, int n_tokens, int top, int E, int H,
                    float* __restrict__ y) {
    pdl_wait();
    pdl_launch_next();
    const int p = blockIdx.x;
    if (ids[p] < E) return;
    const int t = p / top, c = p % top;
    const float w = wts[p];
    const T* xr = x + (size_t)t * ldx;
    float* yr = y + ((size_t)c * n_tokens + t) * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) yr[i] = w * to_f32(xr[i]);
}
}  // namespace

AGV_API int agv_moe_identity(const void* x, long long ldx, int dtype, const int* ids,
                             const float* wts, int T, int top, int E, int H, float* y,
                             cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && top > 0 && E >= 0 && H > 0 && ldx >= H, "moe_identity: bad sizes");
    if (T == 0) return 0;
    const unsigned grid = (unsigned)(T * top);
    if (dtype == AGV_F32)
        agv_launch(moe_identity_kernel<float>, grid, 256, 0, stream, (const float*)x, ldx, ids, wts,
                   T, top, E, H, y);
    else if (dtype == AGV_BF16)
        agv_launch(moe_identity_kernel<__nv_bfloat16>, grid, 256, 0, stream,
                   (const __nv_bfloat16*)x, ldx, ids, wts, T, top, E, H, y);
    else
        return agv_fail(-1, "moe_identity: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("moe_identity_kernel");
    return 0;
}
