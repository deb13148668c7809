// Softmax attention, one warp per (query token, head), keys visited one by one
// with a running maximum and sum.  It reads keys and values either from the
// step's own projection output (prompts that start at position 0) or from the
// paged cache (decoding), and serves the 32-bit path and small or odd shapes
// of the bfloat16 path.  Scores, softmax and the weighted sum are 32-bit.
//
// Reference: score = (q . k) * scale, head h uses kv head h / (nh / nkv), softmax
// with the maximum subtracted (src/backend/kernels/cpu/sdpa.zig:36-37,58,184-234);
// causal bound src/backend/kernels/cuda/sdpa_prefill.zig:50; window start
// sl - W for sl = p + 1 > W (src/models/gemma4.zig:1153-1155).  No value row is
// skipped for a small weight (the reference skips below 1e-6,
// src/backend/kernels/cuda/sdpa.zig:14,99).
//
// Two options beyond that: a value head size hdv that differs from the query / key head
// size hd, and a sink per query head: a learned logit whose exponential is one more term of
// the softmax denominator (unscaled; nothing is added to the weighted sum for it).
// With a sliding window, the sequence's first keep_first keys may stay visible behind it.
// A bias per (distance, head) may be added to the scaled score, and the cache's value rows
// may lie at a stride of their own (values that are the leading part of the key rows).
#include "common.cuh"

constexpr int AT_WARPS = 4;
constexpr int AT_MAX_I = 24;          // head_dim <= 32 * AT_MAX_I

struct PagedKV {
    const void* k_pool;        // [n_pages, page, n_kv, hd] of this layer
    const void* v_pool;
    const int* page_table;     // [n_slots, max_pages]
    const int* slots;          // [B]
    int max_pages, page, cap;
    int v_row;                 // elements between two positions' value rows (0: nkv * hdv)
};

// A learned bias per (head, distance) added to the scaled score: bias[h, min(p - j, n - 1)].
struct DistanceBias {
    const float* bias;         // [nh, n] or null
    int n;
};

template <typename T, bool PAGED>
__global__ void __launch_bounds__(AT_WARPS * 32)
attention_simt_kernel(const T* __restrict__ q, long long q_stride, const T* __restrict__ k,
                      const T* __restrict__ v, long long kv_stride, T* __restrict__ out,
                      const int* __restrict__ positions, const int* __restrict__ seq_index,
                      const int* __restrict__ cu_seqlens, PagedKV pk, int n_tokens, int nh, int nkv,
                      int hd, float scale, int window, int hdv, long long v_stride,
                      const float* __restrict__ sinks, DistanceBias db, int keep_first) {
    pdl_wait();
    pdl_launch_next();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * AT_WARPS + warp;
    if (item >= (long long)n_tokens * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int g = h / (nh / nkv);
    const int b = seq_index[t];
    T* o = out + ((size_t)t * nh + h) * hdv;
    int slot = 0;
    if (PAGED) {
        slot = pk.slots[b];
        if (slot < 0) {
            for (int e = lane; e < hdv; e += 32) o[e] = from_f32<T>(0.f);
            return;
        }
    }
    const int p = positions[t];
    const int lo = first_visible(p, window);
    const T* qp = q + (size_t)t * q_stride + (size_t)h * hd;
    float qr[AT_MAX_I], acc[AT_MAX_I];
#pragma unroll
    for (int i = 0; i < AT_MAX_I; ++i) {
        const int e = lane + 32 * i;
        qr[i] = e < hd ? to_f32(qp[e]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const size_t base = PAGED ? 0 : (size_t)cu_seqlens[b];
    // (with a window, the sequence's first keep_first keys stay visible behind it)
    const int kept = min(keep_first, lo);
    for (int j = kept > 0 ? 0 : lo; j <= p; ++j) {
        if (j == kept && j < lo) j = lo;
        const T *kp, *vp;
        if (PAGED) {
            const int row = j % pk.cap;
            const int page = pk.page_table[(size_t)slot * pk.max_pages + row / pk.page];
            const size_t at = (size_t)page * pk.page + row % pk.page;
            kp = (const T*)pk.k_pool + (at * nkv + g) * hd;
            vp = (const T*)pk.v_pool + at * pk.v_row + (size_t)g * hdv;
        } else {
            kp = k + (base + j) * kv_stride + (size_t)g * hd;
            vp = v + (base + j) * v_stride + (size_t)g * hdv;
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < AT_MAX_I; ++i) {
            const int e = lane + 32 * i;
            if (e < hd) s = fmaf(qr[i], to_f32(kp[e]), s);
        }
        s = warp_sum(s) * scale;
        if (db.bias) s += db.bias[(size_t)h * db.n + min(p - j, db.n - 1)];
        const float mn = fmaxf(m, s);
        const float alpha = expf(m - mn);      // exp(-inf) = 0 on the first key
        const float w = expf(s - mn);
        l = l * alpha + w;
#pragma unroll
        for (int i = 0; i < AT_MAX_I; ++i) {
            const int e = lane + 32 * i;
            if (e < hdv) acc[i] = acc[i] * alpha + w * to_f32(vp[e]);
        }
        m = mn;
    }
    if (sinks) {
        // the sink joins the denominator as one more term, on the running maximum's scale
        const float sk = sinks[h];
        const float mn = fmaxf(m, sk);
        const float alpha = expf(m - mn);
        l = l * alpha + expf(sk - mn);
#pragma unroll
        for (int i = 0; i < AT_MAX_I; ++i) acc[i] *= alpha;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
    for (int i = 0; i < AT_MAX_I; ++i) {
        const int e = lane + 32 * i;
        if (e < hdv) o[e] = from_f32<T>(acc[i] * inv);
    }
}

static int check_attn(int n_tokens, int nh, int nkv, int hd, int window, int hdv = 1) {
    AGV_REQUIRE(hdv > 0 && hdv <= 32 * AT_MAX_I, "attention: value head size %d outside 1..%d", hdv,
                32 * AT_MAX_I);
    AGV_REQUIRE(n_tokens >= 0 && nh > 0 && nkv > 0 && hd > 0, "attention: bad sizes");
    AGV_REQUIRE(nh % nkv == 0, "attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    AGV_REQUIRE(hd <= 32 * AT_MAX_I, "attention: head_dim %d exceeds %d", hd, 32 * AT_MAX_I);
    return 0;
}

// Whole prompts that start at position 0.  q: [T, nh, hd] with row stride
// q_stride; k, v: [T, nkv, hd] with row stride kv_stride (both may point into
// the fused projection output); out: [T, nh * hd] dense.  Token t of batch
// entry b = seq_index[t] has position positions[t] and sees the tokens
// cu_seqlens[b] + j for lo <= j <= position.  window 0: no window.
// hdv: the value head size (v: [T, nkv, hdv] with row stride v_stride, out: [T, nh * hdv]);
// sinks: [nh] 32-bit sink logits or null.
AGV_API int agv_attention_prefill_simt_ex(const void* q, long long q_stride, const void* k,
                                          const void* v, long long kv_stride, void* out, int dtype,
                                          const int* positions, const int* seq_index,
                                          const int* cu_seqlens, int n_tokens, int nh, int nkv,
                                          int hd, float scale, int window, int hdv,
                                          long long v_stride, const float* sinks,
                                          const float* dist_bias, int n_dist, int keep_first,
                                          cudaStream_t stream) {
    if (int rc = check_attn(n_tokens, nh, nkv, hd, window, hdv)) return rc;
    AGV_REQUIRE(!dist_bias || n_dist > 0, "attention: an empty distance table");
    if (n_tokens == 0) return 0;
    DistanceBias db{dist_bias, n_dist};
    const long long items = (long long)n_tokens * nh;
    const unsigned grid = (unsigned)((items + AT_WARPS - 1) / AT_WARPS);
    PagedKV pk{};
    if (dtype == AGV_F32)
        agv_launch(attention_simt_kernel<float, false>, grid, AT_WARPS * 32, 0, stream, (const float*)q, q_stride, (const float*)k, (const float*)v, kv_stride, (float*)out,
            positions, seq_index, cu_seqlens, pk, n_tokens, nh, nkv, hd, scale, window, hdv,
            v_stride, sinks, db, keep_first);
    else if (dtype == AGV_BF16)
        agv_launch(attention_simt_kernel<__nv_bfloat16, false>, grid, AT_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)k, (const __nv_bfloat16*)v,
            kv_stride, (__nv_bfloat16*)out, positions, seq_index, cu_seqlens, pk, n_tokens, nh,
            nkv, hd, scale, window, hdv, v_stride, sinks, db, keep_first);
    else
        return agv_fail(-1, "attention: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("attention_simt_kernel");
    return 0;
}

AGV_API int agv_attention_prefill_simt(const void* q, long long q_stride, const void* k,
                                       const void* v, long long kv_stride, void* out, int dtype,
                                       const int* positions, const int* seq_index,
                                       const int* cu_seqlens, int n_tokens, int nh, int nkv, int hd,
                                       float scale, int window, cudaStream_t stream) {
    return agv_attention_prefill_simt_ex(q, q_stride, k, v, kv_stride, out, dtype, positions,
                                         seq_index, cu_seqlens, n_tokens, nh, nkv, hd, scale,
                                         window, hd, kv_stride, nullptr, nullptr, 0, 0, stream);
}

// Queries against the paged cache (the query's own key is already stored).
// Token t of entry b = seq_index[t] at positions[t] sees cache positions
// lo..positions[t] of slot slots[b]; a negative slot yields zeros.
// hdv: the value head size (v_pool rows of nkv * hdv, out: [T, nh * hdv]); sinks: [nh] or null.
AGV_API int agv_attention_paged_simt_ex(const void* q, long long q_stride, void* out, int dtype,
                                        const void* k_pool, const void* v_pool,
                                        const int* page_table, const int* slots,
                                        const int* positions, const int* seq_index, int max_pages,
                                        int page, int cap, int n_tokens, int nh, int nkv, int hd,
                                        float scale, int window, int hdv, const float* sinks,
                                        const float* dist_bias, int n_dist, int v_row, int keep_first,
                                        cudaStream_t stream) {
    if (int rc = check_attn(n_tokens, nh, nkv, hd, window, hdv)) return rc;
    AGV_REQUIRE(!dist_bias || n_dist > 0, "attention: an empty distance table");
    AGV_REQUIRE(v_row == 0 || v_row >= nkv * hdv, "attention: value rows overlap");
    DistanceBias db{dist_bias, n_dist};
    AGV_REQUIRE(page > 0 && cap > 0 && max_pages > 0, "attention: bad cache geometry");
    AGV_REQUIRE(window <= cap, "attention: window %d exceeds the ring of %d rows",
                window, cap);
    AGV_REQUIRE(keep_first >= 0 && (keep_first == 0 || window >= 0),
                "attention: kept first keys go with a sliding window or none");
    if (n_tokens == 0) return 0;
    const long long items = (long long)n_tokens * nh;
    const unsigned grid = (unsigned)((items + AT_WARPS - 1) / AT_WARPS);
    PagedKV pk{k_pool, v_pool, page_table, slots, max_pages, page, cap, v_row ? v_row : nkv * hdv};
    if (dtype == AGV_F32)
        agv_launch(attention_simt_kernel<float, true>, grid, AT_WARPS * 32, 0, stream, (const float*)q, q_stride, nullptr, nullptr, 0, (float*)out, positions, seq_index,
            nullptr, pk, n_tokens, nh, nkv, hd, scale, window, hdv, 0LL, sinks, db, keep_first);
    else if (dtype == AGV_BF16)
        agv_launch(attention_simt_kernel<__nv_bfloat16, true>, grid, AT_WARPS * 32, 0, stream, (const __nv_bfloat16*)q, q_stride, nullptr, nullptr, 0, (__nv_bfloat16*)out, positions,
            seq_index, nullptr, pk, n_tokens, nh, nkv, hd, scale, window, hdv, 0LL, sinks, db, keep_first);
    else
        return agv_fail(-1, "attention: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("attention_simt_kernel");
    return 0;
}

AGV_API int agv_attention_paged_simt(const void* q, long long q_stride, void* out, int dtype,
                                     const void* k_pool, const void* v_pool, const int* page_table,
                                     const int* slots, const int* positions, const int* seq_index,
                                     int max_pages, int page, int cap, int n_tokens, int nh,
                                     int nkv, int hd, float scale, int window,
                                     cudaStream_t stream) {
    return agv_attention_paged_simt_ex(q, q_stride, out, dtype, k_pool, v_pool, page_table, slots,
                                       positions, seq_index, max_pages, page, cap, n_tokens, nh,
                                       nkv, hd, scale, window, hd, nullptr, nullptr, 0, 0, 0, stream);
}
