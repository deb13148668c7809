// What an attention mixer with a short causal convolution does to a token's row of its
// stacked projection  q | k | v | g  before it attends (k and v absent for a layer that
// attends to another layer's keys and values; g absent without an output gate):
//
//   y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]      on every channel c of q, k and v
//
// with zeros before the sequence's first token, then the rotation of the first rot_dim
// dimensions of every q and k head (pairs (i, i + rot_dim / 2)), then the store of k and v in
// the paged cache; q | k | v | g leave in the compute dtype (g: the gate's logits as they
// came).  The convolution's inputs of earlier steps, u of the last taps - 1 positions, are
// part of the sequence's fixed-size state: a ring by position (position p in row
// p % (taps - 1)), which the kernel reads for positions before the step's first and brings
// up to date.  A channel belongs to one thread, which reads the ring row it then overwrites.
// Sums over partial products, the convolution and the angles' products are 32-bit.
#include "common.cuh"
#include "cache_write.cuh"
#include "row_in.cuh"

namespace {

struct ConvState {
    float* state;              // [n_slots, stride]; the ring starts at off
    long long stride, off;
    const int* cu;             // [B + 1] first token of each sequence in the step
    const int* positions;      // [T]
};

// One warp per (token, head of q | k | v); the gate's logits are copied by the warps of the
// q heads.
template <typename T>
__global__ void __launch_bounds__(128)
conv_rope_store_kernel(RowIn<float> in, int n_tokens, int nh, int nkv, int hd, int hdv,
                       int taps, const float* __restrict__ conv_w, const float* __restrict__ cos_t,
                       const float* __restrict__ sin_t, int rot_dim, int gate, ConvState cs,
                       CacheWrite cw, T* __restrict__ out, long long ldo) {
    pdl_wait();
    pdl_launch_next();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int units = nh + 2 * nkv;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)n_tokens * units) return;
    const int t = (int)(item / units), u = (int)(item % units);
    const int b = cw.seq_index[t];
    const int slot = cw.slots[b];
    const int p = cs.positions[t];
    const int first = cs.cu[b];                 // the sequence's first token of this step
    const int nq = nh * hd, nk = nkv * hd, nv = nkv * hdv;
    const int C = nq + nk + nv;
    // section of this unit: 0 q, 1 k, 2 v
    const int sec = u < nh ? 0 : u < nh + nkv ? 1 : 2;
    const int head = sec == 0 ? u : sec == 1 ? u - nh : u - nh - nkv;
    const int width = sec == 2 ? hdv : hd;
    const int c0 = sec == 0 ? head * hd : sec == 1 ? nq + head * hd : nq + nk + head * hdv;
    const int ring = taps - 1;
    float* rg = slot >= 0 && ring > 0 ? cs.state + (size_t)slot * cs.stride + cs.off : nullptr;
    const bool keep = slot >= 0 && p >= cw.lens[b] - ring;      // among the sequence's last inputs
    T* orow = out + (size_t)t * ldo;

    auto conv = [&](int c) -> float {
        float y = 0.f, cur = 0.f;
        for (int j = 0; j < taps; ++j) {
            const int back = taps - 1 - j;                     // how many positions before p
            float x = 0.f;
            if (back == 0) x = cur = in.at(t, c);
            else if (p - back < 0) x = 0.f;
            else if (t - back >= first) x = in.at(t - back, c);
            else if (rg) x = rg[(size_t)((p - back) % ring) * C + c];
            y = fmaf(conv_w[(size_t)c * taps + j], x, y);
        }
        if (rg && keep) rg[(size_t)(p % ring) * C + c] = cur;
        return y;
    };

    // where k and v of this token go in the cache (null: not stored)
    T* crow = nullptr;
    if (sec != 0 && cw.k_pool && slot >= 0 && p >= cw.lens[b] - cw.cap) {
        const int r = p % cw.cap;
        const int page = cw.page_table[(size_t)slot * cw.max_pages + r / cw.page];
        const size_t at = (size_t)page * cw.page + r % cw.page;
        crow = sec == 1 ? (T*)cw.k_pool + (at * nkv + head) * hd
                        : (T*)cw.v_pool + (at * nkv + head) * hdv;
    }
    const int half = sec == 2 ? 0 : rot_dim / 2;
    for (int e = lane; e < half; e += 32) {
        const float a = conv(c0 + e), bb = conv(c0 + e + half);
        const float c = cos_t[(size_t)t * half + e], s = sin_t[(size_t)t * half + e];
        const T ra = from_f32<T>(a * c - bb * s), rb = from_f32<T>(bb * c + a * s);
        orow[c0 + e] = ra;
        orow[c0 + e + half] = rb;
        if (crow) { crow[e] = ra; crow[e + half] = rb; }
    }
    for (int e = 2 * half + lane; e < width; e += 32) {
        const T r = from_f32<T>(conv(c0 + e));
        orow[c0 + e] = r;
        if (crow) crow[e] = r;
    }
    if (gate && sec == 0)
        for (int e = lane; e < hdv; e += 32)
            orow[C + head * hdv + e] = from_f32<T>(in.at(t, C + head * hdv + e));
}

}  // namespace

// row / part: the projection [T, W] 32-bit or [n_splits, T, W] partial sums, W = C + (gate ?
// nh * hdv : 0), C = nh * hd + nkv * (hd + hdv); nkv may be 0.  conv_w [C, taps] 32-bit.
// cos, sin [T, rot_dim / 2] or null (rot_dim 0).  state: the ring of the convolution's inputs,
// (taps - 1) * C values per slot from state_off on.  out [T, ldo] receives q | k | v | g.
AGV_API int agv_conv_rope_store(const float* row, long long ld, const float* part, int n_splits,
                                int dtype, int T, int nh, int nkv, int hd, int hdv, int taps,
                                const float* conv_w, const float* cos_t, const float* sin_t,
                                int rot_dim, int gate, float* state, long long state_stride,
                                long long state_off, const int* cu_seqlens, const int* positions,
                                void* k_pool, void* v_pool, const int* page_table,
                                const int* slots, const int* lens, const int* seq_index,
                                int max_pages, int page, int cap, void* out, long long ldo,
                                cudaStream_t stream) {
    AGV_REQUIRE(T >= 0 && nh > 0 && nkv >= 0 && hd > 0 && hdv > 0 && taps >= 1,
                "conv_rope_store: bad sizes");
    AGV_REQUIRE(rot_dim >= 0 && rot_dim % 2 == 0 && rot_dim <= hd,
                "conv_rope_store: %d rotated dimensions in a head of %d", rot_dim, hd);
    AGV_REQUIRE(rot_dim == 0 || (cos_t && sin_t), "conv_rope_store: a rotation needs its tables");
    AGV_REQUIRE((row != nullptr) != (part != nullptr && n_splits > 0),
                "conv_rope_store: the projection comes as rows or as partial sums");
    const int C = nh * hd + nkv * (hd + hdv);
    const int W = C + (gate ? nh * hdv : 0);
    AGV_REQUIRE(part || ld >= W, "conv_rope_store: row stride shorter than a row");
    AGV_REQUIRE(ldo >= W, "conv_rope_store: output row stride shorter than a row");
    AGV_REQUIRE(taps == 1 || (state && state_stride >= state_off + (long long)(taps - 1) * C),
                "conv_rope_store: the state has no room for the convolution's inputs");
    AGV_REQUIRE(!k_pool || (page > 0 && cap > 0 && max_pages > 0), "conv_rope_store: bad cache "
                "geometry");
    if (T == 0) return 0;
    RowIn<float> in{row, ld, part, n_splits, (long long)T * W, W};
    ConvState cs{state, state_stride, state_off, cu_seqlens, positions};
    CacheWrite cw{k_pool, v_pool, page_table, slots, lens, seq_index, max_pages, page, cap};
    const unsigned grid = (unsigned)(((long long)T * (nh + 2 * nkv) + 3) / 4);
    if (dtype == AGV_F32)
        agv_launch(conv_rope_store_kernel<float>, grid, 128, 0, stream, in, T, nh, nkv, hd, hdv,
                   taps, conv_w, cos_t, sin_t, rot_dim, gate, cs, cw, (float*)out, ldo);
    else if (dtype == AGV_BF16)
        agv_launch(conv_rope_store_kernel<__nv_bfloat16>, grid, 128, 0, stream, in, T, nh, nkv, hd,
                   hdv, taps, conv_w, cos_t, sin_t, rot_dim, gate, cs, cw, (__nv_bfloat16*)out,
                   ldo);
    else
        return agv_fail(-1, "conv_rope_store: unknown dtype %d", dtype);
    AGV_LAUNCH_OK("conv_rope_store_kernel");
    return 0;
}
