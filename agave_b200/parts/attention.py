"""Grouped-query softmax attention over the paged cache, as a mixer part.

Interface of a mixer part (what a block needs):
  ``param_specs(spec, hidden) -> {local name: ParamSpec}``      (class method)
  ``cache_request() -> KVRequest | StateRequest | None``
  ``load(tensors, dtype, device)``
  ``forward(x [T, hidden], ctx, cache_entry, writes_cache) -> y [T, hidden]``
  (y may also be ``[S, T, hidden]`` 32-bit partial sums; the norm that follows
  adds them)

Order of operations (src/models/gemma3.zig:714-820): q, k, v projections (one
fused product here), per-head RMS norm of q and k, rotation, store of k and v,
attention with the spec's scale and window, output projection.

Prompts are attended from the step's own keys and values (every sequence of a
prompt step starts at position 0), so a window ring never has to hold a whole
prompt; decoding attends from the cache after the new key is stored (where the
sizes allow, the decode attention kernel takes the projection's partial sums and does
the norm, the rotation and that store itself).  A call
that does not write the cache reads what the owning call stored: during a
prompt step through ``ctx.step_kv``, during decoding through the cache.

Options of the spec, each a parameter of the kernels: value heads of another size
than the keys' (``value_dim``), a sink logit per query head that joins the softmax
denominator once (``sink``; tensor ``sink``), a query temperature that multiplies q by
1 + coef * ln(floor((p + 1) / every) + 1) at position p (``q_temp``), and no key / value
projections at all (``own_kv`` False: the layer attends with its own queries to the keys
and values of the cache entry the run order names); q and k normed over the whole
projection instead of head by head (``qk_norm_whole``), a sink of constant logit
(``fixed_sink``), and a learned bias by distance added to the scaled scores
(``distance_bias``; tensor ``distance_bias`` [rows, heads], expanded at load time into one
row per distance); a bias that falls linearly with distance at a slope per head
(``distance_slope``: the same table, filled from the slopes); a mask of blocks counted from
position 0 instead of a sliding window (``chunk``: the kernels take it as a negative window,
the cache as a ring that holds one block); values mixed with an earlier layer's of the same
token before they are cached (``value_mix``; tensor ``value_mix``, a scalar); the sequence's
first keys kept visible behind a sliding window (``keep_first``: the cache then keeps every
key); a short causal convolution over time on every channel of q, k and v, between the
projection and the rotation (``conv_taps``; tensors ``q_conv.weight`` ...; the last
conv_taps - 1 projected rows of a sequence live in its fixed-size state, so such a layer asks
the cache for keys and values *and* for state); and an output gate sigmoid(W_g x) on the
concatenated heads (``out_gate``; tensor ``g_proj.weight``, stacked under q | k | v).
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import kernels
from ..config.base import AttentionSpec
from ..engine.batch import DECODE, PREFILL
from .base import KVRequest, ParamSpec, StateRequest, position_class, register_mixer
from .linear import Linear


class AttentionMixer:
    def __init__(self, spec: AttentionSpec, hidden_size: int, dtype: torch.dtype,
                 device: torch.device):
        if spec.n_heads % spec.n_kv_heads:
            raise ValueError("n_heads must be a multiple of n_kv_heads")
        self.spec, self.hidden_size, self.dtype, self.device = spec, hidden_size, dtype, device
        self.position = (position_class(spec.position.kind)(spec.position, spec.head_dim)
                         if spec.position is not None else None)
        self.qkv: Optional[Linear] = None
        self.out: Optional[Linear] = None
        self.q_norm_weight = self.k_norm_weight = None
        self.sinks: Optional[torch.Tensor] = None
        self.own_kv = bool(getattr(spec, "own_kv", True))
        self.value_dim = int(getattr(spec, "value_dim", 0) or spec.head_dim)
        qt = getattr(spec, "q_temp", None)
        self.q_temp = (float(qt.coef), int(qt.every)) if qt is not None and qt.coef != 0 else None
        if self.q_temp is not None and self.q_temp[1] < 1:
            raise ValueError("the query temperature's period must be at least 1")
        self.whole_norm = bool(getattr(spec, "qk_norm_whole", False))
        self.dist_spec = getattr(spec, "distance_bias", None)
        self.dist_bias: Optional[torch.Tensor] = None
        fixed = getattr(spec, "fixed_sink", None)
        self.fixed_sink = None if fixed is None else float(fixed)
        self.slope_spec = getattr(spec, "distance_slope", None)
        self.chunk = getattr(spec, "chunk", None)
        self.value_mix = getattr(spec, "value_mix", None)
        self.mix_weight = 0.0
        self.keep_first = int(getattr(spec, "keep_first", 0) or 0)
        self.conv_taps = int(getattr(spec, "conv_taps", 0) or 0)
        self.out_gate = bool(getattr(spec, "out_gate", False))
        self.conv_w: Optional[torch.Tensor] = None
        if self.keep_first < 0 or self.conv_taps < 0:
            raise ValueError("keep_first and conv_taps cannot be negative")
        if self.keep_first and self.chunk is not None:
            raise ValueError("kept first keys go with a sliding window, not with a mask of blocks")
        if (self.conv_taps or self.out_gate) and (
                spec.qk_norm is not None or self.q_temp is not None or self.value_mix is not None
                or (self.position is not None and getattr(self.position, "interleaved", False))):
            raise ValueError("a convolution on q, k and v or an output gate goes without q/k "
                             "norms, a query temperature or mixed values")
        if self.chunk is not None and (self.chunk < 1 or spec.window is not None):
            raise ValueError("a mask of blocks needs a positive size and goes without a window")
        if self.slope_spec is not None and (self.dist_spec is not None or
                                            self.slope_spec.reach < 1):
            raise ValueError("a bias by distance is either a learned table or a slope per head, "
                             "and a slope needs the greatest distance a query can see")
        if self.value_mix is not None and not self.whole_norm:
            raise ValueError("mixed values go with the norm over the whole projection (its "
                             "kernel mixes them)")
        if self.whole_norm and (spec.qk_norm is None or self.position is not None or
                                self.q_temp is not None or not self.own_kv):
            raise ValueError("a norm over the whole projection needs qk_norm and goes without a "
                             "rotation, a query temperature or borrowed keys and values")
        if self.fixed_sink is not None and getattr(spec, "sink", False):
            raise ValueError("a sink is either learned or a constant, not both")
        if self.position is not None and getattr(self.position, "interleaved", False):
            raise ValueError("this mixer rotates split halves only")
        # the options the standard kernels' callers do not pass
        self.plain = (self.own_kv and self.value_dim == spec.head_dim and self.q_temp is None
                      and not getattr(spec, "sink", False) and not self.whole_norm
                      and self.dist_spec is None and self.fixed_sink is None
                      and self.slope_spec is None and self.chunk is None
                      and self.value_mix is None and not self.keep_first
                      and not self.conv_taps and not self.out_gate)

    @classmethod
    def param_specs(cls, spec: AttentionSpec, hidden_size: int) -> Dict[str, ParamSpec]:
        q, kv = spec.n_heads * spec.head_dim, spec.n_kv_heads * spec.head_dim
        vd = getattr(spec, "value_dim", 0) or spec.head_dim
        own_kv = getattr(spec, "own_kv", True)
        p = {"q_proj.weight": ParamSpec((q, hidden_size))}
        if own_kv:
            p["k_proj.weight"] = ParamSpec((kv, hidden_size))
            p["v_proj.weight"] = ParamSpec((spec.n_kv_heads * vd, hidden_size))
        p["o_proj.weight"] = ParamSpec((hidden_size, spec.n_heads * vd))
        if spec.qk_norm is not None:
            zc = spec.qk_norm.zero_centered
            whole = getattr(spec, "qk_norm_whole", False)
            p["q_norm.weight"] = ParamSpec((q if whole else spec.head_dim,), "norm",
                                           zero_centered=zc)
            if own_kv:
                p["k_norm.weight"] = ParamSpec((kv if whole else spec.head_dim,), "norm",
                                               zero_centered=zc)
        if getattr(spec, "sink", False):
            p["sink"] = ParamSpec((spec.n_heads,), "float32")
        db = getattr(spec, "distance_bias", None)
        if db is not None:
            p["distance_bias"] = ParamSpec((db.rows, spec.n_heads), "float32")
        if getattr(spec, "value_mix", None) is not None:
            p["value_mix"] = ParamSpec((), "float32")
        taps = int(getattr(spec, "conv_taps", 0) or 0)
        if taps:
            p["q_conv.weight"] = ParamSpec((q, taps), "float32")
            if own_kv:
                p["k_conv.weight"] = ParamSpec((kv, taps), "float32")
                p["v_conv.weight"] = ParamSpec((spec.n_kv_heads * vd, taps), "float32")
        if getattr(spec, "out_gate", False):
            p["g_proj.weight"] = ParamSpec((spec.n_heads * vd, hidden_size))
        return p

    @staticmethod
    def distance_rows(rows: int, far: float, n: int):
        """The table row of each distance 0..n-1: a row each for the first rows/2 distances,
        then rows that grow logarithmically and end at ``far``."""
        half = rows // 2
        out = []
        for dist in range(n):
            if dist < half:
                out.append(dist)
            else:
                out.append(min(rows - 1, half + int(math.floor(
                    math.log(dist / half) / math.log(far / half) * (rows - half)))))
        return out

    def cache_request(self):
        if not self.own_kv:
            return None
        # (a mask of blocks needs the keys of one block: a ring of that many rows; a window
        # behind which the first keys stay visible keeps every key)
        window = self.chunk if self.chunk is not None else self.spec.window
        if self.keep_first or getattr(self.spec, "keep_all_keys", False):
            window = None
        kv = KVRequest(self.spec.n_kv_heads, self.spec.head_dim, window,
                       0 if self.value_dim == self.spec.head_dim else self.value_dim)
        st = self.state_request()
        return kv if st is None else (kv, st)

    def state_request(self):
        """The fixed-size state of a sequence: the convolution's last conv_taps - 1 inputs (a
        layer without keys and values of its own keeps those of its queries)."""
        if self.conv_taps <= 1:
            return None
        return StateRequest((self.conv_taps - 1) * self._conv_channels())

    def _conv_channels(self) -> int:
        s = self.spec
        n_own = s.n_kv_heads if self.own_kv else 0
        return s.n_heads * s.head_dim + n_own * (s.head_dim + self.value_dim)

    def load(self, tensors: Dict[str, torch.Tensor], dtype: torch.dtype,
             device: torch.device) -> None:
        def mat(name):
            return tensors[name].to(device=device, dtype=dtype)
        # one product for q | k | v: rows of q first, then k, then v (q alone for a layer
        # without keys and values of its own)
        stack = [mat("q_proj.weight")]
        if self.own_kv:
            stack += [mat("k_proj.weight"), mat("v_proj.weight")]
        if self.out_gate:
            stack.append(mat("g_proj.weight"))
        self.qkv = Linear(torch.cat(stack, dim=0).contiguous() if len(stack) > 1 else
                          stack[0].contiguous(), role="qkv")
        if self.conv_taps or self.out_gate:
            def f32(name):
                return tensors[name].to(device=device, dtype=torch.float32)
            if self.conv_taps:
                names = ["q_conv.weight"] + (["k_conv.weight", "v_conv.weight"]
                                             if self.own_kv else [])
                self.conv_w = torch.cat([f32(n) for n in names], dim=0).contiguous()
            else:
                self.conv_w = torch.ones((self._conv_channels(), 1), dtype=torch.float32,
                                         device=device)
        self.out = Linear(mat("o_proj.weight").contiguous(), role="out_proj")
        if self.spec.qk_norm is not None:
            add = 1.0 if self.spec.qk_norm.zero_centered else 0.0
            self.q_norm_weight = (tensors["q_norm.weight"].to(device=device, dtype=torch.float32)
                                  + add).contiguous()
            if self.own_kv:
                self.k_norm_weight = (tensors["k_norm.weight"].to(device=device,
                                                                  dtype=torch.float32)
                                      + add).contiguous()
        if getattr(self.spec, "sink", False):
            self.sinks = tensors["sink"].to(device=device, dtype=torch.float32).contiguous()
        if self.fixed_sink is not None:
            self.sinks = torch.full((self.spec.n_heads,), self.fixed_sink, dtype=torch.float32,
                                    device=device)
        if self.dist_spec is not None:
            # one row per distance a query can see; the last row stands for all farther ones
            # (from ``far`` on every distance has the table's last row)
            db = self.dist_spec
            n = int(math.ceil(db.far)) + 1
            if self.spec.window:
                n = min(n, int(self.spec.window))
            idx = torch.tensor(self.distance_rows(db.rows, db.far, max(n, 1)), device=device)
            table = tensors["distance_bias"].to(device=device, dtype=torch.float32)
            self.dist_bias = table[idx].t().contiguous()          # [heads, distances]
        if self.slope_spec is not None:
            # the same table from the slopes: entry [a, n] = -slope_a * n, made in 64-bit
            sl = self.slope_spec
            n = int(sl.reach) if self.chunk is None else min(int(sl.reach), int(self.chunk))
            heads = torch.arange(1, self.spec.n_heads + 1, dtype=torch.float64)
            slopes = torch.pow(torch.tensor(2.0, dtype=torch.float64),
                               -float(sl.exponent) * heads / self.spec.n_heads)
            dist = torch.arange(max(n, 1), dtype=torch.float64)
            self.dist_bias = (-(slopes[:, None] * dist[None, :])).to(
                device=device, dtype=torch.float32).contiguous()
        if self.value_mix is not None and self.value_mix.source is not None:
            self.mix_weight = float(tensors["value_mix"].to(torch.float32).reshape(()).item())

    def forward(self, x: torch.Tensor, ctx, cache_entry: int, writes_cache: bool) -> torch.Tensor:
        if self.conv_taps or self.out_gate:
            return self._forward_conv(x, ctx, cache_entry, writes_cache)
        if not self.plain:
            return self._forward_options(x, ctx, cache_entry, writes_cache)
        s = self.spec
        nh, nkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        T = x.shape[0]
        cos = sin = None
        rotary_dim = 0
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary_dim = self.position.rotary_dim
        view = ctx.cache.kv_view(cache_entry)
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        window = s.window or 0
        if ctx.mode == PREFILL and kernels.qkv_prefill_supported(x, self.qkv.weight, hd,
                                                                 rotary_dim):
            # a prompt step on the tensor cores: norm, rotation, the cache store and the
            # transposed values are the epilogue of the q/k/v product
            qkv = ctx.new(T, (nh + 2 * nkv) * hd)
            vt = None
            if writes_cache and kernels.attention_prefill_wants_transposed_values(qkv, hd):
                vt = kernels.prefill_values_scratch(T, ctx.batch, nkv, hd, qkv.device)
            pools = dict(k_pool=view.k_pool, v_pool=view.v_pool, page_table=view.page_table,
                         slots=ctx.slots, lens=ctx.lens, page=view.page,
                         cap=view.cap) if writes_cache else {}
            kernels.qkv_prefill(x, self.qkv.weight, qkv, nh, nkv, hd, self.q_norm_weight,
                                self.k_norm_weight, eps, cos, sin, ctx.positions, ctx.seq_index,
                                vt=vt, cu_seqlens=ctx.cu_seqlens, **pools)
            return self._attend_prompt(qkv, vt, ctx, cache_entry, writes_cache, window)
        proj = self.qkv.partial(x, cheap_sum=True)
        part = proj if proj.dim() == 3 else None
        if (ctx.mode == DECODE and part is not None and
                kernels.attention_decode_fused_supported(self.dtype, hd, rotary_dim)):
            # decoding: norm, rotation and the store of the new key and value happen inside
            # the attention kernel, on the projection's partial sums
            out = ctx.new(T, nh * hd)
            kernels.attention_decode_fused(part, self.q_norm_weight, self.k_norm_weight, eps, cos,
                                           sin, writes_cache, out, view, ctx, nh, nkv, hd, s.scale,
                                           window)
            return self.out.partial(out)
        qkv = proj if part is None else ctx.new(T, (nh + 2 * nkv) * hd)
        if writes_cache:
            # a prompt step on the tcgen05 attention kernel reads the values transposed:
            # the same launch writes that copy
            vt = None
            if ctx.mode == PREFILL and kernels.attention_prefill_wants_transposed_values(qkv, hd):
                vt = kernels.prefill_values_scratch(T, ctx.batch, nkv, hd, qkv.device)
            kernels.qk_norm_rope_store(
                qkv, nh, nkv, hd, self.q_norm_weight, self.k_norm_weight, eps, cos, sin,
                rotary_dim, ctx.positions, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                ctx.lens, ctx.seq_index, view.page, view.cap, partial=part, vt=vt,
                cu_seqlens=ctx.cu_seqlens, max_len=ctx.max_new)
        else:
            kernels.qk_norm_rope_store(qkv, nh, nkv, hd, self.q_norm_weight, self.k_norm_weight,
                                       eps, cos, sin, rotary_dim, ctx.positions, partial=part)
        if ctx.mode == PREFILL:
            return self._attend_prompt(qkv, vt if writes_cache else None, ctx, cache_entry,
                                       writes_cache, window)
        out = ctx.new(T, nh * hd)
        kernels.attention_decode(qkv[:, :nh * hd], out, view, ctx, nh, nkv, hd, s.scale, window)
        return self.out.partial(out)

    def _forward_options(self, x: torch.Tensor, ctx, cache_entry: int,
                         writes_cache: bool) -> torch.Tensor:
        """The same flow for a spec with a sink, a query temperature, value heads of their
        own size or no keys and values of its own: the projection's 32-bit sums are normed,
        rotated, tempered and rounded once; keys and values go to the cache; prompts attend
        from the step's tensors and decoding from the cache."""
        s = self.spec
        nh, nkv, hd, hdv = s.n_heads, s.n_kv_heads, s.head_dim, self.value_dim
        if writes_cache != self.own_kv:
            raise ValueError("a layer without key / value projections must read another call's "
                             "cache entry, and one with them must write its own")
        T = x.shape[0]
        cos = sin = None
        rotary_dim = 0
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary_dim = self.position.rotary_dim
        view = ctx.cache.kv_view(cache_entry)
        eps = s.qk_norm.eps if s.qk_norm is not None else 0.0
        window = s.window or 0
        if self.chunk is not None:
            window = -int(self.chunk)
        if abs(window) >= ctx.cache.max_seq_len:
            # a window (or block) no sequence of this cache can outgrow is none (its group
            # keeps every key, in rows that may be fewer than the window)
            window = 0
        n_own = nkv if self.own_kv else 0
        width = (nh + n_own) * hd + n_own * hdv
        proj = self.qkv.partial(x, cheap_sum=True)
        part = proj if proj.dim() == 3 else None
        if (ctx.mode == DECODE and part is not None and hdv == hd and not self.whole_norm and
                self.dist_bias is None and not self.keep_first and
                kernels.attention_decode_fused_supported(self.dtype, hd, rotary_dim)):
            out = ctx.new(T, nh * hdv)
            kernels.attention_decode_fused(part, self.q_norm_weight, self.k_norm_weight, eps, cos,
                                           sin, self.own_kv, out, view, ctx, nh, nkv, hd, s.scale,
                                           window, sinks=self.sinks, q_temp=self.q_temp,
                                           q_only=not self.own_kv)
            return self.out.partial(out)
        qkv = proj if part is None else ctx.new(T, width)
        vt = None
        if self.whole_norm:
            v_first = None
            if self.value_mix is not None and self.value_mix.source is not None:
                v_first = ctx.step_values[self.value_mix.source]
            kernels.proj_norm_store(qkv, nh * hd, nkv * hd, nkv * hdv, self.q_norm_weight,
                                    self.k_norm_weight, eps, ctx.positions, view, ctx,
                                    partial=part, v_first=v_first, v_mix=self.mix_weight)
            if self.value_mix is not None and self.value_mix.source is None:
                # the values as projected, for the layers that lean on them
                ctx.step_values[cache_entry] = qkv[:, (nh + nkv) * hd:]
        elif self.own_kv:
            if ctx.mode == PREFILL and kernels.attention_prefill_wants_transposed_values(
                    qkv, hd, hdv):
                vt = kernels.prefill_values_scratch(T, ctx.batch, nkv, hd, qkv.device)
            kernels.qk_norm_rope_store(
                qkv, nh, nkv, hd, self.q_norm_weight, self.k_norm_weight, eps, cos, sin,
                rotary_dim, ctx.positions, view.k_pool, view.v_pool, view.page_table, ctx.slots,
                ctx.lens, ctx.seq_index, view.page, view.cap, partial=part, vt=vt,
                cu_seqlens=ctx.cu_seqlens, max_len=ctx.max_new, value_dim=hdv,
                q_temp=self.q_temp)
        else:
            kernels.qk_norm_rope_store(qkv, nh, 0, hd, self.q_norm_weight, None, eps, cos, sin,
                                       rotary_dim, ctx.positions, partial=part, value_dim=hdv,
                                       q_temp=self.q_temp)
        q = qkv[:, :nh * hd]
        out = ctx.new(T, nh * hdv)
        if ctx.mode == PREFILL:
            if self.own_kv:
                k = qkv[:, nh * hd:(nh + nkv) * hd]
                v = qkv[:, (nh + nkv) * hd:]
                ctx.step_kv[cache_entry] = (k, v, vt)
            else:
                k, v, vt = ctx.step_kv[cache_entry]
            kernels.attention_prefill(q, k, v, out, ctx, nh, nkv, hd, s.scale, window, vt=vt,
                                      value_dim=hdv, sinks=self.sinks, dist_bias=self.dist_bias,
                                      keep_first=self.keep_first)
        else:
            kernels.attention_decode(q, out, view, ctx, nh, nkv, hd, s.scale, window,
                                     value_dim=hdv, sinks=self.sinks, dist_bias=self.dist_bias,
                                     keep_first=self.keep_first)
        return self.out.partial(out)

    def _forward_conv(self, x: torch.Tensor, ctx, cache_entry: int,
                      writes_cache: bool) -> torch.Tensor:
        """The flow of a layer with a convolution on q, k and v or an output gate: one stacked
        product q | k | v | g into 32-bit sums; one row kernel (convolution from the step's
        rows and the sequence's stored inputs, rotation, cache store, everything rounded once);
        attention from the step's tensors (prompts) or the cache (decoding); the gate; the
        output product."""
        from .matrix_memory import project_f32
        s = self.spec
        nh, nkv, hd, hdv = s.n_heads, s.n_kv_heads, s.head_dim, self.value_dim
        if writes_cache != self.own_kv:
            raise ValueError("a layer without key / value projections must read another call's "
                             "cache entry, and one with them must write its own")
        T = x.shape[0]
        cos = sin = None
        rotary_dim = 0
        if self.position is not None:
            cos, sin = self.position.tables(ctx)
            rotary_dim = self.position.rotary_dim
        view = ctx.cache.kv_view(cache_entry)
        window = s.window or 0
        if self.chunk is not None:
            window = -int(self.chunk)
        if abs(window) >= ctx.cache.max_seq_len:
            window = 0
        n_own = nkv if self.own_kv else 0
        C = (nh + n_own) * hd + n_own * hdv
        row, part = project_f32(self.qkv, x)
        qkvg = ctx.new(T, C + (nh * hdv if self.out_gate else 0))
        state = None
        taps = max(self.conv_taps, 1)
        if taps > 1:
            entry = cache_entry if self.own_kv else getattr(ctx, "state_entry", None)
            if entry is None:
                raise ValueError("a layer that borrows its keys and values needs a cache entry "
                                 "for the state of its own convolution")
            state = ctx.cache.state_view(entry).state
        kernels.conv_rope_store(row, part, qkvg, nh, n_own, hd, hdv, taps, self.conv_w, cos, sin,
                                rotary_dim, self.out_gate, state, 0, ctx,
                                view if self.own_kv else None)
        q = qkvg[:, :nh * hd]
        out = ctx.new(T, nh * hdv)
        if ctx.mode == PREFILL:
            if self.own_kv:
                k = qkvg[:, nh * hd:(nh + nkv) * hd]
                v = qkvg[:, (nh + nkv) * hd:C]
                ctx.step_kv[cache_entry] = (k, v, None)
            else:
                k, v, _ = ctx.step_kv[cache_entry]
            kernels.attention_prefill(q, k, v, out, ctx, nh, nkv, hd, s.scale, window,
                                      value_dim=hdv, sinks=self.sinks, dist_bias=self.dist_bias,
                                      keep_first=self.keep_first)
        else:
            kernels.attention_decode(q, out, view, ctx, nh, nkv, hd, s.scale, window,
                                     value_dim=hdv, sinks=self.sinks, dist_bias=self.dist_bias,
                                     keep_first=self.keep_first)
        if self.out_gate:
            kernels.gate_sigmoid(out, qkvg[:, C:])
        return self.out.partial(out)

    def _attend_prompt(self, qkv: torch.Tensor, vt, ctx, cache_entry: int, writes_cache: bool,
                       window: int) -> torch.Tensor:
        """Prompt attention from the step's own keys and values, then the output projection."""
        s = self.spec
        nh, nkv, hd = s.n_heads, s.n_kv_heads, s.head_dim
        if writes_cache:
            k = qkv[:, nh * hd:(nh + nkv) * hd]
            v = qkv[:, (nh + nkv) * hd:]
            ctx.step_kv[cache_entry] = (k, v, vt)
        else:
            k, v, vt = ctx.step_kv[cache_entry]
        out = ctx.new(qkv.shape[0], nh * hd)
        kernels.attention_prefill(qkv[:, :nh * hd], k, v, out, ctx, nh, nkv, hd, s.scale, window,
                                  vt=vt)
        return self.out.partial(out)


register_mixer("attention", AttentionMixer)
