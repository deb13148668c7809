"""Kadavik on the GPU against the plain implementation (tests/plain/kadavik_plain.py): each
mechanism alone, then whole models of three small configurations through the engine: the
stream after every layer, whole prompts, the last tokens one by one, unequal batches against
each request alone, slots, pages and states used again, lengths round page borders and window
edges, long decoding, greedy generation through the scheduler, and trace replay as a process.

Where random weights would hide a fault, the inputs are made so that it shows: one key (at the
window's last place, just behind it, the last kept first key, the one after it, or far back
among hundreds) gets a score that stands out, so an output that includes or misses the wrong
one is far off; the matrix memory's forget gates are set close to one and one far token's
input gate high, so that what was written hundreds of tokens ago still decides the read-out.
"""
import json
import math
import os
import shutil
import subprocess
import sys
import tempfile

import numpy as np
import pytest
import torch

from kadavik_util import CONFIGS, folder_for, plain_logits, tokens
from plain import kadavik_plain as P
from util import ROOT

pytestmark = pytest.mark.gpu
DEV = "cuda"
DTYPES = ["float32", "bfloat16"]
TD = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def rel_err(got, ref):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    return ((got - ref).abs().max() / ref.abs().max().clamp_min(1e-30)).item()


def rows_agree(got, ref, dtype, what=""):
    """Logit rows against reference rows: max error over the row's greatest logit.  32-bit:
    every row within 3e-4, which is the sharp comparison.  bfloat16: the test models' weights
    are strong, so that faults show, and one rounding can move a whole row (an expert chosen
    by a close call); so all but one row in twenty-five (at least two) within 0.12, and every
    row of the right size."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all()
    err = (got - ref).abs().amax(dim=1) / ref.abs().amax(dim=1)
    worst = f"{what}: row {err.argmax().item()} of {len(err)} off by {err.max().item():.2e}"
    if dtype == "float32":
        assert err.max().item() <= 3e-4, worst
    else:
        assert err.max().item() <= 1.0, worst
        over = int((err > 0.12).sum().item())
        assert over <= max(2, len(err) // 25), f"{what}: {over} of {len(err)} rows off; " + worst


def rnd(*shape, seed=0, std=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * std


def summed(y):
    """A part's output: [T, H], or partial sums [S, T, H] the block adds up."""
    return y.float().sum(dim=0) if y.dim() == 3 else y.float()


class _Cache:
    """A cache of one entry and step contexts over it, as a mixer finds them."""

    def __init__(self, request, n_seqs, td, room=4096):
        from agave_b200.cache import Cache
        self.cache = Cache([request], room * (n_seqs + 1), room, n_seqs + 2, td,
                           torch.device(DEV))
        self.td = td
        spare = self.cache.acquire()          # slots in another order than the batch
        self.slots = [self.cache.acquire() for _ in range(n_seqs)]
        self.cache.release(spare)
        self.lens = [0] * n_seqs

    def step(self, new, live=None):
        """A context in which sequence b brings ``new[b]`` more tokens (``live``: which)."""
        from agave_b200.engine.batch import DECODE, PREFILL, StepContext
        live = list(range(len(self.slots))) if live is None else live
        i32 = dict(dtype=torch.int32, device=DEV)
        pos, seq, cu, lens = [], [], [0], []
        starts = [self.lens[b] for b in live]
        for r, (b, k) in enumerate(zip(live, new)):
            self.cache.reserve(self.slots[b], self.lens[b] + k)
            pos += list(range(self.lens[b], self.lens[b] + k))
            self.lens[b] += k
            self.cache.book.set_length(self.slots[b], self.lens[b])
            lens.append(self.lens[b])
            seq += [r] * k
            cu.append(cu[-1] + k)
        self.cache.flush()
        mode = DECODE if max(new) == 1 and min(starts) > 0 else PREFILL
        return StepContext(mode=mode, n_tokens=len(pos), batch=len(live), tokens=None,
                           positions=torch.tensor(pos, **i32), seq_index=torch.tensor(seq, **i32),
                           cu_seqlens=torch.tensor(cu, **i32),
                           slots=torch.tensor([self.slots[b] for b in live], **i32),
                           lens=torch.tensor(lens, **i32), max_len=max(lens),
                           max_new=max(new), cache=self.cache, dtype=self.td,
                           device=torch.device(DEV), state_entry=0)

    def again(self, b):
        """Sequence b ends; another takes a slot (the freed one or the spare)."""
        self.cache.release(self.slots[b])
        self.slots[b] = self.cache.acquire()
        self.lens[b] = 0


# ------------------------------------------------------------ small mechanisms
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, n, wide", [(1, 5, 35), (70, 16, 16), (300, 24, 120)])
def test_token_rows_gated_by_the_gelu_of_a_projection(dtype, T, n, wide):
    from agave_b200 import kernels
    td = TD[dtype]
    z = rnd(T, n, seed=1, std=1.5).float()
    table = rnd(T, wide, seed=2).float()
    off = wide - n
    out = torch.empty(T, n, dtype=td, device=DEV)
    kernels.gelu_mul_rows(z.to(DEV), table.to(DEV)[:, off:off + n], out)
    ref = P.gelu_tanh(z.double()) * table.double()[:, off:off + n]
    assert rel_err(out, ref) < (1e-6 if dtype == "float32" else 6e-3)


def test_scaled_frequencies_on_the_device_tables():
    """cos and sin of a rotation whose frequencies are scaled band by band, against the plain
    list of frequencies, at positions up to a few thousand."""
    from agave_b200.config.base import BandScalingSpec, RotarySpec
    from agave_b200.engine.batch import PREFILL, StepContext
    from agave_b200.parts.rope import RotaryEmbedding
    dims, base, sc = 32, 500.0, (4.0, 2.0, 8.0, 64)
    rope = RotaryEmbedding(RotarySpec(theta=base, rotary_dim=dims, scaling=BandScalingSpec(
        factor=sc[0], low=sc[1], high=sc[2], original=sc[3])), 48)
    pos = torch.tensor([0, 1, 2, 77, 1000, 4099], dtype=torch.int32, device=DEV)
    ctx = StepContext(mode=PREFILL, n_tokens=6, batch=1, tokens=None, positions=pos,
                      seq_index=None, cu_seqlens=None, slots=None, lens=None, max_len=0,
                      max_new=0, cache=None, dtype=torch.float32, device=torch.device(DEV))
    cos, sin = rope.tables(ctx)
    f = torch.tensor(P.scaled_frequencies(dims, base, dict(zip(
        ("factor", "low", "high", "original"), sc))), dtype=torch.float64)
    a = pos.cpu().double()[:, None] * f[None, :]
    assert (cos.cpu().double() - torch.cos(a)).abs().max() < 1e-6
    assert (sin.cpu().double() - torch.sin(a)).abs().max() < 1e-6
    # the three bands are all there: a kept, a blended and a divided frequency
    plain = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    ratios = [x / y for x, y in zip(f.tolist(), plain)]
    assert ratios[0] == 1.0 and abs(ratios[-1] - 1 / sc[0]) < 1e-12
    assert any(1 / sc[0] + 1e-6 < r < 1 - 1e-6 for r in ratios)


def _moe_weights(H, E, I, ff, shared, seed, td):
    lin = 1.0 / H ** 0.5
    W = {"router": rnd(E + I, H, seed=seed, std=3.0 * lin), "correction": rnd(E + I, seed=seed + 1,
                                                                              std=0.05)}
    for e in range(E):
        W[f"e{e}.gate"] = rnd(ff, H, seed=seed + 10 + 3 * e, std=1.5 * lin)
        W[f"e{e}.up"] = rnd(ff, H, seed=seed + 11 + 3 * e, std=1.5 * lin)
        W[f"e{e}.down"] = rnd(H, ff, seed=seed + 12 + 3 * e, std=1.0 / ff ** 0.5)
    if shared:
        W["shared.gate"] = rnd(shared, H, seed=seed + 5, std=1.5 * lin)
        W["shared.up"] = rnd(shared, H, seed=seed + 6, std=1.5 * lin)
        W["shared.down"] = rnd(H, shared, seed=seed + 7, std=1.0 / shared ** 0.5)
        W["shared.sg"] = rnd(1, H, seed=seed + 8, std=2.0 * lin)
    return {k: v.to(td) for k, v in W.items()}


def _moe_part(W, H, E, I, top, ff, shared, scale, td):
    from agave_b200.config.base import RoutedFeedForwardSpec
    from agave_b200.parts.moe import RoutedFeedForward
    spec = RoutedFeedForwardSpec(n_experts=E, top=top, intermediate_size=ff, activation="silu",
                                 correction=True, weighting="softmax_all", route_scale=scale,
                                 n_identity=I, shared_size=shared)
    part = RoutedFeedForward(spec, H, td, torch.device(DEV))
    t = {"router.weight": W["router"], "router.correction": W["correction"]}
    for e in range(E):
        for n in ("gate", "up", "down"):
            t[f"experts.{e}.{n}_proj.weight"] = W[f"e{e}.{n}"]
    if shared:
        for n in ("gate", "up", "down"):
            t[f"shared.{n}_proj.weight"] = W[f"shared.{n}"]
        t["shared.gate.weight"] = W["shared.sg"]
    assert set(t) == set(RoutedFeedForward.param_specs(spec, H))
    part.load(t, td, torch.device(DEV))
    return part


MOE = [(1, 72, 5, 1, 2, 24, 0, 1.5), (40, 96, 1, 0, 1, 32, 0, 1.0), (33, 128, 4, 0, 4, 64, 8, 1.0),
       (200, 128, 7, 2, 3, 64, 96, 2.5), (130, 80, 3, 3, 2, 16, 20, 0.7), (9, 64, 2, 4, 6, 24, 0, 2.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, E, I, top, ff, shared, scale", MOE)
def test_router_with_softmax_scores_and_identity_experts(dtype, T, H, E, I, top, ff, shared, scale):
    """Scores are the softmax over experts and identities together, the correction only
    chooses, the chosen scores are renormalised and scaled.  Tokens whose choice is a close
    call are left out of the comparison of ids."""
    td = TD[dtype]
    W = _moe_weights(H, E, I, ff, shared, 300 + T, td)
    x = rnd(T, H, seed=301).to(td)
    part = _moe_part(W, H, E, I, top, ff, shared, scale, td)
    ids, wts = part.route(x.to(DEV))
    f = {"router": {"experts": E, "identity": I, "top": top, "scale": scale}}
    Wd = {k: v.double() for k, v in W.items()}
    ref_ids, ref_w = P.route(x.double(), f, Wd, "")
    s = torch.softmax(x.double() @ Wd["router"].T, -1) + Wd["correction"]
    srt = s.sort(-1, descending=True).values
    clear = torch.ones(T, dtype=torch.bool) if top == E + I else \
        (srt[:, top - 1] - srt[:, top]) > 1e-5      # (both read the same rounded inputs)
    assert clear.sum() >= T // 2
    got_sets = [set(r) for r in ids.cpu().tolist()]
    for t in range(T):
        if clear[t]:
            assert got_sets[t] == set(ref_ids[t].tolist()), t
            order = {e: k for k, e in enumerate(ids[t].cpu().tolist())}
            mine = torch.tensor([wts[t, order[int(e)]].item() for e in ref_ids[t]])
            assert (mine.double() - ref_w[t]).abs().max() < 3e-6 * scale
    assert abs(wts.sum(-1).double().cpu() - scale).max() < 1e-4 * scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, E, I, top, ff, shared, scale", MOE)
def test_routed_experts_identities_and_a_gated_shared_one(dtype, T, H, E, I, top, ff, shared,
                                                          scale):
    """The whole feed-forward under the experts the library chose: grouped products, the rows
    of identity pairs, the shared expert times its gate, summed."""
    td = TD[dtype]
    W = _moe_weights(H, E, I, ff, shared, 400 + T, td)
    x = rnd(T, H, seed=401).to(td)
    part = _moe_part(W, H, E, I, top, ff, shared, scale, td)
    ids, _ = part.route(x.to(DEV))
    y = summed(part.forward(x.to(DEV), None))
    f = {"router": {"experts": E, "identity": I, "top": top, "scale": scale},
         "shared": {"ff": shared} if shared else None}
    ref = P.moe(x.double(), f, {k: v.double() for k, v in W.items()}, "", chosen=ids.cpu().long())
    assert rel_err(y, ref) < (2e-5 if dtype == "float32" else 3e-2)


# ------------------------------------------------------------ matrix memory
def _mlstm_weights(A, d, dv, H, seed, td, forget=4.0):
    lin = 1.0 / H ** 0.5
    W = {"q": rnd(A * d, H, seed=seed, std=1.5 * lin), "k": rnd(A * d, H, seed=seed + 1, std=1.5 * lin),
         "v": rnd(A * dv, H, seed=seed + 2, std=lin), "g": rnd(A * dv, H, seed=seed + 3, std=1.5 * lin),
         "i": rnd(A, H, seed=seed + 4, std=2.0 * lin), "i.b": rnd(A, seed=seed + 5, std=0.5),
         "f": rnd(A, H, seed=seed + 6, std=lin), "f.b": rnd(A, seed=seed + 7, std=0.5) + forget,
         "norm": rnd(A * dv, seed=seed + 8, std=0.3) + 1.0,
         "o": rnd(H, A * dv, seed=seed + 9, std=1.0 / (A * dv) ** 0.5)}
    return {k: v.to(td) for k, v in W.items()}


def _mlstm_part(W, A, d, dv, H, cap, td, eps=1e-5):
    from agave_b200.config.base import MatrixMemorySpec
    from agave_b200.parts.matrix_memory import MatrixMemoryMixer
    spec = MatrixMemorySpec(n_heads=A, head_dim=d, value_dim=dv, gate_cap=cap, eps=eps)
    part = MatrixMemoryMixer(spec, H, td, torch.device(DEV))
    t = {"q_proj.weight": W["q"], "k_proj.weight": W["k"], "v_proj.weight": W["v"],
         "g_proj.weight": W["g"], "i_proj.weight": W["i"], "i_proj.bias": W["i.b"],
         "f_proj.weight": W["f"], "f_proj.bias": W["f.b"], "out_norm.weight": W["norm"],
         "o_proj.weight": W["o"]}
    assert set(t) == set(MatrixMemoryMixer.param_specs(spec, H))
    part.load(t, td, torch.device(DEV))
    return part


MLSTM = [(3, 12, 10, 72, 8.0), (4, 64, 64, 128, 12.0), (1, 16, 48, 96, 1.0), (2, 20, 6, 80, 15.0),
         (2, 128, 128, 64, 5.0), (1, 200, 24, 40, 3.0), (5, 8, 8, 48, 30.0)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("A, d, dv, H, cap", MLSTM)
def test_matrix_memory_as_prompt_in_portions_and_token_by_token(dtype, A, d, dv, H, cap):
    """The mixer alone against the plain one: the whole sequence in one step; a prompt and
    then tokens one by one; portions down to two tokens (each going on from the state the one
    before left)."""
    td = TD[dtype]
    T = 90
    W = _mlstm_weights(A, d, dv, H, 70, td)
    h = rnd(T, H, seed=71).to(td)
    m = {"heads": A, "dim": d, "vdim": dv, "gate_cap": cap}
    ref = P.mlstm_mixer(h.double(), m, {k: v.double() for k, v in W.items()}, "", 1e-5)
    part = _mlstm_part(W, A, d, dv, H, cap, td)
    tol = 5e-5 if dtype == "float32" else 4e-2
    for new in ([T], [50] + [1] * 40, [1] * 12 + [78], [2, 1, 3, 37, 47], [17, 16, 2, 55]):
        oc = _Cache(part.cache_request(), 1, td)
        got, at = [], 0
        for n in new:
            got.append(summed(part.forward(h[at:at + n].to(DEV), oc.step([n]), 0, True)))
            at += n
        assert rel_err(torch.cat(got), ref) < tol, new[:3]


@pytest.mark.parametrize("dtype", DTYPES)
def test_matrix_memory_unequal_batches_and_slots_used_again(dtype):
    """Three sequences of unequal lengths start together and go on one token at a time, the
    shortest ending first; then another sequence takes a freed slot, whose state (the running
    maximum too) must start at zero.  Each against the plain mixer on that sequence alone."""
    td = TD[dtype]
    A, d, dv, H, cap = 4, 32, 24, 96, 12.0
    W = _mlstm_weights(A, d, dv, H, 90, td)
    Wd = {k: v.double() for k, v in W.items()}
    m = {"heads": A, "dim": d, "vdim": dv, "gate_cap": cap}
    part = _mlstm_part(W, A, d, dv, H, cap, td)
    tol = 5e-5 if dtype == "float32" else 4e-2
    oc = _Cache(part.cache_request(), 3, td)
    for round_, (starts, totals) in enumerate([((40, 1, 7), (52, 4, 20)), ((2, 30, 3), (9, 33, 5))]):
        hs = [rnd(n, H, seed=100 + 10 * round_ + i).to(td) for i, n in enumerate(totals)]
        refs = [P.mlstm_mixer(x.double(), m, Wd, "", 1e-5) for x in hs]
        got = [[] for _ in hs]
        ctx = oc.step(list(starts))
        y = summed(part.forward(torch.cat([x[:n] for x, n in zip(hs, starts)]).to(DEV), ctx, 0,
                                True))
        o = 0
        for i, n in enumerate(starts):
            got[i].append(y[o:o + n])
            o += n
        at = list(starts)
        while any(a < n for a, n in zip(at, totals)):
            live = [i for i in range(3) if at[i] < totals[i]]
            ctx = oc.step([1] * len(live), live)
            y = summed(part.forward(torch.cat([hs[i][at[i]:at[i] + 1] for i in live]).to(DEV),
                                    ctx, 0, True))
            for r, i in enumerate(live):
                got[i].append(y[r:r + 1])
                at[i] += 1
        for i in range(3):
            assert rel_err(torch.cat(got[i]), refs[i]) < tol, (round_, i)
            oc.again(i)


@pytest.mark.parametrize("dtype", DTYPES)
def test_what_the_memory_took_in_hundreds_of_tokens_ago_decides(dtype):
    """Forget gates next to one, input gates low except at one early token (whose stream has
    a component the input gate's projection picks up): the read-out 600 tokens later is that
    token's value, and decoding from the state must still have it."""
    td = TD[dtype]
    A, d, dv, H, cap = 2, 32, 16, 64, 15.0
    W = _mlstm_weights(A, d, dv, H, 500, td, forget=9.0)
    u = torch.zeros(H, dtype=torch.float64)
    u[5] = 1.0
    W["f"] = torch.zeros(A, H).to(td)
    W["i"] = (8.0 * u[None, :].repeat(A, 1)).to(td)
    W["i.b"] = torch.full((A,), -6.0).to(td)
    T, far = 640, 9
    h = rnd(T, H, seed=501)
    h[:, 5] = 0.0
    h[far, 5] = 2.5
    h = h.to(td)
    m = {"heads": A, "dim": d, "vdim": dv, "gate_cap": cap}
    Wd = {k: v.double() for k, v in W.items()}
    ref = P.mlstm_mixer(h.double(), m, Wd, "", 1e-5)
    # the far token matters: without it the last rows differ by much
    h2 = h.clone()
    h2[far] = rnd(H, seed=502).to(td)
    h2[far, 5] = 0
    other = P.mlstm_mixer(h2.double(), m, Wd, "", 1e-5)
    assert (other[-20:] - ref[-20:]).abs().max() > 0.2 * ref[-20:].abs().max()
    part = _mlstm_part(W, A, d, dv, H, cap, td)
    oc = _Cache(part.cache_request(), 1, td)
    got = [summed(part.forward(h[:600].to(DEV), oc.step([600]), 0, True))]
    for t in range(600, T):
        got.append(summed(part.forward(h[t:t + 1].to(DEV), oc.step([1]), 0, True)))
    got = torch.cat(got)
    tol = 3e-4 if dtype == "float32" else 5e-2
    assert rel_err(got[-40:], ref[-40:]) < tol
    # (among 640 rows some queries are nearly orthogonal to the one key that fills the memory:
    # numerator and denominator are both small there, and rounding shows three times as much)
    assert rel_err(got, ref) < 3 * tol


# ------------------------------------------------------------ attention
def _attention_weights(A, G, d, dv, H, taps, own, seed, td):
    lin = 1.0 / H ** 0.5
    W = {"q": rnd(A * d, H, seed=seed, std=1.5 * lin), "g": rnd(A * dv, H, seed=seed + 1, std=1.5 * lin),
         "o": rnd(H, A * dv, seed=seed + 2, std=1.0 / (A * dv) ** 0.5)}
    if taps:
        W["q.conv"] = rnd(A * d, taps, seed=seed + 3, std=0.5) + 0.4
    if own:
        W["k"] = rnd(G * d, H, seed=seed + 4, std=1.5 * lin)
        W["v"] = rnd(G * dv, H, seed=seed + 5, std=lin)
        if taps:
            W["k.conv"] = rnd(G * d, taps, seed=seed + 6, std=0.5) + 0.4
            W["v.conv"] = rnd(G * dv, taps, seed=seed + 7, std=0.5) + 0.4
    return {k: v.to(td) for k, v in W.items()}


def _attention_part(W, m, H, td):
    """The library's attention mixer for the plain mixer description ``m``."""
    from agave_b200.config.base import AttentionSpec, BandScalingSpec, RotarySpec
    from agave_b200.parts.attention import AttentionMixer
    position = None
    if m.get("rot"):
        r = m["rot"]
        sc = r.get("scaling")
        position = RotarySpec(theta=r["base"], rotary_dim=0 if r["dims"] == m["dim"] else r["dims"],
                              scaling=None if sc is None else BandScalingSpec(
                                  factor=sc["factor"], low=sc["low"], high=sc["high"],
                                  original=sc["original"]))
    mask = m.get("mask") or {}
    spec = AttentionSpec(n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"],
                         scale=m["scale"], window=mask.get("size"), position=position,
                         value_dim=0 if m["vdim"] == m["dim"] else m["vdim"],
                         keep_first=mask.get("keep_first", 0) if mask.get("size") else 0,
                         conv_taps=m.get("conv") or 0, out_gate=True)
    part = AttentionMixer(spec, H, td, torch.device(DEV))
    t = {"q_proj.weight": W["q"], "k_proj.weight": W["k"], "v_proj.weight": W["v"],
         "g_proj.weight": W["g"], "o_proj.weight": W["o"]}
    if m.get("conv"):
        t.update({"q_conv.weight": W["q.conv"], "k_conv.weight": W["k.conv"],
                  "v_conv.weight": W["v.conv"]})
    assert set(t) == set(AttentionMixer.param_specs(spec, H))
    part.load(t, td, torch.device(DEV))
    return part


def _plain_attention(h, m, W):
    Wd = {k: v.double() for k, v in W.items()}
    k, v = P.attention_keys_values(h.double(), m, Wd, "")
    return P.attention_mixer(h.double(), m, Wd, "", k, v)


def _run_alone(part, h, new, td):
    oc = _Cache(part.cache_request(), 1, td)
    got, at = [], 0
    for n in new:
        got.append(summed(part.forward(h[at:at + n].to(DEV), oc.step([n]), 0, True)))
        at += n
    return torch.cat(got)


def _mixer(A, G, d, dv, scale, conv=None, size=None, keep=None, rot=None):
    m = {"heads": A, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale}
    if conv is not None:
        m["conv"] = conv
    if size is not None:
        m["mask"] = {"size": size, "keep_first": keep or 0}
    if rot is not None:
        m["rot"] = rot
    return m


SC = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 16}
ATTENTION = [
    # T, H, mixer
    (90, 72, _mixer(4, 2, 10, 14, 0.4, conv=2, size=7, keep=2, rot={"base": 1e4, "dims": 6, "scaling": SC})),
    (200, 128, _mixer(4, 1, 64, 64, 0.13, conv=4, size=100, keep=3, rot={"base": 500.0, "dims": 32})),
    (150, 64, _mixer(2, 2, 24, 8, 0.3, size=64, keep=64, rot={"base": 50.0, "dims": 24})),
    (70, 96, _mixer(1, 1, 16, 16, 0.3, conv=1, size=1, keep=1)),
    (140, 64, _mixer(2, 1, 32, 32, 0.25, conv=5)),
    (300, 128, _mixer(4, 2, 64, 64, 0.12, conv=2, size=70, keep=0, rot={"base": 1e4, "dims": 64})),
    (130, 80, _mixer(6, 3, 128, 48, 0.09, conv=3, size=64, keep=5, rot={"base": 1e5, "dims": 64})),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, m", ATTENTION)
def test_attention_with_convolution_window_kept_keys_rotation_and_gate(dtype, T, H, m):
    """The mixer alone as a prompt, and as a prompt followed by tokens one by one (the
    convolution goes on from the stored inputs, the keys come from the cache), from cuts at
    the first token, inside the window and at a page border."""
    td = TD[dtype]
    W = _attention_weights(m["heads"], m["kv_heads"], m["dim"], m["vdim"], H, m.get("conv"), True,
                           600, td)
    h = rnd(T, H, seed=601).to(td)
    ref = _plain_attention(h, m, W)
    part = _attention_part(W, m, H, td)
    tol = 5e-5 if dtype == "float32" else 4e-2
    for new in ([T], [1] + [1] * (T - 1), [T - 30] + [1] * 30, [64] + [1] * (T - 64), [5] + [1] * (T - 5)):
        assert rel_err(_run_alone(part, h, new, td), ref) < tol, new[:2]


def _marked(T, H, mark, seed, amp=6.0):
    """A stream whose token ``mark`` alone has a component along axis 0, all tokens having one
    along axis 1: with the projections below, every query scores that token's key highest."""
    h = rnd(T, H, seed=seed)
    h[:, 0] = 0.0
    h[:, 1] = 1.0
    h[mark, 0] = amp
    return h


def _mark_weights(W, m, td, strength=1.6):
    """The last (unrotated) dimension of every q head reads axis 1, of every k head axis 0;
    their convolutions pass the current token alone."""
    d = m["dim"]
    for name, axis, heads in (("q", 1, m["heads"]), ("k", 0, m["kv_heads"])):
        w = W[name].double()
        for a in range(heads):
            w[a * d + d - 1] = 0.0
            w[a * d + d - 1, axis] = strength / m["scale"] ** 0.5
            if m.get("conv"):
                c = W[name + ".conv"].double()
                c[a * d + d - 1] = 0.0
                c[a * d + d - 1, -1] = 1.0
                W[name + ".conv"] = c.to(td)
        W[name] = w.to(td)
    return W


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("size, keep, taps, d, dv", [(76, 6, 4, 64, 64), (20, 3, 2, 24, 16),
                                                      (64, 1, 3, 32, 32), (130, 7, None, 16, 16),
                                                      (100, 70, 2, 128, 128), (90, 5, 3, 64, 32)])
def test_the_key_at_a_window_edge_or_a_kept_place_decides(dtype, size, keep, taps, d, dv):
    """One key scores far above the rest.  It is placed at the last kept first place, at the
    first place that is not kept, and so that it lies just inside or just outside the window
    of the rows compared, in a prompt and when decoding: a mask that is off by one gives
    another row altogether."""
    td = TD[dtype]
    A, G, H = 4, 2, 64
    T = 2 * size + 40
    m = _mixer(A, G, d, dv, 0.2, conv=taps, size=size, keep=keep, rot={"base": 1e4, "dims": d // 2})
    tol = 1e-4 if dtype == "float32" else 5e-2
    for mark in (keep - 1, keep, T - size - 2, 64, size + keep):
        W = _mark_weights(_attention_weights(A, G, d, dv, H, taps, True, 700, td), m, td)
        h = _marked(T, H, mark, 701 + mark).to(td)
        ref = _plain_attention(h, m, W)
        # the marked key decides: the row just inside and the row just outside its window differ
        if mark >= keep and mark + size < T:
            a, b = ref[mark + size - 1], ref[mark + size]
            assert (a - b).abs().max() > 0.3 * max(a.abs().max(), b.abs().max())
        part = _attention_part(W, m, H, td)
        for new in ([T], [mark + 3] + [1] * (T - mark - 3), [T - 9] + [1] * 9):
            assert rel_err(_run_alone(part, h, new, td), ref) < tol, (mark, new[:2])


@pytest.mark.parametrize("hd, window, keep, T", [(64, 76, 6, 300), (128, 100, 70, 260),
                                                 (32, 64, 1, 200), (64, 130, 65, 400)])
def test_kept_keys_in_every_form_of_the_prompt_kernels(hd, window, keep, T):
    """bfloat16: the one-warp, the mma.sync and the tcgen05 prompt kernels on the same q, k, v
    (two sequences of unequal lengths, peaked scores) against sums written out in torch."""
    from agave_b200 import kernels
    nh, nkv = 4, 2
    lens = [T, T // 3]
    q = rnd(sum(lens), nh * hd, seed=5, std=1.0).to(torch.bfloat16).to(DEV)
    k = rnd(sum(lens), nkv * hd, seed=6, std=1.0).to(torch.bfloat16).to(DEV)
    v = rnd(sum(lens), nkv * hd, seed=7, std=1.0).to(torch.bfloat16).to(DEV)
    scale = 2.0 / hd ** 0.5
    i32 = dict(dtype=torch.int32, device=DEV)
    cu = torch.tensor([0, lens[0], sum(lens)], **i32)
    pos = torch.tensor(list(range(lens[0])) + list(range(lens[1])), **i32)
    seq = torch.tensor([0] * lens[0] + [1] * lens[1], **i32)
    ref = torch.zeros(sum(lens), nh, hd, dtype=torch.float64)
    o = 0
    for n in lens:
        i = torch.arange(n)[:, None]
        j = torch.arange(n)[None, :]
        see = (j <= i) & ((i - j < window) | (j < keep))
        for a in range(nh):
            g = a // (nh // nkv)
            sc = q[o:o + n, a * hd:(a + 1) * hd].double().cpu() @ \
                k[o:o + n, g * hd:(g + 1) * hd].double().cpu().T * scale
            sc = torch.where(see, sc, torch.full_like(sc, -math.inf))
            ref[o:o + n, a] = torch.softmax(sc, -1) @ v[o:o + n, g * hd:(g + 1) * hd].double().cpu()
        o += n
    ref = ref.reshape(sum(lens), nh * hd)
    out = torch.empty(sum(lens), nh * hd, dtype=torch.bfloat16, device=DEV)
    kernels.attention_prefill_simt(q, k, v, out, pos, seq, cu, nh, nkv, hd, scale, window,
                                   keep_first=keep)
    assert rel_err(out, ref) < 2e-2
    out.zero_()
    kernels.attention_prefill_mma(q, k, v, out, cu, max(lens), nh, nkv, hd, scale, window,
                                  keep_first=keep)
    assert rel_err(out, ref) < 2e-2
    if hd % 16 == 0:
        out.zero_()
        kernels.attention_prefill_tc(q, k, v, out, cu, max(lens), nh, nkv, hd, scale, window,
                                     keep_first=keep)
        assert kernels.attention_tc_status() == 0
        assert rel_err(out, ref) < 2e-2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_decides_in_attention(dtype):
    """No mask: a key 900 tokens back outscores all others; prompt rows and decoded rows."""
    td = TD[dtype]
    A, G, d, dv, H, T = 4, 1, 32, 48, 64, 930
    m = _mixer(A, G, d, dv, 0.18, conv=3, rot={"base": 1e4, "dims": 8})
    W = _mark_weights(_attention_weights(A, G, d, dv, H, 3, True, 800, td), m, td)
    h = _marked(T, H, 11, 801).to(td)
    ref = _plain_attention(h, m, W)
    h2 = h.clone()
    h2[11, 0] = 0
    assert (_plain_attention(h2, m, W)[-10:] - ref[-10:]).abs().max() > 0.3 * ref[-10:].abs().max()
    part = _attention_part(W, m, H, td)
    tol = 1e-4 if dtype == "float32" else 5e-2
    assert rel_err(_run_alone(part, h, [T], td), ref) < tol
    assert rel_err(_run_alone(part, h, [900] + [1] * 30, td)[-30:], ref[-30:]) < tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_unequal_batches_and_slots_used_again(dtype):
    """Three sequences start together with unequal lengths and are decoded together; then
    others take the freed slots, whose stored convolution inputs must start at zero."""
    td = TD[dtype]
    H = 96
    m = _mixer(4, 2, 32, 16, 0.2, conv=4, size=40, keep=2, rot={"base": 1e4, "dims": 16})
    W = _attention_weights(4, 2, 32, 16, H, 4, True, 900, td)
    part = _attention_part(W, m, H, td)
    tol = 5e-5 if dtype == "float32" else 4e-2
    oc = _Cache(part.cache_request(), 3, td)
    for round_, (starts, totals) in enumerate([((70, 1, 7), (82, 5, 60)), ((2, 65, 3), (9, 70, 50))]):
        hs = [rnd(n, H, seed=910 + 10 * round_ + i).to(td) for i, n in enumerate(totals)]
        refs = [_plain_attention(x, m, W) for x in hs]
        got = [[] for _ in hs]
        y = summed(part.forward(torch.cat([x[:n] for x, n in zip(hs, starts)]).to(DEV),
                                oc.step(list(starts)), 0, True))
        o = 0
        for i, n in enumerate(starts):
            got[i].append(y[o:o + n])
            o += n
        at = list(starts)
        while any(a < n for a, n in zip(at, totals)):
            live = [i for i in range(3) if at[i] < totals[i]]
            y = summed(part.forward(torch.cat([hs[i][at[i]:at[i] + 1] for i in live]).to(DEV),
                                    oc.step([1] * len(live), live), 0, True))
            for r, i in enumerate(live):
                got[i].append(y[r:r + 1])
                at[i] += 1
        for i in range(3):
            assert rel_err(torch.cat(got[i]), refs[i]) < tol, (round_, i)
            oc.again(i)


# ------------------------------------------------------------ whole models
_ENGINES = {}


def engine_for(name, dtype, max_tokens=8192):
    key = (name, dtype)
    if key not in _ENGINES:
        from agave_b200.engine.api import Engine
        folder = folder_for(name, TD[dtype])
        _ENGINES[key] = (Engine(folder, dtype=dtype, max_tokens=max_tokens), folder)
    return _ENGINES[key]


def vocab(name):
    return CONFIGS[name]["vocab"]


NAMES = sorted(CONFIGS)


def chosen_by(eng, toks):
    """The experts the library's routers choose for a request run alone, by layer."""
    from agave_b200.parts.moe import RoutedFeedForward
    rec = {}
    keep = RoutedFeedForward.route

    def route(self, x):
        ids, wts = keep(self, x)
        rec[id(self)] = ids.cpu().long()
        return ids, wts
    RoutedFeedForward.route = route
    try:
        s = eng.acquire()
        eng.step([(s, toks)], [[len(toks) - 1]])
        eng.release(s)
    finally:
        RoutedFeedForward.route = keep
    return {i: rec[id(b.ffn)] for i, b in enumerate(eng.model.blocks) if id(b.ffn) in rec}


class RecordedRoutes:
    """While active, every routed feed-forward's choice is kept, step by step: ``steps[k][i]`` is
    the ids [tokens of step k, top] of layer i.  ``of_rows`` puts a request's rows together
    again from (step, first row, rows) pieces, as the plain model's ``chosen`` wants them."""

    def __init__(self, eng):
        self.eng, self.steps, self._cur = eng, [], None

    def __enter__(self):
        from agave_b200.parts.moe import RoutedFeedForward
        self._cls, self._keep = RoutedFeedForward, RoutedFeedForward.route
        layer_of = {id(b.ffn): i for i, b in enumerate(self.eng.model.blocks)}
        rec = self

        def route(part, x):
            ids, wts = rec._keep(part, x)
            rec._cur[layer_of[id(part)]] = ids.cpu().long()
            return ids, wts
        RoutedFeedForward.route = route
        return self

    def __exit__(self, *exc):
        self._cls.route = self._keep

    def step(self, entries, want):
        self._cur = {}
        out = self.eng.step(entries, want)
        self.steps.append(self._cur)
        return out

    def of_rows(self, pieces):
        layers = self.steps[pieces[0][0]].keys()
        return {i: torch.cat([self.steps[k][i][a:a + n] for k, a, n in pieces]) for i in layers}


def reference(eng, folder, toks, dtype):
    """The plain model's logits; in bfloat16 under the experts the library chose, since a
    close call that falls the other way moves a row far more than rounding does."""
    if dtype == "float32":
        return plain_logits(folder, toks)
    return plain_logits(folder, toks, chosen=chosen_by(eng, toks))


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(name):
    """32-bit: the residual stream after each layer against the plain model's, so that a
    fault names its layer."""
    import dataclasses
    eng, folder = engine_for(name, "float32")
    toks = tokens(25, vocab(name), 9)
    streams = []
    plain_logits(folder, toks, streams)
    model = eng.model
    for upto in range(1, len(model.spec.schedule) + 1):
        s = eng.acquire()
        ctx = eng.runner.context([(s, toks)])
        keep = model.spec
        model.spec = dataclasses.replace(keep, schedule=keep.schedule[:upto])
        try:
            h = model.hidden_states(ctx)
        finally:
            model.spec = keep
        eng.runner.cache.trim(s)
        eng.release(s)
        assert rel_err(h, streams[upto - 1]) < 2e-5, f"layer {upto - 1}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_alone(name, dtype):
    """Every row of prompts of 1, 2, a window's and a page's length, and of 300 tokens."""
    eng, folder = engine_for(name, dtype)
    for n in (1, 2, 7, 8, 64, 65, 300):
        toks = tokens(n, vocab(name), 20 + n)
        s = eng.acquire()
        got = eng.step([(s, toks)], [list(range(n))])
        eng.release(s)
        rows_agree(got, reference(eng, folder, toks, dtype), dtype, f"{name} {n} tokens")


def alone(eng, toks, cut):
    """A request by itself: ``cut`` tokens as the prompt, the rest one by one; all rows."""
    s = eng.acquire()
    got = [eng.step([(s, toks[:cut])], [list(range(cut))])]
    for p in range(cut, len(toks)):
        got.append(eng.step([(s, [toks[p]])], [[0]]))
    eng.release(s)
    return torch.cat(got)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_tokens_one_by_one(name, dtype):
    """The prompt's end, then the rest decoded through the cache and the state, against the
    whole sequence at once: decoding starts after one token, inside the first window, at a
    page border, and runs past several windows' edges."""
    eng, folder = engine_for(name, dtype)
    for n, cut in ((100, 60), (41, 1), (200, 127), (140, 64), (12, 2)):
        toks = tokens(n, vocab(name), 11 + n)
        rows_agree(alone(eng, toks, cut), reference(eng, folder, toks, dtype), dtype,
                   f"{name} {n}/{cut}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_and_slots_used_again(name, dtype):
    """Requests of unequal lengths start together and are decoded together, the shorter ones
    ending earlier; then other requests take the freed slots, pages and states.  Every row
    against the plain model run on that request alone."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    for round_, lens in enumerate([(130, 3, 64, 1), (1, 65, 20), (63, 70, 5)]):
        seqs = [tokens(n + 6 + 3 * i, V, 50 + 10 * round_ + i) for i, n in enumerate(lens)]
        slots = [eng.acquire() for _ in seqs]
        got = [[] for _ in seqs]
        out = eng.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)],
                       [list(range(n)) for n in lens])
        o = 0
        for i, n in enumerate(lens):
            got[i].append(out[o:o + n])
            o += n
        at = list(lens)
        while any(a < len(s) for a, s in zip(at, seqs)):
            live = [i for i in range(len(seqs)) if at[i] < len(seqs[i])]
            out = eng.step([(slots[i], [seqs[i][at[i]]]) for i in live], [[0]] * len(live))
            for r, i in enumerate(live):
                got[i].append(out[r:r + 1])
                at[i] += 1
                if at[i] == len(seqs[i]):
                    eng.release(slots[i])
        for i in range(len(seqs)):
            rows_agree(torch.cat(got[i]), reference(eng, folder, seqs[i], dtype), dtype,
                       f"{name} round {round_} request {i}")


@pytest.mark.parametrize("name", NAMES)
def test_lengths_round_page_borders_and_window_edges(name):
    """32-bit: prompts that end just before, on and just after a page border, the windows'
    edges and the kept first keys, each followed by three decoded tokens."""
    eng, folder = engine_for(name, "float32")
    edges = {63, 64, 65, 127, 128, 129}
    for l in CONFIGS[name]["layers"]:
        mask = l["mixer"].get("mask") if l["type"] == "attention" else None
        if mask:
            w, k = mask["size"], mask.get("keep_first") or 0
            edges |= {max(1, w - 1), w, w + 1, w + k, w + k + 1, 2 * w, 2 * w + 1}
    for n in sorted(edges):
        toks = tokens(n + 3, vocab(name), n)
        ref = plain_logits(folder, toks)
        s = eng.acquire()
        got = [eng.step([(s, toks[:n])], [[0, n - 1]])]
        for p in range(n, n + 3):
            got.append(eng.step([(s, [toks[p]])], [[0]]))
        eng.release(s)
        rows_agree(torch.cat(got), ref[[0, n - 1, n, n + 1, n + 2]], "float32", f"{name} {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["K1", "K2"])
def test_long_decoding(name, dtype):
    """300 tokens decoded after a prompt of 5: several pages and windows, the rings wrap more
    than once, the state goes through 300 updates."""
    eng, folder = engine_for(name, dtype)
    toks = tokens(305, vocab(name), 77)
    rows_agree(alone(eng, toks, 5), reference(eng, folder, toks, dtype), dtype, name)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_the_entry_point(name, dtype):
    """``Engine.generate`` (scheduler, CUDA graphs, the arg max in the head's epilogue): every
    generated token is the plain model's best, or within rounding of it."""
    eng, folder = engine_for(name, dtype)
    V = vocab(name)
    prompts = [tokens(n, V, 300 + n) for n in (4, 37, 70, 9, 130)]
    outs = eng.generate(prompts, max_new_tokens=12, stop_token_ids=[])
    slack = 2e-3 if dtype == "float32" else 8e-2
    misses = 0
    for p, g in zip(prompts, outs):
        assert len(g) == 12
        ref = reference(eng, folder, p + g, dtype)
        for k, t in enumerate(g):
            row = ref[len(p) - 1 + k]
            if float(row.max() - row[t]) > slack * float(row.abs().max()):
                misses += 1
    assert misses <= (0 if dtype == "float32" else 3), misses


@pytest.mark.parametrize("dtype", DTYPES)
def test_generation_in_batches_of_the_slot_limit(dtype):
    """More prompts than slots: the scheduler cuts them into batches and uses slots (and
    their states) again; the tokens are the same as with room for all."""
    from agave_b200.engine.api import Engine
    folder = folder_for("K1", TD[dtype])
    V = vocab("K1")
    prompts = [tokens(n, V, 900 + n) for n in (5, 66, 17, 3, 40, 21, 8)]
    wide = Engine(folder, dtype=dtype, max_tokens=4096)
    narrow = Engine(folder, dtype=dtype, max_tokens=4096, max_batch=3)
    a = wide.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    b = narrow.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    same = sum(x == y for x, y in zip(a, b))
    assert same >= (len(prompts) if dtype == "float32" else len(prompts) - 2)


def test_sampling_runs_on_this_architecture():
    eng, _ = engine_for("K1", "bfloat16")
    V = vocab("K1")
    kw = dict(max_new_tokens=8, temperature=0.8, top_k=20, top_p=0.9, seed=5, stop_token_ids=[])
    outs = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], **kw)
    again = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], **kw)
    assert outs == again and all(len(o) == 8 and all(0 <= t < V for t in o) for o in outs)


def test_random_weights_from_a_configuration():
    """``Engine.from_config``: a model with drawn weights steps and generates."""
    from agave_b200.engine.api import Engine
    raw = CONFIGS["K1"]
    eng = Engine.from_config(raw, seed=3, max_tokens=1024)
    outs = eng.generate([tokens(9, raw["vocab"], 1)], max_new_tokens=5, stop_token_ids=[])
    assert len(outs[0]) == 5
    info = eng.model_info()
    assert info["architecture"] == "Kadavik" and info["weight_bytes"] > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype):
    name = "K2"
    folder = folder_for(name, TD[dtype])
    V = vocab(name)
    a, b = tokens(210, V, 5), tokens(33, V, 6)
    eng, _ = engine_for(name, dtype)
    refs = {"a": reference(eng, folder, a, dtype), "b": reference(eng, folder, b, dtype)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:195], "want": [0, 100, 194]},
                                     {"id": "b", "tokens": b[:30], "want": [29]}], "end": []}]
    for k in range(15):
        ent, end = [{"id": "a", "tokens": [a[195 + k]], "want": [0]}], []
        if k < 3:
            ent.append({"id": "b", "tokens": [b[30 + k]], "want": [0] if k != 1 else []})
            if k == 2:
                end.append("b")
        if k == 14:
            end.append("a")
        steps.append({"step": k + 1, "entries": ent, "end": end})
    out = tempfile.mkdtemp(prefix="kadavik_trace_")
    try:
        r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model",
                            folder, "--dtype", dtype, "--out", out, "--max-tokens", "300"],
                           input="\n".join(json.dumps(s) for s in steps) + "\n", text=True,
                           capture_output=True, timeout=900)
        assert r.returncode == 0, r.stderr[-2000:]
        assert [l for l in r.stdout.split("\n") if l.startswith("done")] == \
            [f"done {k}" for k in range(16)]
        got = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(4, V))
        rows_agree(got, torch.stack([refs["a"][0], refs["a"][100], refs["a"][194], refs["b"][29]]),
                   dtype, "step 0")
        rows = []
        for k in range(15):
            want = [refs["a"][195 + k]]
            if k < 3 and k != 1:
                want.append(refs["b"][30 + k])
            g = np.fromfile(os.path.join(out, f"{k + 1}.f32"), dtype="<f4").reshape(len(want), V)
            rows.append((torch.from_numpy(g), torch.stack(want)))
        rows_agree(torch.cat([g for g, _ in rows]), torch.cat([w for _, w in rows]), dtype,
                   "decoded")
    finally:
        shutil.rmtree(out, ignore_errors=True)


def test_command_line_on_this_architecture():
    """``python -m agave_b200`` picks the model class from config.json: greedy tokens equal the
    plain model's, --model-info names the architecture, --profile lists this design's
    operations, --random-weights draws a model from a config.json."""
    name = "K2"
    folder = folder_for(name, torch.float32)
    V = vocab(name)
    prompt = tokens(9, V, 31)

    def run(*args):
        env = dict(os.environ)
        env["PYTHONPATH"] = ROOT + os.pathsep + env.get("PYTHONPATH", "")
        return subprocess.run([sys.executable, "-m", "agave_b200", *args], capture_output=True,
                              text=True, timeout=900, env=env, cwd=ROOT)
    toks = ",".join(str(t) for t in prompt)
    r = run(folder, "--tokens", toks, "-n", "6", "--json", "--dtype", "float32")
    assert r.returncode == 0, r.stderr[-2000:]
    out = json.loads(r.stdout.strip().splitlines()[-1])["output_ids"]
    assert len(out) == 6
    ref = plain_logits(folder, prompt + out)
    for k, t in enumerate(out):
        row = ref[len(prompt) - 1 + k]
        assert float(row.max() - row[t]) <= 2e-3 * float(row.abs().max()), (k, t)
    r = run(folder, "--model-info", "--json")
    assert r.returncode == 0 and "Kadavik" in r.stdout, r.stderr[-2000:]
    r = run(folder, "--tokens", toks, "-n", "3", "--profile", "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr[-2000:]
    for op in ("norm", "qkv", "attention", "conv_rope_store", "mlstm_prepare", "mlstm_scan",
               "mlstm_out", "router", "experts_gate_up", "experts_down", "out_proj",
               "token_side_gate", "down", "lm_head", "TOTAL"):
        assert op in r.stderr, (op, r.stderr[-1500:])
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(CONFIGS[name], f)
        outs = []
        for seed in ("3", "3", "4"):
            r = run(d, "--random-weights", seed, "--tokens", toks, "-n", "5", "--json")
            assert r.returncode == 0, r.stderr[-2000:]
            outs.append(json.loads(r.stdout.strip().splitlines()[-1])["output_ids"])
        assert outs[0] == outs[1] and len(outs[0]) == 5


@pytest.mark.parametrize("name, room", [("K1", 60), ("K2", 90), ("K3", 64), ("K5", 100)])
def test_a_cache_shorter_than_a_page_or_a_window(name, room):
    """32-bit: a cache of one or two pages.  A window that still fits a sequence keeps its
    edge (and the kept keys behind it); a window no sequence can outgrow is none."""
    from agave_b200.engine.api import Engine
    folder = folder_for(name, torch.float32)
    eng = Engine(folder, dtype="float32", max_tokens=room, ctx_size=room, max_batch=1)
    toks = tokens(room, vocab(name), 5)
    rows_agree(alone(eng, toks, room - 15), plain_logits(folder, toks), "float32", name)
