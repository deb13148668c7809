"""Bovozen on the GPU against the plain implementation (tests/plain/bovozen_plain.py): each
mechanism alone, then whole models of three small configurations through the engine: the
stream after every layer, whole prompts, the last tokens one by one, unequal batches
against each request alone, slots and pages used again, lengths round page borders and
block edges, long decoding, greedy generation through the scheduler, and trace replay as a
process.

Where random weights would hide a fault, the inputs are made so that it shows: a key at the
first place of a block and the one before it (or far back among hundreds) are given scores
that stand out, so an output that includes or misses the wrong one is far off; the recurrent
mixer's decays are set close to one, so that what was written hundreds of tokens ago still
decides the read-out.
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

from bovozen_util import CONFIGS, RANKS, folder_for, plain_logits, tokens
from plain import bovozen_plain as P
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
    by a close call, a read-out whose norm is close to zero at a sequence's first tokens); so
    all but one row in twenty-five (at least two) within 0.12, and every row of the right
    size."""
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
                           device=torch.device(DEV))

    def again(self, b):
        """Sequence b ends; another takes a slot (the freed one or the spare)."""
        self.cache.release(self.slots[b])
        self.slots[b] = self.cache.acquire()
        self.lens[b] = 0


# ------------------------------------------------------------ small mechanisms
def test_learned_position_rows():
    from agave_b200 import kernels
    for td in (torch.float32, torch.bfloat16):
        table = rnd(50, 72, seed=1).to(td).to(DEV)
        h = rnd(9, 72, seed=2).float().to(DEV)
        pos = torch.tensor([0, 1, 2, 49, 7, 7, 0, 30, 31], dtype=torch.int32, device=DEV)
        want = h.double() + table.double()[pos.long()]
        kernels.add_position_rows(pos, table, h, 1.0)
        assert rel_err(h, want) < 1e-6


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, ff", [(1, 72, 40), (7, 128, 192), (150, 96, 48), (300, 192, 512)])
def test_dense_feed_forward_with_the_erf_gelu(dtype, T, H, ff):
    from agave_b200.config.base import DenseFeedForwardSpec
    from agave_b200.parts.feedforward import DenseFeedForward
    td = TD[dtype]
    W = {"up": rnd(ff, H, seed=3, std=H ** -0.5).to(td), "down": rnd(H, ff, seed=4, std=ff ** -0.5).to(td)}
    x = rnd(T, H, seed=5, std=2.0).to(td)          # arguments on both sides of the bend
    part = DenseFeedForward(DenseFeedForwardSpec(intermediate_size=ff, activation="gelu_erf"), H,
                            td, torch.device(DEV))
    part.load({"up_proj.weight": W["up"], "down_proj.weight": W["down"]}, td, torch.device(DEV))
    got = summed(part.forward(x.to(DEV), None))
    ref = P.dense_ff(x.double(), {k: v.double() for k, v in W.items()}, "")
    assert rel_err(got, ref) < (2e-5 if dtype == "float32" else 2e-2)
    # the tanh form differs from the erf form by more than that
    z = x.double() @ W["up"].double().T
    tanh = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    if dtype == "float32":
        assert rel_err(tanh @ W["down"].double().T, ref) > 1e-4


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, E, top", [(1, 72, 5, 2), (40, 96, 1, 1), (33, 128, 4, 4),
                                          (200, 192, 12, 2), (64, 64, 70, 7), (9, 40, 6, 1)])
def test_router_with_a_bias_and_softmax_over_the_chosen(dtype, T, H, E, top):
    from agave_b200 import kernels
    td = TD[dtype]
    x = rnd(T, H, seed=6).to(td)
    Wr = rnd(E, H, seed=7, std=2.0 * H ** -0.5).to(td)
    # a bias that changes the choice: without it other experts would win
    b = rnd(E, seed=8, std=2.0).float()
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, dtype=torch.float32, device=DEV)
    kernels.moe_route(x.to(DEV), Wr.to(DEV), None, 1, 1, top, ids, wts, bias=b.to(DEV),
                      softmax_top=True)
    z = x.double() @ Wr.double().T + b.double()
    rid, rw = P.route(x.double(), Wr.double(), b.double(), top)
    nob, _ = P.route(x.double(), Wr.double(), torch.zeros(E, dtype=torch.float64), top)
    if E > top and T > 8:
        assert (nob.sort(dim=1).values != rid.sort(dim=1).values).any()
    ids, wts = ids.cpu().long(), wts.cpu().double()
    assert (wts.sum(dim=1) - 1).abs().max() < 1e-5
    for t in range(T):
        got = dict(zip(ids[t].tolist(), wts[t].tolist()))
        assert len(got) == top
        want = dict(zip(rid[t].tolist(), rw[t].tolist()))
        if set(got) != set(want):
            # a close call between the last chosen and the first left out
            lo = min(z[t, e].item() for e in set(got) | set(want))
            hi = sorted(z[t].tolist())[-top]
            assert abs(hi - lo) < 1e-4 * (1 + abs(hi)), (t, got, want)
            continue
        for e in got:
            assert abs(got[e] - want[e]) < 2e-5, (t, e, got[e], want[e])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, H, E, top, ff, shared", [
    (1, 72, 5, 2, 24, 0), (50, 72, 3, 3, 16, 20), (7, 96, 1, 1, 32, 8), (130, 128, 8, 2, 64, 128),
    (260, 128, 8, 3, 64, 64), (20, 96, 6, 1, 16, 0)])
def test_routed_experts_beside_a_gated_shared_one(dtype, T, H, E, top, ff, shared):
    from agave_b200.config.base import RoutedFeedForwardSpec
    from agave_b200.parts.moe import RoutedFeedForward
    td = TD[dtype]
    W, lin = {}, H ** -0.5
    for e in range(E):
        W[f"e{e}.gate"] = rnd(ff, H, seed=10 + 3 * e, std=1.5 * lin).to(td)
        W[f"e{e}.up"] = rnd(ff, H, seed=11 + 3 * e, std=1.5 * lin).to(td)
        W[f"e{e}.down"] = rnd(H, ff, seed=12 + 3 * e, std=ff ** -0.5).to(td)
    W["router"] = rnd(E, H, seed=400, std=8.0 * lin).to(td)      # no close calls
    W["router.b"] = rnd(E, seed=401, std=1.0).float()
    if shared:
        W["shared.gate"] = rnd(shared, H, seed=402, std=1.5 * lin).to(td)
        W["shared.up"] = rnd(shared, H, seed=403, std=1.5 * lin).to(td)
        W["shared.down"] = rnd(H, shared, seed=404, std=shared ** -0.5).to(td)
        W["shared.sg"] = rnd(1, H, seed=405, std=2.0 * lin).to(td)
    x = rnd(T, H, seed=9).to(td)
    spec = RoutedFeedForwardSpec(n_experts=E, top=top, intermediate_size=ff, activation="silu",
                                 n_groups=1, keep_groups=1, correction=False, router_bias=True,
                                 weighting="softmax_top", shared_size=shared)
    part = RoutedFeedForward(spec, H, td, torch.device(DEV))
    names = {"router.weight": W["router"], "router.bias": W["router.b"]}
    for e in range(E):
        for n in ("gate", "up", "down"):
            names[f"experts.{e}.{n}_proj.weight"] = W[f"e{e}.{n}"]
    if shared:
        names.update({"shared.gate_proj.weight": W["shared.gate"],
                      "shared.up_proj.weight": W["shared.up"],
                      "shared.down_proj.weight": W["shared.down"],
                      "shared.gate.weight": W["shared.sg"]})
    part.load(names, td, torch.device(DEV))
    got = summed(part.forward(x.to(DEV), None))
    f = {"router": {"top": top}, "shared": {"ff": shared} if shared else None}
    ref = P.routed_ff(x.double(), {k: v.double() for k, v in W.items()}, "", f)
    assert rel_err(got, ref) < (3e-5 if dtype == "float32" else 3e-2)
    if shared:
        without = P.routed_ff(x.double(), {k: v.double() for k, v in W.items()}, "",
                              dict(f, shared=None))
        assert rel_err(without, ref) > 0.05          # the shared expert is no small part


# --------------------------------------------------------- the attention mixer
def _attention_weights(A, G, d, dv, H, seed, td):
    lin = H ** -0.5
    W = {"q": rnd(A * d, H, seed=seed, std=lin), "k": rnd(G * d, H, seed=seed + 1, std=lin),
         "v": rnd(G * dv, H, seed=seed + 2, std=lin),
         "q.norm": rnd(A * d, seed=seed + 3, std=0.3) + 1.2,
         "k.norm": rnd(G * d, seed=seed + 4, std=0.3) + 1.2,
         "o": rnd(H, A * dv, seed=seed + 5, std=(A * dv) ** -0.5),
         "vmix": torch.tensor(0.37, dtype=torch.float64)}
    return {k: v.to(td) for k, v in W.items()}


def _attention_part(W, A, G, d, dv, H, scale, block, mix_source, reach, td):
    from agave_b200.config.base import (AttentionSpec, DistanceSlopeSpec, NormSpec,
                                        ValueMixSpec)
    from agave_b200.parts.attention import AttentionMixer
    mix = None if mix_source is False else ValueMixSpec(source=mix_source)
    spec = AttentionSpec(n_heads=A, n_kv_heads=G, head_dim=d, scale=scale, window=None,
                         qk_norm=NormSpec(eps=1e-5, zero_centered=False), qk_norm_whole=True,
                         position=None, value_dim=0 if dv == d else dv, chunk=block,
                         distance_slope=DistanceSlopeSpec(exponent=8.0, reach=reach),
                         value_mix=mix)
    part = AttentionMixer(spec, H, td, torch.device(DEV))
    part.load({"q_proj.weight": W["q"], "k_proj.weight": W["k"], "v_proj.weight": W["v"],
               "o_proj.weight": W["o"], "q_norm.weight": W["q.norm"],
               "k_norm.weight": W["k.norm"], "value_mix": W["vmix"]}, td, torch.device(DEV))
    return part


ATTENTION = [
    # T, A, G, d, dv, H, block
    (40, 4, 2, 10, 14, 72, 7),            # odd sizes, a block shorter than a page
    (330, 4, 1, 64, 64, 128, 100),        # tensor-core sizes, a block that crosses pages
    (200, 3, 3, 16, 16, 96, 64),          # a block of exactly one page
    (30, 2, 2, 24, 8, 96, 1),             # a block of one: every token sees itself only
    (300, 1, 1, 32, 32, 64, None),        # one head, no mask: the slope alone
    (280, 6, 2, 48, 32, 192, 129),        # a block one longer than two pages
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mixing", [False, True])
@pytest.mark.parametrize("T, A, G, d, dv, H, block", ATTENTION)
def test_attention_mixer_blocks_slopes_whole_norm_and_mixed_values(dtype, mixing, T, A, G, d, dv,
                                                                   H, block):
    """The mixer alone, as a prompt and token by token through the cache, against the plain
    one.  The inputs of the last block's first position and of the position before it are
    made the same strong vector the last token has, so that their keys score highest: the
    first counts, the second must not."""
    td = TD[dtype]
    scale = 1.3 / d ** 0.5
    W = _attention_weights(A, G, d, dv, H, 20, td)
    # a group's key projection is that of its first query head: a key made from the same
    # input as a query then scores about scale * 1.4 * d, far above the random ones (a
    # norm over the whole projection undoes any scaling of the input itself)
    per = A // G
    W["k"] = W["q"].view(A, d, H)[::per].reshape(G * d, H).clone()
    W["k.norm"] = W["q.norm"].view(A, d)[::per].reshape(G * d).clone()
    h = rnd(T, H, seed=30)
    first =((T - 1) // block) * block if block else 0
    for p in (first, first - 1):
        if 0 <= p < T - 1:
            h[p] = h[T - 1] * (3.0 if p == first else 4.0)
    h = h.to(td)
    v_first = rnd(T, G * dv, seed=31).to(td) if mixing else None
    m = {"heads": A, "kv_heads": G, "dim": d, "vdim": dv, "scale": scale, "v_mix": mixing}
    if block:
        m["mask"] = {"size": block}
    shared = {"first": v_first.double()} if mixing else {}
    ref = P.attention_mixer(h.double(), {k: v.double() for k, v in W.items()}, "", m, 1e-5, shared)
    part = _attention_part(W, A, G, d, dv, H, scale, block, 5 if mixing else False, 1000, td)
    tol = 3e-5 if dtype == "float32" else 3e-2
    cut = T - min(T - 1, 70)
    for new in ([T], [cut] + [1] * (T - cut)):
        oc = _Cache(part.cache_request(), 1, td)
        got, at = [], 0
        for n in new:
            ctx = oc.step([n])
            if mixing:
                ctx.step_values[5] = v_first[at:at + n].to(DEV)
            got.append(summed(part.forward(h[at:at + n].to(DEV), ctx, 0, True)))
            at += n
        assert rel_err(torch.cat(got), ref) < tol, new[:2]
    # what a wrong edge would give is far from the reference
    if block and block > 1 and first >= 1:
        wrong = dict(m, mask={"size": block + 1})
        other = P.attention_mixer(h.double(), {k: v.double() for k, v in W.items()}, "", wrong,
                                  1e-5, dict(shared))
        assert rel_err(other[T - 1:], ref[T - 1:]) > 10 * tol


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_key_among_hundreds_decides_in_attention(dtype):
    """No mask, 900 keys: position 3's key is made to match the last query of the flattest
    head as well as the last token's own key does (the key projection is that head's query
    projection, the input the last token's), against the slope's pull (that head's slope
    times 896 is 3.5), and its value is forty times as large, so that it is the greater part
    of that head's output; a prompt and a decoded token."""
    td = TD[dtype]
    T, A, G, d, dv, H = 900, 2, 1, 64, 64, 128
    W = _attention_weights(A, G, d, dv, H, 50, td)
    W["k"], W["k.norm"] = W["q"][d:].clone(), W["q.norm"][d:].clone()
    h = rnd(T, H, seed=51)
    h[3] = h[T - 1] * 40.0
    h = h.to(td)
    m = {"heads": A, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.5, "v_mix": False}
    Wd = {k: v.double() for k, v in W.items()}
    ref = P.attention_mixer(h.double(), Wd, "", m, 1e-5, {})
    h2 = h.clone()
    h2[3] = h[4]
    assert rel_err(P.attention_mixer(h2.double(), Wd, "", m, 1e-5, {})[T - 1:], ref[T - 1:]) > 0.2
    part = _attention_part(W, A, G, d, dv, H, 0.5, None, False, 1024, td)
    tol = 3e-5 if dtype == "float32" else 3e-2
    for new in ([T], [T - 2, 1, 1]):
        oc = _Cache(part.cache_request(), 1, td)
        got, at = [], 0
        for n in new:
            got.append(summed(part.forward(h[at:at + n].to(DEV), oc.step([n]), 0, True)))
            at += n
        assert rel_err(torch.cat(got)[T - 1:], ref[T - 1:]) < tol


# -------------------------------------------------------- the recurrent mixer
def _delta_weights(A, G, d, dv, taps, ra, rg, H, seed, td, a_log=-3.0):
    lin = H ** -0.5
    W = {"q": rnd(G * d, H, seed=seed, std=1.5 * lin), "k": rnd(G * d, H, seed=seed + 1, std=1.5 * lin),
         "v": rnd(A * dv, H, seed=seed + 2, std=1.5 * lin),
         "q.conv": rnd(G * d, taps, seed=seed + 3, std=0.6) + 0.3,
         "k.conv": rnd(G * d, taps, seed=seed + 4, std=0.6) + 0.3,
         "v.conv": rnd(A * dv, taps, seed=seed + 5, std=0.6) + 0.3,
         "b": rnd(A, H, seed=seed + 6, std=1.5 * lin),
         "A_log": rnd(A, seed=seed + 7, std=0.7) + a_log,
         "norm": rnd(dv, seed=seed + 8, std=0.3) + 1.0,
         "a1": rnd(ra, H, seed=seed + 9, std=lin), "a2": rnd(A * d, ra, seed=seed + 10, std=ra ** -0.5),
         "dt_bias": rnd(A * d, seed=seed + 11),
         "g1": rnd(rg, H, seed=seed + 12, std=lin),
         "g2": rnd(A * dv, rg, seed=seed + 13, std=1.5 * rg ** -0.5),
         "o": rnd(H, A * dv, seed=seed + 14, std=(A * dv) ** -0.5)}
    return {k: v.to(td) for k, v in W.items()}


def _delta_part(W, A, G, d, dv, taps, ra, rg, H, td, eps=1e-5):
    from agave_b200.config.base import ChannelDeltaSpec
    from agave_b200.parts.delta import ChannelDeltaMixer
    spec = ChannelDeltaSpec(n_heads=A, n_qk_heads=G, head_dim=d, value_dim=dv, conv_taps=taps,
                            decay_rank=ra, gate_rank=rg, eps=eps, unit_eps=1e-6)
    part = ChannelDeltaMixer(spec, H, td, torch.device(DEV))
    part.load({"q_proj.weight": W["q"], "k_proj.weight": W["k"], "v_proj.weight": W["v"],
               "q_conv.weight": W["q.conv"], "k_conv.weight": W["k.conv"],
               "v_conv.weight": W["v.conv"], "beta_proj.weight": W["b"], "a_log": W["A_log"],
               "dt_bias": W["dt_bias"], "decay_down.weight": W["a1"], "decay_up.weight": W["a2"],
               "gate_down.weight": W["g1"], "gate_up.weight": W["g2"],
               "out_norm.weight": W["norm"], "o_proj.weight": W["o"]}, td, torch.device(DEV))
    return part


DELTA = [
    # A, G, d, dv, taps, ra, rg, H
    (4, 2, 12, 10, 2, 6, 5, 72),          # odd sizes, two heads per query/key head
    (4, 4, 64, 64, 4, 24, 24, 192),       # keys of 64: four lanes a column
    (2, 1, 32, 128, 5, 8, 16, 128),       # value heads wider than the keys
    (1, 1, 16, 48, 1, 1, 1, 96),          # one head, one tap: no convolution state
    (3, 3, 8, 8, 4, 12, 3, 40),           # keys shorter than a lane's rows
    (2, 2, 136, 24, 3, 4, 4, 64),         # keys that do not fill their lanes
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("A, G, d, dv, taps, ra, rg, H", DELTA)
def test_delta_mixer_as_prompt_in_portions_and_token_by_token(dtype, A, G, d, dv, taps, ra, rg, H):
    """The mixer alone against the plain one: the whole sequence in one step; a prompt and
    then tokens one by one; portions of 2, 1, 3, 37 and the rest (each going on from the
    state and the convolution's inputs the one before left)."""
    td = TD[dtype]
    T = 90
    W = _delta_weights(A, G, d, dv, taps, ra, rg, H, 70, td)
    h = rnd(T, H, seed=71).to(td)
    m = {"heads": A, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    ref = P.delta_mixer(h.double(), {k: v.double() for k, v in W.items()}, "", m, 1e-5)
    part = _delta_part(W, A, G, d, dv, taps, ra, rg, H, td)
    tol = 5e-5 if dtype == "float32" else 4e-2
    for new in ([T], [50] + [1] * 40, [1] * 12 + [78], [2, 1, 3, 37, 47], [3, 2, 2, 83]):
        oc = _Cache(part.cache_request(), 1, td)
        got, at = [], 0
        for n in new:
            got.append(summed(part.forward(h[at:at + n].to(DEV), oc.step([n]), 0, True)))
            at += n
        assert rel_err(torch.cat(got), ref) < tol, new[:3]


@pytest.mark.parametrize("dtype", DTYPES)
def test_delta_mixer_unequal_batches_and_slots_used_again(dtype):
    """Three sequences of unequal lengths start together and go on one token at a time, the
    shortest ending first; then another sequence takes a freed slot, whose state must start
    at zero.  Each against the plain mixer on that sequence alone."""
    td = TD[dtype]
    A, G, d, dv, taps, ra, rg, H = 4, 2, 32, 24, 4, 8, 6, 96
    W = _delta_weights(A, G, d, dv, taps, ra, rg, H, 90, td)
    Wd = {k: v.double() for k, v in W.items()}
    m = {"heads": A, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    part = _delta_part(W, A, G, d, dv, taps, ra, rg, H, td)
    tol = 5e-5 if dtype == "float32" else 4e-2
    oc = _Cache(part.cache_request(), 3, td)
    for round_, (starts, totals) in enumerate([((40, 1, 7), (52, 4, 20)), ((2, 30, 3), (9, 33, 5))]):
        hs = [rnd(n, H, seed=100 + 10 * round_ + i).to(td) for i, n in enumerate(totals)]
        refs = [P.delta_mixer(x.double(), Wd, "", m, 1e-5) for x in hs]
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
def test_what_the_state_took_in_hundreds_of_tokens_ago_decides(dtype):
    """Decays close to one (A_log round -9): what the fourth token wrote is still the greater
    part of the read-out after 600 tokens, in one step and across 500 decoded tokens.  Queries
    are made like keys (same projection and taps) from the first half of the input and values
    from the second half; tokens 1 to 3 have the last three tokens' first halves, so the last
    query is the fourth token's key, and the fourth token's second half is thirty times as
    large, so its write outweighs the hundreds of partly matching ones after it."""
    td = TD[dtype]
    A, G, d, dv, taps, ra, rg, H = 2, 2, 64, 32, 3, 8, 8, 128
    T = 600
    W = _delta_weights(A, G, d, dv, taps, ra, rg, H, 120, td, a_log=-9.0)
    W["q"], W["q.conv"] = W["k"].clone(), W["k.conv"].clone()
    W["q"][:, H // 2:] = 0
    W["k"][:, H // 2:] = 0
    W["v"][:, :H // 2] = 0
    Wd = {k: v.double() for k, v in W.items()}
    h = rnd(T, H, seed=121)
    h[1:4, :H // 2] = h[T - 3:, :H // 2]
    h[3, H // 2:] *= 30.0
    h = h.to(td)
    m = {"heads": A, "kv_heads": G, "dim": d, "vdim": dv, "conv": taps}
    ref = P.delta_mixer(h.double(), Wd, "", m, 1e-5)
    h2 = h.clone()
    h2[1:4] = h[5:8]
    assert rel_err(P.delta_mixer(h2.double(), Wd, "", m, 1e-5)[T - 1:], ref[T - 1:]) > 0.1
    part = _delta_part(W, A, G, d, dv, taps, ra, rg, H, td)
    tol = 1e-4 if dtype == "float32" else 5e-2
    for new in ([T], [100] + [1] * 500):
        oc = _Cache(part.cache_request(), 1, td)
        got, at = [], 0
        for n in new:
            got.append(summed(part.forward(h[at:at + n].to(DEV), oc.step([n]), 0, True)))
            at += n
        assert rel_err(torch.cat(got)[T - 1:], ref[T - 1:]) < tol


# ------------------------------------------------------------- whole models
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
    """Every row of prompts of 1, 2, a block's and a page's length, and of 300 tokens."""
    eng, folder = engine_for(name, dtype)
    for n in (1, 2, 7, 8, 64, 65, 300):
        toks = tokens(n, vocab(name), 20 + n)
        s = eng.acquire()
        got = eng.step([(s, toks)], [list(range(n))])
        eng.release(s)
        rows_agree(got, plain_logits(folder, toks), dtype, f"{name} {n} tokens")


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
    whole sequence at once: decoding starts after one token, inside the first block, at a
    page border, and runs past several blocks' edges."""
    eng, folder = engine_for(name, dtype)
    for n, cut in ((100, 60), (41, 1), (200, 127), (140, 64), (12, 2)):
        toks = tokens(n, vocab(name), 11 + n)
        rows_agree(alone(eng, toks, cut), plain_logits(folder, toks), dtype, f"{name} {n}/{cut}")


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
            rows_agree(torch.cat(got[i]), plain_logits(folder, seqs[i]), dtype,
                       f"{name} round {round_} request {i}")


@pytest.mark.parametrize("name", NAMES)
def test_lengths_round_page_borders_and_block_edges(name):
    """32-bit: prompts that end just before, on and just after a page border and the blocks'
    edges, each followed by three decoded tokens."""
    eng, folder = engine_for(name, "float32")
    blocks = {l["mixer"]["mask"]["size"] for l in CONFIGS[name]["layers"]
              if l["type"] == "attention" and l["mixer"].get("mask")}
    edges = {63, 64, 65, 127, 128, 129}
    for w in blocks:
        edges |= {max(1, w - 1), w, w + 1, 2 * w - 1, 2 * w, 2 * w + 1}
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
@pytest.mark.parametrize("name", ["V1", "V2"])
def test_long_decoding(name, dtype):
    """300 tokens decoded after a prompt of 5: several pages and blocks, the rings wrap more
    than once, the state goes through 300 updates."""
    eng, folder = engine_for(name, dtype)
    toks = tokens(305, vocab(name), 77)
    rows_agree(alone(eng, toks, 5), plain_logits(folder, toks), dtype, name)


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
        ref = plain_logits(folder, p + g)
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
    folder = folder_for("V1", TD[dtype])
    V = vocab("V1")
    prompts = [tokens(n, V, 900 + n) for n in (5, 66, 17, 3, 40, 21, 8)]
    wide = Engine(folder, dtype=dtype, max_tokens=4096)
    narrow = Engine(folder, dtype=dtype, max_tokens=4096, max_batch=3)
    a = wide.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    b = narrow.generate(prompts, max_new_tokens=10, stop_token_ids=[])
    same = sum(x == y for x, y in zip(a, b))
    assert same >= (len(prompts) if dtype == "float32" else len(prompts) - 2)


def test_sampling_runs_on_this_architecture():
    eng, _ = engine_for("V1", "bfloat16")
    V = vocab("V1")
    kw = dict(max_new_tokens=8, temperature=0.8, top_k=20, top_p=0.9, seed=5, stop_token_ids=[])
    outs = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], **kw)
    again = eng.generate([tokens(6, V, 1), tokens(30, V, 2)], **kw)
    assert outs == again and all(len(o) == 8 and all(0 <= t < V for t in o) for o in outs)


def _with_ranks(name):
    import copy
    raw = copy.deepcopy(CONFIGS[name])
    for i, (ra, rg) in RANKS[name].items():
        raw["layers"][i]["mixer"].update(decay_rank=ra, gate_rank=rg)
    return raw


def test_random_weights_from_a_configuration():
    """``Engine.from_config`` with the bottlenecks' widths written into the configuration: a
    model with drawn weights steps and generates."""
    from agave_b200.engine.api import Engine
    raw = _with_ranks("V1")
    eng = Engine.from_config(raw, seed=3, max_tokens=1024)
    outs = eng.generate([tokens(9, raw["vocab"], 1)], max_new_tokens=5, stop_token_ids=[])
    assert len(outs[0]) == 5
    info = eng.model_info()
    assert info["architecture"] == "Bovozen" and info["weight_bytes"] > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_replay_as_a_process(dtype):
    name = "V2"
    folder = folder_for(name, TD[dtype])
    V = vocab(name)
    a, b = tokens(210, V, 5), tokens(33, V, 6)
    refs = {"a": plain_logits(folder, a), "b": plain_logits(folder, b)}
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
    out = tempfile.mkdtemp(prefix="bovozen_trace_")
    text = "".join(json.dumps(s) + "\n" for s in steps)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder,
                        "--dtype", dtype, "--out", out, "--max-tokens", "512"],
                       input=text, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done ")] == \
        [f"done {s['step']}" for s in steps]
    got0 = torch.from_numpy(np.fromfile(os.path.join(out, "0.f32"), dtype="<f4").reshape(4, V))
    rows_agree(got0, torch.cat([refs["a"][[0, 100, 194]], refs["b"][[29]]]), dtype, "step 0")
    rows, want = [], []
    for k in range(15):
        g = torch.from_numpy(np.fromfile(os.path.join(out, f"{k + 1}.f32"), dtype="<f4").reshape(-1, V))
        rows.append(g)
        want.append(refs["a"][195 + k:196 + k])
        if k in (0, 2):
            want.append(refs["b"][30 + k:31 + k])
    rows_agree(torch.cat(rows), torch.cat(want), dtype, "decoded")
    shutil.rmtree(out, ignore_errors=True)


def test_command_line_on_this_architecture():
    """``python -m agave_b200`` picks the model class from config.json: greedy tokens equal the
    plain model's, --model-info names the architecture, --profile lists this design's
    operations, --random-weights draws a model from a config.json that states the
    bottlenecks' widths."""
    name = "V2"
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
    assert r.returncode == 0 and "Bovozen" in r.stdout, r.stderr[-2000:]
    r = run(folder, "--tokens", toks, "-n", "3", "--profile", "--dtype", "bfloat16")
    assert r.returncode == 0, r.stderr[-2000:]
    for op in ("norm", "qkv", "attention", "delta_prepare", "delta_scan", "delta_out", "router",
               "experts_gate_up", "experts_down", "out_proj", "up", "down", "lm_head", "TOTAL"):
        assert op in r.stderr, (op, r.stderr[-1500:])
    with tempfile.TemporaryDirectory() as d:
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(_with_ranks(name), f)
        outs = []
        for seed in ("3", "3", "4"):
            r = run(d, "--random-weights", seed, "--tokens", toks, "-n", "5", "--json")
            assert r.returncode == 0, r.stderr[-2000:]
            outs.append(json.loads(r.stdout.strip().splitlines()[-1])["output_ids"])
        assert outs[0] == outs[1] and len(outs[0]) == 5


@pytest.mark.parametrize("name, room", [("V1", 60), ("V2", 90), ("V3", 64)])
def test_a_cache_shorter_than_a_page_or_a_block(name, room):
    """32-bit: a cache of one or two pages.  A block that still fits a sequence keeps its
    edge although its group is no ring; a block no sequence can outgrow is none."""
    from agave_b200.engine.api import Engine
    folder = folder_for(name, torch.float32)
    eng = Engine(folder, dtype="float32", max_tokens=room, ctx_size=room, max_batch=1)
    toks = tokens(room, vocab(name), 5)
    rows_agree(alone(eng, toks, room - 15), plain_logits(folder, toks), "float32", name)
