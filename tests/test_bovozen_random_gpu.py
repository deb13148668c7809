"""Bovozen configurations drawn from seeds: random sizes (odd ones and those the tensor-core
kernels take), random order of the two mixers, layers without a feed-forward, dense and
routed feed-forwards with and without a shared expert, blocks from one token to longer than
the prompt or none, value mixing that starts at any attention layer or nowhere, one to five
taps.  Each model runs a cut request, an unequal batch that is decoded together, and greedy
generation, in both precisions, against the plain model."""
import random
import shutil

import pytest
import torch

from bovozen_util import attention, config, delta, dense, moe, plain_logits, tokens, write_folder
from test_bovozen_gpu import TD, alone, rows_agree

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(1000 + seed)
    wide = seed % 2 == 1                       # every second model has tensor-core sizes
    mult = 8 if wide else 2
    width = rng.choice([64, 128, 192]) if wide else 2 * rng.randint(17, 60)
    vocab = rng.randint(60, 400)
    # the values of the layers that mix are of one shape
    mix_kv = rng.choice([1, 2, 3])
    mix_vdim = rng.choice([16, 32, 64]) if wide else mult * rng.randint(2, 8)
    mixing_from = rng.choice([0, 1, 2, 99])     # attention layers before this one do not mix

    seen = [0]

    def one_mixer():
        if rng.random() < 0.5:
            nth = seen[0]
            seen[0] += 1
            mixes = nth >= mixing_from
            kv = mix_kv if mixes else rng.choice([1, 2, 3, 4])
            heads = kv * rng.choice([1, 2, 4])
            dim = rng.choice([16, 32, 48, 64, 80]) if wide else mult * rng.randint(2, 8)
            vdim = mix_vdim if mixes else (dim if rng.random() < 0.5 else mult * rng.randint(2, 8))
            block = rng.choice([None, 1, 2, 5, 33, 64, 65, 100, 128, 500])
            return attention(heads, kv, dim, vdim, 1.3 / dim ** 0.5, block=block, v_mix=mixes)
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2])
        dim = rng.choice([16, 32, 64, 128]) if wide else mult * rng.randint(2, 12)
        vdim = rng.choice([16, 32, 64]) if wide else mult * rng.randint(2, 10)
        return delta(heads, kv, dim, vdim, rng.randint(1, 5), rng.randint(1, 12),
                     rng.randint(1, 12))

    def one_ff():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.5:
            return dense(mult * rng.randint(3, 20))
        experts = rng.randint(1, 9)
        shared = None if rng.random() < 0.4 else mult * rng.randint(1, 10)
        return moe(experts, rng.randint(1, experts), mult * rng.randint(2, 10), shared)

    layers = [(one_mixer(), one_ff()) for _ in range(rng.randint(2, 6))]
    return config(width, vocab, 600, layers, eps=rng.choice([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(10))
def test_a_drawn_configuration(seed, dtype):
    from agave_b200.engine.api import Engine
    cfg, ranks = draw(seed)
    folder = write_folder(cfg, ranks, seed, TD[dtype], prefix=f"bovozen_draw{seed}_")
    try:
        eng = Engine(folder, dtype=dtype, max_tokens=4096)
        V = cfg["vocab"]
        # a cut request: most of it at once, the rest token by token
        toks = tokens(150 + 7 * seed, V, seed)
        rows_agree(alone(eng, toks, len(toks) - 20), plain_logits(folder, toks), dtype,
                   f"seed {seed} alone")
        # an unequal batch decoded together; the shorter request ends first
        seqs = [tokens(n, V, 100 + seed + n) for n in (70 + seed, 9, 1 + seed)]
        lens = [len(s) - 4 - 2 * i for i, s in enumerate(seqs)]
        lens = [max(1, n) for n in lens]
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
        for sl in slots:
            eng.release(sl)
        for i, s in enumerate(seqs):
            rows_agree(torch.cat(got[i]), plain_logits(folder, s), dtype,
                       f"seed {seed} request {i}")
        # greedy generation through the scheduler
        prompts = [tokens(n, V, 500 + seed + n) for n in (3, 40)]
        outs = eng.generate(prompts, max_new_tokens=6, stop_token_ids=[])
        slack = 2e-3 if dtype == "float32" else 8e-2
        misses = 0
        for p, g in zip(prompts, outs):
            ref = plain_logits(folder, p + g)
            for k, t in enumerate(g):
                row = ref[len(p) - 1 + k]
                misses += float(row.max() - row[t]) > slack * float(row.abs().max())
        assert misses <= (0 if dtype == "float32" else 2), misses
    finally:
        shutil.rmtree(folder, ignore_errors=True)
