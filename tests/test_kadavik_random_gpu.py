"""Kadavik configurations drawn from seeds: random sizes (odd ones and those the tensor-core
kernels take), random order of the two mixers, layers without a feed-forward, dense and routed
feed-forwards with and without identity experts and a shared expert, windows from one token to
longer than the prompt or none, kept keys from none to more than the window, one to five taps
or no convolution, rotations of part of the head, of all of it or none, with and without scaled
frequencies, layers that borrow an earlier layer's keys and values through a mask of their own,
with and without the token input and the two multipliers.  Each model runs a cut request, an
unequal batch that is decoded together, and greedy generation, in both precisions, against the
plain model."""
import random
import shutil

import pytest
import torch

from kadavik_util import (attention, config, dense, mlstm, moe, plain_logits, rotation, tokens,
                          write_folder)
from test_kadavik_gpu import TD, RecordedRoutes, reference, rows_agree

pytestmark = pytest.mark.gpu


def draw(seed):
    rng = random.Random(4000 + seed)
    wide = seed % 2 == 1                       # every second model has tensor-core sizes
    mult = 8 if wide else 2
    width = rng.choice([64, 128, 192]) if wide else 2 * rng.randint(17, 60)
    vocab = rng.randint(60, 400)
    owners = []                                # (layer, kv heads, dim, vdim, rot) with keys of their own

    def mask():
        size = rng.choice([None, 1, 2, 5, 33, 64, 65, 100, 128, 500])
        if size is None:
            return None, None
        return size, rng.choice([None, 0, 1, 3, 64, 70])

    def one_mixer(i):
        if rng.random() < 0.5:
            cap = rng.choice([1.0, 5.0, 15.0, 40.0])
            if wide:
                return mlstm(rng.choice([1, 2, 4]), rng.choice([16, 32, 64, 128]),
                             rng.choice([16, 32, 64, 96]), cap)
            return mlstm(rng.randint(1, 4), mult * rng.randint(2, 20), mult * rng.randint(2, 20), cap)
        size, keep = mask()
        conv = rng.choice([None, 1, 2, 3, 4, 5])
        if owners and rng.random() < 0.35:
            j, kv, dim, vdim, rot = rng.choice(owners)
            heads = kv * rng.choice([1, 2, 4])
            return attention(heads, kv, dim, vdim, 1.3 / dim ** 0.5, conv=conv, size=size,
                             keep_first=keep, rot=rot, kv_from=j)
        kv = rng.choice([1, 2, 3])
        heads = kv * rng.choice([1, 2, 4])
        dim = rng.choice([16, 32, 48, 64, 128]) if wide else mult * rng.randint(2, 12)
        vdim = dim if rng.random() < 0.5 else (rng.choice([16, 32, 64]) if wide
                                               else mult * rng.randint(2, 10))
        rot = None
        if rng.random() < 0.8:
            dims = dim if rng.random() < 0.4 else 2 * rng.randint(1, dim // 2)
            sc = None
            if rng.random() < 0.6:
                low = rng.choice([0.5, 1.0, 2.0])
                sc = (rng.choice([2.0, 4.0, 8.0]), low, low * rng.choice([2.0, 4.0]),
                      rng.choice([8, 32, 256]))
            rot = rotation(dims, rng.choice([50.0, 1e4, 5e5]), sc)
        owners.append((i, kv, dim, vdim, rot))
        return attention(heads, kv, dim, vdim, 1.3 / dim ** 0.5, conv=conv, size=size,
                         keep_first=keep, rot=rot)

    def one_ff():
        r = rng.random()
        if r < 0.2:
            return None
        if r < 0.45:
            return dense(mult * rng.randint(3, 20))
        experts = rng.randint(1, 9)
        identity = rng.choice([None, 0, 1, 2, 3])
        shared = None if rng.random() < 0.4 else mult * rng.randint(1, 10)
        return moe(experts, identity, rng.randint(1, experts + (identity or 0)),
                   mult * rng.randint(2, 10), scale=rng.choice([None, 0.5, 2.5]), shared=shared)

    layers = [(one_mixer(i), one_ff()) for i in range(rng.randint(2, 6))]
    return config(width, vocab, layers, eps=rng.choice([1e-6, 1e-5, 1e-3]),
                  embed_scale=rng.choice([None, 4.0, 11.5]),
                  logit_scale=rng.choice([None, 0.25, 3.0]),
                  # (a token input one wide is a sign: y / rms(y) jumps where its gate crosses zero,
                  # and no comparison holds there)
                  side=rng.choice([None, 2, 6, 16]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("seed", range(12))
def test_a_drawn_configuration(seed, dtype):
    from agave_b200.engine.api import Engine
    cfg = draw(seed)
    folder = write_folder(cfg, seed, TD[dtype], prefix=f"kadavik_draw{seed}_")
    try:
        eng = Engine(folder, dtype=dtype, max_tokens=4096)
        V = cfg["vocab"]
        # (bfloat16: the plain model runs under the experts the library chose in the very
        # steps that are compared; a close call may fall differently from step to step)
        def plain(toks, rec, pieces):
            if dtype == "float32":
                return plain_logits(folder, toks)
            return plain_logits(folder, toks, chosen=rec.of_rows(pieces))
        # a cut request: most of it at once, the rest token by token
        toks = tokens(150 + 7 * seed, V, seed)
        cut = len(toks) - 20
        with RecordedRoutes(eng) as rec:
            s0 = eng.acquire()
            got = [rec.step([(s0, toks[:cut])], [list(range(cut))])]
            for p in range(cut, len(toks)):
                got.append(rec.step([(s0, [toks[p]])], [[0]]))
            eng.release(s0)
        pieces = [(0, 0, cut)] + [(k, 0, 1) for k in range(1, len(toks) - cut + 1)]
        rows_agree(torch.cat(got), plain(toks, rec, pieces), dtype, f"seed {seed} alone")
        # an unequal batch decoded together; the shorter request ends first
        seqs = [tokens(n, V, 100 + seed + n) for n in (70 + seed, 9, 1 + seed)]
        lens = [len(s) - 4 - 2 * i for i, s in enumerate(seqs)]
        lens = [max(1, n) for n in lens]
        slots = [eng.acquire() for _ in seqs]
        got = [[] for _ in seqs]
        pieces = [[] for _ in seqs]
        with RecordedRoutes(eng) as rec:
            out = rec.step([(sl, s[:n]) for sl, s, n in zip(slots, seqs, lens)],
                           [list(range(n)) for n in lens])
            o = 0
            for i, n in enumerate(lens):
                got[i].append(out[o:o + n])
                pieces[i].append((0, o, n))
                o += n
            at = list(lens)
            while any(a < len(s) for a, s in zip(at, seqs)):
                live = [i for i in range(len(seqs)) if at[i] < len(seqs[i])]
                out = rec.step([(slots[i], [seqs[i][at[i]]]) for i in live], [[0]] * len(live))
                for r, i in enumerate(live):
                    got[i].append(out[r:r + 1])
                    pieces[i].append((len(rec.steps) - 1, r, 1))
                    at[i] += 1
        for sl in slots:
            eng.release(sl)
        for i, s in enumerate(seqs):
            rows_agree(torch.cat(got[i]), plain(s, rec, pieces[i]), dtype,
                       f"seed {seed} request {i}")
        # greedy generation through the scheduler
        prompts = [tokens(n, V, 500 + seed + n) for n in (3, 40)]
        outs = eng.generate(prompts, max_new_tokens=6, stop_token_ids=[])
        slack = 2e-3 if dtype == "float32" else 8e-2
        misses = 0
        for p, g in zip(prompts, outs):
            ref = reference(eng, folder, p + g, dtype)
            for k, t in enumerate(g):
                row = ref[len(p) - 1 + k]
                misses += float(row.max() - row[t]) > slack * float(row.abs().max())
        assert misses <= (0 if dtype == "float32" else 2), misses
    finally:
        shutil.rmtree(folder, ignore_errors=True)
