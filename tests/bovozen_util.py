"""Small Bovozen configurations and a writer of model folders for the tests.

The writer makes every tensor under its checkpoint name from the configuration dictionary
alone (it does not ask the library which names it expects), with scales chosen so that
faults show: scores of order one to two, decays close enough to one that a state lost
hundreds of tokens ago is missed, router logits and gates spread round zero.
"""
import atexit
import json
import os
import shutil
import tempfile

import torch


def attention(heads, kv_heads, dim, vdim, scale, block=None, v_mix=False):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "v_mix": v_mix,
         "vdim": vdim}
    if block is not None:
        m["mask"] = {"size": block}
    return "attention", m, None


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    m = {"conv": conv, "dim": dim, "heads": heads, "kv_heads": kv_heads, "vdim": vdim}
    return "channel_delta", m, (decay_rank, gate_rank)


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, top, ff, shared=None):
    f = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def config(width, vocab, positions, layers, eps=1e-5):
    """``layers``: (mixer tuple, feed-forward or None).  Returns the configuration and, per
    recurrent layer, the widths of its two bottlenecks (config.json does not carry them)."""
    out, ranks = [], {}
    for i, (mix, ff) in enumerate(layers):
        kind, m, extra = mix
        if extra is not None:
            ranks[i] = extra
        out.append({"mixer": m, "mlp": ff, "type": kind})
    cfg = {"architecture": "Bovozen", "layers": out, "max_positions": positions,
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    return cfg, ranks


# V1: small odd sizes (every kernel's general form): a recurrent layer first, a block
# shorter than a page, a layer without a feed-forward, value mixing that starts at the third
# layer, experts without a shared one, two taps, two heads per query/key head in both mixers.
V1 = config(72, 210, 700, [
    (delta(4, 2, 12, 10, 2, 6, 5), dense(40)),
    (attention(4, 2, 10, 14, 0.45, block=7), None),
    (attention(6, 3, 8, 6, 0.5, block=50, v_mix=True), moe(5, 2, 24)),
    (delta(2, 2, 20, 6, 3, 4, 9), moe(3, 3, 16, shared=20)),
    (attention(3, 3, 12, 6, 0.4, block=33, v_mix=True), dense(56)),
    (attention(3, 3, 4, 6, 0.6, v_mix=True), None),
], eps=1e-5)

# V2: the sizes that take the tensor-core kernels (head sizes 64, four query heads per kv
# head, a block that crosses pages), attention without a mask, five taps.
V2 = config(128, 320, 1024, [
    (attention(4, 1, 64, 64, 0.16, block=100, v_mix=True), moe(8, 2, 64, shared=128)),
    (delta(4, 2, 64, 32, 5, 16, 8), moe(8, 3, 64, shared=64)),
    (attention(4, 1, 64, 64, 0.16, v_mix=True), dense(192)),
    (delta(2, 1, 32, 128, 4, 8, 16), dense(128)),
], eps=1e-6)

# V3: values the other two make unequal are equal here or 1: one head, as many kv heads as
# heads, a block of exactly one page, a block of one, one tap (no convolution state), one
# expert of one, every expert chosen, value heads wider than the keys, a single v_mix layer.
V3 = config(96, 150, 400, [
    (attention(3, 3, 16, 16, 0.35, block=64), moe(1, 1, 32)),
    (delta(1, 1, 16, 48, 1, 1, 1), moe(4, 4, 24, shared=8)),
    (attention(2, 2, 24, 8, 0.3, block=1, v_mix=True), dense(48)),
    (delta(3, 3, 8, 8, 4, 12, 3), None),
    (attention(1, 1, 32, 32, 0.25), moe(6, 1, 16)),
], eps=3e-6)

CONFIGS = {"V1": V1[0], "V2": V2[0], "V3": V3[0]}
RANKS = {"V1": V1[1], "V2": V2[1], "V3": V3[1]}


def make_tensors(cfg, ranks, seed, dtype):
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    H, V = cfg["width"], cfg["vocab"]
    t = {"embed": rnd(V, H, std=1.0), "pos": rnd(cfg["max_positions"], H, std=0.5),
         "final.norm": rnd(H, std=0.2)}
    lin = 1.0 / H ** 0.5                                   # unit outputs from a unit stream
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        t[p + "norm1"] = rnd(H, std=0.2, mean=-0.3)
        A, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            t[p + "mix.q"] = rnd(A * d, H, std=lin)
            t[p + "mix.k"] = rnd(G * d, H, std=lin)
            t[p + "mix.v"] = rnd(G * dv, H, std=lin)
            t[p + "mix.q.norm"] = rnd(A * d, std=0.3, mean=1.2)
            t[p + "mix.k.norm"] = rnd(G * d, std=0.3, mean=1.2)
            t[p + "mix.vmix"] = (torch.rand((), generator=g) * 0.6 + 0.2).to(dtype)
        else:
            ra, rg = ranks[i]
            taps = m["conv"]
            t[p + "mix.q"] = rnd(G * d, H, std=1.5 * lin)
            t[p + "mix.k"] = rnd(G * d, H, std=1.5 * lin)
            t[p + "mix.v"] = rnd(A * dv, H, std=1.5 * lin)
            for name, rows in (("q", G * d), ("k", G * d), ("v", A * dv)):
                t[p + f"mix.{name}.conv"] = rnd(rows, taps, std=0.6, mean=0.3)
            t[p + "mix.b"] = rnd(A, H, std=1.5 * lin)
            t[p + "mix.A_log"] = rnd(A, std=0.7, mean=-3.0)
            t[p + "mix.norm"] = rnd(dv, std=0.3, mean=1.0)
            t[p + "mix.a1"] = rnd(ra, H, std=lin)
            t[p + "mix.a2"] = rnd(A * d, ra, std=1.0 / ra ** 0.5)
            t[p + "mix.dt_bias"] = rnd(A * d, std=1.0)
            t[p + "mix.g1"] = rnd(rg, H, std=lin)
            t[p + "mix.g2"] = rnd(A * dv, rg, std=1.5 / rg ** 0.5)
        t[p + "mix.o"] = rnd(H, A * dv, std=1.0 / (A * dv) ** 0.5)
        f = layer["mlp"]
        if f is None:
            continue
        t[p + "norm2"] = rnd(H, std=0.2, mean=-0.3)
        q = p + "mlp."
        if f["kind"] == "dense":
            t[q + "up"] = rnd(f["ff"], H, std=lin)
            t[q + "down"] = rnd(H, f["ff"], std=1.0 / f["ff"] ** 0.5)
            continue
        ff = f["expert"]["ff"]
        E = f["router"]["experts"]
        for e in range(E):
            t[f"{q}e{e}.gate"] = rnd(ff, H, std=1.5 * lin)
            t[f"{q}e{e}.up"] = rnd(ff, H, std=1.5 * lin)
            t[f"{q}e{e}.down"] = rnd(H, ff, std=1.0 / ff ** 0.5)
        t[q + "router"] = rnd(E, H, std=2.0 * lin)
        t[q + "router.b"] = rnd(E, std=0.5)
        if f.get("shared"):
            sf = f["shared"]["ff"]
            t[q + "shared.gate"] = rnd(sf, H, std=1.5 * lin)
            t[q + "shared.up"] = rnd(sf, H, std=1.5 * lin)
            t[q + "shared.down"] = rnd(H, sf, std=1.0 / sf ** 0.5)
            t[q + "shared.sg"] = rnd(1, H, std=2.0 * lin)
    return t


_FOLDERS = {}


def write_folder(cfg, ranks, seed, dtype, prefix="bovozen_"):
    from safetensors.torch import save_file
    d = tempfile.mkdtemp(prefix=prefix)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in make_tensors(cfg, ranks, seed, dtype).items()},
              os.path.join(d, "model.safetensors"))
    return d


def folder_for(name, dtype=torch.float32, seed=0):
    """A temporary model folder of configuration ``name`` (made once per run)."""
    key = (name, dtype, seed)
    if key not in _FOLDERS:
        _FOLDERS[key] = write_folder(CONFIGS[name], RANKS[name], seed, dtype,
                                     prefix=f"bovozen_{name}_")
    return _FOLDERS[key]


def _cleanup():
    for d in _FOLDERS.values():
        shutil.rmtree(d, ignore_errors=True)


atexit.register(_cleanup)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def plain_logits(folder, toks, streams=None):
    from plain import bovozen_plain as P
    return P.forward(P.read_config(folder), P.read_weights(folder), toks, streams)
