"""Small Kadavik configurations and a writer of model folders for the tests.

The writer makes every tensor under its checkpoint name from the configuration dictionary
alone (it does not ask the library which names it expects), with scales chosen so that faults
show: scores of order one, forget gates close enough to one that a state lost hundreds of
tokens ago is missed, router logits and gates spread round zero.
"""
import atexit
import json
import os
import shutil
import tempfile

import torch


def attention(heads, kv_heads, dim, vdim, scale, conv=None, size=None, keep_first=None, rot=None,
              kv_from=None):
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "scale": scale, "vdim": vdim}
    if conv is not None:
        m["conv"] = conv
    if size is not None:
        m["mask"] = {"size": size}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot is not None:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return "attention", m


def rotation(dims, base, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def mlstm(heads, dim, vdim, cap):
    return "mlstm", {"dim": dim, "gate_cap": cap, "heads": heads, "vdim": vdim}


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(experts, identity, top, ff, scale=None, shared=None):
    r = {"experts": experts, "top": top}
    if identity is not None:
        r["identity"] = identity
    if scale is not None:
        r["scale"] = scale
    f = {"expert": {"ff": ff}, "kind": "moe", "router": r}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


def config(width, vocab, layers, eps=1e-5, embed_scale=None, logit_scale=None, side=None):
    cfg = {"architecture": "Kadavik",
           "layers": [{"mixer": m, "mlp": ff, "type": kind} for (kind, m), ff in layers],
           "norm": {"eps": eps}, "vocab": vocab, "width": width}
    if embed_scale is not None:
        cfg["embedding"] = {"scale": embed_scale}
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    if side is not None:
        cfg["token_side"] = {"dim": side}
    return cfg


# K1: small odd sizes (every kernel's general form): attention first, with a window shorter
# than a page behind which two keys stay, a rotation of part of the head with scaled
# frequencies; a layer without a feed-forward; a layer that borrows keys and values and looks
# at them through another mask; identity experts with and without a shared expert; value heads
# wider and narrower than the keys.
K1 = config(72, 210, [
    (attention(4, 2, 10, 14, 0.4, conv=2, size=7, keep_first=2,
               rot=rotation(6, 10000.0, (8.0, 1.0, 4.0, 16))), dense(40)),
    (mlstm(3, 12, 10, 8.0), None),
    (attention(4, 2, 10, 14, 0.45, conv=3, size=20, keep_first=0,
               rot=rotation(6, 10000.0, (8.0, 1.0, 4.0, 16)), kv_from=0),
     moe(5, 1, 2, 24, scale=1.5)),
    (mlstm(2, 20, 6, 15.0), moe(3, 2, 3, 16, scale=0.7, shared=20)),
    (attention(3, 3, 12, 6, 0.35, conv=3, rot=rotation(12, 300.0)), dense(56)),
], eps=1e-5, embed_scale=3.0, logit_scale=0.5, side=5)

# K2: the sizes that take the tensor-core kernels (head sizes 64, four query heads per kv
# head, windows that cross pages), a window without kept keys (a ring in the cache), four taps.
K2 = config(128, 320, [
    (mlstm(4, 64, 64, 12.0), moe(7, 2, 3, 64, scale=2.5, shared=96)),
    (attention(4, 1, 64, 64, 0.13, conv=4, size=100, keep_first=3,
               rot=rotation(32, 500.0, (4.0, 2.0, 8.0, 64))), moe(8, 1, 2, 64, scale=1.0)),
    (mlstm(2, 32, 128, 10.0), dense(192)),
    (attention(4, 1, 64, 64, 0.13, conv=2, size=100, keep_first=3,
               rot=rotation(32, 500.0, (4.0, 2.0, 8.0, 64)), kv_from=1), dense(128)),
    (attention(4, 2, 64, 64, 0.12, conv=2, size=70, keep_first=0, rot=rotation(64, 10000.0)),
     moe(4, 0, 2, 64, scale=1.0, shared=64)),
    # (it looks further back than the layer whose keys it borrows: that layer's cache must
    # keep more than its own window)
    (attention(4, 2, 64, 64, 0.12, size=150, rot=rotation(64, 10000.0), kv_from=4), None),
], eps=1e-6, embed_scale=8.0, logit_scale=3.0, side=16)

# K3: values the other two make unequal are equal here or 1, and what may be absent is: one
# head, as many kv heads as heads, one tap and no convolution at all, a window of one with one
# kept key, a window of exactly a page, no rotation, one expert of one, every expert chosen, no
# identity experts, no token input, no multipliers.
K3 = config(96, 150, [
    (attention(1, 1, 16, 16, 0.3, conv=1, size=1, keep_first=1), moe(1, 0, 1, 32)),
    (mlstm(1, 16, 48, 1.0), moe(4, None, 4, 24, shared=8)),
    (attention(2, 2, 24, 8, 0.3, size=64, keep_first=64, rot=rotation(24, 50.0)), dense(48)),
    (mlstm(3, 8, 8, 30.0), None),
    (attention(2, 1, 32, 32, 0.25, conv=5), moe(6, 3, 1, 16, scale=2.0)),
], eps=3e-6)

# K4: a width, a vocabulary and inner sizes that are no multiples of 8 (no product takes the
# tensor cores), attention layers only at the end, a source with two readers.
K4 = config(76, 211, [
    (mlstm(2, 18, 22, 6.0), moe(3, 1, 2, 20, scale=1.2, shared=12)),
    (mlstm(1, 40, 10, 12.0), dense(36)),
    (attention(2, 1, 20, 12, 0.3, conv=2, size=33, keep_first=1, rot=rotation(10, 2000.0)),
     moe(2, 2, 3, 28, scale=1.0)),
    (attention(2, 1, 20, 12, 0.3, conv=4, size=9, keep_first=5, rot=rotation(10, 2000.0),
               kv_from=2), None),
    (attention(2, 1, 20, 12, 0.35, size=200, rot=rotation(10, 2000.0), kv_from=2), dense(44)),
], eps=2e-5, embed_scale=5.0, logit_scale=1.7, side=3)

# K5: windows without kept keys, so that the cache keeps rings of them, each read by a second
# layer through the same mask.
K5 = config(128, 200, [
    (attention(4, 2, 64, 64, 0.15, conv=3, size=70, keep_first=0, rot=rotation(32, 1e4)), dense(64)),
    (mlstm(2, 32, 32, 10.0), None),
    (attention(8, 2, 64, 64, 0.15, conv=2, size=70, keep_first=0, rot=rotation(32, 1e4), kv_from=0),
     dense(64)),
    (attention(2, 1, 16, 16, 0.3, size=130), None),
    (attention(2, 1, 16, 16, 0.3, size=130, kv_from=3), dense(32)),
], eps=1e-5, embed_scale=2.0, side=4)

CONFIGS = {"K1": K1, "K2": K2, "K3": K3, "K4": K4, "K5": K5}


def make_tensors(cfg, seed, dtype):
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, std=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * std + mean).to(dtype)

    H, V = cfg["width"], cfg["vocab"]
    L = len(cfg["layers"])
    scale = (cfg.get("embedding") or {}).get("scale", 1.0)
    t = {"embed": rnd(V, H, std=1.0 / scale), "final.norm": rnd(H, std=0.2, mean=1.0)}
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        t["side.embed"] = rnd(V, L * side, std=1.0)
    lin = 1.0 / H ** 0.5                                   # unit outputs from a unit stream
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        t[p + "norm1"] = rnd(H, std=0.2, mean=0.8)
        t[p + "norm1b"] = rnd(H, std=0.2, mean=0.7)
        A, d, dv = m["heads"], m["dim"], m["vdim"]
        if layer["type"] == "attention":
            G = m.get("kv_heads", A)
            taps = m.get("conv")
            t[p + "mix.q"] = rnd(A * d, H, std=1.5 * lin)
            if taps:
                t[p + "mix.q.conv"] = rnd(A * d, taps, std=0.5, mean=0.4)
            if m.get("kv_from") is None:
                t[p + "mix.k"] = rnd(G * d, H, std=1.5 * lin)
                t[p + "mix.v"] = rnd(G * dv, H, std=lin)
                if taps:
                    t[p + "mix.k.conv"] = rnd(G * d, taps, std=0.5, mean=0.4)
                    t[p + "mix.v.conv"] = rnd(G * dv, taps, std=0.5, mean=0.4)
        else:
            t[p + "mix.q"] = rnd(A * d, H, std=1.5 * lin)
            t[p + "mix.k"] = rnd(A * d, H, std=1.5 * lin)
            t[p + "mix.v"] = rnd(A * dv, H, std=lin)
            t[p + "mix.i"] = rnd(A, H, std=2.0 * lin)
            t[p + "mix.i.b"] = rnd(A, std=0.5)
            t[p + "mix.f"] = rnd(A, H, std=lin)
            t[p + "mix.f.b"] = rnd(A, std=0.5, mean=4.0)
            t[p + "mix.norm"] = rnd(A * dv, std=0.3, mean=1.0)
        t[p + "mix.g"] = rnd(A * dv, H, std=1.5 * lin)
        t[p + "mix.o"] = rnd(H, A * dv, std=1.0 / (A * dv) ** 0.5)
        if side:
            t[p + "side.gate"] = rnd(side, H, std=lin)
            t[p + "side.proj"] = rnd(H, side, std=1.0 / side ** 0.5)
            t[p + "side.norm"] = rnd(H, std=0.2, mean=0.5)
        f = layer["mlp"]
        if f is None:
            continue
        t[p + "norm2"] = rnd(H, std=0.2, mean=0.8)
        t[p + "norm2b"] = rnd(H, std=0.2, mean=0.7)
        q = p + "mlp."
        if f["kind"] == "dense":
            t[q + "gate"] = rnd(f["ff"], H, std=1.5 * lin)
            t[q + "up"] = rnd(f["ff"], H, std=lin)
            t[q + "down"] = rnd(H, f["ff"], std=1.0 / f["ff"] ** 0.5)
            continue
        ff = f["expert"]["ff"]
        E = f["router"]["experts"]
        n_out = E + (f["router"].get("identity") or 0)
        for e in range(E):
            t[f"{q}e{e}.gate"] = rnd(ff, H, std=1.5 * lin)
            t[f"{q}e{e}.up"] = rnd(ff, H, std=1.5 * lin)
            t[f"{q}e{e}.down"] = rnd(H, ff, std=1.0 / ff ** 0.5)
        t[q + "router"] = rnd(n_out, H, std=2.0 * lin)
        t[q + "correction"] = rnd(n_out, std=0.1)
        if f.get("shared"):
            sf = f["shared"]["ff"]
            t[q + "shared.gate"] = rnd(sf, H, std=1.5 * lin)
            t[q + "shared.up"] = rnd(sf, H, std=1.5 * lin)
            t[q + "shared.down"] = rnd(H, sf, std=1.0 / sf ** 0.5)
            t[q + "shared.sg"] = rnd(1, H, std=2.0 * lin)
    return t


_FOLDERS = {}


def write_folder(cfg, seed, dtype, prefix="kadavik_"):
    from safetensors.torch import save_file
    d = tempfile.mkdtemp(prefix=prefix)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in make_tensors(cfg, seed, dtype).items()},
              os.path.join(d, "model.safetensors"))
    return d


def folder_for(name, dtype=torch.float32, seed=0):
    """A temporary model folder of configuration ``name`` (made once per run)."""
    key = (name, dtype, seed)
    if key not in _FOLDERS:
        _FOLDERS[key] = write_folder(CONFIGS[name], seed, dtype, prefix=f"kadavik_{name}_")
    return _FOLDERS[key]


def _cleanup():
    for d in _FOLDERS.values():
        shutil.rmtree(d, ignore_errors=True)


atexit.register(_cleanup)


def tokens(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def read_folder(folder):
    from safetensors.torch import load_file
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, load_file(os.path.join(folder, "model.safetensors"))


_READ = {}


def plain_logits(folder, toks, streams=None, chosen=None):
    from plain import kadavik_plain as P
    if folder not in _READ:
        _READ[folder] = read_folder(folder)
    cfg, w = _READ[folder]
    return P.forward(cfg, w, toks, chosen=chosen, layers_out=streams)
