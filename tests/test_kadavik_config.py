"""Kadavik without a GPU: the configuration reader and its errors, the lowering to part
specs and a run order, tensor names and the loader, what the cache is asked for, and the plain
implementation's mechanisms on cases worked out by hand."""
import copy
import json
import math

import pytest
import torch

from agave_b200.config import ConfigError, load_config, resolve_architecture
from agave_b200.config.base import (AttentionSpec, BandScalingSpec, GatedFeedForwardSpec,
                                    MatrixMemorySpec, NormSpec, RoutedFeedForwardSpec,
                                    TokenSideSpec)
from agave_b200.config.kadavik import KadavikConfig
from agave_b200.models.decoder import decoder_param_specs
from agave_b200.weights import WeightsError, load_weights
from kadavik_util import CONFIGS, folder_for, make_tensors
from plain import kadavik_plain as P


# ------------------------------------------------------------------- reading
def test_registry_finds_the_architecture():
    assert resolve_architecture({"architecture": "Kadavik"}).name == "Kadavik"
    assert resolve_architecture({"model_type": "kadavik"}).name == "Kadavik"


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_reading_and_writing_round_trip(name):
    cfg = KadavikConfig.from_dict(CONFIGS[name])
    again = KadavikConfig.from_dict(cfg.to_dict())
    assert again == cfg
    assert len(cfg.layers) == len(CONFIGS[name]["layers"])


def test_what_may_be_absent_reads_as_none():
    cfg = KadavikConfig.from_dict(CONFIGS["K3"])
    assert (cfg.embed_scale, cfg.logit_scale, cfg.side_dim) == (1.0, 1.0, 0)
    m = cfg.layers[4].mixer
    assert (m.window, m.keep_first, m.rot, m.conv, m.kv_from) == (None, 0, None, 5, None)
    assert cfg.layers[2].mixer.conv == 0
    f = cfg.layers[1].mlp
    assert (f.identity, f.route_scale, f.shared_ff) == (0, 1.0, 8)
    assert cfg.layers[3].mlp is None


@pytest.mark.parametrize("path, value, match", [
    (("vocab",), None, "vocab"),
    (("width",), 0, "positive"),
    (("norm", "eps"), None, "norm.eps"),
    (("layers", 0, "type"), "conv", "not a mixer"),
    (("layers", 0, "mixer", "kv_heads"), 3, "multiple"),
    (("layers", 0, "mixer", "scale"), None, "scale"),
    (("layers", 0, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 0, "mixer", "dim"), 2.5, "integer"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mixer", "rot", "scaling", "high"), 0.5, "rot.scaling"),
    (("layers", 1, "mixer", "gate_cap"), None, "gate_cap"),
    (("layers", 2, "mixer", "kv_from"), 3, "earlier layer"),
    (("layers", 2, "mixer", "kv_from"), 1, "no keys and values"),
    (("layers", 2, "mixer", "vdim"), 8, "must equal"),
    (("layers", 0, "mlp", "kind"), "glu", "not a feed-forward"),
    (("layers", 2, "mlp", "router", "top"), 7, "top"),
    (("layers", 2, "mlp", "expert"), None, "expert"),
    (("layers", 3, "mlp", "shared", "ff"), None, "shared.ff"),
    (("token_side", "dim"), None, "token_side.dim"),
])
def test_errors_name_the_key(path, value, match):
    raw = copy.deepcopy(CONFIGS["K1"])
    d = raw
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        KadavikConfig.from_dict(raw)


# ------------------------------------------------------------------ lowering
def test_lowering_to_parts_and_run_order():
    cfg = KadavikConfig.from_dict(CONFIGS["K1"])
    spec = cfg.to_model_spec()
    assert len(spec.blocks) == 5 and spec.tie_embeddings
    assert (spec.embed_scale, spec.logit_scale, spec.token_side_width) == (3.0, 0.5, 25)
    # the third layer reads the first one's keys and values and keeps its own state
    assert [(c.block, c.cache, c.writes_cache, c.state) for c in spec.schedule] == \
        [(0, 0, True, None), (1, 1, True, None), (2, 0, False, 2), (3, 3, True, None),
         (4, 4, True, None)]
    assert spec.n_cache_entries() == 5
    norm = NormSpec(eps=1e-5, zero_centered=False)
    assert all(b.arrangement == "sandwich" and b.norm == norm for b in spec.blocks)
    assert spec.final_norm == norm
    assert [b.token_side for b in spec.blocks] == \
        [TokenSideSpec(dim=5, offset=5 * i, eps=1e-5) for i in range(5)]
    b0, b1, b2, b3, b4 = spec.blocks
    m = b0.mixer
    assert isinstance(m, AttentionSpec) and m.own_kv and m.out_gate and m.qk_norm is None
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.value_dim, m.scale) == (4, 2, 10, 14, 0.4)
    assert (m.window, m.keep_first, m.conv_taps) == (7, 2, 2)
    assert (m.position.theta, m.position.rotary_dim, m.position.interleaved) == (1e4, 6, False)
    assert m.position.scaling == BandScalingSpec(factor=8.0, original=16.0, low=1.0, high=4.0)
    # its reader looks through another mask: the cache keeps every key
    assert m.keep_all_keys
    assert b0.feed_forward == GatedFeedForwardSpec(intermediate_size=40, activation="gelu_tanh")
    assert b1.mixer == MatrixMemorySpec(n_heads=3, head_dim=12, value_dim=10, gate_cap=8.0,
                                        eps=1e-5, den_eps=1e-6)
    assert b1.feed_forward is None
    assert not b2.mixer.own_kv and (b2.mixer.window, b2.mixer.keep_first, b2.mixer.conv_taps) == \
        (20, 0, 3)
    f = b2.feed_forward
    assert isinstance(f, RoutedFeedForwardSpec)
    assert (f.n_experts, f.n_identity, f.top, f.intermediate_size, f.activation) == \
        (5, 1, 2, 24, "silu")
    assert (f.weighting, f.route_scale, f.correction, f.shared_size) == \
        ("softmax_all", 1.5, True, 0)
    assert b3.feed_forward.shared_size == 20 and b3.feed_forward.n_identity == 2
    # a rotation of the whole head is written as such; no mask, no kept keys
    assert b4.mixer.position.rotary_dim == 0 and b4.mixer.position.scaling is None
    assert (b4.mixer.window, b4.mixer.keep_first, b4.mixer.keep_all_keys) == (None, 0, False)
    # equal masks on both sides leave the owner's window alone
    k2 = KadavikConfig.from_dict(CONFIGS["K2"]).to_model_spec()
    assert not k2.blocks[1].mixer.keep_all_keys and k2.blocks[4].mixer.keep_all_keys


def test_what_the_cache_is_asked_for():
    """Keys and values and a state for an attention layer with a convolution; every key where
    first keys stay visible; a state alone for the layer that borrows; S, n and m for the
    matrix memory."""
    from agave_b200.parts.base import KVRequest, StateRequest
    from agave_b200.parts.block import Block
    import agave_b200.models       # registers the parts
    spec = KadavikConfig.from_dict(CONFIGS["K1"]).to_model_spec()
    dev = torch.device("cpu")
    blocks = [Block(b, 72, torch.float32, dev) for b in spec.blocks]
    kv, st = blocks[0].cache_request()
    assert kv == KVRequest(2, 10, None, 14) and st == StateRequest(1 * (40 + 20 + 28))
    assert blocks[1].cache_request() == StateRequest(3 * 12 * 10 + 3 * 12 + 3 * 2)
    assert blocks[2].cache_request() is None and blocks[2].state_request() == StateRequest(2 * 40)
    spec3 = KadavikConfig.from_dict(CONFIGS["K3"]).to_model_spec()
    b = [Block(x, 96, torch.float32, dev) for x in spec3.blocks]
    assert b[0].cache_request() == KVRequest(1, 16, None, 0)          # one tap: no state
    assert b[2].cache_request() == KVRequest(2, 24, None, 8)
    spec2 = KadavikConfig.from_dict(CONFIGS["K2"]).to_model_spec()
    b = [Block(x, 128, torch.float32, dev) for x in spec2.blocks]
    assert b[4].cache_request()[0].window is None                      # a reader looks further


def test_tensor_names_and_loader():
    folder = folder_for("K1")
    entry, cfg = load_config(folder)
    assert entry.name == "Kadavik"
    specs = decoder_param_specs(cfg.to_model_spec())
    names = entry.weight_names(cfg)
    want = {names.checkpoint_name(n, "") for n in specs}
    assert want == set(make_tensors(CONFIGS["K1"], 0, torch.float32))
    assert names.checkpoint_name("blocks.0.mixer.q_conv.weight", "") == "l0.mix.q.conv"
    assert names.checkpoint_name("blocks.1.mixer.i_proj.bias", "") == "l1.mix.i.b"
    assert names.checkpoint_name("blocks.1.mixer.out_norm.weight", "") == "l1.mix.norm"
    assert names.checkpoint_name("blocks.3.ffn.shared.gate.weight", "") == "l3.mlp.shared.sg"
    assert names.checkpoint_name("blocks.2.ffn.router.correction", "") == "l2.mlp.correction"
    assert names.checkpoint_name("blocks.2.ffn.experts.4.down_proj.weight", "") == \
        "l2.mlp.e4.down"
    assert names.checkpoint_name("blocks.4.side.gate_proj.weight", "") == "l4.side.gate"
    assert names.checkpoint_name("blocks.0.post_ffn_norm.weight", "") == "l0.norm2b"
    assert names.checkpoint_name("token_side.weight", "") == "side.embed"
    tensors = load_weights(folder, specs, names.checkpoint_name, names.prefixes, strict=True)
    assert tensors["blocks.0.mixer.k_conv.weight"].shape == (20, 2)
    assert tensors["blocks.2.ffn.router.weight"].shape == (6, 72)
    assert tensors["token_side.weight"].shape == (210, 25)
    assert "blocks.2.mixer.k_proj.weight" not in tensors


def test_loader_reports_what_is_wrong(tmp_path):
    from safetensors.torch import save_file
    t = make_tensors(CONFIGS["K1"], 0, torch.float32)
    del t["l3.mlp.correction"]
    t["l1.mix.i"] = t["l1.mix.i"][:2].contiguous()
    t["l1.norm2"] = torch.ones(72)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(CONFIGS["K1"], f)
    save_file(t, str(tmp_path / "model.safetensors"))
    entry, cfg = load_config(str(tmp_path))
    names = entry.weight_names(cfg)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path), decoder_param_specs(cfg.to_model_spec()),
                     names.checkpoint_name, names.prefixes)
    assert e.value.missing == ["l3.mlp.correction"]
    assert e.value.unexpected == ["l1.norm2"]
    assert [w[0] for w in e.value.wrong_shape] == ["l1.mix.i"]


def test_scaled_frequencies_of_the_rotation_part():
    """The library's list of frequencies against the plain one, and the bands by hand."""
    from agave_b200.config.base import RotarySpec
    from agave_b200.parts.rope import RotaryEmbedding
    sc = {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 16}
    rope = RotaryEmbedding(RotarySpec(theta=100.0, rotary_dim=8, scaling=BandScalingSpec(
        factor=8.0, original=16, low=1.0, high=4.0)), 12)
    f, mult = rope.frequencies()
    assert mult == 1.0 and f == pytest.approx(P.scaled_frequencies(8, 100.0, sc), rel=1e-14)
    # wavelengths 6.28 (> 16 / 4: blended), 19.9, 62.8, 198.7 (> 16: divided)
    plain = [100.0 ** (-2.0 * i / 8) for i in range(4)]
    s = (16 / (2 * math.pi) - 1.0) / 3.0
    assert f[0] == pytest.approx((1 - s) * plain[0] / 8 + s * plain[0])
    assert f[1:] == pytest.approx([x / 8 for x in plain[1:]])
    # a short wavelength is kept
    assert P.scaled_frequencies(2, 100.0, {**sc, "original": 64})[0] == 1.0


# -------------------------------------------------- mechanisms of the plain model, by hand
def test_window_and_kept_keys_by_hand():
    see = [[P.visible(i, j, 3, 2) for j in range(7)] for i in range(7)]
    assert see[2] == [True, True, True, False, False, False, False]
    assert see[4] == [True, True, True, True, True, False, False]
    assert see[5] == [True, True, False, True, True, True, False]
    assert see[6] == [True, True, False, False, True, True, True]
    assert [P.visible(6, j, 3, 0) for j in range(7)] == [False] * 4 + [True] * 3
    assert all(P.visible(6, j, None, 0) for j in range(7))


def test_convolution_by_hand():
    x = torch.tensor([[1.0], [2.0], [-3.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, -1.0, 2.0]], dtype=torch.float64)        # oldest .. current
    want = [2.0 * 1, 2.0 * 2 - 1.0 * 1, 2.0 * -3 - 1.0 * 2 + 0.5 * 1]
    assert P.causal_conv(x, w)[:, 0].tolist() == pytest.approx(want)


def test_partial_rotation_by_hand():
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=torch.float64).repeat(2, 1, 1)
    y = P.rotate(x, torch.tensor([0, 3]), {"dims": 4, "base": 100.0})
    assert y[0, 0].tolist() == pytest.approx([1, 2, 3, 4, 5])
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5
    want = [1 * math.cos(a0) - 3 * math.sin(a0), 2 * math.cos(a1) - 4 * math.sin(a1),
            3 * math.cos(a0) + 1 * math.sin(a0), 4 * math.cos(a1) + 2 * math.sin(a1), 5.0]
    assert y[1, 0].tolist() == pytest.approx(want)


def test_matrix_memory_by_hand():
    """One head, d = 2, dv = 1, two tokens, gates set through the biases alone."""
    H = 2
    eye = torch.eye(2, dtype=torch.float64)
    cap = 100.0
    i_pre, f_pre = 1.0, 2.0
    w = {"q": eye * math.sqrt(2.0), "k": eye, "v": torch.tensor([[1.0, 1.0]], dtype=torch.float64),
         "i": torch.zeros(1, 2, dtype=torch.float64), "i.b": torch.tensor([i_pre], dtype=torch.float64),
         "f": torch.zeros(1, 2, dtype=torch.float64), "f.b": torch.tensor([f_pre], dtype=torch.float64),
         "g": torch.zeros(1, 2, dtype=torch.float64), "norm": torch.ones(1, dtype=torch.float64),
         "o": torch.ones(2, 1, dtype=torch.float64)}
    h = torch.tensor([[1.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    y = P.mlstm_mixer(h, {"heads": 1, "dim": 2, "vdim": 1, "gate_cap": cap}, w, "", 0.0)
    i = cap * math.tanh(i_pre / cap)
    f = -math.log1p(math.exp(-cap * math.tanh(f_pre / cap)))
    # token 0: m = max(f + 0, i) = i; S = exp(0) k v = [1, 0]; n = [1, 0]; q = [1, 0]
    m0 = max(f, i)
    S0 = math.exp(i - m0) * 1.0
    o0 = S0 / (max(abs(S0), math.exp(-m0)) + 1e-6)
    # token 1: k = [0, 2], v = 2, q = [0, 2]
    m1 = max(f + m0, i)
    S1 = [math.exp(f + m0 - m1) * S0, math.exp(i - m1) * 2 * 2]
    n1 = [math.exp(f + m0 - m1) * S0, math.exp(i - m1) * 2]
    o1 = 2 * S1[1] / (max(abs(2 * n1[1]), math.exp(-m1)) + 1e-6)
    # one value channel: over its root mean square it is its sign; the gate is sigmoid(0)
    for t, o in ((0, o0), (1, o1)):
        assert y[t].tolist() == pytest.approx([0.5 * o / abs(o)] * 2)
    # the read-out itself, through a wider value head
    w2 = dict(w, v=torch.tensor([[1.0, 1.0], [0.0, 0.0]], dtype=torch.float64),
              g=torch.zeros(2, 2, dtype=torch.float64), norm=torch.ones(2, dtype=torch.float64),
              o=torch.tensor([[1.0, 0.0]], dtype=torch.float64))
    y2 = P.mlstm_mixer(h, {"heads": 1, "dim": 2, "vdim": 2, "gate_cap": cap}, w2, "", 0.0)
    assert y2[:, 0].tolist() == pytest.approx([0.5 * math.sqrt(2.0)] * 2)


def test_router_by_hand():
    h = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    w = {"router": torch.tensor([[1.0, 0.0], [2.0, 0.0], [0.0, 5.0], [3.0, 0.0]],
                                dtype=torch.float64),
         "correction": torch.tensor([0.0, 0.0, 1.0, -1.0], dtype=torch.float64)}
    f = {"router": {"experts": 3, "identity": 1, "top": 2, "scale": 3.0}}
    z = [1.0, 2.0, 0.0, 3.0]
    s = [math.exp(x) / sum(math.exp(y) for y in z) for x in z]
    # the correction lifts the third output above all and sinks the fourth (an identity)
    ids, wt = P.route(h, f, w, "")
    assert ids.tolist() == [[2, 1]]
    assert wt[0].tolist() == pytest.approx([3.0 * s[2] / (s[2] + s[1]), 3.0 * s[1] / (s[2] + s[1])])
    w["correction"] = torch.zeros(4, dtype=torch.float64)
    ids, wt = P.route(h, f, w, "")
    assert ids.tolist() == [[3, 1]]                     # index 3 is the identity expert
    y = P.moe(h, {**f, "shared": None}, {**w, **{f"e{e}.{n}": torch.zeros(2, 2, dtype=torch.float64)
                                                for e in range(3) for n in ("gate", "up", "down")}}, "")
    assert y[0].tolist() == pytest.approx([float(wt[0, 0]), 0.0])


def test_norm_gelu_and_token_input_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([0.0, 1.0, -0.5, 0.5], dtype=torch.float64)
    assert torch.allclose(P.rms_norm(x, w, 0.5), x / math.sqrt(12.5 + 0.5) * w)
    z = 0.7
    want = 0.5 * z * (1 + math.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    assert P.gelu_tanh(torch.tensor(z, dtype=torch.float64)).item() == pytest.approx(want)
    cfg = {"token_side": {"dim": 1}, "norm": {"eps": 0.0}}
    wt = {"side.embed": torch.tensor([[9.0, 2.0]], dtype=torch.float64),
          "l1.side.gate": torch.tensor([[1.0, 0.0]], dtype=torch.float64),
          "l1.side.proj": torch.tensor([[3.0], [4.0]], dtype=torch.float64),
          "l1.side.norm": torch.tensor([1.0, 2.0], dtype=torch.float64)}
    h = torch.tensor([[0.7, 5.0]], dtype=torch.float64)
    y = P.side_input(h, torch.tensor([0]), 1, cfg, wt)
    r = math.sqrt((9 + 16) / 2)
    assert y[0].tolist() == pytest.approx([0.7 + 3 / r, 5.0 + 2 * 4 / r])
