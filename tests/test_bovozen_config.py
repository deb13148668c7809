"""Bovozen without a GPU: the configuration reader and its errors, the lowering to part
specs and a run order, tensor names and the loader, and the plain implementation's
mechanisms on cases worked out by hand."""
import copy
import json
import math

import pytest
import torch

from agave_b200.config import ConfigError, load_config, resolve_architecture
from agave_b200.config.base import (AttentionSpec, ChannelDeltaSpec, DenseFeedForwardSpec,
                                    NormSpec, RoutedFeedForwardSpec)
from agave_b200.config.bovozen import BovozenConfig
from agave_b200.models.decoder import decoder_param_specs
from agave_b200.weights import WeightsError, load_weights
from bovozen_util import CONFIGS, RANKS, folder_for, make_tensors
from plain import bovozen_plain as P


def with_ranks(name):
    """The configuration with the bottlenecks' widths written into it (what a folder's
    tensor shapes give otherwise)."""
    raw = copy.deepcopy(CONFIGS[name])
    for i, (ra, rg) in RANKS[name].items():
        raw["layers"][i]["mixer"].update(decay_rank=ra, gate_rank=rg)
    return raw


# ------------------------------------------------------------------- reading
def test_registry_finds_the_architecture():
    assert resolve_architecture({"architecture": "Bovozen"}).name == "Bovozen"
    assert resolve_architecture({"model_type": "bovozen"}).name == "Bovozen"


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_reading_and_writing_round_trip(name):
    cfg = BovozenConfig.from_dict(with_ranks(name))
    again = BovozenConfig.from_dict(cfg.to_dict())
    assert again == cfg
    assert len(cfg.layers) == len(CONFIGS[name]["layers"])


def test_widths_of_the_bottlenecks_come_from_the_folder():
    folder = folder_for("V1")
    entry, cfg = load_config(folder)
    assert entry.name == "Bovozen"
    assert (cfg.layers[0].mixer.decay_rank, cfg.layers[0].mixer.gate_rank) == (6, 5)
    assert (cfg.layers[3].mixer.decay_rank, cfg.layers[3].mixer.gate_rank) == (4, 9)
    with pytest.raises(ConfigError, match="bottlenecks are unknown"):
        BovozenConfig.from_dict(CONFIGS["V1"])


def test_positions_from_the_table_when_the_key_is_absent():
    raw = with_ranks("V3")
    del raw["max_positions"]
    with pytest.raises(ConfigError, match="max_positions"):
        BovozenConfig.from_dict(raw)
    cfg = BovozenConfig.from_dict(raw, shapes=lambda n: (333, 96) if n == "pos" else None)
    assert cfg.max_positions == 333


@pytest.mark.parametrize("path, value, match", [
    (("vocab",), None, "vocab"),
    (("width",), 0, "positive"),
    (("norm", "eps"), None, "norm.eps"),
    (("layers", 0, "type"), "conv", "not a mixer"),
    (("layers", 0, "mixer", "conv"), None, "conv"),
    (("layers", 0, "mixer", "kv_heads"), 3, "multiple"),
    (("layers", 1, "mixer", "scale"), None, "scale"),
    (("layers", 1, "mixer", "mask", "size"), 0, "mask.size"),
    (("layers", 1, "mixer", "dim"), 2.5, "integer"),
    (("layers", 4, "mixer", "vdim"), 8, "v_mix"),
    (("layers", 0, "mlp", "kind"), "glu", "not a feed-forward"),
    (("layers", 2, "mlp", "router", "top"), 6, "top"),
    (("layers", 2, "mlp", "expert"), None, "expert"),
    (("layers", 3, "mlp", "shared", "ff"), None, "shared.ff"),
])
def test_errors_name_the_key(path, value, match):
    raw = with_ranks("V1")
    d = raw
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError, match=match):
        BovozenConfig.from_dict(raw)


# ------------------------------------------------------------------ lowering
def test_lowering_to_parts_and_run_order():
    cfg = BovozenConfig.from_dict(with_ranks("V1"))
    spec = cfg.to_model_spec()
    assert len(spec.blocks) == 6 and spec.tie_embeddings and spec.embed_scale == 1.0
    assert [(c.block, c.cache, c.writes_cache) for c in spec.schedule] == \
        [(i, i, True) for i in range(6)]
    assert all(b.arrangement == "pre" and b.norm == NormSpec(eps=1e-5, zero_centered=True)
               for b in spec.blocks)
    assert spec.final_norm == NormSpec(eps=1e-5, zero_centered=True)
    assert spec.max_positions == 700
    b0, b1, b2, b3, b4, b5 = spec.blocks
    assert b0.mixer == ChannelDeltaSpec(n_heads=4, n_qk_heads=2, head_dim=12, value_dim=10,
                                        conv_taps=2, decay_rank=6, gate_rank=5, eps=1e-5,
                                        unit_eps=1e-6)
    assert b0.feed_forward == DenseFeedForwardSpec(intermediate_size=40, activation="gelu_erf")
    m = b1.mixer
    assert isinstance(m, AttentionSpec) and b1.feed_forward is None
    assert (m.window, m.chunk, m.qk_norm_whole, m.position, m.value_mix) == \
        (None, 7, True, None, None)
    assert (m.n_heads, m.n_kv_heads, m.head_dim, m.value_dim, m.scale) == (4, 2, 10, 14, 0.45)
    assert m.qk_norm == NormSpec(eps=1e-5, zero_centered=False)
    assert (m.distance_slope.exponent, m.distance_slope.reach) == (8.0, 700)
    # the first v_mix layer is the source of the later ones
    assert b2.mixer.value_mix.source is None
    assert b4.mixer.value_mix.source == 2 and b5.mixer.value_mix.source == 2
    assert b5.mixer.chunk is None
    f = b2.feed_forward
    assert isinstance(f, RoutedFeedForwardSpec)
    assert (f.n_experts, f.top, f.intermediate_size, f.activation) == (5, 2, 24, "silu")
    assert (f.router_bias, f.weighting, f.shared_size, f.correction) == \
        (True, "softmax_top", 0, False)
    assert b3.feed_forward.shared_size == 20 and b3.feed_forward.top == 3


def test_tensor_names_and_loader():
    folder = folder_for("V1")
    entry, cfg = load_config(folder)
    specs = decoder_param_specs(cfg.to_model_spec())
    names = entry.weight_names(cfg)
    want = {names.checkpoint_name(n, "") for n in specs}
    made = set(make_tensors(CONFIGS["V1"], RANKS["V1"], 0, torch.float32))
    # (a layer that mixes no values may carry the scalar all the same; it is passed over)
    assert names.ignore_prefixes == ("l1.mix.vmix",)
    assert want == made - {"l1.mix.vmix"}
    assert names.checkpoint_name("blocks.0.mixer.q_conv.weight", "") == "l0.mix.q.conv"
    assert names.checkpoint_name("blocks.0.mixer.decay_up.weight", "") == "l0.mix.a2"
    assert names.checkpoint_name("blocks.2.mixer.value_mix", "") == "l2.mix.vmix"
    assert names.checkpoint_name("blocks.3.ffn.shared.gate.weight", "") == "l3.mlp.shared.sg"
    assert names.checkpoint_name("blocks.2.ffn.experts.4.down_proj.weight", "") == \
        "l2.mlp.e4.down"
    assert names.checkpoint_name("stream_position.table.weight", "") == "pos"
    tensors = load_weights(folder, specs, names.checkpoint_name, names.prefixes,
                           ignore_prefixes=names.ignore_prefixes)
    assert tensors.ignored == ["l1.mix.vmix"]
    assert tensors["blocks.0.mixer.k_conv.weight"].shape == (24, 2)
    assert tensors["blocks.3.ffn.router.bias"].shape == (3,)
    assert tensors["stream_position.table.weight"].shape == (700, 72)


def test_loader_reports_what_is_wrong(tmp_path):
    from safetensors.torch import save_file
    t = make_tensors(CONFIGS["V1"], RANKS["V1"], 0, torch.float32)
    del t["l3.mlp.router.b"]
    del t["l1.mix.vmix"]                 # unused there: its absence is no fault
    t["l0.mix.a2"] = t["l0.mix.a2"][:5].contiguous()
    t["l1.norm2"] = torch.ones(72)
    with open(tmp_path / "config.json", "w") as f:
        json.dump(CONFIGS["V1"], f)
    save_file(t, str(tmp_path / "model.safetensors"))
    entry, cfg = load_config(str(tmp_path))
    names = entry.weight_names(cfg)
    with pytest.raises(WeightsError) as e:
        load_weights(str(tmp_path), decoder_param_specs(cfg.to_model_spec()),
                     names.checkpoint_name, names.prefixes,
                     ignore_prefixes=names.ignore_prefixes)
    assert e.value.missing == ["l3.mlp.router.b"]
    assert e.value.unexpected == ["l1.norm2"]
    assert [w[0] for w in e.value.wrong_shape] == ["l0.mix.a2"]


# -------------------------------------------------- mechanisms of the plain model, by hand
def test_slopes_and_blocks_by_hand():
    assert P.head_slopes(4).tolist() == pytest.approx([0.25, 1 / 16, 1 / 64, 1 / 256])
    assert P.head_slopes(1).tolist() == pytest.approx([2.0 ** -8])
    see = P.visible(7, 3)
    assert see[2].tolist() == [True, True, True, False, False, False, False]
    assert see[3].tolist() == [False, False, False, True, False, False, False]
    assert see[6].tolist() == [False] * 6 + [True]
    assert P.visible(3, None).tolist() == [[True, False, False], [True, True, False],
                                           [True, True, True]]


def test_biased_attention_by_hand():
    # one head (slope 2^-8), keys c_j e_1, values the position
    q = torch.zeros(4, 1, 2, dtype=torch.float64); q[:, 0, 0] = 1.0
    k = torch.zeros(4, 1, 2, dtype=torch.float64); k[:, 0, 0] = torch.tensor([0.0, 1.0, 2.0, 3.0])
    v = torch.arange(4, dtype=torch.float64).view(4, 1, 1)
    s = 2.0 ** -8
    o = P.biased_softmax_attention(q, k, v, 0.5, None)
    w = [math.exp(0.5 * j - s * (3 - j)) for j in range(4)]
    assert o[3, 0, 0].item() == pytest.approx(sum(j * w[j] for j in range(4)) / sum(w))
    o = P.biased_softmax_attention(q, k, v, 0.5, 2)        # blocks {0, 1}, {2, 3}
    assert o[2, 0, 0].item() == pytest.approx(2.0)
    assert o[3, 0, 0].item() == pytest.approx((2 * w[2] + 3 * w[3]) / (w[2] + w[3]))
    assert o[1, 0, 0].item() == pytest.approx(math.exp(0.5) / (math.exp(-s) + math.exp(0.5)))


def test_convolution_and_unit_vectors_by_hand():
    x = torch.tensor([[1.0], [2.0], [-3.0]], dtype=torch.float64)
    w = torch.tensor([[0.5, -1.0, 2.0]], dtype=torch.float64)        # oldest .. current
    y = [2.0 * 1, 2.0 * 2 - 1.0 * 1, 2.0 * -3 - 1.0 * 2 + 0.5 * 1]
    want = [a / (1 + math.exp(-a)) for a in y]
    assert P.causal_conv_silu(x, w)[:, 0].tolist() == pytest.approx(want)
    u = P.unit(torch.tensor([3.0, 4.0], dtype=torch.float64), eps=11.0)
    assert u.tolist() == pytest.approx([0.5, 4 / 6])


def test_delta_rule_by_hand():
    # one head, d = 2, dv = 1, two tokens
    k = torch.tensor([[[1.0, 0.0]], [[0.6, 0.8]]], dtype=torch.float64)
    q = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]]], dtype=torch.float64)
    v = torch.tensor([[[2.0]], [[1.0]]], dtype=torch.float64)
    beta = torch.tensor([[0.5], [1.0]], dtype=torch.float64)
    decay = torch.tensor([[[0.9, 0.8]], [[0.5, 0.25]]], dtype=torch.float64)
    o, S = P.delta_recurrence(q, k, v, beta, decay)
    # token 0: S = 0; u = 0.5 * 2 = 1; S = [1, 0]; o = 1
    # token 1: S = [0.5, 0]; S^T k = 0.3; u = 0.7; S = [0.5 + 0.42, 0.56]; o = 0.56
    assert o[:, 0, 0].tolist() == pytest.approx([1.0, 0.56])
    assert S[0, :, 0].tolist() == pytest.approx([0.92, 0.56])
    # carried on from a state equals the run in one
    o2, S2 = P.delta_recurrence(q[1:], k[1:], v[1:], beta[1:], decay[1:],
                                S0=torch.tensor([[[1.0], [0.0]]], dtype=torch.float64))
    assert o2[0, 0, 0].item() == pytest.approx(0.56) and torch.allclose(S2, S)


def test_decay_by_hand():
    low = torch.tensor([[2.0]], dtype=torch.float64)
    g = P.channel_decay(low, torch.tensor([[0.5], [-1.0]], dtype=torch.float64),
                        torch.tensor([0.0, 1.0], dtype=torch.float64),
                        torch.tensor([math.log(2.0)], dtype=torch.float64), 1, 2)
    want = [math.exp(-2.0 * math.log1p(math.exp(1.0))), math.exp(-2.0 * math.log1p(math.exp(-1.0)))]
    assert g.view(-1).tolist() == pytest.approx(want)


def test_router_by_hand():
    h = torch.tensor([[1.0, 0.0]], dtype=torch.float64)
    Wr = torch.tensor([[1.0, 0.0], [2.0, 0.0], [0.0, 5.0], [3.0, 0.0]], dtype=torch.float64)
    b = torch.tensor([0.0, 0.0, 2.5, -2.0], dtype=torch.float64)      # logits 1, 2, 2.5, 1
    ids, w = P.route(h, Wr, b, 2)
    assert ids.tolist() == [[2, 1]]
    assert w[0].tolist() == pytest.approx([1 / (1 + math.exp(-0.5)), 1 / (1 + math.exp(0.5))])
    ids, w = P.route(h, Wr, b, 1)
    assert ids.tolist() == [[2]] and w.tolist() == [[1.0]]


def test_norms_and_gelu_by_hand():
    x = torch.tensor([[1.0, 2.0, 3.0, 6.0]], dtype=torch.float64)
    w = torch.tensor([0.0, 1.0, -0.5, 0.5], dtype=torch.float64)
    assert torch.allclose(P.norm_around_zero(x, w, 0.5), x / math.sqrt(12.5 + 0.5) * (1 + w))
    assert P.gelu_erf(torch.tensor(1.0, dtype=torch.float64)).item() == \
        pytest.approx(0.5 * (1 + math.erf(1 / math.sqrt(2))))
