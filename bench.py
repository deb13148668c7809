#!/usr/bin/env python3
"""Measures decoding and prefill of Gemma 3 layer sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl ours|reference]
                    [--shapes 1b|4b|27b] [--prompt-lens LO HI] [--prefill-tokens N]

Prints ONE JSON line.  ``value`` is decoded tokens per second of K decode
steps (random bfloat16 weights, context 8,192), timed on the device with CUDA
events; ``e2e`` is the same through ``Engine.generate`` with host token ids in
and out every step.  ``prefill`` is one 2,048-token prompt: ``ms`` for a
length whose step has been recorded, ``first_seen_ms`` for lengths never run
before (no recording: the host launches the step, through the library's C++
step function), ``first_seen_128_tokens_ms`` the same for prompts of about 128
tokens.
``roofline`` relates the decode step to the bytes it has to read; ``points``
holds decoding at the other batch sizes of the schedule.

Schedules (``--shapes``; the default, 1b, is the benchmark configuration):
  1b   batch 8 (and 1, 64), prompts of unequal lengths 128..2,048, K steps
  4b   batch 8, prompts of unequal lengths 256..4,096, 256 decoded tokens
  27b  batch 16 (and 1), prompts of 2,048 tokens, 128 decoded tokens (54 GB of weights)
A step's inputs (the weights, gigabytes) are larger than the 126 MB L2, so
every timed iteration reads them from HBM; ``config.l2`` says how many bytes.
``--layers``, ``--prompt-lens`` and ``--prefill-tokens`` measure fewer layers,
other contexts and other prompts; what they were is in ``config`` and
``prefill``.

``--compare ramilorn`` is another measurement altogether (the default workload and its
JSON line are untouched by it): the Ramilorn decoder at a few layer sizes beside a
Gemma 3 decoder of equal size (same width, heads, head size, layers and vocabulary, a
dense feed-forward as wide as the experts a token uses), random weights, one JSON line
with, per size and model, prefill and decode throughput (recorded steps, CUDA events)
and every operation's device time with its share of the measured peaks
(``agave_b200.perf``, steps run launch by launch).  ``--compare zazerax`` does the same for the
Zazerax decoder (layers alternating latent attention of both kinds with windowed attention,
dense squared-relu feed-forward) beside a Gemma 3 decoder of equal width, heads, layers and
vocabulary whose every second layer has the same window and whose gated feed-forward has as
many weights.  ``--compare bovozen`` sets the Bovozen decoder (attention over blocks of positions
alternating with the gated delta rule, routed experts beside a gated shared one) beside the
Ramilorn decoder of equal width, heads, experts, layers and vocabulary.  ``--compare kadavik``
sets the Kadavik decoder (attention with a convolution on q, k and v, a window behind which the
first keys stay visible and an output gate, alternating with the matrix memory; routed experts
with identity experts beside a gated shared one; a per-layer token input) beside the Bovozen
decoder of equal width, heads, head size, experts, layers and vocabulary.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Gemma 3 1B layer sizes (random weights, seed 2, N(0, 0.02) bfloat16)
CONFIG_1B = {
    "architectures": ["Gemma3ForCausalLM"], "model_type": "gemma3_text",
    "num_hidden_layers": 26, "hidden_size": 1152, "num_attention_heads": 4,
    "num_key_value_heads": 1, "head_dim": 256, "query_pre_attn_scalar": 256,
    "intermediate_size": 6912, "vocab_size": 262144, "sliding_window": 512,
    "sliding_window_pattern": 6, "rope_local_base_freq": 10000.0, "rope_theta": 1000000.0,
    "rope_scaling": None, "rms_norm_eps": 1e-6, "tie_word_embeddings": True,
    "max_position_embeddings": 32768, "hidden_activation": "gelu_pytorch_tanh",
    "bos_token_id": 2, "eos_token_id": 1,
}
# layer sizes of the larger family members (--shapes 4b / 27b); the default run is 1b
CONFIG_4B = dict(CONFIG_1B, num_hidden_layers=34, hidden_size=2560, num_attention_heads=8,
                 num_key_value_heads=4, head_dim=256, query_pre_attn_scalar=256,
                 intermediate_size=10240, vocab_size=262208, sliding_window=1024,
                 rope_scaling={"rope_type": "linear", "factor": 8.0}, max_position_embeddings=131072)
CONFIG_27B = dict(CONFIG_4B, num_hidden_layers=62, hidden_size=5376, num_attention_heads=32,
                  num_key_value_heads=16, head_dim=128, query_pre_attn_scalar=168,
                  intermediate_size=21504)
SHAPES = {"1b": (CONFIG_1B, 2), "4b": (CONFIG_4B, 3), "27b": (CONFIG_27B, 4)}
# per shape: headline batch, the other batch sizes, prompt lengths, decode steps (None: --steps)
SCHEDULES = {"1b": dict(batch=8, others=(1, 64), lens=(128, 2048), steps=None),
             "4b": dict(batch=8, others=(), lens=(256, 4096), steps=256),
             "27b": dict(batch=16, others=(1,), lens=(2048, 2048), steps=128)}
CONTEXT = 8192
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        try:
            with open(path) as f:
                p = json.load(f)
            return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                    "source": "measured"}
        except Exception:
            pass
    return {**FALLBACK_PEAKS, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.samples, self.proc = [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", "0", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "20"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        mhz = sorted(int(s[0]) for s in self.samples if s and s[0].isdigit())
        mx = [int(s[1]) for s in self.samples if len(s) > 1 and s[1].isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({names[i] for s in self.samples if len(s) >= 6
                          for i in range(4) if s[2 + i].lower().startswith("active")})
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(mhz)}


def layer_kinds(cfg):
    P = cfg["sliding_window_pattern"]
    return [(P > 0 and (l + 1) % P != 0) for l in range(cfg["num_hidden_layers"])]


def decode_bytes(cfg, lens):
    """Bytes one decode step must read: every weight once, and the live cache."""
    H, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    L = cfg["num_hidden_layers"]
    per_layer = (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * ff) * 2 + (4 * H + 2 * hd) * 4
    weights = L * per_layer + V * H * 2 + H * 4
    kv = 0
    W = cfg["sliding_window"]
    for local in layer_kinds(cfg):
        for n in lens:
            kv += (min(n, W) if local else n) * nkv * hd * 2 * 2
    return weights + kv


def prefill_flops(cfg, T, rows):
    H, ff, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    W = cfg["sliding_window"]
    lin = 2 * T * (H * (nh + 2 * nkv) * hd + nh * hd * H + 3 * H * ff)
    total = 0
    for local in layer_kinds(cfg):
        vis = sum(min(t + 1, W) if local else t + 1 for t in range(T))
        total += lin + 4 * nh * hd * vis
    return total + 2 * rows * H * V


def run_reference(args):
    print(json.dumps({
        "impl": "reference",
        "unavailable": "maci0/agave is a Zig program (build.zig); pip reports 'Neither setup.py "
                       "nor pyproject.toml found' and no zig toolchain is installed, so it "
                       "cannot be built or run here"}))
    return 0


def timed_decode(engine, torch, batch, steps, warmup, seed, lo=128, hi=2048):
    """K decode steps at one batch size, device-timed; returns (ms/step, lens, launches/step).

    The steps are the engine's own: each is staged by ``Engine._stage_step`` (the routine
    the generation loop stages its steps with), kept in a device array, and replayed
    through the engine's recorded decode step; only the token ids are this function's."""
    from agave_b200.engine.generate import RequestState
    from agave_b200.sampling import SamplingParams
    g = torch.Generator().manual_seed(seed)
    V = engine.spec.vocab_size
    lens = torch.linspace(lo, hi, batch).round().int().tolist() if batch > 1 else [(lo + hi) // 2]
    prompts = [torch.randint(3, V, (n,), generator=g).tolist() for n in lens]
    reqs = [RequestState(i, p, 1 << 30, output=[3]) for i, p in enumerate(prompts)]
    for r in reqs:
        r.slot = engine.acquire()
    # prompts in chunks of sequences, to bound the prompt step's activations
    for i in range(0, batch, 8):
        part = reqs[i:i + 8]
        engine.step([(r.slot, r.prompt) for r in part], [[] for _ in part])
    params = SamplingParams()
    total = warmup + steps
    toks = torch.randint(3, V, (total, batch), generator=g, dtype=torch.int32)
    staged = None
    for k in range(total):
        graph = engine._stage_step(reqs, params, 0, k, 0)       # the step k steps ahead
        a = graph.hosts_np[0]
        a[:batch] = toks[k].numpy()
        a[graph.flag_at] = 0                                    # token ids come from the host
        if staged is None:
            staged = torch.zeros((total, a.size), dtype=torch.int32)
        staged[k] = graph.hosts[0]
    engine.runner.cache.flush()
    staged_dev = staged.to(engine.device)
    torch.cuda.synchronize()
    per_step = graph.kernels_per_step
    for k in range(warmup):
        graph.dev.copy_(staged_dev[k])
        graph.graph.replay()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for k in range(warmup, total):
        graph.dev.copy_(staged_dev[k])
        graph.graph.replay()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    # the last step's choices are real tokens of the vocabulary (the step ran, on these ids)
    chosen = graph.next_dev[:batch].cpu()
    assert int(chosen.min()) >= 0 and int(chosen.max()) < V, "the decode step chose no tokens"
    book = engine.runner.cache.book
    final_lens = [book.length[r.slot] + total for r in reqs]
    for r in reqs:
        engine.release(r.slot)
    return ms, final_lens, per_step


# Ramilorn layer sizes for --compare: (width, heads, kv heads, head size, experts, experts per
# token, expert width, groups, groups kept, layers, vocabulary).  Every second layer
# attends to the keys and values of the layer before it.
COMPARE_SIZES = {
    "small": (1024, 16, 4, 64, 16, 2, 512, 4, 2, 8, 32768),
    "medium": (2048, 16, 4, 128, 32, 4, 768, 8, 4, 8, 65536),
    "large": (4096, 32, 8, 128, 64, 6, 1408, 8, 4, 4, 65536),
}


def compare_configs(size):
    H, A, G, d, E, top, ff, groups, keep, L, V = COMPARE_SIZES[size]
    mixer = {"dim": d, "heads": A, "kv_heads": G, "q_temp": {"coef": 0.1, "every": 1024},
             "scale": d ** -0.5, "vdim": d}
    mlp = {"expert": {"ff": ff}, "kind": "moe",
           "router": {"experts": E, "groups": {"count": groups, "keep": keep}, "top": top}}
    layers = []
    for l in range(L):
        m = dict(mixer)
        if l % 2 == 1:
            m["kv_from"] = l - 1
        layers.append({"mixer": m, "mlp": mlp, "type": "attention"})
    ramilorn = {"architecture": "Ramilorn", "layers": layers, "logit_softcap": 30.0,
                "norm": {"eps": 1e-5}, "residual_mult": 0.5, "vocab": V, "width": H}
    gemma = dict(CONFIG_1B, num_hidden_layers=L, hidden_size=H, num_attention_heads=A,
                 num_key_value_heads=G, head_dim=d, query_pre_attn_scalar=d,
                 intermediate_size=top * ff, vocab_size=V, sliding_window=None,
                 sliding_window_pattern=0, hidden_activation="silu")
    return ramilorn, gemma


# Zazerax layer sizes for --compare: width, heads; latent attention: unrotated and rotated
# head part, value head, kv latent, query latent (second kind); windowed attention: kv heads,
# head size, window; feed-forward width; layers; vocabulary.
ZAZERAX_SIZES = {
    "small": dict(H=1024, A=16, d=32, r=32, dv=64, R=96, Rq=256, G=4, hd=64, window=512, ff=3072,
                  L=8, V=32768),
    "medium": dict(H=2048, A=16, d=64, r=64, dv=128, R=192, Rq=512, G=4, hd=128, window=1024,
                   ff=6144, L=8, V=65536),
    "large": dict(H=4096, A=32, d=128, r=64, dv=128, R=192, Rq=768, G=8, hd=128, window=1024,
                  ff=12288, L=4, V=65536),
}


def compare_configs_zazerax(size):
    z = ZAZERAX_SIZES[size]
    rot = {"base": 10000.0, "dims": z["r"]}
    lat = {"dim": z["d"], "heads": z["A"], "kv_rank": z["R"], "rot_dim": z["r"],
           "scale": (z["d"] + z["r"]) ** -0.5, "vdim": z["dv"]}
    first = dict(lat, rot=dict(rot, scaling={"factor": 4.0, "original": 4096, "fast": 32.0,
                                             "slow": 1.0}))
    second = dict(lat, rot=rot, q_rank=z["Rq"])
    win = {"bias_max": 4 * z["window"], "bias_rows": 32, "dim": z["hd"], "heads": z["A"],
           "kv_heads": z["G"], "mask": {"size": z["window"]}, "scale": z["hd"] ** -0.5,
           "vdim": z["hd"]}
    mlp = {"ff": z["ff"], "kind": "dense"}
    kinds = [("latent_attention", first), ("attention", win), ("latent_attention_2", second),
             ("attention", win)]
    layers = [{"mixer": kinds[l % 4][1], "mlp": mlp, "type": kinds[l % 4][0]}
              for l in range(z["L"])]
    zazerax = {"architecture": "Zazerax", "embedding": {"scale": 1.0}, "layers": layers,
               "norm": {"eps": 1e-5}, "vocab": z["V"], "width": z["H"]}
    # (a gated feed-forward has three matrices where the dense one has two)
    gemma = dict(CONFIG_1B, num_hidden_layers=z["L"], hidden_size=z["H"],
                 num_attention_heads=z["A"], num_key_value_heads=z["G"], head_dim=z["hd"],
                 query_pre_attn_scalar=z["hd"], intermediate_size=z["ff"] * 2 // 3 // 128 * 128,
                 vocab_size=z["V"], sliding_window=z["window"], sliding_window_pattern=2,
                 hidden_activation="silu")
    return zazerax, gemma


def compare_configs_bovozen(size):
    """Bovozen beside Ramilorn, the library's other decoder with routed experts: equal width,
    heads, head size, experts, layers and vocabulary.  Bovozen's layers alternate attention
    over blocks of 1,024 positions (values leaning towards the first layer's) with the gated
    delta rule (as many heads, state head size x head size per head, four taps); its experts
    have a shared one of twice their width beside them."""
    H, A, G, d, E, top, ff, groups, keep, L, V = COMPARE_SIZES[size]
    att = {"dim": d, "heads": A, "kv_heads": G, "mask": {"size": 1024}, "scale": d ** -0.5,
           "v_mix": True, "vdim": d}
    rec = {"conv": 4, "dim": d, "heads": A, "kv_heads": G, "vdim": d, "decay_rank": 64,
           "gate_rank": 64}
    mlp = {"expert": {"ff": ff}, "kind": "moe", "router": {"experts": E, "top": top},
           "shared": {"ff": 2 * ff}}
    layers = [{"mixer": rec if l % 2 else att, "mlp": mlp,
               "type": "channel_delta" if l % 2 else "attention"} for l in range(L)]
    bovozen = {"architecture": "Bovozen", "layers": layers, "max_positions": 4096,
               "norm": {"eps": 1e-6}, "vocab": V, "width": H}
    return bovozen, compare_configs(size)[0]


def compare_configs_kadavik(size):
    """Kadavik beside Bovozen, the library's other decoder with a recurrent mixer, routed
    experts and a shared one: equal width, heads, head size, experts, layers and vocabulary.
    Kadavik's layers alternate attention (four taps on q, k and v, half the head rotated, a
    window of 1,024 behind which eight keys stay, an output gate) with the matrix memory (as
    many heads, state head size x head size per head); its routers have two identity outputs
    beyond the experts; every layer takes a token input 64 wide."""
    H, A, G, d, E, top, ff, groups, keep, L, V = COMPARE_SIZES[size]
    att = {"conv": 4, "dim": d, "heads": A, "kv_heads": G,
           "mask": {"keep_first": 8, "size": 1024},
           "rot": {"base": 1000000.0, "dims": d // 2,
                   "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}},
           "scale": d ** -0.5, "vdim": d}
    rec = {"dim": d, "gate_cap": 15.0, "heads": A, "vdim": d}
    mlp = {"expert": {"ff": ff}, "kind": "moe",
           "router": {"experts": E, "identity": 2, "scale": 1.5, "top": top},
           "shared": {"ff": 2 * ff}}
    layers = [{"mixer": rec if l % 2 else att, "mlp": mlp,
               "type": "mlstm" if l % 2 else "attention"} for l in range(L)]
    kadavik = {"architecture": "Kadavik", "embedding": {"scale": H ** 0.5}, "layers": layers,
               "logit_scale": 1.0, "norm": {"eps": 1e-6}, "token_side": {"dim": 64}, "vocab": V,
               "width": H}
    return kadavik, compare_configs_bovozen(size)[0]


COMPARE_BUILDERS = {"ramilorn": (compare_configs, "gemma3"),
                    "kadavik": (compare_configs_kadavik, "bovozen"),
                    "zazerax": (compare_configs_zazerax, "gemma3"),
                    "bovozen": (compare_configs_bovozen, "ramilorn")}


def run_compare(args):
    import torch
    from agave_b200 import kernels
    from agave_b200.config import resolve_architecture
    from agave_b200.engine.api import Engine
    from agave_b200.models.decoder import decoder_param_specs
    from agave_b200.perf import PerfCounters
    from agave_b200.weights import random_tensors
    pk = peaks()
    batch, ctx_len, n_pre = 8, 1024, args.prefill_tokens
    builder, beside = COMPARE_BUILDERS[args.compare]
    out = {"compare": f"{args.compare} beside {beside} at equal size", "dtype": "bf16",
           "data": "synthetic", "decode_batch": batch, "decode_context": ctx_len,
           "prefill_tokens": n_pre, "peaks": pk, "sizes": {}}
    for size in (args.compare_sizes or sorted(COMPARE_SIZES)):
        entry = {}
        for name, cfg in zip((args.compare, beside), builder(size)):
            arch = resolve_architecture(cfg)
            specs = decoder_param_specs(arch.config_class.from_dict(cfg).to_model_spec())
            tensors = random_tensors(specs, 11, 0.02, 0.1, torch.bfloat16, "cuda:0")
            for k, t in tensors.items():
                if k.endswith("router.weight"):
                    t.mul_(60.0)      # router logits of order one: tokens spread over the experts
            engine = Engine(None, _raw_config=cfg, _tensors=tensors, dtype="bfloat16",
                            max_tokens=batch * 4096, ctx_size=4096, max_batch=batch)
            del tensors
            V = engine.spec.vocab_size
            g = torch.Generator().manual_seed(3)
            prompt = torch.randint(3, V, (n_pre,), generator=g).tolist()

            def timed_prompt(tokens):
                s = engine.acquire()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                torch.cuda.synchronize()
                e0.record()
                engine.step([(s, tokens)], [[len(tokens) - 1]])
                e1.record()
                torch.cuda.synchronize()
                engine.release(s)
                return e0.elapsed_time(e1)
            pre = sorted(timed_prompt(prompt) for _ in range(3 + 5))[:5]
            pre_ms = pre[len(pre) // 2]
            ms, _, launches = timed_decode(engine, torch, batch, args.steps, max(3, args.warmup), 8,
                                           ctx_len, ctx_len)
            # every operation's device time, launch by launch
            ops = {}
            for what in ("prefill", "decode"):
                counters = PerfCounters()
                if what == "prefill":
                    for rep in range(3):
                        slot = engine.acquire()
                        if rep == 2:
                            counters.__enter__()
                        engine.step([(slot, prompt)], [[n_pre - 1]])
                        engine.release(slot)
                else:
                    slots = [engine.acquire() for _ in range(batch)]
                    engine.step([(s, prompt[:ctx_len - 7 * i]) for i, s in enumerate(slots)],
                                [[] for _ in slots])
                    chosen = []                    # the experts each routed layer picks (device)
                    routed = [b.ffn for b in engine.model.blocks
                              if getattr(b, "ffn", None) is not None and hasattr(b.ffn, "route")]
                    for ffn in routed:
                        def route(x, _r=ffn.route):
                            ids, wts = _r(x)
                            chosen.append(ids)
                            return ids, wts
                        ffn.route = route
                    for rep in range(3):
                        if rep == 2:
                            del chosen[:]
                            counters.__enter__()
                        engine.step([(s, [5 + rep + i]) for i, s in enumerate(slots)],
                                    [[0] for _ in slots])
                    for ffn in routed:
                        del ffn.route                # back to the class's method
                    for s in slots:
                        engine.release(s)
                table = counters.table()
                counters.__exit__()
                if what == "decode" and chosen:
                    # a decode step reads only the experts some token chose: the spans' byte
                    # counts assume min(experts, pairs) of them, the truth is counted here
                    used = sum(int(c.unique().numel()) for c in chosen) / len(chosen)
                    E = routed[0].spec.n_experts
                    assumed = min(E, batch * routed[0].spec.top)
                    for op in ("experts_gate_up", "experts_down"):
                        if op in table:
                            table[op]["bytes"] = int(table[op]["bytes"] * used / assumed)
                    entry_extra = {"experts_read_per_layer": round(used, 1), "experts": E}
                else:
                    entry_extra = {}
                if what == "decode":
                    decode_extra = entry_extra
                rows = {}
                for op, r in table.items():
                    sec = r["total_us"] * 1e-6
                    gbs = r["bytes"] / sec / 1e9 if sec > 0 else 0.0
                    tf = r["flops"] / sec / 1e12 if sec > 0 else 0.0
                    rows[op] = {"calls": r["calls"], "us": round(r["total_us"] / r["calls"], 2),
                                "gbs": round(gbs, 1), "tflops": round(tf, 2),
                                "of_peak": round(max(gbs / pk["hbm_gbs"], tf / pk["bf16_tflops"]), 4)}
                ops[what] = rows
            entry[name] = {"prefill_ms": round(pre_ms, 3),
                           "prefill_tokens_per_s": round(n_pre / pre_ms * 1e3, 1),
                           "decode_ms_per_step": round(ms, 4),
                           "decode_tokens_per_s": round(batch / ms * 1e3, 1),
                           "kernels_per_decode_step": launches,
                           "weight_gb": round(engine.model.weight_bytes() / 1e9, 3), "ops": ops,
                           **decode_extra}
            del engine
            torch.cuda.empty_cache()
        out["sizes"][size] = entry
    print(json.dumps(out))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0,
                    help="run fewer layers than the configuration has (0 = all)")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shapes", default="1b", choices=sorted(SHAPES),
                    help="layer sizes to run (the default, 1b, is the benchmark configuration)")
    ap.add_argument("--prompt-lens", type=int, nargs=2, default=None, metavar=("LO", "HI"),
                    help="the decode batches' prompt lengths run from LO to HI (default: the "
                         "schedule's, 128 to 2,048 for the benchmark configuration)")
    ap.add_argument("--prefill-tokens", type=int, default=PREFILL_TOKENS,
                    help="length of the timed prompt (default: the benchmark configuration's)")
    ap.add_argument("--compare", default=None, choices=sorted(COMPARE_BUILDERS),
                    help="instead of the benchmark: this architecture beside the closest other "
                         "one at equal layer sizes (see the module text)")
    ap.add_argument("--compare-sizes", nargs="+", default=None, choices=sorted(COMPARE_SIZES),
                    help="the sizes --compare runs (default: all)")
    args = ap.parse_args()
    if args.compare and args.impl == "ours":
        if args.gpus != 1:
            print("bench.py: this library runs on one GPU; --gpus must be 1")
            return 2
        return run_compare(args)
    sched = SCHEDULES[args.shapes]
    lo, hi = args.prompt_lens or sched["lens"]
    steps = args.steps if sched["steps"] is None else sched["steps"]
    n_pre = args.prefill_tokens
    if not (0 < lo <= hi and hi + steps + max(3, args.warmup) + 1 <= CONTEXT
            and 8 <= n_pre <= CONTEXT):
        print(f"bench.py: prompts and the decoded tokens must fit the context of {CONTEXT}")
        return 2
    if args.impl == "reference":
        return run_reference(args)
    if args.gpus != 1:
        print("bench.py: this library runs on one GPU; --gpus must be 1")
        return 2
    args.warmup = max(3, args.warmup)

    import torch
    from agave_b200.engine.api import Engine

    base_cfg, seed = SHAPES[args.shapes]
    cfg = dict(base_cfg)
    full_layers = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    batch = sched["batch"]
    max_batch = max((batch,) + tuple(sched["others"]))
    engine = Engine.from_config(cfg, seed=seed, std=0.02, norm_std=0.1, dtype="bfloat16",
                                max_tokens=max_batch * CONTEXT, ctx_size=CONTEXT,
                                max_batch=max_batch)
    V = engine.spec.vocab_size
    g = torch.Generator().manual_seed(5)

    def timed_prompt(tokens):
        s = engine.acquire()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        engine.step([(s, tokens)], [[len(tokens) - 1]])
        e1.record()
        torch.cuda.synchronize()
        engine.release(s)
        return e0.elapsed_time(e1)

    # ---- prefill: one prompt (2,048 tokens by default), logits of its last token ----
    prompt = torch.randint(3, V, (n_pre,), generator=g).tolist()
    # lengths never run before: no recorded step, the host launches kernel by kernel
    # (the first of them also pays what a kernel's first use costs, so it is not counted)
    first_seen = sorted(timed_prompt(prompt[:n_pre - k]) for k in (7, 5, 3, 1))[:3]
    first_seen_ms = sorted(first_seen)[1]
    # the same for short prompts (time to the first token of a chat turn): what the host
    # needs to launch a step bounds these
    short = sorted(timed_prompt(prompt[:128 - k]) for k in (7, 5, 3, 1))[:3]
    short_ms = sorted(short)[1]
    pre_ms = [timed_prompt(prompt) for _ in range(3 + 5)][3:]
    pre_ms = sorted(pre_ms)[len(pre_ms) // 2]
    pflops = prefill_flops(cfg, n_pre, 1)
    prefill = {"value": round(n_pre / pre_ms * 1e3, 1), "tokens": n_pre,
               "ms": round(pre_ms, 3),
               "frac": round(pflops / (pre_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
               "first_seen_ms": round(first_seen_ms, 3),
               "first_seen_128_tokens_ms": round(short_ms, 3)}

    # ---- decode at the headline batch, with clocks sampled meanwhile ----
    clocks = ClockSampler()
    clocks.start()
    ms_b, lens_b, launches = timed_decode(engine, torch, batch, steps, args.warmup, 8, lo, hi)
    clock_rec = clocks.stop()
    value = batch / ms_b * 1e3
    nbytes = decode_bytes(cfg, lens_b)
    achieved = nbytes / (ms_b * 1e-3) / 1e9
    roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"],
                "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4),
                "of": pk["source"], "bytes_per_step": nbytes}

    # ---- the other batch sizes ----
    points = {}
    for b in sched["others"]:
        k = steps if b <= 16 else max(8, steps // 2)
        ms, _, _ = timed_decode(engine, torch, b, k, args.warmup, b, lo, hi)
        points[f"decode_b{b}"] = round(b / ms * 1e3, 1)

    # ---- end to end through the Python entry point ----
    lens = torch.linspace(lo, hi, batch).round().int().tolist()
    prompts = [torch.randint(3, V, (n,), generator=g).tolist() for n in lens]
    n_new = steps + 1
    engine.generate(prompts, max_new_tokens=4, stop_token_ids=[])           # warm-up
    engine.generate(prompts, max_new_tokens=n_new, stop_token_ids=[])
    st = engine.stats
    e2e_val = st["decode_tokens"] / st["decode_seconds"]
    graph = next(iter(engine._graphs.values()))
    e2e = {"value": round(e2e_val, 1), "unit": "tokens/s",
           "h2d_bytes_per_step": int(graph.hosts[0].numel() * 4),
           "d2h_bytes_per_step": int(graph.next_hosts[0].numel() * 4)}

    weight_gb = (decode_bytes(cfg, [0]) / 1e9)
    out = {
        "metric": f"Gemma3-{args.shapes.upper()} bf16 decode tokens/s at batch {batch} "
                  f"(context {CONTEXT})",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(ms_b, 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {
            "model": f"gemma3-{args.shapes}-shapes-random", "layers": cfg["num_hidden_layers"],
            "layers_full": full_layers, "hidden": cfg["hidden_size"],
            "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
            "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"],
            "vocab": cfg["vocab_size"], "sliding_window": cfg["sliding_window"],
            "local_per_global": cfg["sliding_window_pattern"] - 1, "global_batch": batch,
            "seq_len": CONTEXT, "prompt_lens": f"{lo}..{hi}" + (" unequal" if lo != hi else ""),
            "seed": seed, "parallelism": "single-gpu", "cache": "paged bf16",
            "l2": f"inputs larger than L2 ({weight_gb:.1f} GB weights per step)"},
        "prefill": prefill, "roofline": roofline, "points": points, "e2e": e2e,
        "gpu_launches": int(launches * steps), "clocks": clock_rec,
    }
    print(json.dumps(out))
    return 0


if __name__ == "__main__":
    sys.exit(main())
