"""Typed descriptions of a decoder, one small record per part.

A model configuration (read from an architecture's own ``config.json`` keys)
is lowered into these records; the generic decoder in ``agave_b200.models``
builds parts from them through the part registries and never looks at the
architecture's name.  Every size and constant of a part is a field here, so
that two layers of one model may carry different mixers, feed-forwards,
windows or rotary bases.

The reference keeps the same facts as flat fields of one model struct
(src/models/gemma3.zig:59-85) and decides "local or global" per layer inside
the forward pass (src/models/gemma3.zig:736); here that decision is data.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Tuple


class ConfigError(ValueError):
    """A configuration that cannot be built; the message names the key."""


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding on split halves (i, i + rotary_dim/2).

    angle(p, i) = (p / factor) * theta ** (-2 i / rotary_dim)
    (src/backend/kernels/cpu/rope.zig:11-47, src/models/gemma3.zig:884-902).
    """
    kind: str = "rotary"
    theta: float = 10000.0
    factor: float = 1.0
    rotary_dim: int = 0          # 0 means the whole head
    # pairs (2i, 2i + 1) instead of (i, i + rotary_dim/2); a mixer that rotates honours it
    interleaved: bool = False
    # frequencies blended between wavelength bounds, and a multiplier on cos and sin
    # (``WavelengthScalingSpec``), or divided band by band (``BandScalingSpec``)
    scaling: Optional[object] = None

    def key(self) -> Tuple:
        return (self.kind, float(self.theta), float(self.factor), int(self.rotary_dim),
                self.scaling)


@dataclass(frozen=True)
class WavelengthScalingSpec:
    """Frequency scaling by wavelength (the YaRN form).  With pair(t) = dims * ln(original /
    (2 pi t)) / (2 ln theta), lo = max(floor(pair(fast)), 0), hi = min(ceil(pair(slow)),
    dims - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns with
    f_i / factor * ramp_i + f_i * (1 - ramp_i); cos and sin are multiplied by
    0.1 ln(factor) + 1."""
    factor: float = 1.0
    original: float = 0.0
    fast: float = 32.0
    slow: float = 1.0


@dataclass(frozen=True)
class BandScalingSpec:
    """Frequency scaling in three bands of wavelength l = 2 pi / f: f is kept where
    l < original / high, divided by ``factor`` where l > original / low, and between the two,
    with s = (original / l - low) / (high - low), becomes (1 - s) f / factor + s f.  cos and
    sin are not multiplied."""
    factor: float = 1.0
    original: float = 0.0
    low: float = 1.0
    high: float = 4.0


@dataclass(frozen=True)
class NormSpec:
    """RMS norm; ``zero_centered`` stores w and applies (1 + w)
    (src/models/gemma3.zig:199-202,943-949)."""
    kind: str = "rmsnorm"
    eps: float = 1e-6
    zero_centered: bool = True


@dataclass(frozen=True)
class LayerNormSpec:
    """Layer norm with weight and bias: (x - mean) / sqrt(var + eps) * w + b, the variance
    being the mean of the squared deviations; ``bias`` False leaves b out."""
    kind: str = "layernorm"
    eps: float = 1e-5
    bias: bool = True


@dataclass(frozen=True)
class IdentityNormSpec:
    """No norm at all: a branch reads the stream itself (rounded to the compute dtype)."""
    kind: str = "identity"


@dataclass(frozen=True)
class DistanceBiasSpec:
    """A learned table [rows, heads] added to the scaled score by distance n = t - j >= 0:
    row n for n < rows/2, else min(rows - 1, rows/2 + floor(ln(n / (rows/2)) / ln(far /
    (rows/2)) * (rows - rows/2)))."""
    rows: int = 0
    far: float = 0.0


@dataclass(frozen=True)
class DistanceSlopeSpec:
    """A bias that falls linearly with distance: slope_a * (t - j) is taken off the scaled
    score of head a, slope_a = 2 ** (-exponent * (a + 1) / n_heads) for a = 0 .. n_heads - 1.
    ``reach``: the greatest distance a query can see plus one (the model's positions, or the
    mask's size where that is less); it sizes the table the kernels index by distance."""
    exponent: float = 8.0
    reach: int = 0


@dataclass(frozen=True)
class ValueMixSpec:
    """Values that lean towards an earlier layer's: v <- (1 - m) v + m v_first, m a learned
    scalar (tensor ``value_mix``), v_first the values the call named ``source`` (a cache entry
    of the run order) made for the same token before its own mixing.  ``source`` None: this
    layer is the source; it mixes nothing and keeps its values for the others (its own
    ``value_mix`` tensor exists and is unused)."""
    source: Optional[int] = None


@dataclass(frozen=True)
class QueryTemperatureSpec:
    """The queries at position p are multiplied by 1 + coef * ln(floor((p + 1) / every) + 1):
    attention sharpens in steps as the context grows."""
    coef: float = 0.0
    every: int = 1


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query softmax attention over a key/value cache.

    ``window`` None keeps every key; an integer W lets position p see the keys
    j with p - W < j <= p (src/models/gemma4.zig:1153-1155).  ``scale``
    multiplies the dot product (src/backend/kernels/cpu/sdpa.zig:58).
    """
    kind: str = "attention"
    n_heads: int = 0
    n_kv_heads: int = 0
    head_dim: int = 0
    scale: float = 1.0
    window: Optional[int] = None
    qk_norm: Optional[NormSpec] = None      # per-head norm of q and k, before the rotation
    position: Optional[RotarySpec] = None
    # the size of a value head where it differs from head_dim (0: the same)
    value_dim: int = 0
    # a learned logit per query head whose exponential is one more term of the softmax
    # denominator (unscaled; nothing enters the weighted sum for it)
    sink: bool = False
    q_temp: Optional[QueryTemperatureSpec] = None
    # False: the layer has no key / value projections and attends to what the call that
    # writes its cache entry stored (the run order names that entry)
    own_kv: bool = True
    # q and k are RMS-normed over their whole projection (all heads at once, a weight of
    # that width) instead of head by head; eps and centring come from ``qk_norm``
    qk_norm_whole: bool = False
    # a sink whose logit is this constant instead of a learned tensor (0.0: one is added to
    # the softmax denominator)
    fixed_sink: Optional[float] = None
    distance_bias: Optional[DistanceBiasSpec] = None
    # position p sees j <= p only inside its own block of this many positions, counted from
    # position 0 of the sequence (floor(p / chunk) == floor(j / chunk)); not with ``window``
    chunk: Optional[int] = None
    distance_slope: Optional[DistanceSlopeSpec] = None
    value_mix: Optional[ValueMixSpec] = None
    # with ``window``: the sequence's first keep_first keys stay visible behind the window
    # (position p sees j <= p if p - j < window or j < keep_first), at their true positions
    keep_first: int = 0
    # a causal convolution over this many tokens on every channel of q, k and v (tensors
    # ``q_conv.weight`` ... [channels, taps], no bias, no activation), right after the
    # projection and before the rotation; 0: none.  The last conv_taps - 1 projected rows of a
    # sequence are part of its fixed-size state
    conv_taps: int = 0
    # the concatenated heads are multiplied element by element by sigmoid(W_g x) (tensor
    # ``g_proj.weight``) before the output projection
    out_gate: bool = False
    # the cache keeps every key of this layer whatever its own mask: another call reads the
    # entry through a mask that reaches further back
    keep_all_keys: bool = False

    @property
    def v_dim(self) -> int:
        return self.value_dim or self.head_dim


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal softmax attention whose keys and values are rebuilt from a cached latent.

    Per position the cache holds c = rmsnorm(W_dkv x)[:kv_rank] and one rotated key part kr
    (rot_dim wide) that all heads share.  Head a scores (q_a[:head_dim] . (W_uk c)_a +
    rot(q_a[head_dim:]) . kr) * scale and weighs (W_uv c)_a.  ``q_rank`` > 0: the queries
    come through a normed latent of that size too.  ``gate``: the heads' outputs are
    multiplied by sigmoid(W_g x), "element" by element or one value per "head"."""
    kind: str = "latent_attention"
    n_heads: int = 0
    head_dim: int = 0            # unrotated part of a query / key head
    rot_dim: int = 0             # rotated part
    value_dim: int = 0
    kv_rank: int = 0
    q_rank: int = 0
    scale: float = 1.0
    eps: float = 1e-6
    position: Optional[RotarySpec] = None
    gate: Optional[str] = None


@dataclass(frozen=True)
class ChannelDeltaSpec:
    """A recurrent mixer: the gated delta rule with a decay per key channel.

    q, k (``n_qk_heads`` heads of ``head_dim``) and v (``n_heads`` heads of ``value_dim``)
    pass a causal convolution over ``conv_taps`` tokens per channel and silu; q and k heads
    become unit vectors (x / sqrt(sum x^2 + unit_eps)), q times head_dim ** -0.5.  Per head,
    with beta = sigmoid(W_b x) and the decay g = exp(-exp(A_log) * softplus(W_a2 W_a1 x +
    dt_bias)) per key channel:  S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T;
    o = S^T q.  o / rms(o) (``eps``) * weight * sigmoid(W_g2 W_g1 x) feeds the output
    product.  ``decay_rank`` and ``gate_rank`` are the widths of the two bottlenecks.  The
    state (S in 32-bit and the convolution's last conv_taps - 1 inputs) is a fixed size per
    sequence."""
    kind: str = "channel_delta"
    n_heads: int = 0
    n_qk_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    conv_taps: int = 1
    decay_rank: int = 0
    gate_rank: int = 0
    eps: float = 1e-6
    unit_eps: float = 1e-6


@dataclass(frozen=True)
class MatrixMemorySpec:
    """A recurrent mixer: a matrix memory with exponential gates (the mLSTM of xLSTM).

    q = W_q x * head_dim ** -0.5 and k = W_k x (``n_heads`` heads of ``head_dim``), v = W_v x
    (heads of ``value_dim``).  Per head a log input gate i = cap * tanh((W_i x + b_i) / cap)
    and a log forget gate f = logsigmoid(cap * tanh((W_f x + b_f) / cap)), cap = ``gate_cap``.
    With a running maximum m that starts at 0:  m_t = max(f + m_(t-1), i);
    S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T;  n_t likewise with k alone;
    o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + ``den_eps``).  Every head's o is divided by its
    root mean square (``eps``), the heads are multiplied by a weight per channel and by
    sigmoid(W_g x) and go through the output product.  S, n and m (32-bit) are a fixed size
    per sequence."""
    kind: str = "matrix_memory"
    n_heads: int = 0
    head_dim: int = 0
    value_dim: int = 0
    gate_cap: float = 15.0
    eps: float = 1e-6
    den_eps: float = 1e-6


@dataclass(frozen=True)
class TokenSideSpec:
    """A per-layer input from the token itself, after the layer's feed-forward: with e the
    slice [offset, offset + dim) of the token's row of a table shared by the layers
    (``ModelSpec.token_side_width`` wide), g = gelu_tanh(W_gate h) * e, y = W_proj g and
    h += y / rms(y) * w (an RMS norm with a plain weight and ``eps``)."""
    dim: int = 0
    offset: int = 0
    eps: float = 1e-6


@dataclass(frozen=True)
class GatedFeedForwardSpec:
    """down(act(gate x) * up x), dense (src/models/gemma3.zig:840-872)."""
    kind: str = "gated_dense"
    intermediate_size: int = 0
    activation: str = "gelu_tanh"


@dataclass(frozen=True)
class DenseFeedForwardSpec:
    """down(act(up x)), dense, no gate; "relu2" is max(z, 0)^2, "gelu_erf" is
    z / 2 * (1 + erf(z / sqrt 2))."""
    kind: str = "dense"
    intermediate_size: int = 0
    activation: str = "relu2"


@dataclass(frozen=True)
class RoutedFeedForwardSpec:
    """A mixture of gated experts, down(act(gate x) * up x) each, of which a token uses
    ``top``.  Router: s = sigmoid(W_r x) in 32-bit; s + correction chooses, s weighs (not
    renormalised).  The experts form ``n_groups`` equal groups of neighbours; a group's score
    is the sum of its two largest choice scores, and only experts of the ``keep_groups`` best
    groups can be chosen."""
    kind: str = "routed"
    n_experts: int = 0
    top: int = 1
    intermediate_size: int = 0
    activation: str = "silu"
    n_groups: int = 1
    keep_groups: int = 1
    correction: bool = True
    # a bias [n_experts] added to the router's logits (tensor ``router.bias``)
    router_bias: bool = False
    # "sigmoid": as above; "softmax_top": the logits choose (with ``correction`` False) and the
    # chosen experts' weights are the softmax over their logits alone; "softmax_all": the
    # scores s are the softmax over all the router's outputs, s + correction chooses, and the
    # chosen experts' s, divided by their sum (+ 1e-20) and times ``route_scale``, weigh
    weighting: str = "sigmoid"
    route_scale: float = 1.0
    # the router has this many outputs beyond ``n_experts``: identity experts without tensors,
    # whose output is the feed-forward's input itself (times the weight)
    n_identity: int = 0
    # an expert of the same form that every token uses, of this width (0: none); its output is
    # multiplied by sigmoid(w_sg . x), one number per token (tensor ``shared.gate.weight``)
    shared_size: int = 0


@dataclass(frozen=True)
class LearnedPositionSpec:
    """A learned vector per position (tensor ``table.weight`` [positions, hidden]) added to the
    stream after the embedding, times ``scale``."""
    kind: str = "learned"
    positions: int = 0
    scale: float = 1.0


@dataclass(frozen=True)
class BlockSpec:
    """One layer: a mixer and a feed-forward between norms.

    arrangement "sandwich": h += post(mixer(pre(h))); h += post(ffn(pre(h)))
    (src/models/gemma3.zig:708-709,824-826,835-836,876-878);
    arrangement "pre": the same without the two post norms;
    arrangement "post": the same without the two pre norms (the branches read the stream
    itself).
    ``kind`` names the block class in the block registry; "sequential" is the
    class that runs the mixer and then the feed-forward, as above.  Another
    arrangement of parts (both branches from one norm, no feed-forward at all)
    is another block class under another kind, with a spec of its own if it
    needs other fields.
    """
    mixer: object = None
    feed_forward: object = None        # None: the layer has no feed-forward branch
    norm: object = NormSpec()
    arrangement: str = "sandwich"
    kind: str = "sequential"
    # every branch joins the stream times this: h += residual_mult * post(branch(pre(h)))
    residual_mult: float = 1.0
    # a per-layer input from the token, added after the feed-forward (None: none)
    token_side: Optional[TokenSideSpec] = None


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``block`` indexes ``ModelSpec.blocks`` (a block may be called twice);
    ``cache`` names the cache entry the mixer uses and ``writes_cache`` says
    whether this call appends to it (False: it reads what another call wrote).
    ``state``: the cache entry of the call's own fixed-size state where that is not
    ``cache`` (a call that reads another's keys and values and still has state of its own).
    """
    block: int
    cache: int
    writes_cache: bool = True
    state: Optional[int] = None


@dataclass(frozen=True)
class ModelSpec:
    """The whole decoder as data."""
    hidden_size: int
    vocab_size: int
    embed_scale: float
    blocks: Tuple[BlockSpec, ...]
    schedule: Tuple[LayerCall, ...]
    final_norm: object
    tie_embeddings: bool = True
    max_positions: int = 0
    bos_token_id: Optional[int] = None
    eos_token_ids: Tuple[int, ...] = ()
    # a position encoding that is added to the stream after the embedding (a learned
    # table, say), by its kind in the stream-position registry; None: there is none
    stream_position: Optional[object] = None
    # logits <- cap * tanh(logits / cap); None: no cap
    logit_softcap: Optional[float] = None
    # the logits are multiplied by this (before a cap)
    logit_scale: float = 1.0
    # width of the table of per-layer token inputs (tensor ``token_side.weight`` [vocab,
    # width]); the blocks' ``TokenSideSpec`` name their slices.  0: there is none
    token_side_width: int = 0

    def n_cache_entries(self) -> int:
        if not self.schedule:
            return 0
        return 1 + max(max(c.cache, c.state if c.state is not None else 0)
                       for c in self.schedule)


def default_schedule(n_blocks: int) -> Tuple[LayerCall, ...]:
    return tuple(LayerCall(block=i, cache=i) for i in range(n_blocks))
