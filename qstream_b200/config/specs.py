"""Typed descriptions of the parts a model is put together from.

A spec says which part to build (`kind`, looked up in the part registries), with
which sizes and constants, and under which checkpoint names its tensors lie
(`names`: the part's own tensor name -> the name in the safetensors file).  A spec
holds no weights and no code.  An architecture's configuration produces one
`ModelSpec`; nothing below it knows the architecture's name.

Any object with a `kind` attribute may serve as a spec of a part registered under
that kind, so a new part brings its own spec class.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """LayerNorm: mean and biased variance over `size`, eps inside the root,
    weight and (if `bias`) bias (QStream src/kernels_scalar.c:151-171)."""
    size: int
    eps: float
    bias: bool = True
    kind: str = "layernorm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class RmsNormSpec:
    """RMS norm: x / sqrt(mean(x^2) + eps) * (offset + weight), eps inside the root.  `offset` 1 is for
    weights stored around zero, 0 for plain weights."""
    size: int
    eps: float
    offset: float = 0.0
    kind: str = "rmsnorm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class StreamNormSpec:
    """A norm with a weight and no bias that reads a residual stream in its own type (32-bit, say) and writes the
    engine's: the layer norm (x - mean) / sqrt(variance + eps) * w (`center`) or the RMS norm x / sqrt(mean(x^2) + eps)
    * w, eps inside the root.  It can also add a branch to the stream first, the branch normed with another such
    norm's weight, in the same kernel (layers that norm a branch before they add it)."""
    size: int
    eps: float
    center: bool = True
    kind: str = "stream_norm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class RotaryHalfSpec:
    """Rotary position encoding on the first `rotary_dim` dims of a vector, element i paired with i + rotary_dim/2,
    angle position * f_i, f_i = base^(-2i / rotary_dim).  `scaling` (factor, original, fast, slow) rescales the
    frequencies in the YaRN manner: with dim(t) = rotary_dim ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(dim(fast)), 0), hi = min(ceil(dim(slow)), rotary_dim - 1) and
    ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), f_i becomes f_i / factor * ramp_i + f_i (1 - ramp_i), and cos
    and sin are multiplied by 0.1 ln(factor) + 1.  `layout` "interleaved" pairs element 2i with 2i + 1 instead (same
    angles); the kernels that rotate are told which."""
    rotary_dim: int
    base: float
    scaling: Optional[Mapping[str, float]] = None
    kind: str = "rotary_half"
    layout: str = "half"


@dataclass(frozen=True)
class PositionSpec:
    """Rotary position encoding on the first `rotary_dim` dims of each head,
    pairs (i, i+1) (QStream src/engine.c:205-234 with head_dim -> rotary_dim)."""
    rotary_dim: int
    base: float
    max_positions: int
    kind: str = "rotary_interleaved"


@dataclass(frozen=True)
class PositionHalfSpec:
    """Rotary position encoding on the first `rotary_dim` dims of each head, element i paired with element
    i + rotary_dim / 2, angle position * base^(-2i / rotary_dim); the angles come from a table of `max_positions`
    rows, and attention fuses the rotation with its cache write."""
    rotary_dim: int
    base: float
    max_positions: int
    kind: str = "rotary_half_table"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal softmax attention over the sequence's cache.

    `window` = 0 reads all keys, w > 0 the last w (the query's own included).
    `shares_cache`: the layer projects queries only and reads the keys and values
    that another layer of the schedule wrote.
    `v_head_dim`: the values' head size where it differs from that of queries and keys.
    `score_scale`: the factor on q.k (default head_dim^-1/2).  `softcap` c > 0: scores
    become c tanh(s / c) before the softmax.  `gate`: the concatenated heads are multiplied
    by sigmoid(W_g h) before the output projection.  `value_mix`: "first" keeps the layer's
    values for later layers of the same step, "blend" caches (1 - l) v + l v_first with its
    scalar tensor "value_mix" as l.
    `chunk` c > 0: a query sees only the keys of its own chunk of c positions; chunks tile the sequence from its first token (no window then).
    `keep_first` n > 0 with a window: the sequence's first n keys stay visible to every later query.
    `sink`: a learned number per query head (tensor "sink") whose exponential joins the softmax's denominator without a
    key or a value.  `maps` = 2 (differential attention): q and k hold two maps per head side by side, each an attention
    of its own over the same values; with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + `diff` (four vectors of head_dim),
    o = a1 - lambda a2 per head, divided by its root mean square over the head's values (`eps` inside the root), times
    (1 - diff).
    `qk_norm` "whole": q = W_q h and k = W_k h each pass one RMS norm over the whole projection (all heads at once,
    plain weights "q_norm" and "k_norm" of that size, `eps` inside the root) before they are split into heads and rotated.
    `values_from_keys`: there is no W_v; a key head's values are its keys as projected, before norm and rotation.
    `fixed_sink`: a number whose exponential joins every softmax's denominator without a key or a value (0.0: one
    more term of exp(0) = 1), with no tensor behind it.
    """
    width: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    position: Optional[PositionSpec] = None
    window: int = 0
    qkv_bias: bool = False
    out_bias: bool = False
    shares_cache: bool = False
    kind: str = "attention"
    names: Mapping[str, str] = field(default_factory=dict)
    v_head_dim: Optional[int] = None
    score_scale: Optional[float] = None
    softcap: float = 0.0
    gate: bool = False
    value_mix: Optional[str] = None
    chunk: int = 0
    keep_first: int = 0
    sink: bool = False
    maps: int = 1
    diff: float = 0.0
    eps: float = 0.0
    qk_norm: Optional[str] = None
    values_from_keys: bool = False
    fixed_sink: Optional[float] = None

    @property
    def scale(self) -> float:
        return self.head_dim ** -0.5 if self.score_scale is None else float(self.score_scale)

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_head_dim is None else self.v_head_dim


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal softmax attention whose keys and values are linear maps of one cached latent per token.

    Queries: c_q = RMSnorm(W_dq h) (rank `q_rank`), q = W_uq c_q, per head [head_dim unrotated | rot_dim rotated].
    W_dkv h gives the latent c (rank `kv_rank`, RMS-normed) and one rotated key part of `rot_dim` shared by all heads;
    only these are cached.  Per head the unrotated key is W_uk c and the value W_uv c (`v_head_dim`).  The score is
    (q_unrotated . k_unrotated + q_rotated . k_rotated) * `score_scale`.  `shares_cache`: the layer has no W_dkv and
    reads the latents another layer cached, with its own W_uk, W_uv and queries.  `sink`: a learned number per head
    (tensor "sink") whose exponential joins the softmax's denominator, unscaled, without key or value.  `head_gate`:
    head h's output is multiplied by sigmoid(W_g h)_h, W_g ("g") having one row per head."""
    width: int
    n_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    score_scale: float
    eps: float
    position: Optional[object] = None
    shares_cache: bool = False
    kind: str = "latent_attention"
    names: Mapping[str, str] = field(default_factory=dict)
    sink: bool = False
    head_gate: bool = False


@dataclass(frozen=True)
class MlstmSpec:
    """Matrix memory with exponential gates (the mLSTM of xLSTM): q = W_q h key_dim^-1/2, k = W_k h, v = W_v h per head,
    log gates i = cap tanh((W_i h + b_i) / cap), f = logsigmoid(cap tanh((W_f h + b_f) / cap)) (`gate_cap` 0: no cap);
    m_t = max(f + m_{t-1}, i) with m_0 = 0; S_t = exp(f + m_{t-1} - m_t) S_{t-1} + exp(i - m_t) k v^T, n_t likewise with
    k alone; o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6); each head's o divided by its root mean square, times a
    weight, times sigmoid(W_g h), then W_o.  State per sequence in 32-bit: S and n ([heads, value_dim + 1, key_dim])
    and m ([heads])."""
    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    eps: float
    kind: str = "mlstm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class DecayAttentionSpec:
    """Linear attention with a fixed decay per head: S_t = decay_h S_{t-1} + k_t v_t^T, o_t = S_t^T q_t, with
    `activation` on q, k and v; the concatenated heads get one RMS norm (plain weight), a sigmoid gate from
    the mixer's input, and the output projection.  State: [heads, value_dim, key_dim] in 32-bit per sequence.
    Options: `position` rotates q and k before the recurrence; `key_scale` multiplies k; `norm_per_head` takes each
    head's root mean square instead of the whole vector's; `norm_weight` False: the norm has no weight;
    `gate_activation` names the gate's function."""
    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    decay: Tuple[float, ...]
    eps: float
    activation: Optional[str] = "silu"
    kind: str = "lightning"
    names: Mapping[str, str] = field(default_factory=dict)
    position: Optional[object] = None
    key_scale: float = 1.0
    norm_per_head: bool = False
    norm_weight: bool = True
    gate_activation: str = "sigmoid"


@dataclass(frozen=True)
class GlaSpec:
    """Gated linear attention: q = W_q h key_dim^-1/2, k = W_k h, v = W_v h per head; a decay per token, head and key
    channel w = sigmoid(W_a2 (W_a1 h) + b)^(1 / `tau`) from a two-matrix bottleneck (`decay_rank`, -1: whatever the
    checkpoint holds); S_t = diag(w_t) S_{t-1} + k_t v_t^T, o_t = S_t^T q_t.  Each head's o gets an RMS norm over
    value_dim with a weight of that size shared by the heads; the concatenated heads are multiplied by silu(W_g h) and
    projected by W_o.  State per sequence: S [heads, value_dim, key_dim] in 32-bit; the decays and the walk are 32-bit."""
    width: int
    n_heads: int
    key_dim: int
    value_dim: int
    tau: float
    eps: float
    decay_rank: int = -1
    kind: str = "gla"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class GatedDeltaSpec:
    """The gated delta rule.  q, k = W h (`n_qk_heads` heads of key_dim), v = W h (`n_heads` heads of value_dim); each
    passes a causal convolution over time per channel (`conv_taps` taps, the last the current token's) and silu; q and k
    become unit vectors per head (x / sqrt(sum x^2 + `unit_eps`)), q times key_dim^-1/2.  Step size beta = sigmoid(W_b h)
    per head; decay per head and key channel g = exp(-exp(A_log_h) softplus(W_a2 W_a1 h + dt_bias)).  Per head, on
    S [key_dim, value_dim]: S <- diag(g) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q.  Each head's o is divided by
    its root mean square (`eps`), times a weight of value_dim shared by the heads, times sigmoid(W_g2 W_g1 h); then W_o.
    State per sequence: S in 32-bit and the convolutions' last conv_taps - 1 inputs.  The ranks of the two bottlenecks
    (-1: whatever the checkpoint holds)."""
    width: int
    n_heads: int
    n_qk_heads: int
    key_dim: int
    value_dim: int
    conv_taps: int
    eps: float
    unit_eps: float = 1e-6
    decay_rank: int = -1
    gate_rank: int = -1
    kind: str = "gated_delta"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class PairMixerSpec:
    """Two mixers side by side that read the same input: left_scale * left(h) + right_scale * right(h).  Each keeps its
    own cache entry (a schedule run names two)."""
    left: object
    right: object
    left_scale: float = 1.0
    right_scale: float = 1.0
    kind: str = "pair"

    @property
    def names(self) -> Mapping[str, str]:
        """The two mixers' tensors under "left.<name>" and "right.<name>"."""
        return {**{"left." + k: v for k, v in self.left.names.items()}, **{"right." + k: v for k, v in self.right.names.items()}}


@dataclass(frozen=True)
class WkvSpec:
    """RWKV-style time mixing: five mixes of the input with the previous token's, r/k/v/gate projections,
    a decay exp(-exp(.)) per token and channel from a two-matrix bottleneck of `decay_rank` (-1: whatever
    the checkpoint holds), a bonus for the current token, a unit RMS per head, a weight, the gate, and the
    output projection.  State: [heads, head_dim, head_dim] in 32-bit and the previous input per sequence."""
    width: int
    n_heads: int
    head_dim: int
    eps: float
    decay_rank: int = -1
    kind: str = "wkv"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class MlpSpec:
    """Dense feed-forward: up projection, activation, down projection
    (QStream src/engine.c:1150-1170), with biases if `bias`."""
    width: int
    inner: int
    activation: str
    bias: bool = True
    kind: str = "mlp"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class GatedMlpSpec:
    """Gated feed-forward: down(act(gate h) * (up h)), every projection with a bias if `bias`."""
    width: int
    inner: int
    activation: str = "silu"
    kind: str = "gated_mlp"
    names: Mapping[str, str] = field(default_factory=dict)
    bias: bool = False


@dataclass(frozen=True)
class HyperConnectionSpec:
    """How one sublayer meets a residual stream kept in `streams` copies x_1 .. x_S: it reads u = sum_s in[s] x_s and its
    result y returns as x_t <- sum_s mix[s][t] x_s + out[t] * (scale . y) for all t at once, `scale` a vector of the
    width (`layer_scale`).  `mixing` False: no in, mix, out tensors (ones, the identity, ones), which with one copy is the
    plain residual sum."""
    streams: int
    width: int
    mixing: bool = True
    layer_scale: bool = True
    kind: str = "hyper_connection"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class StreamSumNormSpec:
    """The RMS norm of the sum of a residual stream's `streams` copies (one row holds them side by side):
    x = sum_s x_s; x / sqrt(mean(x^2) + eps) * (offset + weight)."""
    size: int
    streams: int
    eps: float
    offset: float = 0.0
    kind: str = "stream_sum_rmsnorm"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class RoutedExpertsSpec:
    """A mixture of `n_experts` small feed-forward layers W_down act(W_up h) without biases, of which a token uses `top`.

    Router: scores s = sigmoid(W_router h) in 32-bit; choice scores s + correction; the experts form `groups` equal
    groups of neighbours, a group's score is the sum of its two largest choice scores, and only experts of the best
    `keep` groups can be chosen; the `top` largest choice scores win; their weights are s * `route_scale`, not
    renormalised.  `shared_inner` > 0: one more expert of that size runs for every token and is added, multiplied by
    sigmoid(w_sg . h).
    Options: `scores` "softmax": s = softmax(z) over all experts; `group_score` "max": a group's score is its largest
    choice score; `correction` False: no correction tensor; `shared_gate` False: the shared expert is added as it is.
    `gated`: every expert (the shared one too) is W_down y with g = min(W_gate h, limit), u = clamp(W_up h, -limit,
    limit), y = g sigmoid(`glu_alpha` g) (u + `glu_shift`) (tensors "gate<e>", "shared_gate_proj"); `limit` for the
    routed experts, `shared_limit` for the shared one (0: no clamp)."""
    width: int
    n_experts: int
    inner: int
    top: int
    groups: int = 1
    keep: int = 1
    route_scale: float = 1.0
    activation: str = "relu2"
    shared_inner: int = 0
    kind: str = "routed_experts"
    names: Mapping[str, str] = field(default_factory=dict)
    scores: str = "sigmoid"
    group_score: str = "top2"
    correction: bool = True
    shared_gate: bool = True
    gated: bool = False
    limit: float = 0.0
    shared_limit: float = 0.0
    glu_alpha: float = 1.702
    glu_shift: float = 1.0


@dataclass(frozen=True)
class BlockSpec:
    """One layer: its norms, mixer and feed-forward, and how they are wired.

    arrangement "parallel": h = norm(x); x + mixer(h) + ffn(h)   (norms: "input")
    arrangement "sequential": x += mixer(norm_1(x)); x += ffn(norm_2(x))
                                                     (norms: "input", "post_mixer")
    arrangement "scaled_residual": the same with x kept in 32-bit whatever the engine's type and
        every branch multiplied by `residual_scale`: x += m mixer(norm_1(x)); x += m ffn(norm_2(x));
        `ffn` may be None (then only "input" is needed).
    arrangement "sandwich": a norm before and after each sublayer, x in 32-bit:
        x += norm_1b(mixer(norm_1(x))); x += norm_2b(ffn(norm_2(x)))
                                        (norms: "input", "post_input", and with a feed-forward "post_mixer", "post_ffn")
    arrangement "post_norm": the sublayers read the 32-bit stream itself and a norm meets their results only:
        x += norm_1(mixer(x)); x += norm_2(ffn(x))      (norms: "post_input", and with a feed-forward "post_ffn")
    arrangement "hyper": the stream in several copies, in 32-bit; each sublayer reads and writes it as its
        `HyperConnectionSpec` says (`connections`: "mixer", and with a feed-forward "ffn"); norms "input", "post_mixer".
    """
    mixer: object
    ffn: object
    norms: Mapping[str, object]
    arrangement: str = "parallel"
    residual_scale: float = 1.0
    connections: Mapping[str, object] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerRun:
    """One entry of the schedule: run layer `layer` against cache entry `cache`.
    A layer may appear in several runs; two runs may name the same cache entry
    when the later one only reads it.  For a layer with several parts that use the
    cache, `cache` is a tuple with one entry id per such part."""
    layer: int
    cache: object


@dataclass(frozen=True)
class EmbeddingSpec:
    vocab_size: int
    width: int
    kind: str = "embedding"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class PairEmbeddingSpec:
    """x = table[token] * scale + pair[(previous token * mul_prev + token * mul_cur) mod buckets], the pair
    table's last row (number `buckets`) for a sequence's first token; `buckets` 0: no pair table.
    `stream_dtype`: the type of x where it is not the engine's ("float32": a 32-bit residual stream)."""
    vocab_size: int
    width: int
    scale: float = 1.0
    buckets: int = 0
    mul_prev: int = 0
    mul_cur: int = 0
    stream_dtype: Optional[str] = None
    kind: str = "pair_embedding"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class NormedEmbeddingSpec:
    """x = norm(table[token]): the token's row followed by a norm with a weight and no bias (layer norm if `center`,
    else RMS), delivered in `stream_dtype` ("float32": a 32-bit residual stream; None: the engine's type)."""
    vocab_size: int
    width: int
    eps: float
    center: bool = True
    stream_dtype: Optional[str] = None
    offset: float = 0.0                 # RMS only: the weight is stored around zero (offset 1)
    kind: str = "normed_embedding"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class HeadSpec:
    """Output projection to the vocabulary, logits in 32-bit.  `tied` reuses the
    embedding table as its weight."""
    vocab_size: int
    width: int
    bias: bool = True
    tied: bool = False
    kind: str = "lm_head"
    names: Mapping[str, str] = field(default_factory=dict)


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    width: int
    max_positions: int
    embedding: object
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[LayerRun, ...]
    final_norm: Optional[object]            # None: the head sees the last layer's output as it is
    head: object
    stop_tokens: Tuple[int, ...] = ()
    bos_token_id: Optional[int] = None

    def n_cache_entries(self) -> int:
        ids = [c for r in self.schedule for c in (r.cache if isinstance(r.cache, (tuple, list)) else (r.cache,))]
        return 1 + max(ids, default=-1)
