"""What a model is made of, as data: one small record for each part of each layer.

A configuration class (`gemma2.Gemma2Config`) turns config.json into a `ModelSpec`; the
engine builds parts from it through `kapel_b200.parts.registry` by each record's `kind`.
Nothing here knows a model family: sizes, constants and tensor names are all fields.

Kapel keeps one struct of switches for every family (crates/kapel-models/src/config.rs:98-166);
here a layer names its own mixer, feed-forward, norms and position encoding, so two layers
of one model may differ in all of them.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Mapping, Optional, Tuple


@dataclass(frozen=True)
class NormSpec:
    """y = x / sqrt(mean(x^2) + eps) * (offset + w) for kind "rms"; kind "layer" takes the row's mean
    off first: y = (x - mean) / sqrt(mean((x - mean)^2) + eps) * (offset + w), without a bias."""

    width: int
    eps: float
    offset: float
    weight: str                      # tensor name
    kind: str = "rms"


@dataclass(frozen=True)
class RopeScaling:
    """Frequencies stretched by wavelength: with r rotated components and base theta, the pair that
    turns t times over `original` positions is number n(t) = r ln(original / (2 pi t)) / (2 ln theta);
    lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), r - 1), ramp_j = clamp((j - lo) / max(hi - lo,
    0.001), 0, 1); pair j turns at f_j / factor * ramp_j + f_j (1 - ramp_j), and cos and sin are both
    multiplied by 0.1 ln(factor) + 1."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class PositionSpec:
    """kind "rope": rotation of the first `rotary_dim` components, pairing "half" (j, j+r/2) or
    "neighbours" (2j, 2j+1), by the angle position * theta^(-2j/r) / `divisor` (a divisor above 1
    stretches the positions); with `scaling` the frequencies follow `RopeScaling` instead."""

    kind: str = "rope"
    theta: float = 10000.0
    rotary_dim: int = 0
    pairing: str = "half"
    divisor: float = 1.0
    scaling: Optional[RopeScaling] = None


@dataclass(frozen=True)
class AttentionSpec:
    """Grouped-query attention over a paged cache.

    `window` None sees every key; else a query at position p sees keys j with p - j < window,
    and also the keys j < `keep_first` however far back. `scale` multiplies q.k; `softcap` c turns
    a score s into c*tanh(s/c) before the mask. `weights` maps the roles q, k, v, o to tensor
    names, each [out, in]; with `gated`, role g as well: the heads' outputs are multiplied by
    sigmoid(g(h)) ahead of o. `v_head_dim` None: values have the keys' size. `q_norm` / `k_norm`:
    a norm over the whole projection (all heads' rows at once) ahead of the split into heads.
    `q_head_norm` / `k_head_norm`: an RMS norm over each head's vector with one weight of the head's
    size for all heads, ahead of the rotation.

    `bias`: q, k and v have biases (roles q_bias, k_bias, v_bias). `pool` P > 0 (with a window): beside
    the window's tokens a query sees one key and value for every block of P positions that lies wholly
    below its window, the means of the block's keys and values as the cache holds them, in the same
    softmax; `pool_blocks` is the most blocks a request can have (its position limit / P). `head_temp`:
    a head's scores are multiplied by its number of role temp [heads]. `talk`: after the softmax the
    heads' weights are mixed, w'_h = sum_g talk[h, g] w_g (role talk [heads, heads]), and head h applies
    w'_h to the values of its own kv head. `value_mix` "source": this layer's values (of this step's
    rows, before they are cached) are kept for later layers; "mix": v <- (1 - l) v + l v_source with l
    the one value of role vmix, and the mixed v is what is cached; the layers of one `value_mix_key`
    share a source.

    `conv` t > 0: every channel of the query and of the key projection goes through a causal convolution
    over the last t rows (roles q_conv, k_conv: [channels, t], the last weight for the row itself; zeros
    before a request's first row; no activation), directly after the projection and its bias; the last
    t - 1 projected rows are state of a request. `values_are_keys`: there is no v; a key as it is cached is
    also the value. `block_mask` B > 0: a query at position i sees a key j <= i only if floor(i / B) =
    floor(j / B), blocks counted from position 0. `unit_sink`: 1 joins the softmax's denominator (a key
    of score 0 without a value). `out_bias`: o has a bias (role o_bias); with `qk_bias` q and k have
    biases and v has none.
    """

    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    softcap: Optional[float]
    window: Optional[int]
    position: PositionSpec
    weights: Mapping[str, str]
    kind: str = "attention"
    keep_first: int = 0
    v_head_dim: Optional[int] = None
    q_norm: Optional[NormSpec] = None
    k_norm: Optional[NormSpec] = None
    gated: bool = False
    q_head_norm: Optional[NormSpec] = None
    k_head_norm: Optional[NormSpec] = None
    bias: bool = False
    pool: int = 0
    pool_blocks: int = 0
    head_temp: bool = False
    talk: bool = False
    value_mix: Optional[str] = None
    value_mix_key: str = "values"
    conv: int = 0
    values_are_keys: bool = False
    block_mask: int = 0
    unit_sink: bool = False
    qk_bias: bool = False
    out_bias: bool = False


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Attention whose queries and whose keys and values come through low-rank latents.

    c_q = rms(dq h) [q_rank]; every head's query is uq c_q: `head_dim` plain components, then
    `rot_dim` rotated ones. dkv h gives the latent c [kv_rank] (RMS-normed) and, behind it, one
    rotated key part [rot_dim] shared by all heads (not normed). A head's plain key is uk c, its
    value uv c; score = (q_plain . k_plain + q_rot . k_rot) * `scale`. Only c and the rotated part
    are kept in the cache. With `sink`, e^(sink[head]) joins the softmax's denominator; with
    `gated`, the heads' outputs are multiplied by sigmoid(g(h)) ahead of o. `weights`: dq, dq_norm,
    uq, dkv, dkv_norm, uk, uv, o, and sink, g where used.
    """

    hidden: int
    num_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    scale: float
    eps: float
    position: PositionSpec
    weights: Mapping[str, str]
    sink: bool = False
    gated: bool = False
    kind: str = "latent_attention"


@dataclass(frozen=True)
class DeltaSpec:
    """The gated delta rule: a matrix memory S [head_dim, v_head_dim] a head and request.

    q, k [kv_heads, head_dim] and v [heads, v_head_dim] from the input, each through a causal
    convolution over `conv` rows per channel and silu; q and k made unit vectors per head
    (x / sqrt(sum x^2 + `unit_eps`)), q times head_dim^-1/2; step size beta = sigmoid(b h) and decay
    g = exp(-exp(A_log) softplus(a h + dt_bias)) per head. Per row: S <- g S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q. Each head's o is divided by its root mean square (`eps`), times the
    weight `norm` [v_head_dim] (one for all heads), times silu(g h), then o. `weights`: q, k, v,
    q_conv, k_conv, v_conv, b, a, A_log, dt_bias, norm, g, o.
    """

    hidden: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    conv: int
    eps: float
    weights: Mapping[str, str]
    unit_eps: float = 1e-6
    kind: str = "delta"


@dataclass(frozen=True)
class GeneralDeltaSpec:
    """The generalized delta rule: a matrix memory S [head_dim, head_dim] a head and request with a
    decay a key channel and the removal of what lies along the unit key.

    r, k, v [heads, head_dim] from the input. Per head and key channel the decay
    w = exp(-`decay_scale` sigmoid(w2 tanh(w1 h) + w0)) and the removal rate a = sigmoid(a h + a_bias).
    With u = k / sqrt(sum k^2 + `unit_eps`): S <- diag(w) S - (a u)(u^T S) + k v^T (both first terms
    read the old S); o = S^T r. Each head's o is divided by its root mean square (`eps`), times the
    weight `norm` [heads head_dim], times sigmoid(g h), then o. `weights`: r, k, v, g, a, a_bias, w1,
    w2, w0, norm, o; the small net's hidden width is w1's number of rows (`lora`).
    """

    hidden: int
    num_heads: int
    head_dim: int
    lora: int
    eps: float
    weights: Mapping[str, str]
    decay_scale: float = 0.6065306597126334          # e^(-1/2)
    unit_eps: float = 1e-6
    kind: str = "general_delta"


@dataclass(frozen=True)
class ForgetGateSpec:
    """Gated linear attention with tied gates, the input gate being one minus the forget gate (HGRN2): a matrix memory
    S [head_dim, v_head_dim] a head and request.

    q = silu(q h) [heads, head_dim], v = v h [heads, v_head_dim], f = l + (1 - l) sigmoid(f h + f_bias)
    per head and channel with the lower bound l (role lower, [heads head_dim]). S <- diag(f) S +
    (1 - f) v^T; o = S^T q. Each head's o is RMS-normed over v_head_dim (`eps`) with the weight `norm`
    [v_head_dim] shared by the heads, then o. `weights`: q, f, f_bias, lower, v, norm, o.
    """

    hidden: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    eps: float
    weights: Mapping[str, str]
    kind: str = "forget_gate"


@dataclass(frozen=True)
class ParallelMixerSpec:
    """Two mixers side by side that read the same input: `left_scale` left(h) + `right_scale` right(h).
    Each keeps its own pages and state; at most one of them may ask for pages."""

    left: object
    right: object
    left_scale: float
    right_scale: float
    kind: str = "parallel"


@dataclass(frozen=True)
class MLSTMSpec:
    """A matrix memory with exponential gates (xLSTM's mLSTM), one state a head and request.

    q (times head_dim^-1/2), k [heads, head_dim] and v [heads, v_head_dim] from the input; log input
    gate cap*tanh(z_i/cap), log forget gate logsigmoid(cap*tanh(z_f/cap)) with z = W h + b per
    head; memory S, normaliser n and running maximum m start at zero; the read-out S^T q is divided
    by max(|n.q|, exp(-m)) + `floor`, then each head by its root mean square (`eps`), times the
    weight `norm`, times sigmoid(g(h)), then o. `weights`: q, k, v, g, o, i, i_bias, f, f_bias, norm.
    """

    hidden: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    gate_cap: float
    eps: float
    weights: Mapping[str, str]
    floor: float = 1e-6
    kind: str = "mlstm"


@dataclass(frozen=True)
class MoESpec:
    """A mixture of small feed-forwards: down(act(up(h))) for the `top` experts a token chooses,
    added up with the router's weights.

    Router scores s = `scoring`(router(h)) ("sigmoid", "softmax" over all experts, or "softmax_chosen":
    the logits choose and the chosen experts are weighted by the softmax over their logits alone);
    with `gated` an expert is down(act(gate(h)) * up(h)) (pattern `gate`); `shared`: the spec of a
    feed-forward that every token runs and whose output is added. Experts are chosen by s + the tensor `correction`
    (where one is named) but weighted by s; with `groups` > 1 the experts form that many equal
    groups of neighbours, a group scores the sum of its `group_top` best choice scores, and only
    experts of the best `keep_groups` groups can be chosen; `renormalize` divides the chosen
    weights by their sum. `weights`: router, correction (or absent), and the patterns `up` and
    `down` with `{e}` for the expert's number. The gated activation "clamped_swish" with `limit` L and
    `swish_alpha` a: g = min(gate h, L), u = clamp(up h, -L, L), the unit is g sigmoid(a g) (u + 1).
    """

    hidden: int
    experts: int
    top: int
    intermediate: int
    activation: str                  # "relu2": the square of relu; or one of the gated unit's names
    weights: Mapping[str, str]
    groups: int = 1
    keep_groups: int = 1
    group_top: int = 2
    scoring: str = "sigmoid"
    renormalize: bool = False
    gated: bool = False
    shared: Optional[object] = None
    limit: Optional[float] = None
    swish_alpha: float = 1.702
    kind: str = "moe"


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(h)) * up(h)); `activation` is "gelu_tanh" or "silu"."""

    hidden: int
    intermediate: int
    activation: str
    weights: Mapping[str, str]       # roles gate, up, down
    kind: str = "gated_mlp"


@dataclass(frozen=True)
class MLPSpec:
    """down(act(up(h))); `activation` is "relu2" (the square of relu), "gelu_tanh" or "silu"."""

    hidden: int
    intermediate: int
    activation: str
    weights: Mapping[str, str]       # roles up, down
    kind: str = "mlp"


@dataclass(frozen=True)
class BlockSpec:
    """The arrangement of one layer.

    kind "sandwich": norms `pre_mixer`, `post_mixer`, `pre_ffn`, `post_ffn` around both
    branches (`ffn` None: a layer of its mixer alone, with the first two norms);
    kind "prenorm": `pre_mixer` and `pre_ffn` only; kind "postnorm": the branches read
    the residual itself and only their outputs are normed (`post_mixer`, `post_ffn`), and `ffn`
    may be None for a layer without a feed-forward. kind "parallel": one norm `pre`, and both branches
    read its output h: x <- x + (mixer(h) + ffn(h)); with `scales` = (name, name) each branch is first
    multiplied, channel by channel, by a weight [hidden] (the second is absent without a feed-forward);
    with `shift` (a tensor [hidden]) the mixer, and only the mixer, reads h_t + (h_(t-1) - h_t) * shift,
    h_(t-1) the row before (zeros for a request's first row), which is state of a request.
    """

    mixer: object
    ffn: object
    norms: Mapping[str, NormSpec]
    kind: str = "sandwich"
    scales: Optional[Tuple[str, Optional[str]]] = None
    shift: Optional[str] = None


@dataclass(frozen=True)
class ScheduleEntry:
    """One layer run: which layer, and whose cache it reads (its own when `cache_of == layer`).

    A layer named twice runs twice; a layer whose `cache_of` is another layer's index reads
    that layer's keys and values and writes none. `replica` > 0 gives a run of the same layer a
    cache (pages, state) of its own: a layer that runs several times with the same weights keeps
    one cache a run. `before`: the spec of a part of category "merge" that rewrites the residual
    stream ahead of this run (`InputMixSpec`), or None.
    """

    layer: int
    cache_of: int
    replica: int = 0
    before: Optional[object] = None


@dataclass(frozen=True)
class InputMixSpec:
    """x <- W [x; x0]: the stream and the embedding's output x0 side by side through one matrix
    `weight` [hidden, 2 hidden] (the stream's columns first)."""

    hidden: int
    weight: str
    kind: str = "input_mix"


@dataclass(frozen=True)
class InputAddSpec:
    """x <- x + x0: the embedding's output x0 is added to the stream."""

    hidden: int
    kind: str = "input_add"


@dataclass(frozen=True)
class EmbedSpec:
    """x = table[token] * scale; with `positions` (a tensor [max_positions, hidden]) plus that table's
    row of the token's position, not scaled."""

    weight: str
    scale: float                     # exact; rounded to the activation dtype when `round_scale`
    round_scale: bool = True
    kind: str = "embedding"
    positions: Optional[str] = None
    max_positions: int = 0


@dataclass(frozen=True)
class HeadSpec:
    weight: str                      # the table [vocab, hidden]; the embedding's when tied
    softcap: Optional[float]
    kind: str = "vocab_head"


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    vocab_size: int
    hidden_size: int
    embed: EmbedSpec
    layers: Tuple[BlockSpec, ...]
    schedule: Tuple[ScheduleEntry, ...]
    final_norm: NormSpec
    head: HeadSpec
    max_positions: Optional[int] = None
    extra: Mapping[str, object] = field(default_factory=dict)


def default_schedule(n_layers: int) -> Tuple[ScheduleEntry, ...]:
    """Each layer once, in order, with a cache of its own."""
    return tuple(ScheduleEntry(i, i) for i in range(n_layers))
