"""Lokedra's configuration: a list of layers, each naming its mixer and its mixture of experts, and a
loop that runs a run of layers several times.

config.json gives `architecture`, `vocab`, `width`, `norm.eps`, `embedding.scale`, `layers` and `loop`.
A layer record is {type, mixer, mlp}. A layer has ONE norm (an RMS norm whose weight is stored around
zero) and both branches read its output: x <- x + (ls1 * mixer(shift(h)) + ls2 * ffn(h)), with a
weight a channel on each branch and a token shift ahead of the mixer. `type`:

* "general_delta": the generalized delta rule {heads, dim} (the small decay net's hidden width is the
  number of rows of the tensor `w1`; `lora` may also be given here, as a model with random weights needs it);
* "latent_attention": attention through low-rank latents {heads, dim, rot_dim, vdim, q_rank, kv_rank,
  scale, rot{base, dims, scaling{factor, original, fast, slow}}}, neighbouring components rotated;
* "parallel": two mixers side by side, {left, right, left_scale, right_scale}: `left` is grouped-query
  attention behind short convolutions {heads, kv_heads, dim, vdim, conv, scale, mask{size}} whose values
  are its keys, over chunks of `mask.size` positions, with 1 in the softmax's denominator; `right`
  {heads, dim, vdim} is gated linear attention whose input gate is one minus its forget gate.

`mlp` is {kind: "moe", router{experts, top}, expert{ff, limit}} or null. `loop` {start, stop, times}: the
layers start .. stop-1 run `times` times in a row with the same weights and a cache of their own each
time; ahead of every pass but the first the embedding's output is added to the stream. The head is the
embedding table. Every size and constant is read from the file; the constants written here are those
the design fixes (the decay's e^(-1/2), the unit key's 1e-6, the experts' 1.702).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, replace
from typing import Optional, Tuple

from .gemma2 import ConfigError, _MAX_HEAD_DIM, _MAX_HEADS, _MAX_HIDDEN, _MAX_INTERMEDIATE, _MAX_LAYERS, _MAX_VOCAB, _float, _int
from .spec import (
    AttentionSpec,
    BlockSpec,
    EmbedSpec,
    ForgetGateSpec,
    GeneralDeltaSpec,
    HeadSpec,
    InputAddSpec,
    LatentAttentionSpec,
    ModelSpec,
    MoESpec,
    NormSpec,
    ParallelMixerSpec,
    PositionSpec,
    RopeScaling,
    ScheduleEntry,
)

TYPES = ("general_delta", "latent_attention", "parallel")
DECAY_SCALE = math.exp(-0.5)
UNIT_EPS = 1e-6
SWISH_ALPHA = 1.702


def _record(raw, key: str, where: str, required: bool = True) -> Optional[dict]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: `{where}{key}` is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: `{where}{key}` must be an object")
    return v


def _flat(rec: dict, where: str) -> dict:
    return {f"{where}{k}": v for k, v in rec.items()}


@dataclass(frozen=True)
class LokedraRotation:
    dims: int
    base: float
    scaling: Optional[RopeScaling]


@dataclass(frozen=True)
class LokedraDelta:
    heads: int
    dim: int
    lora: Optional[int]                          # None until the tensors' shapes are known


@dataclass(frozen=True)
class LokedraLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: LokedraRotation


@dataclass(frozen=True)
class LokedraChunked:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    scale: float
    chunk: int


@dataclass(frozen=True)
class LokedraGate:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class LokedraParallel:
    left: LokedraChunked
    right: LokedraGate
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class LokedraExperts:
    experts: int
    top: int
    ff: int
    limit: float


@dataclass(frozen=True)
class LokedraLayer:
    type: str
    mixer: object
    mlp: Optional[LokedraExperts]


@dataclass(frozen=True)
class LokedraLoop:
    start: int
    stop: int
    times: int


def _read_rot(m: dict, where: str, rot_dim: int) -> LokedraRotation:
    rot = _record(m, "rot", where)
    f = _flat(rot, f"{where}rot.")
    dims = _int(f, [f"{where}rot.dims"], rot_dim, lo=2, hi=_MAX_HEAD_DIM)
    if dims != rot_dim or dims % 2:
        raise ConfigError(f"config.json: `{where}rot.dims` = {dims} must equal `{where}rot_dim` = {rot_dim}, an even number")
    base = _float(f, [f"{where}rot.base"], required=True)
    scaling = None
    sc = _record(rot, "scaling", f"{where}rot.", required=False)
    if sc is not None:
        g = _flat(sc, f"{where}rot.scaling.")
        scaling = RopeScaling(*(_float(g, [f"{where}rot.scaling.{k}"], required=True) for k in ("factor", "original", "fast", "slow")))
        if base <= 1.0:
            raise ConfigError(f"config.json: `{where}rot.base` = {base} must be above 1 where `scaling` is given")
    return LokedraRotation(dims, base, scaling)


def _read_mixer(kind: str, m: dict, where: str):
    w = f"{where}mixer."
    if kind == "parallel":
        left, right = _record(m, "left", w), _record(m, "right", w)
        fl, fr = _flat(left, f"{w}left."), _flat(right, f"{w}right.")
        heads = _int(fl, [f"{w}left.heads"], hi=_MAX_HEADS)
        kv_heads = _int(fl, [f"{w}left.kv_heads"], heads, hi=_MAX_HEADS)
        if heads % kv_heads:
            raise ConfigError(f"config.json: `{w}left.heads` = {heads} is not a multiple of `{w}left.kv_heads` = {kv_heads}")
        dim = _int(fl, [f"{w}left.dim"], hi=_MAX_HEAD_DIM)
        vdim = _int(fl, [f"{w}left.vdim"], dim, hi=_MAX_HEAD_DIM)
        if vdim != dim:
            raise ConfigError(f"config.json: `{w}left.vdim` = {vdim} must equal `{w}left.dim` = {dim}: this attention has no value projection, it reads its keys")
        mask = _record(left, "mask", f"{w}left.")
        chunked = LokedraChunked(heads, kv_heads, dim, vdim, _int(fl, [f"{w}left.conv"], hi=16),
                                 _float(fl, [f"{w}left.scale"], required=True),
                                 _int(_flat(mask, f"{w}left.mask."), [f"{w}left.mask.size"], hi=1 << 30))
        gdim = _int(fr, [f"{w}right.dim"], hi=_MAX_HEAD_DIM)
        gate = LokedraGate(_int(fr, [f"{w}right.heads"], hi=_MAX_HEADS), gdim, _int(fr, [f"{w}right.vdim"], gdim, hi=_MAX_HEAD_DIM))
        f = _flat(m, w)
        return LokedraParallel(chunked, gate, _float(f, [f"{w}left_scale"], 1.0, positive=False), _float(f, [f"{w}right_scale"], 1.0, positive=False))
    f = _flat(m, w)
    heads = _int(f, [f"{w}heads"], hi=_MAX_HEADS)
    dim = _int(f, [f"{w}dim"], hi=_MAX_HEAD_DIM)
    if kind == "general_delta":
        return LokedraDelta(heads, dim, _int(f, [f"{w}lora"], hi=_MAX_HIDDEN, required=False))
    rot_dim = _int(f, [f"{w}rot_dim"], lo=2, hi=_MAX_HEAD_DIM)
    return LokedraLatent(heads, dim, rot_dim, _int(f, [f"{w}vdim"], dim, hi=_MAX_HEAD_DIM), _int(f, [f"{w}q_rank"], hi=_MAX_HIDDEN),
                         _int(f, [f"{w}kv_rank"], hi=_MAX_HIDDEN), _float(f, [f"{w}scale"], required=True), _read_rot(m, w, rot_dim))


def _read_mlp(m, where: str) -> Optional[LokedraExperts]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: `{where}mlp` must be an object or null")
    if m.get("kind", "moe") != "moe":
        raise ConfigError(f"config.json: `{where}mlp.kind` = {m.get('kind')!r} is not known (\"moe\")")
    router, expert = _record(m, "router", f"{where}mlp."), _record(m, "expert", f"{where}mlp.")
    fr, fe = _flat(router, f"{where}mlp.router."), _flat(expert, f"{where}mlp.expert.")
    experts = _int(fr, [f"{where}mlp.router.experts"], hi=1 << 16)
    return LokedraExperts(experts, _int(fr, [f"{where}mlp.router.top"], hi=experts), _int(fe, [f"{where}mlp.expert.ff"], hi=_MAX_INTERMEDIATE),
                          _float(fe, [f"{where}mlp.expert.limit"], required=True))


@dataclass(frozen=True)
class LokedraConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    layers: Tuple[LokedraLayer, ...]
    loop: Optional[LokedraLoop]

    architecture = "Lokedra"
    model_type = "lokedra"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json(cls, raw: dict) -> "LokedraConfig":
        if not isinstance(raw, dict):
            raise ConfigError("config.json must hold a JSON object")
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw or len(layers_raw) > _MAX_LAYERS:
            raise ConfigError("config.json: `layers` must be a list of 1 to 4096 layer records")
        layers = []
        for i, rec in enumerate(layers_raw):
            where = f"layers[{i}]."
            if not isinstance(rec, dict):
                raise ConfigError(f"config.json: `layers[{i}]` must be an object")
            kind = rec.get("type")
            if kind not in TYPES:
                raise ConfigError(f"config.json: `{where}type` = {kind!r} is not known {TYPES}")
            layers.append(LokedraLayer(kind, _read_mixer(kind, _record(rec, "mixer", where), where), _read_mlp(rec.get("mlp"), where)))
        loop = None
        loop_raw = _record(raw, "loop", "", required=False)
        if loop_raw is not None:
            flat = _flat(loop_raw, "loop.")
            start = _int(flat, ["loop.start"], lo=0, hi=len(layers))
            stop = _int(flat, ["loop.stop"], lo=start, hi=len(layers))
            loop = LokedraLoop(start, stop, _int(flat, ["loop.times"], lo=1, hi=_MAX_LAYERS))
        norm = _record(raw, "norm", "", required=False) or {}
        embedding = _record(raw, "embedding", "", required=False) or {}
        return cls(
            vocab=_int(raw, ["vocab"], hi=_MAX_VOCAB),
            width=_int(raw, ["width"], hi=_MAX_HIDDEN),
            eps=_float({"norm.eps": norm.get("eps")}, ["norm.eps"], 1e-6),
            embed_scale=_float({"embedding.scale": embedding.get("scale")}, ["embedding.scale"], 1.0, positive=False),
            layers=tuple(layers),
            loop=loop,
        )

    def with_shapes(self, shape_of) -> "LokedraConfig":
        """The configuration with the sizes that only the tensors give: `shape_of(name)` is a tensor's
        shape. The hidden width of a delta layer's decay net is the number of rows of its `w1`."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == "general_delta" and l.mixer.lora is None:
                try:
                    shape = tuple(shape_of(f"l{i}.mix.w1"))
                except KeyError:
                    raise ConfigError(f"the tensor `l{i}.mix.w1`, whose rows size layer {i}'s decay net, is missing") from None
                if len(shape) != 2 or shape[0] < 1:
                    raise ConfigError(f"the tensor `l{i}.mix.w1` has shape {shape}, expected [rows, {self.width}]")
                l = replace(l, mixer=replace(l.mixer, lora=int(shape[0])))
            layers.append(l)
        return replace(self, layers=tuple(layers))

    def to_json(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "general_delta":
                mixer = {"heads": m.heads, "dim": m.dim}
                if m.lora is not None:
                    mixer["lora"] = m.lora
            elif l.type == "latent_attention":
                rot = {"base": m.rot.base, "dims": m.rot.dims}
                if m.rot.scaling is not None:
                    s = m.rot.scaling
                    rot["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                         "scale": m.scale, "rot": rot}
            else:
                a, g = m.left, m.right
                mixer = {"left": {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "conv": a.conv, "scale": a.scale,
                                  "mask": {"size": a.chunk}},
                         "right": {"heads": g.heads, "dim": g.dim, "vdim": g.vdim}, "left_scale": m.left_scale, "right_scale": m.right_scale}
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "router": {"experts": l.mlp.experts, "top": l.mlp.top}, "expert": {"ff": l.mlp.ff, "limit": l.mlp.limit}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
               "embedding": {"scale": self.embed_scale}, "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    # ------------------------------------------------------------------ the model as data
    def runs(self):
        """The layers in the order they run: (layer, which pass of the loop it is in, whether the
        embedding's output is added first): ahead of every pass of the loop but the first."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop <= self.loop.start:
            return [(i, 0, False) for i in range(n)]
        lp = self.loop
        out = [(i, 0, False) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t, i == lp.start and t > 0) for i in range(lp.start, lp.stop)]
        return out + [(i, 0, False) for i in range(lp.stop, n)]

    def to_spec(self) -> ModelSpec:
        w = self.width
        blocks = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.mix", l.mixer
            if l.type == "general_delta":
                if m.lora is None:
                    raise ConfigError(f"layer {i}: the decay net's hidden width is known from the tensors only (`with_shapes`), "
                                      f"or from `layers[{i}].mixer.lora`")
                names = {r: f"{p}.{r}" for r in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")}
                names["a_bias"] = f"{p}.a.b"
                mixer = GeneralDeltaSpec(hidden=w, num_heads=m.heads, head_dim=m.dim, lora=m.lora, eps=self.eps, weights=names,
                                         decay_scale=DECAY_SCALE, unit_eps=UNIT_EPS)
            elif l.type == "latent_attention":
                names = {r: f"{p}.{r}" for r in ("dq", "uq", "dkv", "uk", "uv", "o")}
                names.update(dq_norm=f"{p}.dq.norm", dkv_norm=f"{p}.dkv.norm")
                position = PositionSpec(kind="rope", theta=m.rot.base, rotary_dim=m.rot.dims, pairing="neighbours", scaling=m.rot.scaling)
                mixer = LatentAttentionSpec(
                    hidden=w, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_head_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank,
                    scale=m.scale, eps=self.eps, position=position, weights=names, sink=False, gated=False)
            else:
                a, g = m.left, m.right
                names = {"q": f"{p}.left.q", "k": f"{p}.left.k", "o": f"{p}.left.o", "q_bias": f"{p}.left.q.b", "k_bias": f"{p}.left.k.b",
                         "o_bias": f"{p}.left.o.b", "q_conv": f"{p}.left.q.conv", "k_conv": f"{p}.left.k.conv"}
                left = AttentionSpec(
                    hidden=w, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, scale=a.scale, softcap=None, window=None,
                    position=PositionSpec(kind="none"), weights=names, conv=a.conv, values_are_keys=True, block_mask=a.chunk,
                    unit_sink=True, qk_bias=True, out_bias=True)
                gnames = {r: f"{p}.right.{r}" for r in ("q", "f", "lower", "v", "norm", "o")}
                gnames["f_bias"] = f"{p}.right.f.b"
                right = ForgetGateSpec(hidden=w, num_heads=g.heads, head_dim=g.dim, v_head_dim=g.vdim, eps=self.eps, weights=gnames)
                mixer = ParallelMixerSpec(left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
            ffn = None
            if l.mlp is not None:
                f, e = f"l{i}.mlp", l.mlp
                ffn = MoESpec(
                    hidden=w, experts=e.experts, top=e.top, intermediate=e.ff, activation="clamped_swish",
                    weights={"router": f"{f}.router", "correction": f"{f}.correction", "gate": f"{f}.e{{e}}.gate", "up": f"{f}.e{{e}}.up",
                             "down": f"{f}.e{{e}}.down"},
                    scoring="softmax", renormalize=False, gated=True, limit=e.limit, swish_alpha=SWISH_ALPHA)
            norms = {"pre": NormSpec(width=w, eps=self.eps, offset=1.0, weight=f"l{i}.norm1")}
            blocks.append(BlockSpec(kind="parallel", mixer=mixer, ffn=ffn, norms=norms,
                                    scales=(f"l{i}.ls1", f"l{i}.ls2" if ffn is not None else None), shift=f"l{i}.shift"))
        add = InputAddSpec(hidden=w)
        schedule = tuple(ScheduleEntry(i, i, replica=t, before=add if adds else None) for i, t, adds in self.runs())
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=w,
            embed=EmbedSpec(weight="embed", scale=self.embed_scale, round_scale=False),
            layers=tuple(blocks), schedule=schedule,
            final_norm=NormSpec(width=w, eps=self.eps, offset=1.0, weight="final.norm"),
            head=HeadSpec(weight="embed", softcap=None), max_positions=None,
        )

    # ------------------------------------------------------------------ random weights
    def init_std(self, name: str, shape) -> float:
        """Tables N(0, inner width^-1/2) (the embedding, which is also the head, by the model's width); vectors
        (norm weights, biases, branch weights, shifts) and convolution filters N(0, 0.5); the gates' lower bounds N(0, 0.1)."""
        if name.endswith(".lower"):
            return 0.1                  # a lower bound above 1 would make a gate that grows
        if len(shape) <= 1 or name.endswith(".conv"):
            return 0.5
        return float(shape[-1]) ** -0.5
