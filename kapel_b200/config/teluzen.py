"""Teluzen's configuration: a list of layers, each naming its mixer's sizes and its feed-forward.

config.json gives `architecture`, `vocab`, `width`, `max_positions`, `norm.eps` and `layers`: a list of
records {type, mixer, mlp}. The one `type` is "attention": grouped-query attention with biases on q, k
and v, an RMS norm over the whole query and key projections, a rotation of neighbouring components of
the first `rot.dims` of every head (frequencies stretched by `rot.scaling`), a number a head on the
scores, a sliding window with one pooled key and value for every block of `mask.pool` positions below
it, the heads' softmax weights mixed by a matrix, and (with `v_mix`) values mixed with those of the
first such layer. `mlp` is null, a dense feed-forward (down(relu(up h)^2)) or a mixture of gated silu
experts weighted by the softmax over the chosen logits, with a shared expert. A learned position
vector is added to the embedding; every sublayer has a norm before and after it; the head is a table
of its own behind a final norm. Every size and constant is read from the file; what is written here
is what the design fixes (the activations, the pairing, the scaling's rule).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .fusitar import _MAX_EXPERTS, _record
from .gemma2 import ConfigError, _MAX_HEAD_DIM, _MAX_HEADS, _MAX_HIDDEN, _MAX_INTERMEDIATE, _MAX_LAYERS, _MAX_VOCAB, _float, _int
from .spec import (
    AttentionSpec,
    BlockSpec,
    EmbedSpec,
    GatedMLPSpec,
    HeadSpec,
    MLPSpec,
    ModelSpec,
    MoESpec,
    NormSpec,
    PositionSpec,
    RopeScaling,
    default_schedule,
)

_MAX_POSITIONS = 1 << 22


@dataclass(frozen=True)
class TeluzenRotation:
    dims: int
    base: float
    scaling: Optional[RopeScaling]


@dataclass(frozen=True)
class TeluzenAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    pool: int
    rot: Optional[TeluzenRotation]
    v_mix: bool


@dataclass(frozen=True)
class TeluzenMLP:
    kind: str                                    # "dense" or "moe"
    ff: int                                      # the dense layer's, or an expert's
    experts: int = 0
    top: int = 0
    shared_ff: int = 0                           # 0: no shared expert


@dataclass(frozen=True)
class TeluzenLayer:
    type: str
    mixer: TeluzenAttention
    mlp: Optional[TeluzenMLP]


def _flat(rec: dict, where: str) -> dict:
    return {f"{where}{k}": v for k, v in rec.items()}


def _read_rotation(m: dict, where: str, dim: int) -> Optional[TeluzenRotation]:
    rot = _record(m, "rot", where, required=False)
    if rot is None:
        return None
    flat = _flat(rot, f"{where}rot.")
    dims = _int(flat, [f"{where}rot.dims"], hi=dim)
    if dims % 2:
        raise ConfigError(f"config.json: `{where}rot.dims` = {dims} must be even (pairs are rotated)")
    base = _float(flat, [f"{where}rot.base"], required=True)
    scaling = None
    sc = _record(rot, "scaling", f"{where}rot.", required=False)
    if sc is not None:
        f = _flat(sc, f"{where}rot.scaling.")
        scaling = RopeScaling(*(_float(f, [f"{where}rot.scaling.{k}"], required=True) for k in ("factor", "original", "fast", "slow")))
        if base <= 1.0:
            raise ConfigError(f"config.json: `{where}rot.base` = {base} must be above 1 where `scaling` is given")
    return TeluzenRotation(dims, base, scaling)


def _read_mixer(m: dict, where: str) -> TeluzenAttention:
    where = f"{where}mixer."
    flat = _flat(m, where)
    heads = _int(flat, [f"{where}heads"], hi=_MAX_HEADS)
    kv_heads = _int(flat, [f"{where}kv_heads"], heads, hi=_MAX_HEADS)
    if heads % kv_heads:
        raise ConfigError(f"config.json: `{where}heads` = {heads} is not a multiple of `kv_heads` = {kv_heads}")
    dim = _int(flat, [f"{where}dim"], hi=_MAX_HEAD_DIM)
    vdim = _int(flat, [f"{where}vdim"], dim, hi=_MAX_HEAD_DIM)
    mask = _record(m, "mask", where)
    mflat = _flat(mask, f"{where}mask.")
    v_mix = m.get("v_mix", False)
    if not isinstance(v_mix, bool):
        raise ConfigError(f"config.json: `{where}v_mix` must be true or false")
    return TeluzenAttention(
        heads, kv_heads, dim, vdim, _float(flat, [f"{where}scale"], required=True),
        window=_int(mflat, [f"{where}mask.size"]), pool=_int(mflat, [f"{where}mask.pool"], 0, lo=0),
        rot=_read_rotation(m, where, dim), v_mix=v_mix)


def _read_mlp(m, where: str) -> Optional[TeluzenMLP]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: `{where}mlp` must be an object or null")
    where = f"{where}mlp."
    kind = m.get("kind")
    if kind == "dense":
        return TeluzenMLP("dense", _int(_flat(m, where), [f"{where}ff"], hi=_MAX_INTERMEDIATE))
    if kind != "moe":
        raise ConfigError(f"config.json: `{where}kind` = {kind!r} is not known (\"dense\", \"moe\")")
    router = _flat(_record(m, "router", where), f"{where}router.")
    expert = _flat(_record(m, "expert", where), f"{where}expert.")
    shared = _record(m, "shared", where, required=False)
    experts = _int(router, [f"{where}router.experts"], hi=_MAX_EXPERTS)
    return TeluzenMLP(
        "moe", _int(expert, [f"{where}expert.ff"], hi=_MAX_INTERMEDIATE), experts=experts,
        top=_int(router, [f"{where}router.top"], hi=experts),
        shared_ff=_int(_flat(shared, f"{where}shared."), [f"{where}shared.ff"], hi=_MAX_INTERMEDIATE) if shared is not None else 0)


@dataclass(frozen=True)
class TeluzenConfig:
    vocab: int
    width: int
    max_positions: int
    eps: float
    layers: Tuple[TeluzenLayer, ...]

    architecture = "Teluzen"
    model_type = "teluzen"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json(cls, raw: dict) -> "TeluzenConfig":
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
            if rec.get("type") != "attention":
                raise ConfigError(f"config.json: `{where}type` = {rec.get('type')!r} is not known (\"attention\")")
            layers.append(TeluzenLayer("attention", _read_mixer(_record(rec, "mixer", where), where), _read_mlp(rec.get("mlp"), where)))
        mixing = [(l.mixer.kv_heads, l.mixer.vdim) for l in layers if l.mixer.v_mix]
        if len(set(mixing)) > 1:
            raise ConfigError(f"config.json: the layers with `v_mix` have values of different shapes {sorted(set(mixing))} (kv_heads, vdim)")
        norm = _record(raw, "norm", "", required=False) or {}
        max_positions = _int(raw, ["max_positions"], hi=_MAX_POSITIONS)
        return cls(
            vocab=_int(raw, ["vocab"], hi=_MAX_VOCAB),
            width=_int(raw, ["width"], hi=_MAX_HIDDEN),
            max_positions=max_positions,
            eps=_float({"norm.eps": norm.get("eps")}, ["norm.eps"], 1e-6),
            layers=tuple(layers),
        )

    def to_json(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                     "mask": {"size": m.window, "pool": m.pool}, "v_mix": m.v_mix}
            if m.rot is not None:
                mixer["rot"] = {"dims": m.rot.dims, "base": m.rot.base}
                if m.rot.scaling is not None:
                    s = m.rot.scaling
                    mixer["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            mlp = None
            if l.mlp is not None and l.mlp.kind == "dense":
                mlp = {"kind": "dense", "ff": l.mlp.ff}
            elif l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff}, "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
                if l.mlp.shared_ff:
                    mlp["shared"] = {"ff": l.mlp.shared_ff}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "max_positions": self.max_positions,
                "norm": {"eps": self.eps}, "layers": layers}

    # ------------------------------------------------------------------ the model as data
    def _ffn(self, i: int, mlp: Optional[TeluzenMLP]):
        w, f = self.width, f"l{i}.mlp"
        if mlp is None:
            return None
        if mlp.kind == "dense":
            return MLPSpec(hidden=w, intermediate=mlp.ff, activation="relu2", weights={"up": f"{f}.up", "down": f"{f}.down"})
        shared = None
        if mlp.shared_ff:
            shared = GatedMLPSpec(hidden=w, intermediate=mlp.shared_ff, activation="silu",
                                  weights={r: f"{f}.shared.{r}" for r in ("gate", "up", "down")})
        return MoESpec(hidden=w, experts=mlp.experts, top=mlp.top, intermediate=mlp.ff, activation="silu",
                       weights={"router": f"{f}.router", "gate": f + ".e{e}.gate", "up": f + ".e{e}.up", "down": f + ".e{e}.down"},
                       scoring="softmax_chosen", gated=True, shared=shared)

    def to_spec(self) -> ModelSpec:
        w = self.width
        norm = lambda name: NormSpec(width=w, eps=self.eps, offset=0.0, weight=name)
        blocks = []
        source_seen = False
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.mix", l.mixer
            position = PositionSpec(kind="none")
            if m.rot is not None:
                position = PositionSpec(kind="rope", theta=m.rot.base, rotary_dim=m.rot.dims, pairing="neighbours", scaling=m.rot.scaling)
            names = {r: f"{p}.{r}" for r in ("q", "k", "v", "o", "talk", "temp", "vmix")}
            names.update(q_bias=f"{p}.q.b", k_bias=f"{p}.k.b", v_bias=f"{p}.v.b")
            value_mix = None
            if m.v_mix:
                value_mix = "mix" if source_seen else "source"
                source_seen = True
            mixer = AttentionSpec(
                hidden=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale, softcap=None,
                window=m.window, position=position, weights=names, v_head_dim=m.vdim,
                q_norm=NormSpec(width=m.heads * m.dim, eps=self.eps, offset=0.0, weight=f"{p}.q.norm"),
                k_norm=NormSpec(width=m.kv_heads * m.dim, eps=self.eps, offset=0.0, weight=f"{p}.k.norm"),
                bias=True, pool=m.pool, pool_blocks=(self.max_positions // m.pool) if m.pool else 0,
                head_temp=True, talk=True, value_mix=value_mix,
            )
            norms = {"pre_mixer": norm(f"l{i}.norm1"), "post_mixer": norm(f"l{i}.norm1b")}
            if l.mlp is not None:
                norms.update(pre_ffn=norm(f"l{i}.norm2"), post_ffn=norm(f"l{i}.norm2b"))
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, ffn=self._ffn(i, l.mlp), norms=norms))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=w,
            embed=EmbedSpec(weight="embed", scale=1.0, round_scale=False, positions="pos", max_positions=self.max_positions),
            layers=tuple(blocks), schedule=default_schedule(len(blocks)),
            final_norm=norm("final.norm"), head=HeadSpec(weight="head", softcap=None), max_positions=self.max_positions,
        )

    # ------------------------------------------------------------------ random weights
    def init_std(self, name: str, shape) -> float:
        """Tables N(0, in^-1/2); biases, norm weights, head temperatures and the values' weight N(0, 0.5)
        (a norm weight around zero would silence a branch); the heads' mix N(0, heads^-1/2)."""
        if len(shape) <= 1:
            return 0.5
        return float(shape[-1]) ** -0.5
