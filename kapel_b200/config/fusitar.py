"""Fusitar's configuration: a list of layers, each naming its mixer and its feed-forward.

config.json gives `architecture`, `vocab`, `width`, `embedding.scale`, `norm.eps` and `layers`: a
list of records {type, mixer, mlp}. `type` "attention" is grouped-query attention without a
rotation, with a norm over the whole query and key projections, a sliding window that keeps the
first positions, and a sigmoid output gate; `type` "mlstm" is a matrix memory with exponential
gates. `mlp` is a mixture of experts with a grouped sigmoid router, or null. Every branch's
output is normed before it joins the residual ("postnorm" blocks); the head is the embedding
table. Every size and constant is read from the file; the constants written here are those the
design fixes (the floor of the memory's read-out, two scores a group, the experts' activation).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .gemma2 import ConfigError, _MAX_HEAD_DIM, _MAX_HEADS, _MAX_HIDDEN, _MAX_INTERMEDIATE, _MAX_LAYERS, _MAX_VOCAB, _float, _int
from .spec import (
    AttentionSpec,
    BlockSpec,
    EmbedSpec,
    HeadSpec,
    MLSTMSpec,
    ModelSpec,
    MoESpec,
    NormSpec,
    PositionSpec,
    default_schedule,
)

_MAX_EXPERTS = 1 << 12


def _record(raw, key: str, where: str, required: bool = True) -> Optional[dict]:
    v = raw.get(key)
    if v is None:
        if required:
            raise ConfigError(f"config.json: `{where}{key}` is missing")
        return None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: `{where}{key}` must be an object")
    return v


@dataclass(frozen=True)
class FusitarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int
    keep_first: int


@dataclass(frozen=True)
class FusitarMLSTM:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class FusitarMoE:
    experts: int
    top: int
    groups: int
    keep_groups: int
    ff: int


@dataclass(frozen=True)
class FusitarLayer:
    type: str                                    # "attention" or "mlstm"
    mixer: object
    mlp: Optional[FusitarMoE]


def _read_mixer(kind: str, m: dict, where: str):
    named = lambda k: [f"{where}mixer.{k}"]
    flat = {f"{where}mixer.{k}": v for k, v in m.items()}
    heads = _int(flat, named("heads"), hi=_MAX_HEADS)
    dim = _int(flat, named("dim"), hi=_MAX_HEAD_DIM)
    vdim = _int(flat, named("vdim"), dim, hi=_MAX_HEAD_DIM)
    if kind == "mlstm":
        return FusitarMLSTM(heads, dim, vdim, _float(flat, named("gate_cap"), required=True))
    kv_heads = _int(flat, named("kv_heads"), heads, hi=_MAX_HEADS)
    if heads % kv_heads:
        raise ConfigError(f"config.json: `{where}mixer.heads` = {heads} is not a multiple of `kv_heads` = {kv_heads}")
    mask = _record(m, "mask", f"{where}mixer.")
    mflat = {f"{where}mixer.mask.{k}": v for k, v in mask.items()}
    return FusitarAttention(
        heads, kv_heads, dim, vdim, _float(flat, named("scale"), required=True),
        window=_int(mflat, [f"{where}mixer.mask.size"]),
        keep_first=_int(mflat, [f"{where}mixer.mask.keep_first"], 0, lo=0),
    )


def _read_mlp(m: Optional[dict], where: str) -> Optional[FusitarMoE]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: `{where}mlp` must be an object or null")
    if m.get("kind", "moe") != "moe":
        raise ConfigError(f"config.json: `{where}mlp.kind` = {m.get('kind')!r} is not known (\"moe\")")
    router = _record(m, "router", f"{where}mlp.")
    expert = _record(m, "expert", f"{where}mlp.")
    groups = router.get("groups") or {}
    if not isinstance(groups, dict):
        raise ConfigError(f"config.json: `{where}mlp.router.groups` must be an object")
    flat = {f"{where}mlp.router.{k}": v for k, v in router.items()}
    flat.update({f"{where}mlp.router.groups.{k}": v for k, v in groups.items()})
    flat.update({f"{where}mlp.expert.{k}": v for k, v in expert.items()})
    experts = _int(flat, [f"{where}mlp.router.experts"], hi=_MAX_EXPERTS)
    top = _int(flat, [f"{where}mlp.router.top"], hi=experts)
    count = _int(flat, [f"{where}mlp.router.groups.count"], 1, hi=experts)
    keep = _int(flat, [f"{where}mlp.router.groups.keep"], count, hi=count)
    if experts % count:
        raise ConfigError(f"config.json: `{where}mlp.router.experts` = {experts} does not split into {count} equal groups")
    if keep * (experts // count) < top:
        raise ConfigError(f"config.json: `{where}mlp.router`: {keep} groups of {experts // count} experts cannot give {top} experts")
    return FusitarMoE(experts, top, count, keep, _int(flat, [f"{where}mlp.expert.ff"], hi=_MAX_INTERMEDIATE))


@dataclass(frozen=True)
class FusitarConfig:
    vocab: int
    width: int
    embedding_scale: float
    eps: float
    layers: Tuple[FusitarLayer, ...]

    architecture = "Fusitar"
    model_type = "fusitar"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json(cls, raw: dict) -> "FusitarConfig":
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
            if kind not in ("attention", "mlstm"):
                raise ConfigError(f"config.json: `{where}type` = {kind!r} is not known (\"attention\", \"mlstm\")")
            layers.append(FusitarLayer(kind, _read_mixer(kind, _record(rec, "mixer", where), where), _read_mlp(rec.get("mlp"), where)))
        emb = _record(raw, "embedding", "", required=False) or {}
        norm = _record(raw, "norm", "", required=False) or {}
        return cls(
            vocab=_int(raw, ["vocab"], hi=_MAX_VOCAB),
            width=_int(raw, ["width"], hi=_MAX_HIDDEN),
            embedding_scale=_float({"embedding.scale": emb.get("scale")}, ["embedding.scale"], 1.0),
            eps=_float({"norm.eps": norm.get("eps")}, ["norm.eps"], 1e-6),
            layers=tuple(layers),
        )

    def to_json(self) -> dict:
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale,
                         "mask": {"size": m.window, "keep_first": m.keep_first}}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "gate_cap": m.gate_cap}
            mlp = None
            if l.mlp is not None:
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                       "router": {"experts": l.mlp.experts, "top": l.mlp.top, "groups": {"count": l.mlp.groups, "keep": l.mlp.keep_groups}}}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps}, "layers": layers}

    # ------------------------------------------------------------------ the model as data
    def to_spec(self) -> ModelSpec:
        w = self.width
        blocks = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.mix", l.mixer
            if l.type == "attention":
                mixer = AttentionSpec(
                    hidden=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale, softcap=None,
                    window=m.window, position=PositionSpec(kind="none"),
                    weights={r: f"{p}.{r}" for r in ("q", "k", "v", "g", "o")},
                    keep_first=m.keep_first, v_head_dim=m.vdim, gated=True,
                    q_norm=NormSpec(width=m.heads * m.dim, eps=self.eps, offset=0.0, weight=f"{p}.q.norm"),
                    k_norm=NormSpec(width=m.kv_heads * m.dim, eps=self.eps, offset=0.0, weight=f"{p}.k.norm"),
                )
            else:
                names = {r: f"{p}.{r}" for r in ("q", "k", "v", "g", "o", "i", "f", "norm")}
                names.update(i_bias=f"{p}.i.b", f_bias=f"{p}.f.b")
                mixer = MLSTMSpec(hidden=w, num_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, gate_cap=m.gate_cap,
                                  eps=self.eps, weights=names, floor=1e-6)
            ffn = None
            norms = {"post_mixer": NormSpec(width=w, eps=self.eps, offset=0.0, weight=f"l{i}.norm1")}
            if l.mlp is not None:
                f = f"l{i}.mlp"
                ffn = MoESpec(hidden=w, experts=l.mlp.experts, top=l.mlp.top, intermediate=l.mlp.ff, activation="relu2",
                              weights={"router": f"{f}.router", "correction": f"{f}.correction",
                                       "up": f + ".e{e}.up", "down": f + ".e{e}.down"},
                              groups=l.mlp.groups, keep_groups=l.mlp.keep_groups, group_top=2, scoring="sigmoid", renormalize=False)
                norms["post_ffn"] = NormSpec(width=w, eps=self.eps, offset=0.0, weight=f"l{i}.norm2")
            blocks.append(BlockSpec(kind="postnorm", mixer=mixer, ffn=ffn, norms=norms))
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=w,
            embed=EmbedSpec(weight="embed", scale=self.embedding_scale, round_scale=False),
            layers=tuple(blocks), schedule=default_schedule(len(blocks)),
            final_norm=NormSpec(width=w, eps=self.eps, offset=0.0, weight="final.norm"),
            head=HeadSpec(weight="embed", softcap=None), max_positions=None,
        )

    # ------------------------------------------------------------------ random weights
    def init_std(self, name: str, shape) -> float:
        """Norm weights and the router's correction around zero would silence a branch: vectors get
        N(0, 0.5) (biases, corrections, norm weights alike), tables N(0, width^-1/2)."""
        if len(shape) == 1:
            return 0.5
        return float(shape[-1]) ** -0.5
