"""Kofutar's configuration: a list of layers, each naming its mixer and its feed-forward, and a
loop that runs a run of layers several times.

config.json gives `architecture`, `vocab`, `width`, `norm.eps`, `layers` and `loop`. A layer record
is {type, mixer, mlp}. `type` "attention" is grouped-query attention with an RMS norm over every
head's query and key and a rotation of the first `rot.dims` components (`rot.base`, optionally
`rot.scaling.factor`, which divides every frequency); "latent_attention" is attention whose queries
and whose keys and values come through low-rank latents, with a sink in the softmax's denominator
and a sigmoid gate on the heads' outputs; "delta" is the gated delta rule behind short convolutions.
`mlp` is a dense gated feed-forward {kind: "dense", ff} or null. Every branch is normed on its way in
and on its way out by a layer norm with a weight and no bias ("sandwich" blocks). `loop`
{start, stop, times}: the layers start .. stop-1 run `times` times in a row with the same weights
and a cache of their own each time; ahead of each such pass the stream and the embedding's output go
through the matrix `loop.in` side by side. The head is a table of its own. Every size and constant is
read from the file; the constants written here are those the design fixes (the unit vectors' 1e-6,
the feed-forward's activation).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .gemma2 import ConfigError, _MAX_HEAD_DIM, _MAX_HEADS, _MAX_HIDDEN, _MAX_INTERMEDIATE, _MAX_LAYERS, _MAX_VOCAB, _float, _int
from .spec import (
    AttentionSpec,
    BlockSpec,
    DeltaSpec,
    EmbedSpec,
    GatedMLPSpec,
    HeadSpec,
    InputMixSpec,
    LatentAttentionSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
)

TYPES = ("attention", "latent_attention", "delta")


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
class KofutarRot:
    base: float
    dims: int
    factor: float = 1.0                          # every frequency is divided by it


@dataclass(frozen=True)
class KofutarAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot: Optional[KofutarRot]


@dataclass(frozen=True)
class KofutarLatent:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot: KofutarRot


@dataclass(frozen=True)
class KofutarDelta:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int


@dataclass(frozen=True)
class KofutarLayer:
    type: str
    mixer: object
    ff: Optional[int]                            # the dense feed-forward's inner width, or None for no feed-forward


@dataclass(frozen=True)
class KofutarLoop:
    start: int
    stop: int
    times: int


def _read_rot(m: dict, where: str, dims_default: Optional[int], required: bool) -> Optional[KofutarRot]:
    rot = _record(m, "rot", where, required=required)
    if rot is None:
        return None
    flat = {f"{where}rot.{k}": v for k, v in rot.items()}
    scaling = rot.get("scaling")
    if scaling is not None and not isinstance(scaling, dict):
        raise ConfigError(f"config.json: `{where}rot.scaling` must be an object")
    flat.update({f"{where}rot.scaling.{k}": v for k, v in (scaling or {}).items()})
    dims = _int(flat, [f"{where}rot.dims"], dims_default, lo=2, hi=_MAX_HEAD_DIM)
    if dims % 2:
        raise ConfigError(f"config.json: `{where}rot.dims` = {dims} must be even")
    return KofutarRot(_float(flat, [f"{where}rot.base"], required=True), dims, _float(flat, [f"{where}rot.scaling.factor"], 1.0))


def _read_mixer(kind: str, m: dict, where: str):
    w = f"{where}mixer."
    flat = {f"{w}{k}": v for k, v in m.items()}
    heads = _int(flat, [f"{w}heads"], hi=_MAX_HEADS)
    dim = _int(flat, [f"{w}dim"], hi=_MAX_HEAD_DIM)
    vdim = _int(flat, [f"{w}vdim"], dim, hi=_MAX_HEAD_DIM)
    if kind == "latent_attention":
        rot_dim = _int(flat, [f"{w}rot_dim"], lo=2, hi=_MAX_HEAD_DIM)
        rot = _read_rot(m, w, rot_dim, required=True)
        if rot.dims != rot_dim or rot_dim % 2:
            raise ConfigError(f"config.json: `{w}rot.dims` = {rot.dims} must equal `{w}rot_dim` = {rot_dim}, an even number")
        return KofutarLatent(heads, dim, rot_dim, vdim, _int(flat, [f"{w}q_rank"], hi=_MAX_HIDDEN), _int(flat, [f"{w}kv_rank"], hi=_MAX_HIDDEN),
                             _float(flat, [f"{w}scale"], required=True), rot)
    kv_heads = _int(flat, [f"{w}kv_heads"], heads, hi=_MAX_HEADS)
    if heads % kv_heads:
        raise ConfigError(f"config.json: `{w}heads` = {heads} is not a multiple of `{w}kv_heads` = {kv_heads}")
    if kind == "delta":
        return KofutarDelta(heads, kv_heads, dim, vdim, _int(flat, [f"{w}conv"], hi=8))
    rot = _read_rot(m, w, None, required=False)
    if rot is not None and rot.dims > dim:
        raise ConfigError(f"config.json: `{w}rot.dims` = {rot.dims} is more than `{w}dim` = {dim}")
    return KofutarAttention(heads, kv_heads, dim, vdim, _float(flat, [f"{w}scale"], required=True), rot)


def _read_mlp(m, where: str) -> Optional[int]:
    if m is None:
        return None
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: `{where}mlp` must be an object or null")
    if m.get("kind", "dense") != "dense":
        raise ConfigError(f"config.json: `{where}mlp.kind` = {m.get('kind')!r} is not known (\"dense\")")
    return _int({f"{where}mlp.ff": m.get("ff")}, [f"{where}mlp.ff"], hi=_MAX_INTERMEDIATE)


@dataclass(frozen=True)
class KofutarConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[KofutarLayer, ...]
    loop: Optional[KofutarLoop]

    architecture = "Kofutar"
    model_type = "kofutar"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_json(cls, raw: dict) -> "KofutarConfig":
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
            layers.append(KofutarLayer(kind, _read_mixer(kind, _record(rec, "mixer", where), where), _read_mlp(rec.get("mlp"), where)))
        loop = None
        loop_raw = _record(raw, "loop", "", required=False)
        if loop_raw is not None:
            flat = {f"loop.{k}": v for k, v in loop_raw.items()}
            start = _int(flat, ["loop.start"], lo=0, hi=len(layers))
            stop = _int(flat, ["loop.stop"], lo=start, hi=len(layers))
            loop = KofutarLoop(start, stop, _int(flat, ["loop.times"], lo=1, hi=_MAX_LAYERS))
        norm = _record(raw, "norm", "", required=False) or {}
        return cls(
            vocab=_int(raw, ["vocab"], hi=_MAX_VOCAB),
            width=_int(raw, ["width"], hi=_MAX_HIDDEN),
            eps=_float({"norm.eps": norm.get("eps")}, ["norm.eps"], 1e-5),
            layers=tuple(layers),
            loop=loop,
        )

    def to_json(self) -> dict:
        def rot_json(r: KofutarRot) -> dict:
            out = {"base": r.base, "dims": r.dims}
            if r.factor != 1.0:
                out["scaling"] = {"factor": r.factor}
            return out

        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "attention":
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.rot is not None:
                    mixer["rot"] = rot_json(m.rot)
            elif l.type == "latent_attention":
                mixer = {"heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "q_rank": m.q_rank, "kv_rank": m.kv_rank,
                         "scale": m.scale, "rot": rot_json(m.rot)}
            else:
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "conv": m.conv}
            layers.append({"type": l.type, "mixer": mixer, "mlp": None if l.ff is None else {"kind": "dense", "ff": l.ff}})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps}, "layers": layers}
        if self.loop is not None:
            out["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return out

    # ------------------------------------------------------------------ the model as data
    def runs(self):
        """The layers in the order they run: (layer, which pass of the loop it is in, whether it opens a pass)."""
        n = len(self.layers)
        if self.loop is None or self.loop.stop <= self.loop.start:
            return [(i, 0, False) for i in range(n)]
        lp = self.loop
        out = [(i, 0, False) for i in range(lp.start)]
        for t in range(lp.times):
            out += [(i, t, i == lp.start) for i in range(lp.start, lp.stop)]
        return out + [(i, 0, False) for i in range(lp.stop, n)]

    def to_spec(self) -> ModelSpec:
        w = self.width

        def norm(name: str) -> NormSpec:
            return NormSpec(width=w, eps=self.eps, offset=0.0, weight=name, kind="layer")

        def position(r: Optional[KofutarRot]) -> PositionSpec:
            if r is None:
                return PositionSpec(kind="none")
            return PositionSpec(kind="rope", theta=r.base, rotary_dim=r.dims, pairing="half", divisor=r.factor)

        blocks = []
        for i, l in enumerate(self.layers):
            p, m = f"l{i}.mix", l.mixer
            if l.type == "attention":
                mixer = AttentionSpec(
                    hidden=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, scale=m.scale, softcap=None, window=None,
                    position=position(m.rot), weights={r: f"{p}.{r}" for r in ("q", "k", "v", "o")}, v_head_dim=m.vdim,
                    q_head_norm=NormSpec(width=m.dim, eps=self.eps, offset=0.0, weight=f"{p}.q.norm"),
                    k_head_norm=NormSpec(width=m.dim, eps=self.eps, offset=0.0, weight=f"{p}.k.norm"),
                )
            elif l.type == "latent_attention":
                names = {r: f"{p}.{r}" for r in ("dq", "uq", "dkv", "uk", "uv", "sink", "g", "o")}
                names.update(dq_norm=f"{p}.dq.norm", dkv_norm=f"{p}.dkv.norm")
                mixer = LatentAttentionSpec(
                    hidden=w, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, v_head_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank,
                    scale=m.scale, eps=self.eps, position=position(m.rot), weights=names, sink=True, gated=True)
            else:
                names = {r: f"{p}.{r}" for r in ("q", "k", "v", "b", "a", "A_log", "dt_bias", "norm", "g", "o")}
                names.update(q_conv=f"{p}.q.conv", k_conv=f"{p}.k.conv", v_conv=f"{p}.v.conv")
                mixer = DeltaSpec(hidden=w, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim, conv=m.conv,
                                  eps=self.eps, weights=names, unit_eps=1e-6)
            norms = {"pre_mixer": norm(f"l{i}.norm1"), "post_mixer": norm(f"l{i}.norm1b")}
            ffn = None
            if l.ff is not None:
                f = f"l{i}.mlp"
                ffn = GatedMLPSpec(hidden=w, intermediate=l.ff, activation="gelu_tanh", weights={r: f"{f}.{r}" for r in ("gate", "up", "down")})
                norms.update(pre_ffn=norm(f"l{i}.norm2"), post_ffn=norm(f"l{i}.norm2b"))
            blocks.append(BlockSpec(kind="sandwich", mixer=mixer, ffn=ffn, norms=norms))
        mix = InputMixSpec(hidden=w, weight="loop.in")
        schedule = tuple(ScheduleEntry(i, i, replica=t, before=mix if opens else None) for i, t, opens in self.runs())
        return ModelSpec(
            architecture=self.architecture, vocab_size=self.vocab, hidden_size=w,
            embed=EmbedSpec(weight="embed", scale=1.0, round_scale=False),
            layers=tuple(blocks), schedule=schedule,
            final_norm=norm("final.norm"), head=HeadSpec(weight="head", softcap=None), max_positions=None,
        )

    # ------------------------------------------------------------------ random weights
    def init_std(self, name: str, shape) -> float:
        """Vectors (norm weights, sinks, decay rates, biases) N(0, 0.5); convolution filters N(0, 0.5);
        tables N(0, inner width^-1/2)."""
        if len(shape) == 1 or name.endswith(".conv"):
            return 0.5
        return float(shape[-1]) ** -0.5
