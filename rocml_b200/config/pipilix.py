"""Typed configuration of the Pipilix decoder, read from config.json.

A Pipilix model is an embedding (rows times a multiplier, plus a sinusoid position vector), a
list of layers that each name their mixer and feed-forward with their own sizes, an optional
span of layers that runs several times with the same weights (each pass with a cache of its
own), a final RMSNorm and a head whose result is multiplied by a constant.  Every layer is
norm -> sublayer -> norm -> add, twice.

Keys read (every size and every constant that differs between models comes from here)::

    architecture        "Pipilix"
    vocab, width
    embedding.scale
    norm.eps
    layers[i].type      the mixer: "latent_attention"
    layers[i].mixer     heads, dim, vdim, kv_rank, scale, mask.size
    layers[i].mlp       null | {kind: "dense", ff} | {kind: "moe", expert: {ff, limit}, router: {experts, top}}
    loop                optional {start, stop, times}
    logit_scale

Tensor names: ``embed``, ``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.<role>``,
``l<i>.mlp.<role>`` or ``l<i>.mlp.e<k>.<role>``, ``final.norm``, ``head``; no ``.weight`` suffix.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry

ARCHITECTURE = "Pipilix"

# Constants the design fixes.
POSITION_BASE = 10000.0        # the sinusoid position vector's base
EXPERT_SWISH_ALPHA = 1.702     # an expert's gate is g * sigmoid(alpha * g)
MAX_CONTEXT = 1 << 20          # the design names no longest sequence: positions are plain integers

_MIXERS = ("latent_attention",)
_FF_KINDS = ("dense", "moe")


def _get(d: Mapping[str, Any], key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json lacks {where}{key!r}")
    return d[key]


def _int(d, key, where, least=1) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {where}{key!r} must be an integer, found {v!r}")
    if v < least:
        raise ConfigError(f"config.json: {where}{key!r} must be at least {least}, found {v}")
    return v


def _num(d, key, where) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"config.json: {where}{key!r} must be a number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float
    window: int

    @staticmethod
    def from_dict(d, where) -> "LatentAttentionConfig":
        mask = _get(d, "mask", where)
        return LatentAttentionConfig(
            heads=_int(d, "heads", where), dim=_int(d, "dim", where), vdim=_int(d, "vdim", where),
            kv_rank=_int(d, "kv_rank", where), scale=_num(d, "scale", where),
            window=_int(mask, "size", where + "mask."))

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale,
                "mask": {"size": self.window}}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                      # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0
    limit: float = 0.0

    @staticmethod
    def from_dict(d, where) -> "FeedForwardConfig":
        kind = _get(d, "kind", where)
        if kind not in _FF_KINDS:
            raise ConfigError(f"config.json: {where}kind {kind!r} is unknown (known: {', '.join(_FF_KINDS)})")
        if kind == "dense":
            return FeedForwardConfig("dense", _int(d, "ff", where))
        ex, ro = _get(d, "expert", where), _get(d, "router", where)
        cfg = FeedForwardConfig("moe", _int(ex, "ff", where + "expert."), _int(ro, "experts", where + "router."),
                                _int(ro, "top", where + "router."), _num(ex, "limit", where + "expert."))
        if cfg.top > cfg.experts:
            raise ConfigError(f"config.json: {where}router.top {cfg.top} exceeds router.experts {cfg.experts}")
        if not cfg.limit > 0:
            raise ConfigError(f"config.json: {where}expert.limit must be positive, found {cfg.limit}")
        return cfg

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
                "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class PipilixLayer:
    mixer_type: str
    mixer: LatentAttentionConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class PipilixConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[PipilixLayer, ...]
    logit_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None        # (start, stop, times)

    def __post_init__(self):
        if not self.layers:
            raise ConfigError("config.json: 'layers' is empty")
        if not self.norm_eps > 0:
            raise ConfigError(f"config.json: norm.eps must be positive, found {self.norm_eps}")
        if self.loop is not None:
            a, b, n = self.loop
            if not (0 <= a < b <= len(self.layers)) or n < 1:
                raise ConfigError(f"config.json: loop {{start: {a}, stop: {b}, times: {n}}} does not fit "
                                  f"{len(self.layers)} layers")

    @staticmethod
    def from_dict(d: Mapping[str, Any]) -> "PipilixConfig":
        layers = _get(d, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("config.json: 'layers' must be a list")
        out = []
        for i, L in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is unknown (known: {', '.join(_MIXERS)})")
            mixer = LatentAttentionConfig.from_dict(_get(L, "mixer", where), where + "mixer.")
            mlp = L.get("mlp")
            out.append(PipilixLayer(kind, mixer, None if mlp is None else FeedForwardConfig.from_dict(mlp, where + "mlp.")))
        loop = d.get("loop")
        if loop is not None:
            loop = (_int(loop, "start", "loop.", 0), _int(loop, "stop", "loop."), _int(loop, "times", "loop."))
        return PipilixConfig(
            vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
            embedding_scale=_num(_get(d, "embedding", ""), "scale", "embedding."),
            norm_eps=_num(_get(d, "norm", ""), "eps", "norm."), layers=tuple(out),
            logit_scale=_num(d, "logit_scale", "") if d.get("logit_scale") is not None else 1.0, loop=loop)

    def to_dict(self) -> dict:
        d = {
            "architecture": ARCHITECTURE,
            "embedding": {"scale": self.embedding_scale},
            "layers": [{"type": L.mixer_type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers],
            "logit_scale": self.logit_scale,
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    # ---- the architecture, spelled as parts ------------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.norm_eps)
        layers = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            mixer = MixerSpec.make(
                "latent_attention", n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, kv_rank=m.kv_rank,
                latent_norm_eps=self.norm_eps, window=m.window, scale=m.scale, gated=True,
                names={"q": "q", "down": "dkv", "latent_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "o": "o"})
            ff = None
            if L.mlp is not None and L.mlp.kind == "dense":
                ff = FeedForwardSpec.make("gated_mlp", intermediate=L.mlp.ff, activation="silu", bias=False,
                                          names={"gate": "gate", "up": "up", "down": "down"})
            elif L.mlp is not None:
                ff = FeedForwardSpec.make(
                    "routed_mlp", experts=L.mlp.experts, top=L.mlp.top, intermediate=L.mlp.ff,
                    activation="clamped_swish", limit=L.mlp.limit, alpha=EXPERT_SWISH_ALPHA, score="sigmoid",
                    choice_bias=True, renormalize=False,
                    names={"router": "router", "choice_bias": "correction", "expert": "e{e}.", "gate": "gate", "up": "up",
                           "down": "down"})
            layers.append(LayerSpec(
                prefix=f"l{i}", mixer=mixer, feed_forward=ff, mixer_norm=norm, ff_norm=norm, arrangement="sandwich_norm",
                mixer_norm_name="norm1", mixer_name="mix.", ff_norm_name="norm2", ff_name="mlp.",
                mixer_post_norm=norm, ff_post_norm=norm, mixer_post_norm_name="norm1b", ff_post_norm_name="norm2b"))
        n = len(self.layers)
        if self.loop is None:
            schedule = [ScheduleEntry(i) for i in range(n)]
        else:
            a, b, times = self.loop
            schedule = [ScheduleEntry(i) for i in range(a)]
            for t in range(times):
                for i in range(a, b):
                    first = i == a
                    schedule.append(ScheduleEntry(i, add_input=first and t > 0,
                                                  add_row=("loop.step.weight", t, times) if first else None))
            schedule += [ScheduleEntry(i) for i in range(b, n)]
        return ModelSpec(
            architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_position=MAX_CONTEXT,
            layers=tuple(layers), schedule=tuple(schedule), final_norm=norm, tie_embeddings=False,
            embedding_name="embed.weight", final_norm_name="final.norm.weight", head_name="head.weight",
            embedding_scale=self.embedding_scale, input_position=PositionSpec("sinusoid", theta=POSITION_BASE),
            logit_scale=self.logit_scale, weight_suffix="")
