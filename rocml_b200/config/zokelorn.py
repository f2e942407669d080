"""Typed configuration of the Zokelorn decoder, read from config.json.

A Zokelorn model is an embedding, a list of layers that each name their mixer and feed-forward with
their own sizes, an optional span of layers that runs several times in a row with the same weights
(each pass with a cache or state of its own), a final RMSNorm and a head.  Every layer is parallel:
one norm, whose output both the mixer and the feed-forward read, and both results join the stream.
Three mixers: softmax attention over blocks of positions with grouped key/value heads, rotation of
neighbouring pairs (optionally with stretched long wavelengths) and a sigmoid gate per head; lightning
attention and retention, two linear attentions with a fixed decay per head and a state of fixed size.
Two feed-forwards: a dense gated one (gelu in its tanh form) and routed experts (silu) chosen from the
best groups of experts, with weights that sum to one, plus a gated shared expert.

Keys read (every size and every constant that differs between models comes from here)::

    architecture        "Zokelorn"
    vocab, width
    norm.eps
    layers[i].type      "attention" | "lightning" | "retention"
    layers[i].mixer     attention: heads, kv_heads, dim, vdim, scale, mask.size,
                                   rot: {base, dims, scaling: {factor, low, high, original} (optional)}
                        lightning, retention: heads, dim, vdim, decay (one number a head)
    layers[i].mlp       null | {kind: "dense", ff}
                        | {kind: "moe", expert: {ff}, router: {experts, top, groups: {count, keep} (optional)},
                           shared: {ff} (optional)}
    loop                optional {start, stop, times}

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.<q|k|v|g|o|norm>``, ``l<i>.mlp.<gate|up|down>``,
``l<i>.mlp.router``, ``l<i>.mlp.e<k>.<gate|up|down>``, ``l<i>.mlp.shared.<gate|up|down|sg>``,
``final.norm``, ``head``; no ``.weight`` suffix.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import ConfigError
from .pipilix import _get, _int, _num
from .specs import FeedForwardSpec, LayerSpec, MixerSpec, ModelSpec, NormSpec, PositionSpec, ScheduleEntry, _frozen_params

ARCHITECTURE = "Zokelorn"

# Constants the design fixes.
ROUTE_WEIGHT_EPS = 1e-20       # added to the sum of the chosen scores before they are divided by it
MAX_CONTEXT = 1 << 20          # the design names no longest sequence: positions are plain integers

_MIXERS = ("attention", "lightning", "retention")
_FF_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class RotationConfig:
    base: float
    dims: int
    scaling: Optional[Tuple[float, float, float, float]] = None     # factor, low, high, original

    @staticmethod
    def from_dict(d, where) -> "RotationConfig":
        sc = d.get("scaling") if isinstance(d, Mapping) else None
        scaling = None
        if sc is not None:
            w = where + "scaling."
            scaling = (_num(sc, "factor", w), _num(sc, "low", w), _num(sc, "high", w), _num(sc, "original", w))
        cfg = RotationConfig(_num(d, "base", where), _int(d, "dims", where, 0), scaling)
        if cfg.dims % 2:
            raise ConfigError(f"config.json: {where}dims must be even, found {cfg.dims}")
        if not cfg.base > 0:
            raise ConfigError(f"config.json: {where}base must be positive, found {cfg.base}")
        return cfg

    def to_dict(self) -> dict:
        d = {"base": self.base, "dims": self.dims}
        if self.scaling is not None:
            d["scaling"] = dict(zip(("factor", "low", "high", "original"), self.scaling))
        return d


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    block: Optional[int]               # mask.size: a query sees the earlier keys of its own block of positions
    rot: Optional[RotationConfig]

    @staticmethod
    def from_dict(d, where) -> "AttentionConfig":
        mask = d.get("mask") if isinstance(d, Mapping) else None
        rot = d.get("rot") if isinstance(d, Mapping) else None
        cfg = AttentionConfig(
            heads=_int(d, "heads", where), kv_heads=_int(d, "kv_heads", where), dim=_int(d, "dim", where),
            vdim=_int(d, "vdim", where), scale=_num(d, "scale", where),
            block=None if mask is None else _int(mask, "size", where + "mask."),
            rot=None if rot is None else RotationConfig.from_dict(rot, where + "rot."))
        if cfg.heads % cfg.kv_heads:
            raise ConfigError(f"config.json: {where}heads {cfg.heads} is no multiple of kv_heads {cfg.kv_heads}")
        if cfg.rot is not None and cfg.rot.dims > cfg.dim:
            raise ConfigError(f"config.json: {where}rot.dims {cfg.rot.dims} exceeds dim {cfg.dim}")
        return cfg

    def to_dict(self) -> dict:
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.block is not None:
            d["mask"] = {"size": self.block}
        if self.rot is not None:
            d["rot"] = self.rot.to_dict()
        return d


@dataclass(frozen=True)
class DecayConfig:
    """The sizes of a lightning or retention mixer."""

    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]

    @staticmethod
    def from_dict(d, where) -> "DecayConfig":
        decay = _get(d, "decay", where)
        if not isinstance(decay, (list, tuple)) or not all(isinstance(x, (int, float)) and not isinstance(x, bool) for x in decay):
            raise ConfigError(f"config.json: {where}decay must be a list of numbers")
        cfg = DecayConfig(_int(d, "heads", where), _int(d, "dim", where), _int(d, "vdim", where), tuple(float(x) for x in decay))
        if len(cfg.decay) != cfg.heads:
            raise ConfigError(f"config.json: {where}decay has {len(cfg.decay)} numbers for {cfg.heads} heads")
        if not all(0.0 <= x <= 1.0 for x in cfg.decay):
            raise ConfigError(f"config.json: {where}decay must lie in [0, 1]")
        return cfg

    def to_dict(self) -> dict:
        return {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "decay": list(self.decay)}


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                      # "dense" or "moe"
    ff: int
    experts: int = 0
    top: int = 0
    groups: int = 1
    keep: int = 1
    shared_ff: int = 0

    @staticmethod
    def from_dict(d, where) -> "FeedForwardConfig":
        kind = _get(d, "kind", where)
        if kind not in _FF_KINDS:
            raise ConfigError(f"config.json: {where}kind {kind!r} is unknown (known: {', '.join(_FF_KINDS)})")
        if kind == "dense":
            return FeedForwardConfig("dense", _int(d, "ff", where))
        ex, ro = _get(d, "expert", where), _get(d, "router", where)
        gr, sh = ro.get("groups"), d.get("shared")
        cfg = FeedForwardConfig(
            "moe", _int(ex, "ff", where + "expert."), _int(ro, "experts", where + "router."), _int(ro, "top", where + "router."),
            groups=1 if gr is None else _int(gr, "count", where + "router.groups."),
            keep=1 if gr is None else _int(gr, "keep", where + "router.groups."),
            shared_ff=0 if sh is None else _int(sh, "ff", where + "shared."))
        if cfg.top > cfg.experts:
            raise ConfigError(f"config.json: {where}router.top {cfg.top} exceeds router.experts {cfg.experts}")
        if cfg.experts % cfg.groups or cfg.keep > cfg.groups or cfg.keep * (cfg.experts // cfg.groups) < cfg.top:
            raise ConfigError(f"config.json: {where}router.groups {{count: {cfg.groups}, keep: {cfg.keep}}} does not fit "
                              f"{cfg.experts} experts of which {cfg.top} are chosen")
        return cfg

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        router = {"experts": self.experts, "top": self.top}
        if self.groups > 1:
            router["groups"] = {"count": self.groups, "keep": self.keep}
        d = {"kind": "moe", "expert": {"ff": self.ff}, "router": router}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff}
        return d


@dataclass(frozen=True)
class ZokelornLayer:
    mixer_type: str
    mixer: Any                     # AttentionConfig or DecayConfig
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class ZokelornConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[ZokelornLayer, ...]
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
    def from_dict(d: Mapping[str, Any]) -> "ZokelornConfig":
        layers = _get(d, "layers", "")
        if not isinstance(layers, (list, tuple)):
            raise ConfigError("config.json: 'layers' must be a list")
        out = []
        for i, L in enumerate(layers):
            where = f"layers[{i}]."
            kind = _get(L, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"config.json: {where}type {kind!r} is unknown (known: {', '.join(_MIXERS)})")
            m = _get(L, "mixer", where)
            mixer = AttentionConfig.from_dict(m, where + "mixer.") if kind == "attention" else \
                DecayConfig.from_dict(m, where + "mixer.")
            mlp = L.get("mlp")
            out.append(ZokelornLayer(kind, mixer, None if mlp is None else FeedForwardConfig.from_dict(mlp, where + "mlp.")))
        loop = d.get("loop")
        if loop is not None:
            loop = (_int(loop, "start", "loop.", 0), _int(loop, "stop", "loop."), _int(loop, "times", "loop."))
        return ZokelornConfig(vocab=_int(d, "vocab", ""), width=_int(d, "width", ""),
                              norm_eps=_num(_get(d, "norm", ""), "eps", "norm."), layers=tuple(out), loop=loop)

    def to_dict(self) -> dict:
        d = {
            "architecture": ARCHITECTURE,
            "layers": [{"type": L.mixer_type, "mixer": L.mixer.to_dict(), "mlp": None if L.mlp is None else L.mlp.to_dict()}
                       for L in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return d

    # ---- the architecture, spelled as parts ------------------------------------------------------
    def _mixer_spec(self, L: ZokelornLayer) -> MixerSpec:
        m = L.mixer
        if L.mixer_type == "attention":
            position = None
            if m.rot is not None and m.rot.dims > 0:
                params = {}
                if m.rot.scaling is not None:
                    params["scaling"] = dict(zip(("factor", "low", "high", "original"), m.rot.scaling))
                position = PositionSpec("rope_pairs", theta=m.rot.base, rot_dim=m.rot.dims, params_items=_frozen_params(params))
            return MixerSpec.make(
                "attention", position, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                scale=m.scale, chunk=m.block, gated=True, bias=False, qk_norm=False,
                names={"q": "q", "k": "k", "v": "v", "o": "o", "gate": "g"})
        names = {"q": "q", "k": "k", "v": "v", "gate": "g", "o": "o", "out_norm": "norm"}
        if L.mixer_type == "lightning":
            return MixerSpec.make(
                "linear_attention", n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, decay=tuple(m.decay),
                qk_activation="silu", v_activation="silu", k_scale=1.0, out_norm="all_heads", out_norm_eps=self.norm_eps,
                out_norm_weight=True, gate_activation="sigmoid", names=names)
        return MixerSpec.make(
            "linear_attention", n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, decay=tuple(m.decay),
            qk_activation="none", v_activation="none", k_scale=float(m.dim) ** -0.5, out_norm="per_head",
            out_norm_eps=self.norm_eps, out_norm_weight=False, gate_activation="silu", names=names)

    @staticmethod
    def _ff_spec(f: Optional[FeedForwardConfig]) -> Optional[FeedForwardSpec]:
        if f is None:
            return None
        if f.kind == "dense":
            return FeedForwardSpec.make("gated_mlp", intermediate=f.ff, activation="gelu_tanh", bias=False,
                                        names={"gate": "gate", "up": "up", "down": "down"})
        return FeedForwardSpec.make(
            "routed_mlp", experts=f.experts, top=f.top, intermediate=f.ff, activation="silu", score="sigmoid",
            choice_bias=False, renormalize=True, renormalize_eps=ROUTE_WEIGHT_EPS, groups=f.groups, keep_groups=f.keep,
            shared=f.shared_ff, shared_gate=f.shared_ff > 0,
            names={"router": "router", "expert": "e{e}.", "gate": "gate", "up": "up", "down": "down", "shared": "shared.",
                   "shared_gate": "sg"})

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec("rmsnorm", self.norm_eps)
        layers = tuple(
            LayerSpec(prefix=f"l{i}", mixer=self._mixer_spec(L), feed_forward=self._ff_spec(L.mlp), mixer_norm=norm,
                      ff_norm=norm, arrangement="parallel", mixer_norm_name="norm1", mixer_name="mix.", ff_name="mlp.")
            for i, L in enumerate(self.layers))
        n = len(self.layers)
        if self.loop is None:
            order = list(range(n))
        else:
            a, b, times = self.loop
            order = list(range(a)) + list(range(a, b)) * times + list(range(b, n))
        return ModelSpec(
            architecture=ARCHITECTURE, hidden=self.width, vocab=self.vocab, max_position=MAX_CONTEXT, layers=layers,
            schedule=tuple(ScheduleEntry(i) for i in order), final_norm=norm, tie_embeddings=False,
            embedding_name="embed.weight", final_norm_name="final.norm.weight", head_name="head.weight", weight_suffix="")
