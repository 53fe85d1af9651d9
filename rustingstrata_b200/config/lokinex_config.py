"""Typed configuration of the Lokinex decoder, read from its own config.json keys.

    architecture: "Lokinex"; vocab; width; norm: {eps}; canon: {taps} (absent: no input convolution);
    layers: [{type: "rglru" | "latent_attention", mixer: {...}, mlp: null | {kind: "dense", ff} |
             {kind: "moe", expert: {ff}, router: {experts, top}, shared: null | {ff}}}, ...];
    loop: {start, stop, times} (absent: every layer runs once); max_positions (optional).

Every size and constant lives here and reaches the parts as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _require

RGLRU = "rglru"
LATENT_ATTENTION = "latent_attention"
DEFAULT_MAX_POSITIONS = 1 << 20


@dataclass(frozen=True)
class RecurrentMixerConfig:
    width: int
    blocks: int
    conv: int


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str                      # "dense" or "moe"
    ff: int = 0                    # dense: the inner width
    experts: int = 0
    top: int = 0
    expert_ff: int = 0
    shared_ff: int = 0             # 0: no shared expert


@dataclass(frozen=True)
class LokinexLayerConfig:
    type: str
    mixer: Any
    mlp: Optional[FeedForwardConfig]


@dataclass(frozen=True)
class LokinexConfig:
    vocab: int
    width: int
    eps: float
    canon_taps: Optional[int]
    layers: Tuple[LokinexLayerConfig, ...]
    loop: Optional[Tuple[int, int, int]]        # (start, stop, times)
    max_positions: int = DEFAULT_MAX_POSITIONS
    raw: Optional[Mapping[str, Any]] = None     # the mapping it was read from, for writing it back

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str = "config.json") -> "LokinexConfig":
        vocab = _require(d, "vocab", int, where)
        width = _require(d, "width", int, where)
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError(f"{where}: missing required object 'norm'")
        eps = _require(norm, "eps", float, where + " norm")
        canon = d.get("canon")
        taps = _require(canon, "taps", int, where + " canon") if isinstance(canon, Mapping) else None
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must list at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"{where} layers[{i}]"
            if not isinstance(L, Mapping) or not isinstance(L.get("mixer"), Mapping):
                raise ConfigError(f"{w}: a layer is an object with 'type', 'mixer' and 'mlp'")
            m = L["mixer"]
            if L.get("type") == RGLRU:
                mixer = RecurrentMixerConfig(_require(m, "width", int, w), _require(m, "blocks", int, w),
                                             _require(m, "conv", int, w))
                if mixer.width % mixer.blocks:
                    raise ConfigError(f"{w}: width {mixer.width} is not a multiple of {mixer.blocks} blocks")
            elif L.get("type") == LATENT_ATTENTION:
                rot = m.get("rot")
                if not isinstance(rot, Mapping):
                    raise ConfigError(f"{w}: missing required object 'rot'")
                mixer = LatentMixerConfig(_require(m, "heads", int, w), _require(m, "dim", int, w),
                                          _require(m, "rot_dim", int, w), _require(m, "vdim", int, w),
                                          _require(m, "kv_rank", int, w), _require(m, "scale", float, w),
                                          _require(rot, "dims", int, w + " rot"), _require(rot, "base", float, w + " rot"))
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"{w}: rot.dims {mixer.rot_dims} must be even and at most rot_dim {mixer.rot_dim}")
            else:
                raise ConfigError(f"{w}: unknown layer type {L.get('type')!r} (known: {RGLRU}, {LATENT_ATTENTION})")
            mlp = L.get("mlp")
            if mlp is None:
                ff = None
            elif not isinstance(mlp, Mapping):
                raise ConfigError(f"{w}: 'mlp' must be an object or null")
            elif mlp.get("kind") == "dense":
                ff = FeedForwardConfig("dense", ff=_require(mlp, "ff", int, w + " mlp"))
            elif mlp.get("kind") == "moe":
                router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
                if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
                    raise ConfigError(f"{w}: a mixture of experts needs 'router' and 'expert' objects")
                ff = FeedForwardConfig("moe", experts=_require(router, "experts", int, w + " router"),
                                       top=_require(router, "top", int, w + " router"),
                                       expert_ff=_require(expert, "ff", int, w + " expert"),
                                       shared_ff=_require(shared, "ff", int, w + " shared") if isinstance(shared, Mapping) else 0)
                if ff.top > ff.experts:
                    raise ConfigError(f"{w}: top {ff.top} exceeds the {ff.experts} experts")
            else:
                raise ConfigError(f"{w}: unknown mlp kind {mlp.get('kind')!r} (known: dense, moe)")
            layers.append(LokinexLayerConfig(L["type"], mixer, ff))
        loop = d.get("loop")
        if isinstance(loop, Mapping):
            start = loop.get("start", 0)
            stop, times = _require(loop, "stop", int, where + " loop"), _require(loop, "times", int, where + " loop")
            if isinstance(start, bool) or not isinstance(start, int) or not 0 <= start < stop <= len(layers):
                raise ConfigError(f"{where}: loop start {start!r} .. stop {stop} does not lie within the {len(layers)} layers")
            loop_t = (start, stop, times)
        else:
            loop_t = None
        max_pos = d.get("max_positions", DEFAULT_MAX_POSITIONS)
        if isinstance(max_pos, bool) or not isinstance(max_pos, int) or max_pos <= 0:
            raise ConfigError(f"{where}: 'max_positions' must be a positive integer, got {max_pos!r}")
        return cls(vocab=vocab, width=width, eps=float(eps), canon_taps=taps, layers=tuple(layers), loop=loop_t,
                   max_positions=max_pos, raw=dict(d))

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise ValueError("this configuration was not read from a mapping")
