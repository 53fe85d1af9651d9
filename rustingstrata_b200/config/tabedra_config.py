"""Typed configuration of the Tabedra decoder, read from its own config.json keys.

    architecture: "Tabedra"; vocab; width; norm: {eps}; streams (absent: one residual stream, the plain residual sum);
    max_positions (rows of the learned position table); embedding: {bigram: {buckets, mul_prev, mul_cur}} (absent: no
    bigram table);
    layers: [{type: "attention", mixer: {heads, kv_heads, dim, vdim, conv (taps; absent: none), scale, bias_max,
              mask: {size} (absent: every earlier key), kv_from (absent: keys and values of its own)},
              mlp: null | {kind: "moe", expert: {ff}, router: {experts, top}, shared: null | {ff}}}, ...].

Two sizes are not in config.json but in the checkpoint's tensor shapes: the rows of a layer's distance-bias table
(``l<i>.mix.rel``) and of the position table (``pos``); :meth:`TabedraConfig.resolve_shapes` takes them from there.
A configuration for random weights names them itself (``bias_rows`` in a mixer).  Every size and constant lives here
and reaches the parts as parameters.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError, _require

ATTENTION = "attention"


@dataclass(frozen=True)
class TabedraMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    taps: int                       # 0: no convolution
    scale: float
    bias_max: float
    bias_rows: Optional[int]        # rows of the distance-bias table; None: not known yet (the checkpoint says); 0: no bias
    window: Optional[int]
    kv_from: Optional[int]


@dataclass(frozen=True)
class TabedraFeedForwardConfig:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int                  # 0: no shared expert


@dataclass(frozen=True)
class TabedraLayerConfig:
    mixer: TabedraMixerConfig
    mlp: Optional[TabedraFeedForwardConfig]


@dataclass(frozen=True)
class TabedraConfig:
    vocab: int
    width: int
    eps: float
    streams: Optional[int]          # None: a single stream without stream-mixing tensors
    max_positions: int
    position_rows: int              # rows of the learned position table
    bigram: Optional[Tuple[int, int, int]]      # (buckets, mul_prev, mul_cur)
    layers: Tuple[TabedraLayerConfig, ...]
    raw: Optional[Mapping[str, Any]] = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any], where: str = "config.json") -> "TabedraConfig":
        vocab = _require(d, "vocab", int, where)
        width = _require(d, "width", int, where)
        norm = d.get("norm")
        if not isinstance(norm, Mapping):
            raise ConfigError(f"{where}: missing required object 'norm'")
        eps = _require(norm, "eps", float, where + " norm")
        streams = _require(d, "streams", int, where) if d.get("streams") is not None else None
        max_pos = _require(d, "max_positions", int, where)
        emb = d.get("embedding")
        big = emb.get("bigram") if isinstance(emb, Mapping) else None
        bigram = None
        if isinstance(big, Mapping):
            w = where + " embedding.bigram"
            for key in ("mul_prev", "mul_cur"):
                if isinstance(big.get(key), bool) or not isinstance(big.get(key), int):
                    raise ConfigError(f"{w}: key '{key}' must be an integer, got {big.get(key)!r}")
            bigram = (_require(big, "buckets", int, w), int(big["mul_prev"]), int(big["mul_cur"]))
        raw_layers = d.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must list at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            w = f"{where} layers[{i}]"
            if not isinstance(L, Mapping) or not isinstance(L.get("mixer"), Mapping):
                raise ConfigError(f"{w}: a layer is an object with 'type', 'mixer' and 'mlp'")
            if L.get("type") != ATTENTION:
                raise ConfigError(f"{w}: unknown layer type {L.get('type')!r} (known: {ATTENTION})")
            m = L["mixer"]
            mask = m.get("mask")
            window = _require(mask, "size", int, w + " mask") if isinstance(mask, Mapping) else None
            kv_from = m.get("kv_from")
            if kv_from is not None and (isinstance(kv_from, bool) or not isinstance(kv_from, int) or not 0 <= kv_from < i):
                raise ConfigError(f"{w}: 'kv_from' must name an earlier layer, got {kv_from!r}")
            rows = m.get("bias_rows")
            if rows is not None and (isinstance(rows, bool) or not isinstance(rows, int) or rows < 0):
                raise ConfigError(f"{w}: 'bias_rows' must be a non-negative integer, got {rows!r}")
            mixer = TabedraMixerConfig(
                heads=_require(m, "heads", int, w), kv_heads=_require(m, "kv_heads", int, w), dim=_require(m, "dim", int, w),
                vdim=_require(m, "vdim", int, w), taps=_require(m, "conv", int, w) if m.get("conv") is not None else 0,
                scale=_require(m, "scale", float, w),
                bias_max=_require(m, "bias_max", float, w) if m.get("bias_max") is not None else 0.0,
                bias_rows=rows if m.get("bias_max") is not None else 0, window=window, kv_from=kv_from)
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"{w}: {mixer.heads} heads are not a multiple of {mixer.kv_heads} kv_heads")
            mlp = L.get("mlp")
            if mlp is None:
                ff = None
            elif not isinstance(mlp, Mapping) or mlp.get("kind", "moe") != "moe":
                raise ConfigError(f"{w}: 'mlp' must be null or an object of kind 'moe'")
            else:
                router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
                if not isinstance(router, Mapping) or not isinstance(expert, Mapping):
                    raise ConfigError(f"{w}: a mixture of experts needs 'router' and 'expert' objects")
                ff = TabedraFeedForwardConfig(
                    experts=_require(router, "experts", int, w + " router"), top=_require(router, "top", int, w + " router"),
                    expert_ff=_require(expert, "ff", int, w + " expert"),
                    shared_ff=_require(shared, "ff", int, w + " shared") if isinstance(shared, Mapping) else 0)
                if ff.top > ff.experts:
                    raise ConfigError(f"{w}: top {ff.top} exceeds the {ff.experts} experts")
            layers.append(TabedraLayerConfig(mixer, ff))
        for i, L in enumerate(layers):
            j = L.mixer.kv_from
            if j is None:
                continue
            o = layers[j].mixer
            if o.kv_from is not None:
                raise ConfigError(f"{where} layers[{i}]: 'kv_from' names layer {j}, which has no keys and values of its own")
            if (o.kv_heads, o.dim, o.vdim, o.heads) != (L.mixer.kv_heads, L.mixer.dim, L.mixer.vdim, L.mixer.heads):
                raise ConfigError(f"{where} layers[{i}]: head counts and sizes differ from those of layer {j}, whose keys "
                                  f"and values it reads")
        return cls(vocab=vocab, width=width, eps=float(eps), streams=streams, max_positions=max_pos, position_rows=max_pos,
                   bigram=bigram, layers=tuple(layers), raw=dict(d))

    def resolve_shapes(self, shapes: Mapping[str, Tuple[int, ...]]) -> "TabedraConfig":
        """The sizes that only the checkpoint's tensor shapes give (name → shape)."""
        layers = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            if m.bias_rows is None:
                shape = shapes.get(f"l{i}.mix.rel")
                m = replace(m, bias_rows=int(shape[0]) if shape else 0)
            layers.append(replace(L, mixer=m))
        rows = int(shapes["pos"][0]) if "pos" in shapes and len(shapes["pos"]) == 2 else self.position_rows
        return replace(self, layers=tuple(layers), position_rows=rows)

    def to_dict(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise ValueError("this configuration was not read from a mapping")
