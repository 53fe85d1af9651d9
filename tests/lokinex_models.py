"""Small Lokinex configurations with weights made here, for the tests.

The tensor names and shapes are derived here from the configuration (not from the engine's manifest, which is thereby
checked too), the values are drawn with numpy, rounded to bfloat16 and written by a few lines of safetensors writing
of this file's own.  ``sharp=True`` makes faults visible that random weights would hide: the recurrence's ``lam`` is
pushed down so that the state lasts hundreds of tokens, and the attention's scale is raised so that each query looks
at one or two keys only, wherever they lie.
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch


def latent(heads, dim, rot_dim, vdim, kv_rank, rot_dims=None, base=10000.0, scale=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
                      "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims},
                      "scale": (dim + rot_dim) ** -0.5 if scale is None else scale}}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def config(vocab, width, layers, eps=1e-6, canon=None, loop=None):
    c = {"architecture": "Lokinex", "vocab": vocab, "width": width, "norm": {"eps": eps},
         "layers": [dict(l, mlp=m) for l, m in layers]}
    if canon is not None:
        c["canon"] = {"taps": canon}
    if loop is not None:
        c["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return c


# Sizes that differ from each other in every respect; values that a model may happen to make equal or 1 (top, blocks,
# taps, times, rot.dims against rot_dim, vdim against dim) are unequal or not 1 somewhere and equal or 1 elsewhere.
CONFIGS = {
    # a loop in the middle (start > 0, stop < layers), three passes, a layer without feed-forward, padding of the latent row
    "P": config(211, 96, [
        (rglru(64, 4, 3), dense(160)),
        (latent(3, 16, 8, 24, 40, base=10000.0), moe(5, 2, 40, shared=56)),
        (latent(5, 8, 16, 8, 23, rot_dims=8, base=500.0), None),
        (rglru(96, 1, 2), moe(4, 1, 24)),
    ], eps=1e-6, canon=3, loop=(1, 3, 3)),
    # no loop, no input convolution, a width the tensor-core products refuse, every expert used by every token, one tap
    "Q": config(130, 100, [
        (latent(2, 32, 16, 16, 64), dense(72)),
        (rglru(60, 3, 1), moe(3, 3, 20, shared=12)),
    ], eps=1e-5),
    # wider, one pass of a loop over everything, long taps, for long sequences
    "R": config(320, 256, [
        (latent(4, 32, 32, 48, 96, base=100000.0), moe(8, 2, 64, shared=96)),
        (rglru(192, 2, 5), dense(384)),
    ], eps=1e-5, canon=4, loop=(0, 2, 1)),
}


def tensor_shapes(cfg):
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "head": (V, D), "final.norm": ()}
    if cfg.get("loop") is not None:
        s["loop.in"] = (D, 2 * D)
        s["loop.step"] = (cfg["loop"]["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        s[p + "norm1"] = s[p + "norm1b"] = ()
        if cfg.get("canon") is not None:
            s[p + "canon1"] = (D, cfg["canon"]["taps"])
        if L["type"] == "rglru":
            W, B = m["width"], m["blocks"]
            s.update({p + "mix.y": (W, D), p + "mix.y.b": (W,), p + "mix.x": (W, D), p + "mix.x.b": (W,),
                      p + "mix.conv": (W, m["conv"]), p + "mix.conv.b": (W,), p + "mix.ra": (B, W // B, W // B),
                      p + "mix.ra.b": (B, W // B), p + "mix.ri": (B, W // B, W // B), p + "mix.ri.b": (B, W // B),
                      p + "mix.lam": (W,), p + "mix.o": (D, W)})
        else:
            H = m["heads"]
            s.update({p + "mix.q": (H * (m["dim"] + m["rot_dim"]), D), p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], D),
                      p + "mix.dkv.norm": (m["kv_rank"],), p + "mix.uk": (H * m["dim"], m["kv_rank"]),
                      p + "mix.uv": (H * m["vdim"], m["kv_rank"]), p + "mix.o": (D, H * m["vdim"])})
        mlp = L["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = s[p + "norm2b"] = ()
        if mlp["kind"] == "dense":
            s[p + "mlp.up"], s[p + "mlp.down"] = (mlp["ff"], D), (D, mlp["ff"])
        else:
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                s[p + f"mlp.e{e}.gate"] = s[p + f"mlp.e{e}.up"] = (ff, D)
                s[p + f"mlp.e{e}.down"] = (D, ff)
            s[p + "mlp.table"] = (V, mlp["router"]["top"])
            if mlp["shared"] is not None:
                sf = mlp["shared"]["ff"]
                s.update({p + "mlp.shared.gate": (sf, D), p + "mlp.shared.up": (sf, D), p + "mlp.shared.down": (D, sf),
                          p + "mlp.shared.sg": (1, D)})
    return s


def draw_weights(cfg, seed, sharp=False):
    """name → float64 tensor holding bfloat16-representable values (int64 for the expert tables)."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        leaf = name.split(".")[-1]
        if leaf == "table":
            E = next(L["mlp"]["router"]["experts"] for i, L in enumerate(cfg["layers"]) if name.startswith(f"l{i}."))
            out[name] = torch.from_numpy(np.stack([rng.permutation(E)[: shape[1]] for _ in range(shape[0])]).astype(np.int64))
            continue
        if shape == () or name.endswith("dkv.norm"):
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "lam":
            v = (-5.0 if sharp else 0.0) + rng.standard_normal(shape)
        elif leaf == "b" or name == "loop.step":
            v = 0.3 * rng.standard_normal(shape)
        elif leaf in ("conv", "canon1"):
            v = 0.5 * rng.standard_normal(shape)
        elif name in ("embed",):
            v = rng.standard_normal(shape)
        else:
            v = rng.standard_normal(shape) / np.sqrt(shape[-1])
            if sharp and leaf == "q":
                v = v * 6.0                       # peaked attention: a query looks at one or two keys, wherever they lie
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16).to(torch.float64)
    return out


def write_model(path, cfg, weights):
    """config.json and model.safetensors (BF16, integer tables I32) under ``path``."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        if t.dtype == torch.int64:
            raw, tag = t.to(torch.int32).numpy().tobytes(), "I32"
        else:
            raw, tag = t.to(torch.bfloat16).view(torch.int16).numpy().tobytes(), "BF16"
        header[name] = {"dtype": tag, "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    return path


def make(path, name_or_cfg, seed=0, sharp=False):
    cfg = CONFIGS[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    w = draw_weights(cfg, seed, sharp)
    write_model(path, cfg, w)
    return cfg, w
