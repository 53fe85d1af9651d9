"""Small Tabedra configurations with weights made here, for the tests.

The tensor names and shapes are derived here from the configuration (not from the engine's manifest, which is thereby
checked too), the values are drawn with numpy, rounded to bfloat16 and written by a few lines of safetensors writing
of this file's own.  The rows of a layer's distance-bias table are not in config.json: the engine has to take them from
the checkpoint, so they travel beside the configuration (``rows``).

``sharp`` makes faults visible that random weights would hide: the score scale is raised so that a query looks at one
or two keys only, wherever they lie in its window, and the distance-bias tables get large entries, so that a bucket or a
window's edge that is one off moves the logits.  ``steady_router`` spaces the router's corrections so far apart that
the choice of experts does not hang on the last bits of a score (the bfloat16 engine rounds the router's input; the
weights of the chosen experts still come from the live scores).
"""
from __future__ import annotations

import json
import os
import struct

import numpy as np
import torch


def attn(heads, kv_heads, dim, vdim, conv=4, scale=None, bias_max=50.0, rows=12, window=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5 if scale is None else scale,
         "bias_max": bias_max}
    if conv:
        m["conv"] = conv
    if window is not None:
        m["mask"] = {"size": window}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "_rows": rows}


def moe(experts, top, ff, shared=None):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def config(vocab, width, layers, streams=2, eps=1e-5, bigram=(61, 7, 13), max_positions=1024):
    """Returns (config.json contents, rows of each layer's distance-bias table)."""
    rows = [l["_rows"] for l, _ in layers]
    c = {"architecture": "Tabedra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_positions": max_positions,
         "layers": [dict({k: v for k, v in l.items() if k != "_rows"}, mlp=m) for l, m in layers]}
    if streams is not None:
        c["streams"] = streams
    if bigram is not None:
        c["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return c, rows


# Sizes that differ from each other in every respect; values that a model may happen to make equal or 1 (streams, top,
# kv_heads, taps, dim against vdim, window against page and split sizes) are unequal or not 1 somewhere and equal or 1
# elsewhere.
CONFIGS = {
    # key and value sizes differ and are no multiples of 16; a reader of layer 0's cache with a wider window than the
    # owner's and one with a narrower; a layer without feed-forward; windows that are no multiples of the page
    "P": config(211, 96, [
        (attn(6, 2, 24, 40, conv=3, bias_max=40.0, rows=10, window=37), moe(5, 2, 40, shared=56)),
        (attn(4, 4, 16, 16, conv=2, bias_max=90.0, rows=16, window=None), None),
        (attn(6, 2, 24, 40, conv=5, bias_max=33.5, rows=8, window=52, kv_from=0), moe(4, 1, 24)),
        (attn(6, 2, 24, 40, conv=3, bias_max=20.0, rows=6, window=19, kv_from=0), moe(7, 3, 16, shared=8)),
    ], streams=3, eps=1e-6, bigram=(97, 31, 5)),
    # one stream with mixing tensors, no bigram table, one tap, every expert chosen, a width the tensor-core products refuse
    "Q": config(130, 100, [
        (attn(2, 1, 32, 16, conv=1, bias_max=64.0, rows=14, window=64), moe(3, 3, 20, shared=12)),
        (attn(5, 5, 20, 20, conv=4, bias_max=25.0, rows=4, window=30), moe(6, 2, 28)),
    ], streams=1, bigram=None),
    # the plain residual sum (no streams key), no convolution in one layer, head size 64 (tensor-core attention shapes)
    "R": config(320, 256, [
        (attn(4, 2, 64, 64, conv=4, bias_max=100.0, rows=32, window=128), moe(8, 2, 64, shared=96)),
        (attn(4, 1, 64, 64, conv=None, bias_max=300.0, rows=20, window=None), moe(8, 4, 32)),
        (attn(4, 2, 64, 64, conv=2, bias_max=100.0, rows=32, window=200, kv_from=0), None),
    ], streams=None, bigram=(251, 3, 11)),
}


def tensor_shapes(cfg, rows):
    D, V = cfg["width"], cfg["vocab"]
    S = cfg.get("streams")
    s = {"embed": (V, D), "pos": (cfg["max_positions"], D), "head": (V, D), "final.norm": (D,), "final.norm.b": (D,)}
    if cfg.get("embedding"):
        s["bigram"] = (cfg["embedding"]["bigram"]["buckets"] + 1, D)
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        s[p + "norm1"] = s[p + "norm1.b"] = (D,)
        s.update({p + "mix.q": (H * dk, D), p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv), p + "mix.rel": (rows[i], H)})
        if m.get("conv"):
            s[p + "mix.q.conv"] = (H * dk, m["conv"])
        if m.get("kv_from") is None:
            s.update({p + "mix.k": (G * dk, D), p + "mix.v": (G * dv, D)})
            if m.get("conv"):
                s.update({p + "mix.k.conv": (G * dk, m["conv"]), p + "mix.v.conv": (G * dv, m["conv"])})
        if S is not None:
            s.update({p + "hc1.in": (S,), p + "hc1.out": (S,), p + "hc1.mix": (S, S)})
        mlp = L["mlp"]
        if mlp is None:
            continue
        s[p + "norm2"] = s[p + "norm2.b"] = (D,)
        if S is not None:
            s.update({p + "hc2.in": (S,), p + "hc2.out": (S,), p + "hc2.mix": (S, S)})
        E, ff = mlp["router"]["experts"], mlp["expert"]["ff"]
        s[p + "mlp.router"], s[p + "mlp.correction"] = (E, D), (E,)
        for e in range(E):
            s[p + f"mlp.e{e}.up"], s[p + f"mlp.e{e}.down"] = (ff, D), (D, ff)
        if mlp["shared"] is not None:
            s[p + "mlp.shared.up"], s[p + "mlp.shared.down"] = (mlp["shared"]["ff"], D), (D, mlp["shared"]["ff"])
    return s


def draw_weights(cfg, rows, seed, sharp=False, steady_router=False):
    """name → float64 tensor holding bfloat16-representable values."""
    rng = np.random.default_rng(seed)
    out = {}
    for name, shape in tensor_shapes(cfg, rows).items():
        leaf = name.split(".")[-1]
        if leaf in ("norm1", "norm2", "norm") and len(shape) == 1:
            v = 1.0 + 0.2 * rng.standard_normal(shape)
        elif leaf == "b":
            v = 0.3 * rng.standard_normal(shape)
        elif leaf == "conv":
            v = 0.5 * rng.standard_normal(shape)
        elif leaf == "rel":
            v = (2.0 if sharp else 0.7) * rng.standard_normal(shape)
            mixer = cfg["layers"][int(name.split(".")[0][1:])]["mixer"]
            if sharp and mixer.get("mask"):
                # the row that serves the window's last key stands out: the keys at the edge get weight
                from plain_tabedra import distance_bucket
                v[distance_bucket(mixer["mask"]["size"] - 1, shape[0], mixer["bias_max"])] += 4.0
        elif name in ("embed", "pos", "bigram"):
            v = (1.0 if name == "embed" else 0.5) * rng.standard_normal(shape)
        elif leaf == "in":
            v = 1.0 / shape[0] + 0.3 * rng.standard_normal(shape)
        elif leaf == "out":
            v = 1.0 + 0.3 * rng.standard_normal(shape)
        elif leaf == "mix":
            v = np.eye(shape[0]) + 0.2 * rng.standard_normal(shape)
        elif leaf == "correction":
            v = rng.permutation(shape[0]) * 1.0 if steady_router else 0.15 * rng.standard_normal(shape)
        elif leaf == "router":
            v = 2.0 * rng.standard_normal(shape) / np.sqrt(shape[-1])
        else:
            v = rng.standard_normal(shape) / np.sqrt(shape[-1])
        out[name] = torch.from_numpy(np.asarray(v, dtype=np.float32)).to(torch.bfloat16).to(torch.float64)
    return out


def sharpened(cfg, factor=6.0):
    """The configuration with every layer's score scale raised: peaked attention."""
    c = json.loads(json.dumps(cfg))
    for L in c["layers"]:
        L["mixer"]["scale"] *= factor
    return c


def write_model(path, cfg, weights):
    """config.json and model.safetensors (BF16) under ``path``."""
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "config.json"), "w") as f:
        json.dump(cfg, f)
    header, blobs, off = {}, [], 0
    for name, t in weights.items():
        raw = t.to(torch.bfloat16).view(torch.int16).numpy().tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [off, off + len(raw)]}
        blobs.append(raw)
        off += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(os.path.join(path, "model.safetensors"), "wb") as f:
        f.write(struct.pack("<Q", len(text)) + text + b"".join(blobs))
    return path


def make(path, name_or_cfg, seed=0, sharp=False, steady_router=False):
    cfg, rows = CONFIGS[name_or_cfg] if isinstance(name_or_cfg, str) else name_or_cfg
    if sharp:
        cfg = sharpened(cfg)
    w = draw_weights(cfg, rows, seed, sharp, steady_router)
    write_model(path, cfg, w)
    return cfg, w
