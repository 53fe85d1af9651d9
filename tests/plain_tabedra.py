"""A plain, slow implementation of the Tabedra decoder in float64, one function per mechanism.

It runs a whole sequence at once, keeps no cache and no state (every token sees its past by recomputation) and
shares no code with the engine: the engine's kernels, parts and step function are compared with it.  ``weights``
maps checkpoint tensor names to float64 torch tensors on the CPU; ``config`` is the parsed config.json.

Notation: every matrix is stored [out, in] and applied as x @ W.T; X is the set of residual streams [S, T, D].
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def unit_rms(x, eps):
    """x divided by the root of its mean square over the last axis (eps inside the root); no gain."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm(x, w, b, eps):
    """(x - mean) / sqrt(var + eps) * w + b over the last axis, var = mean squared deviation."""
    mu = x.mean(dim=-1, keepdim=True)
    d = x - mu
    var = (d * d).mean(dim=-1, keepdim=True)
    return d / torch.sqrt(var + eps) * w + b


def causal_conv(u, w):
    """Per-channel convolution over time: out[t] = sum_j w[:, j] * u[t - (taps - 1) + j], zeros before the start.
    u [T, C], w [C, taps] (the last column multiplies the current token)."""
    T, C = u.shape
    taps = w.shape[1]
    out = torch.zeros(T, C, dtype=u.dtype)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * u[s]
    return out


def distance_bucket(n, rows, far):
    """Row of the distance-bias table for distance n >= 0: one row per distance below rows/2, then rows spaced
    evenly in the logarithm of the distance up to ``far``, where the last row is reached."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


# ----------------------------------------------------------------------------- embedding
def embedding(tokens, weights, config):
    """Token row + bigram row (hash of previous and current token; a row of its own for a first token) + position row."""
    T = len(tokens)
    x = weights["embed"][torch.tensor(tokens)].clone()
    big = (config.get("embedding") or {}).get("bigram")
    if big is not None:
        n, a, b = int(big["buckets"]), int(big["mul_prev"]), int(big["mul_cur"])
        rows = [n if t == 0 else (tokens[t - 1] * a + tokens[t] * b) % n for t in range(T)]
        x = x + weights["bigram"][torch.tensor(rows)]
    if "pos" in weights:
        x = x + weights["pos"][:T]
    return x


# ----------------------------------------------------------------------------- attention
def keys_values(h, weights, prefix, m, eps):
    """A layer's keys (convolved, unit norm per head) and values (convolved) from its mixer input h [T, D]."""
    G, dk, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    k = h @ weights[prefix + "k"].T
    v = h @ weights[prefix + "v"].T
    if m.get("conv"):
        k = causal_conv(k, weights[prefix + "k.conv"])
        v = causal_conv(v, weights[prefix + "v.conv"])
    k = unit_rms(k.reshape(T, G, dk), eps)
    return k, v.reshape(T, G, dv)


def attention(h, k, v, weights, prefix, m, eps):
    """Windowed softmax attention of the queries made from h over given keys k [T, G, dk] and values v [T, G, dv],
    with a learned bias per bucketed distance and head, a sigmoid gate on the joined heads, and the output matrix."""
    H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    T = h.shape[0]
    q = h @ weights[prefix + "q"].T
    if m.get("conv"):
        q = causal_conv(q, weights[prefix + "q.conv"])
    q = unit_rms(q.reshape(T, H, dk), eps)
    window = int(m["mask"]["size"]) if m.get("mask") else None
    rel = weights.get(prefix + "rel")
    if rel is not None:          # the bias of every distance that can occur, [T, H]
        by_distance = rel[torch.tensor([distance_bucket(n, rel.shape[0], float(m["bias_max"])) for n in range(T)])]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        for i in range(T):
            lo = 0 if window is None else max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, hd]) * float(m["scale"])
            if rel is not None:
                s = s + by_distance[torch.arange(i - lo, -1, -1), hd]        # key j lies i - j back
            p = torch.softmax(s, dim=0)
            out[i, hd] = p @ v[lo:i + 1, g]
    y = out.reshape(T, H * dv)
    if prefix + "g" in weights:
        y = y * torch.sigmoid(h @ weights[prefix + "g"].T)
    return y @ weights[prefix + "o"].T


# ----------------------------------------------------------------------------- feed-forward
def relu2_expert(h, up, down):
    a = torch.relu(h @ up.T)
    return (a * a) @ down.T


def router(h, weights, prefix, top):
    """(chosen experts [T, top], their weights [T, top]): softmax over all experts; the choice adds a correction
    to the scores, the weights do not and are divided by their sum."""
    s = torch.softmax(h @ weights[prefix + "router"].T, dim=-1)
    choice = s + weights[prefix + "correction"] if prefix + "correction" in weights else s
    idx = torch.topk(choice, top, dim=-1).indices
    w = torch.gather(s, 1, idx)
    return idx, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def mixture(h, weights, prefix, mlp):
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    idx, w = router(h, weights, prefix, top)
    out = torch.zeros(h.shape[0], weights[prefix + "e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            assert 0 <= e < E
            out[t] += w[t, j] * relu2_expert(h[t:t + 1], weights[f"{prefix}e{e}.up"], weights[f"{prefix}e{e}.down"])[0]
    if mlp.get("shared"):
        out = out + relu2_expert(h, weights[prefix + "shared.up"], weights[prefix + "shared.down"])
    return out


# ----------------------------------------------------------------------------- streams
def read_streams(X, weights, name):
    """What a sublayer reads: the streams weighted by ``in`` and summed (one stream without the tensors: itself)."""
    if name + ".in" not in weights:
        return X[0]
    return torch.einsum("s,std->td", weights[name + ".in"], X)


def write_streams(X, y, weights, name):
    """All streams at once from the old ones: x_t <- sum_s mix[s, t] x_s + out[t] y (plain x + y without the tensors)."""
    if name + ".in" not in weights:
        return X + y[None]
    return torch.einsum("st,sud->tud", weights[name + ".mix"], X) + weights[name + ".out"][:, None, None] * y[None]


# ----------------------------------------------------------------------------- the model
def forward(tokens, weights, config, layers_out=None):
    """Logits [T, vocab] of a whole sequence.  ``layers_out``: a list that receives the sum of the streams after
    every layer."""
    eps = float(config["norm"]["eps"])
    x = embedding(tokens, weights, config)
    S = int(config["streams"]) if config.get("streams") else 1
    X = torch.stack([x] * S)
    kept = {}
    for i, L in enumerate(config["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        u = read_streams(X, weights, p + "hc1")
        h = layer_norm(u, weights[p + "norm1"], weights[p + "norm1.b"], eps)
        if L["type"] != "attention":
            raise ValueError(L["type"])
        if m.get("kv_from") is None:
            kept[i] = keys_values(h, weights, p + "mix.", m, eps)
            k, v = kept[i]
        else:
            k, v = kept[int(m["kv_from"])]
        X = write_streams(X, attention(h, k, v, weights, p + "mix.", m, eps), weights, p + "hc1")
        if L.get("mlp") is not None:
            u = read_streams(X, weights, p + "hc2")
            h = layer_norm(u, weights[p + "norm2"], weights[p + "norm2.b"], eps)
            X = write_streams(X, mixture(h, weights, p + "mlp.", L["mlp"]), weights, p + "hc2")
        if layers_out is not None:
            layers_out.append(X.sum(dim=0))
    x = X.sum(dim=0)
    x = layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps)
    return x @ weights["head"].T
