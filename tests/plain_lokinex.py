"""A plain, slow implementation of the Lokinex decoder in float64, one function per mechanism.

It runs whole sequences at once, keeps no cache and no state (every token sees its past by recomputation or by an
explicit loop over time) and shares no code with the engine: the engine's kernels, parts and step function are
compared with it.  ``weights`` maps checkpoint tensor names to float64 (or int64) torch tensors on the CPU;
``config`` is the parsed config.json.

Notation: x the residual stream [T, D]; every matrix is stored [out, in] and applied as x @ W.T.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


# ----------------------------------------------------------------------------- small pieces
def rms(x, eps):
    """x divided by the root of its mean square (eps inside the root), over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def scalar_norm(x, gain, eps):
    """RMS norm whose gain is one number for all coordinates."""
    return rms(x, eps) * gain.reshape(())


def vector_norm(x, weight, eps):
    return rms(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def causal_conv(h, w, bias=None):
    """Per-channel convolution over time: out[t] = sum_j w[:, j] * h[t - (taps - 1) + j], zeros before the start.
    h [T, C], w [C, taps] (the last column multiplies the current token)."""
    T, C = h.shape
    taps = w.shape[1]
    out = torch.zeros(T, C, dtype=h.dtype)
    for t in range(T):
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    if bias is not None:
        out = out + bias
    return out


def rotate_interleaved(v, positions, n_rot, base):
    """Rotates the pairs (2i, 2i+1), i < n_rot/2, of the last axis of v [T, ..., d] by position * base^(-2i/n_rot);
    coordinates from n_rot on pass unchanged."""
    out = v.clone()
    half = n_rot // 2
    freq = torch.tensor([base ** (-2.0 * i / n_rot) for i in range(half)], dtype=F64)
    ang = positions.to(F64)[:, None] * freq[None, :]                    # [T, half]
    while ang.dim() < v.dim():
        ang = ang.unsqueeze(1)
    cos, sin = torch.cos(ang), torch.sin(ang)
    a, b = v[..., 0:n_rot:2], v[..., 1:n_rot:2]
    out[..., 0:n_rot:2] = a * cos - b * sin
    out[..., 1:n_rot:2] = b * cos + a * sin
    return out


# ----------------------------------------------------------------------------- mixers
def rglru_mixer(h, w, p, m):
    """Recurrent block: a gated branch y and a branch u that passes a short convolution and a real-gated linear
    recurrence whose gates are block-diagonal maps of u.  ``w(name)`` fetches '<layer>.mix.<name>'."""
    T = h.shape[0]
    width, blocks = m["width"], m["blocks"]
    y = gelu_tanh(h @ w("y").T + w("y.b"))
    u = causal_conv(h @ w("x").T + w("x.b"), w("conv"), w("conv.b"))
    bw = width // blocks
    ub = u.reshape(T, blocks, bw)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w("ra")) + w("ra.b")).reshape(T, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w("ri")) + w("ri.b")).reshape(T, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w("lam"))
    a = torch.exp(log_a)
    S = torch.zeros(width, dtype=F64)
    out = torch.zeros(T, width, dtype=F64)
    for t in range(T):
        S = a[t] * S + torch.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = S
    return (out * y) @ w("o").T


def latent_attention_mixer(h, w, p, m, eps):
    """Attention whose keys and values are expanded from a low-rank latent: per head the key is [W_uk c | shared
    rotated part] and the value W_uv c; the query is [unrotated | rotated] per head."""
    T = h.shape[0]
    H, dim, rot_dim, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w("q").T).reshape(T, H, dim + rot_dim)
    q_nope, q_rot = q[..., :dim], q[..., dim:]
    dkv = h @ w("dkv").T
    c = vector_norm(dkv[:, :rank], w("dkv.norm"), eps)
    k_rot = dkv[:, rank:]                                              # [T, rot_dim], one for all heads
    n_rot, base = m["rot"]["dims"], m["rot"]["base"]
    q_rot = rotate_interleaved(q_rot, pos, n_rot, base)
    k_rot = rotate_interleaved(k_rot, pos, n_rot, base)
    k_nope = (c @ w("uk").T).reshape(T, H, dim)
    v = (c @ w("uv").T).reshape(T, H, vdim)
    scores = (torch.einsum("thd,shd->hts", q_nope, k_nope) + torch.einsum("thd,sd->hts", q_rot, k_rot)) * m["scale"]
    mask = pos[None, :] <= pos[:, None]                                # [t, s]: s <= t
    scores = scores.masked_fill(~mask[None], float("-inf"))
    prob = torch.softmax(scores, dim=-1)
    o = torch.einsum("hts,shd->thd", prob, v).reshape(T, H * vdim)
    return o @ w("o").T


# ----------------------------------------------------------------------------- feed-forwards
def dense_ff(h, w):
    z = torch.relu(h @ w("up").T)
    return (z * z) @ w("down").T


def gated_expert(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def moe_ff(h, tokens, w, mlp):
    """Experts chosen by the token id from a table, each with weight 1/top; a shared expert gated by one sigmoid."""
    top = mlp["router"]["top"]
    table = w("table")
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in table[int(tokens[t])].tolist():
            out[t] += gated_expert(h[t:t + 1], w(f"e{e}.gate"), w(f"e{e}.up"), w(f"e{e}.down"))[0] / top
    if mlp.get("shared") is not None:
        sh = gated_expert(h, w("shared.gate"), w("shared.up"), w("shared.down"))
        out = out + sh * torch.sigmoid(h @ w("shared.sg").T)
    return out


# ----------------------------------------------------------------------------- the model
def layer_forward(x, tokens, weights, config, li):
    eps = config["norm"]["eps"]
    layer = config["layers"][li]
    p = f"l{li}."
    g = lambda n: weights[p + n]                                        # noqa: E731
    h = scalar_norm(x, g("norm1"), eps)
    if config.get("canon") is not None:
        h = h + causal_conv(h, g("canon1"))
    mw = lambda n: weights[p + "mix." + n]                              # noqa: E731
    if layer["type"] == "rglru":
        mixed = rglru_mixer(h, mw, p, layer["mixer"])
    elif layer["type"] == "latent_attention":
        mixed = latent_attention_mixer(h, mw, p, layer["mixer"], eps)
    else:
        raise ValueError(layer["type"])
    x = x + scalar_norm(mixed, g("norm1b"), eps)
    mlp = layer.get("mlp")
    if mlp is not None:
        h = scalar_norm(x, g("norm2"), eps)
        fw = lambda n: weights[p + "mlp." + n]                          # noqa: E731
        ff = dense_ff(h, fw) if mlp["kind"] == "dense" else moe_ff(h, tokens, fw, mlp)
        x = x + scalar_norm(ff, g("norm2b"), eps)
    return x


def run_order(config):
    """(layer index, pass number or None, first of its pass) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop")
    if loop is None:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    order += [(i, None, False) for i in range(loop["stop"], n)]
    return order


def forward(tokens, weights, config, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer run)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x0 = weights["embed"][tokens]
    x = x0
    streams = []
    for li, t, first in run_order(config):
        if first:
            x = torch.cat([x, x0], dim=-1) @ weights["loop.in"].T
            x = x + weights["loop.step"][t]
        x = layer_forward(x, tokens, weights, config, li)
        streams.append(x)
    logits = scalar_norm(x, weights["final.norm"], config["norm"]["eps"]) @ weights["head"].T
    if return_layers:
        return logits, torch.stack(streams)
    return logits
