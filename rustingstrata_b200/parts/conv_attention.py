"""Paged attention whose queries, keys and values pass a short convolution over time, with unit-norm queries and
keys, a learned bias per bucketed distance, and a sigmoid gate on the joined heads.

Per token, from the mixer's input h: q = W_q h, k = W_k h, v = W_v h (no biases); each channel of the three is
convolved over time with ``taps`` taps (zeros before the sequence's start; the last taps - 1 projected rows of a
request are its state); every q and k head is divided by sqrt(mean square + eps); a score is

    (q . k) * scale + rel[bucket(i - j), head]            for 0 <= i - j < window,

with bucket(n) = n below half the table's rows B/2, then evenly spaced in log(n) so that distance ``bias_max`` reaches
the last row: B/2 + floor(log(n / (B/2)) / log(bias_max / (B/2)) * (B - B/2)), capped at B - 1.  Softmax over the
visible keys, the joined heads times sigmoid(W_g h), then W_o.  Keys and values may have different sizes; the cache and
the attention kernels see heads padded with zeros to a common size (a multiple of 16; in the bfloat16 engine the next
size its tensor-core attention kernels take).  A call that reads another call's cache
projects and convolves queries only.

The work lists, split form and workspaces are those of :class:`~rustingstrata_b200.parts.attention.PagedAttention`;
the bias reaches the kernels as a table by distance (one row per distance up to the one from which the last bucket
serves every longer one).
"""
from __future__ import annotations

import math

import numpy as np
import torch

from ..kernels import ops
from .attention import PagedAttention
from .base import CallInfo, StepContext
from .registry import register_part
from .spec import CacheNeed, PartSpec, StateNeed, TensorNeed


def distance_rows(n_rows: int, far: float, n_distances: int) -> np.ndarray:
    """Row of a [n_rows, heads] distance-bias table for each distance 0 .. n_distances - 1 (int64)."""
    half = n_rows // 2
    out = np.empty(n_distances, dtype=np.int64)
    for n in range(n_distances):
        if n < half:
            out[n] = n
        else:
            step = int(math.floor(math.log(n / half) / math.log(far / half) * (n_rows - half)))
            out[n] = min(n_rows - 1, half + step)
    return out


@register_part("mixer", "conv_gated_attention")
class ConvGatedAttention(PagedAttention):
    """params: hidden, n_heads, n_kv_heads, dim (query/key size per head), vdim, taps (0 or None: no convolution),
    unit_norm (bool), eps, window (None: every key), cache_window (what the cache keeps; at least ``window``, more when
    other calls with wider windows read this call's cache), scale, bias_rows (0: no distance bias), bias_max, gate (bool),
    kv_projection (bool).  tensors: q_proj, k_proj, v_proj, o_proj, and q_conv, k_conv, v_conv [channels, taps], rel
    [bias_rows, n_heads], g_proj as the params ask."""
    chain_safe = False

    def __init__(self, spec, runtime, position=None):
        p = spec.params
        self.dk, self.dv = int(p["dim"]), int(p["vdim"])
        self.head_pad = (max(self.dk, self.dv) + 15) // 16 * 16
        if runtime.dtype == torch.bfloat16:
            # up to 128: the next head size the tensor-core attention kernels take
            self.head_pad = next((n for n in (32, 64, 96, 128) if n >= self.head_pad), self.head_pad)
        if self.head_pad > 256:
            raise ValueError(f"conv_gated_attention: head sizes {self.dk} / {self.dv} exceed the 256 the kernels take")
        inner = PartSpec(spec.kind, {"hidden": p["hidden"], "n_heads": p["n_heads"], "n_kv_heads": p["n_kv_heads"],
                                     "head_dim": self.head_pad, "window": p.get("window"), "scale": p["scale"],
                                     "qk_norm": False, "kv_projection": p.get("kv_projection", True)}, spec.tensors)
        super().__init__(inner, runtime, position)
        self.spec = spec
        self.taps = int(p.get("taps") or 0)
        if self.taps > 64:
            raise ValueError(f"conv_gated_attention: {self.taps} taps (up to 64 are supported)")
        self.unit_norm = bool(p.get("unit_norm", True))
        self.eps = float(p.get("eps", 0.0))
        self.gate = bool(p.get("gate", True))
        self.bias_rows = int(p.get("bias_rows") or 0)
        self.bias_max = float(p.get("bias_max") or 0.0)
        if self.bias_rows and (self.bias_rows < 2 or self.bias_max <= self.bias_rows // 2):
            raise ValueError(f"conv_gated_attention: a distance bias of {self.bias_rows} rows needs bias_max above "
                             f"{self.bias_rows // 2}, got {self.bias_max}")
        cw = p.get("cache_window", p.get("window"))
        self.cache_window = int(cw) if cw else 0
        if self.window and self.cache_window and self.cache_window < self.window:
            raise ValueError("conv_gated_attention: the cache must keep at least the mixer's own window")
        self.q_cols = self.n_heads * self.dk
        self.kv_cols = self.n_kv * (self.dk + self.dv) if self.kv_projection else 0
        self.channels = self.q_cols + self.kv_cols                  # what the convolution runs over
        self.g_cols = self.n_heads * self.dv if self.gate else 0
        self.o_in = self.n_heads * self.dv
        rt = runtime
        rt.scratch("conv_proj", rt.max_batch_tokens, self.channels + self.g_cols)
        rt.scratch("gated_heads", rt.max_batch_tokens, self.o_in)
        self.w_in = self.w_conv = self.bias_table = self.bias_table_by_head = None

    # ---------------------------------------------------------------- weights
    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["q_proj"]: TensorNeed((self.q_cols, self.hidden)), t["o_proj"]: TensorNeed((self.hidden, self.o_in))}
        if self.kv_projection:
            needs[t["k_proj"]] = TensorNeed((self.n_kv * self.dk, self.hidden))
            needs[t["v_proj"]] = TensorNeed((self.n_kv * self.dv, self.hidden))
        if self.taps:
            needs[t["q_conv"]] = TensorNeed((self.q_cols, self.taps))
            if self.kv_projection:
                needs[t["k_conv"]] = TensorNeed((self.n_kv * self.dk, self.taps))
                needs[t["v_conv"]] = TensorNeed((self.n_kv * self.dv, self.taps))
        if self.gate:
            needs[t["g_proj"]] = TensorNeed((self.g_cols, self.hidden))
        if self.bias_rows:
            needs[t["rel"]] = TensorNeed((self.bias_rows, self.n_heads))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        kv = ("k", "v") if self.kv_projection else ()
        mats = [tensors[t["q_proj"]]] + [tensors[t[f"{n}_proj"]] for n in kv] + ([tensors[t["g_proj"]]] if self.gate else [])
        if len({m.dtype for m in mats}) != 1:
            raise ValueError("conv_gated_attention: the input projections must share an element type")
        # one [q | k | v | gate] matrix: the mixer's input is read by one product
        self.w_in = torch.cat(mats, dim=0).contiguous()
        self.w_o = tensors[t["o_proj"]].contiguous()
        if self.taps:
            conv = torch.cat([tensors[t["q_conv"]]] + [tensors[t[f"{n}_conv"]] for n in kv], dim=0)
            self.w_conv = conv.t().contiguous()                  # tap-major, as the kernel reads it
        if self.bias_rows:
            # by distance: the last row serves every distance from bias_max on (and none beyond the window is asked for)
            reach = self.window if self.window else self.runtime.max_positions
            n = max(1, min(reach, int(math.ceil(self.bias_max)) + 1))
            rows = torch.from_numpy(distance_rows(self.bias_rows, self.bias_max, n)).to(tensors[t["rel"]].device)
            self.bias_table = tensors[t["rel"]].to(torch.float32)[rows].contiguous()
            self.bias_table_by_head = self.bias_table.t().contiguous()      # the tcgen05 kernel's threads walk one head's row

    # ---------------------------------------------------------------- state
    def cache_need(self):
        return CacheNeed(self.n_kv, self.head_pad, self.cache_window or None)

    def state_need(self):
        return StateNeed((self.taps - 1) * self.channels, "float32") if self.taps > 1 else None

    def _distance_bias(self):
        return self.bias_table

    def _has_distance_bias(self):
        return bool(self.bias_rows)

    def flops_per_token(self) -> float:
        return 2.0 * self.hidden * (self.channels + self.g_cols + self.o_in)

    # ---------------------------------------------------------------- the step
    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T = self.runtime, ctx.n_tokens
        if call.writes_cache != self.kv_projection:
            raise RuntimeError("conv_gated_attention: a call projects keys and values exactly when it owns its cache")
        proj = rt.get_scratch("conv_proj")[:, : self.channels + self.g_cols]
        ops.linear(h, self.w_in, proj, T, status=ctx.status)
        q = rt.get_scratch("qkv")[:, : self.n_heads * self.head_pad]
        ops.conv_norm_kv_write(proj, self.w_conv, call.state, self.n_heads, self.n_kv, self.dk, self.dv, self.head_pad,
                               self.unit_norm, self.eps, q, call.cache, ctx.block_tables[call.cache_group], rt.page_size,
                               ctx.positions, ctx.seq_of_token, ctx.q_start, ctx.state_slots, T, ctx.n_seqs,
                               call.writes_cache, ctx.status)
        out = self._attend(q, ctx, call)
        gated = rt.get_scratch("gated_heads")[:, : self.o_in]
        ops.sigmoid_gate(out, proj[:, self.channels:] if self.gate else None, gated, self.n_heads, self.dv, self.head_pad, T)
        ops.linear(gated, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)
