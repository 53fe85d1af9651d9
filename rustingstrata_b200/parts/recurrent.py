"""Recurrent mixer with a real-gated linear recurrent unit (the recurrent block of Griffin).

Two branches of ``width`` channels from the mixer's input h: y = gelu_tanh(W_y h + b_y), and u = conv(W_x h + b_x), a
short causal convolution per channel.  u is cut into ``blocks`` equal parts; in part b the recurrence gate is
r = sigmoid(A_b u_b + a_b) and the input gate i = sigmoid(I_b u_b + i_b) (square matrices per part).  Per channel

    a_t = exp(-decay * r_t * softplus(lam)),    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,    S = 0 before the start,

and the mixer's output is W_o (S_t * y_t).  Per request the state slot keeps the convolution's last taps - 1 inputs
and S, both float32; gates, decays and the recurrence are float32 in both engines (the projections follow the engine).
"""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import ops
from .base import CallInfo, HostBatch, Mixer, StepContext
from .registry import register_part
from .spec import StateNeed, TensorNeed


@register_part("mixer", "rglru")
class GatedLinearRecurrence(Mixer):
    """params: hidden, width, blocks, taps, decay (the constant in the exponent, 8 in Griffin).
    tensors: y_proj, y_bias, x_proj, x_bias, conv, conv_bias, recurrence_gate [blocks, w, w], recurrence_gate_bias
    [blocks, w], input_gate, input_gate_bias, lam [width], o_proj."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.hidden = int(p["hidden"])
        self.width = int(p["width"])
        self.blocks = int(p["blocks"])
        self.taps = int(p["taps"])
        self.decay = float(p.get("decay", 8.0))
        if self.width % self.blocks:
            raise ValueError(f"rglru: width {self.width} is not a multiple of {self.blocks} blocks")
        if not 1 <= self.taps <= 17:
            raise ValueError(f"rglru: {self.taps} taps (1 to 17 are supported)")
        self.bw = self.width // self.blocks
        self.tail = (self.taps - 1) * self.width
        rt = runtime
        rt.scratch("rglru_yx", rt.max_batch_tokens, 2 * self.width, torch.float32)
        rt.scratch("rglru_u", rt.max_batch_tokens, self.width, torch.float32)
        rt.scratch("rglru_gates", rt.max_batch_tokens, 2 * self.width, torch.float32)
        rt.scratch("rglru_act", rt.max_batch_tokens, self.width)
        max_chunks = rt.max_batch_tokens // self.SCAN_CHUNK + rt.max_seqs
        rt.scratch("rglru_scan", 1, 3 * max_chunks * self.width, torch.float32)

    def tensor_needs(self):
        t, W, B, bw = self.spec.tensors, self.width, self.blocks, self.bw
        return {t["y_proj"]: TensorNeed((W, self.hidden)), t["y_bias"]: TensorNeed((W,)),
                t["x_proj"]: TensorNeed((W, self.hidden)), t["x_bias"]: TensorNeed((W,)),
                t["conv"]: TensorNeed((W, self.taps)), t["conv_bias"]: TensorNeed((W,)),
                t["recurrence_gate"]: TensorNeed((B, bw, bw)), t["recurrence_gate_bias"]: TensorNeed((B, bw)),
                t["input_gate"]: TensorNeed((B, bw, bw)), t["input_gate_bias"]: TensorNeed((B, bw)),
                t["lam"]: TensorNeed((W,)), t["o_proj"]: TensorNeed((self.hidden, W))}

    def load(self, tensors):
        t = self.spec.tensors
        g = lambda k: tensors[t[k]].contiguous()                              # noqa: E731
        self.w_yx = torch.cat([tensors[t["y_proj"]], tensors[t["x_proj"]]], dim=0).contiguous()    # one product for both branches
        self.y_bias, self.x_bias = g("y_bias"), g("x_bias")
        self.conv_w, self.conv_bias = tensors[t["conv"]].t().contiguous(), g("conv_bias")     # tap-major
        # per block the recurrence gate's matrix on top of the input gate's: one block-diagonal product for both
        self.w_gates = torch.cat([tensors[t["recurrence_gate"]], tensors[t["input_gate"]]], dim=1).contiguous()
        self.b_gates = torch.cat([tensors[t["recurrence_gate_bias"]], tensors[t["input_gate_bias"]]], dim=1).contiguous()
        self.lam, self.w_o = g("lam"), g("o_proj")

    def state_need(self):
        return StateNeed(self.tail + self.width, "float32")

    # Portions longer than SCAN_CHUNK tokens are cut into chunks that run side by side (the recurrence is linear in S,
    # so a chunk is a map S -> A S + B); shorter ones, and single tokens, take one thread per channel.
    SCAN_CHUNK = 32

    def plan_key(self):
        return ("recurrence_chunks", self.SCAN_CHUNK)

    def build_plan(self, batch: HostBatch):
        L = self.SCAN_CHUNK
        if batch.bucketed or int(batch.q_lens.max()) <= L:
            return {"n_chunks": 0}
        per_seq = (batch.q_lens + L - 1) // L
        first = np.zeros(batch.n_seqs + 1, np.int32)
        np.cumsum(per_seq, out=first[1:])
        seq = np.repeat(np.arange(batch.n_seqs, dtype=np.int32), per_seq)
        start = (np.arange(int(first[-1]), dtype=np.int32) - np.repeat(first[:-1], per_seq)) * L
        return {"chunk_seq": seq, "chunk_start": start.astype(np.int32), "seq_first_chunk": first, "n_chunks": int(first[-1]),
                "chunk_len": L}

    def flops_per_token(self) -> float:
        return 2.0 * (3 * self.width * self.hidden + 2 * self.width * self.bw)

    def forward(self, h, residual, ctx: StepContext, call: CallInfo):
        rt, T, W = self.runtime, ctx.n_tokens, self.width
        yx = rt.get_scratch("rglru_yx", torch.float32)[:, : 2 * W]
        u = rt.get_scratch("rglru_u", torch.float32)[:, :W]
        gates = rt.get_scratch("rglru_gates", torch.float32)[:, : 2 * W]
        act = rt.get_scratch("rglru_act")[:, :W]
        ops.linear(h, self.w_yx, yx, T, status=ctx.status)
        state = call.state
        conv_state = state[:, : max(1, self.tail)]
        ops.short_conv(yx[:, W:], self.conv_w, u, conv_state, ctx.seq_of_token, ctx.q_start, ctx.state_slots, T, ctx.n_seqs,
                       in_bias=self.x_bias, bias=self.conv_bias)
        ops.block_linear(u, self.w_gates, gates, T, self.bw, 2 * self.bw, bias=self.b_gates)
        plan = ctx.plans[self.plan_key()]
        chunks = dict(plan, work=rt.get_scratch("rglru_scan", torch.float32).view(-1)) if plan["n_chunks"] else None
        ops.gated_linear_recurrence(gates, u, yx[:, :W], self.y_bias, self.lam, act, state[:, self.tail:], ctx.q_start,
                                    ctx.state_slots, ctx.n_seqs, self.decay, chunks=chunks, block_width=self.bw)
        ops.linear(act, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)
