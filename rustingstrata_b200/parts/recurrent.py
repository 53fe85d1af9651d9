"""Recurrent mixer with a real-gated linear recurrent unit (the recurrent block of Griffin).

Two branches of ``width`` channels from the mixer's input h: y = gelu_tanh(W_y h + b_y), and u = conv(W_x h + b_x), a
short causal convolution per channel.  u is cut into ``blocks`` equal parts; in part b the recurrence gate is
r = sigmoid(A_b u_b + a_b) and the input gate i = sigmoid(I_b u_b + i_b) (square matrices per part).  Per channel

    a_t = exp(-decay * r_t * softplus(lam)),    S_t = a_t S_(t-1) + sqrt(1 - a_t^2) * i_t * u_t,    S = 0 before the start,

and the mixer's output is W_o (S_t * y_t).  Per request the state slot keeps the convolution's last taps - 1 inputs
and S, both float32; gates, decays and the recurrence are float32 in both engines (the projections follow the engine).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import CallInfo, Mixer, StepContext
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
        self.conv_w, self.conv_bias = g("conv"), g("conv_bias")
        self.w_r, self.b_r = g("recurrence_gate"), g("recurrence_gate_bias")
        self.w_i, self.b_i = g("input_gate"), g("input_gate_bias")
        self.lam, self.w_o = g("lam"), g("o_proj")

    def state_need(self):
        return StateNeed(self.tail + self.width, "float32")

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
        ops.block_linear(u, self.w_r, gates[:, :W], T, self.bw, self.bw, bias=self.b_r)
        ops.block_linear(u, self.w_i, gates[:, W:], T, self.bw, self.bw, bias=self.b_i)
        ops.gated_linear_recurrence(gates, u, yx[:, :W], self.y_bias, self.lam, act, state[:, self.tail:], ctx.q_start,
                                    ctx.state_slots, ctx.n_seqs, self.decay)
        ops.linear(act, self.w_o, residual, T, accumulate=not ctx.store_output, status=ctx.status)
