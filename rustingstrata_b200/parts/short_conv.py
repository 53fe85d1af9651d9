"""Short causal convolution over time on each channel, with the last inputs kept per request.

out[t] = (x[t] if add_input) + bias + sum_j w[:, j] * x[t - (taps - 1) + j], zeros before a sequence's start.  The
last taps - 1 inputs of every request live in its state slot, so a sequence may be cut into steps anywhere.  Used as
a layer's input convolution (a block's ``input_conv`` role: what the mixer reads becomes h + conv(h)) and, through
:func:`rustingstrata_b200.kernels.ops.short_conv`, inside recurrent mixers.
"""
from __future__ import annotations

from ..kernels import ops
from .base import CallInfo, Mixer, StepContext
from .registry import register_part
from .spec import StateNeed, TensorNeed


@register_part("mixer", "short_conv")
class ShortConv(Mixer):
    """params: channels, taps, add_input (bool), bias (bool).  tensors: weight [channels, taps], and bias [channels].
    ``forward(h, out, ctx, call)`` stores into ``out`` (never adds: it feeds a mixer, not the stream)."""

    def __init__(self, spec, runtime, position=None):
        super().__init__(spec, runtime)
        p = spec.params
        self.channels = int(p["channels"])
        self.taps = int(p["taps"])
        self.add_input = bool(p.get("add_input", False))
        self.has_bias = bool(p.get("bias", False))
        if not 1 <= self.taps <= 17:
            raise ValueError(f"short_conv: {self.taps} taps (1 to 17 are supported)")
        self.weight = self.bias = None

    def tensor_needs(self):
        t = self.spec.tensors
        needs = {t["weight"]: TensorNeed((self.channels, self.taps))}
        if self.has_bias:
            needs[t["bias"]] = TensorNeed((self.channels,))
        return needs

    def load(self, tensors):
        t = self.spec.tensors
        self.weight = tensors[t["weight"]].t().contiguous()            # tap-major, as the kernel reads it
        self.bias = tensors[t["bias"]].contiguous() if self.has_bias else None

    def state_need(self):
        return StateNeed(max(1, (self.taps - 1) * self.channels), "float32")

    def forward(self, h, out, ctx: StepContext, call: CallInfo):
        ops.short_conv(h, self.weight, out, call.state, ctx.seq_of_token, ctx.q_start, ctx.state_slots, ctx.n_tokens,
                       ctx.n_seqs, bias=self.bias, add_input=self.add_input)
