"""RMSNorm: out = x * rsqrt(mean(x^2) + eps) * w   (reference src/ops.rs:3-7; device
src/cuda/kernels.cu:1504-1552).  ``eps`` and the width are parameters.  Two kinds: ``rmsnorm`` with one weight per
coordinate and ``rmsnorm_scalar`` with one number for all coordinates.  Both can also norm a sublayer's output on
its way into the residual stream (``forward_add``: x += norm(delta)), fused with the norm of the stream's next
reader when that is one of these two kinds."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Norm
from .registry import register_part
from .spec import TensorNeed


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: width, eps.  tensors: weight."""
    chain_safe = True
    takes_owed = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.width = int(spec.params["width"])
        self.eps = float(spec.params["eps"])
        self.weight = None

    def tensor_needs(self):
        return {self.spec.tensors["weight"]: TensorNeed((self.width,), "norm")}

    def load(self, tensors):
        self.weight = tensors[self.spec.tensors["weight"]].contiguous()

    def forward(self, x, out, n_rows, rows=None, owed=None):
        ops.rmsnorm(x, self.weight, self.eps, out, rows=rows, n_rows=n_rows, pending=owed)

    def forward_add(self, delta, x, n_rows, then=None, out=None):
        if then is not None and isinstance(then, RMSNorm) and then.width == self.width:
            ops.rmsnorm_add(x, delta, self.gain, self.eps, n_rows, then.gain, then.eps, out)
            return
        ops.rmsnorm_add(x, delta, self.gain, self.eps, n_rows)
        if then is not None:
            then.forward(x, out, n_rows)

    @property
    def gain(self):
        """What multiplies the normed row: [width] values (one value for the scalar kind)."""
        return self.weight


@register_part("norm", "rmsnorm_scalar")
class ScalarRMSNorm(RMSNorm):
    """params: width, eps.  tensors: weight (a single number that scales every coordinate)."""

    def tensor_needs(self):
        return {self.spec.tensors["weight"]: TensorNeed((), "norm")}

    def load(self, tensors):
        self._gain = tensors[self.spec.tensors["weight"]].reshape(1).contiguous()
        # the row kernels shared with the vector kind read one weight per coordinate
        self.weight = self._gain.expand(self.width).contiguous()

    @property
    def gain(self):
        return self._gain
