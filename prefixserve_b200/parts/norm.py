"""RMSNorm, fused with the residual sum that precedes it.

y = gain * (x * rsqrt(mean(x^2) + eps)), everything in float32
(prefixserve/model/llama.py:63-69).  The residual stream is float32; the
pending output of the previous sublayer is added in the same kernel that
normalises (prefixserve/model/llama.py:117,:119,:121).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Norm, ParamSpec, StepContext
from .registry import register_norm


class RMSNorm(Norm):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_pending_products = True  # ``delta`` may be an ops.PendingProduct (a product that has not run yet)

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        # zero_centred: the checkpoint stores the gain as an offset from one (the rows are multiplied by 1 + weight)
        self.zero_centred = bool(params.get("zero_centred", False))
        self.gain: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), role="vector", init="normal" if self.zero_centred else "ones")}

    def load(self, tensors, *, compute_dtype, device):
        gain = tensors["weight"].to(device=device, dtype=torch.float32)
        self.gain = (1.0 + gain if self.zero_centred else gain).contiguous()

    def forward(self, h, delta, ctx: StepContext, rows=None):
        if isinstance(delta, ops.PostNormed):  # the pending result brings a norm of its own: both norms in one kernel
            return ops.norm_add_norm(h, delta.y, delta.gain, delta.eps, self.gain, self.eps, ctx.compute_dtype, rows)
        return ops.add_rmsnorm(h, delta, self.gain, self.eps, ctx.compute_dtype, rows)

    def post(self, y) -> "ops.PostNormed":
        """This norm on a sublayer's result y, to be added to the stream by whoever meets it next."""
        return ops.PostNormed(y, self.gain, self.eps)

    def add_normed(self, h, y, ctx: StepContext, *, gate=None, gate_bias=None, scale: float = 1.0):
        """The norm on a sublayer's result instead of its input: h += scale * norm(y * sigmoid(gate + gate_bias)) in
        place (``gate`` None: norm(y)).  Returns the new stream in the compute type for the next sublayer's products
        (h itself on the float32 path)."""
        copy = ops.gated_norm_add(h, y, gate, gate_bias, self.gain, self.eps, scale, ctx.compute_dtype)
        return h if copy is None else copy

    def defer(self, h, delta, ctx: StepContext, rows=None):
        if isinstance(delta, ops.PostNormed):
            return ops.NormedRows.ready(self.forward(h, delta, ctx, rows), h)
        return ops.NormedRows(h, delta, self.gain, self.eps, ctx.compute_dtype, rows)


register_norm("rms", RMSNorm, replace=True)
