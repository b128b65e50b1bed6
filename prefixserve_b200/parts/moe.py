"""A routed feed-forward: ``experts`` small feed-forwards down_e(act(up_e x)), of which each token uses ``top``.

Router: z = W_r x in float32, scores s = sigmoid(z).  The choice is made on s + correction (a learned offset per
expert), the weights on s.  With ``groups`` > 1 the experts form that many equal groups of neighbours; a group's score
is the sum of its two largest choice scores and only experts of the ``keep`` best groups can be chosen.  The weights
of the chosen experts are their s divided by the sum of those (+ 1e-20), times ``scale``.  A shared expert of the same
form (``shared_size``) may run for every token; its output is multiplied by sigmoid(w_sg . x), one number per token.

The router and the shared expert's gate are one product with float32 sums and float32 output.  The chosen (token, expert) pairs are grouped by
expert on the device and every expert multiplies its own rows only; nothing of the routing comes back to the host.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, ParamSpec, StepContext
from .registry import register_ffn


class RoutedExperts(FeedForward):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.experts = int(params["experts"])
        self.inter = int(params["expert_size"])
        self.top = int(params["top"])
        self.groups = int(params.get("groups") or 1)
        self.keep = int(params.get("keep") or self.groups)
        self.scale = float(params.get("scale", 1.0))
        self.has_correction = bool(params.get("correction", True))
        self.shared_size = params.get("shared_size")
        self.shared_gated = bool(params.get("shared_gate", True)) and self.shared_size is not None
        self.activation = str(params.get("activation", "relu2"))
        if self.activation not in ops.UNARY_ACTIVATIONS or self.activation not in ops.MOE_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not built for routed experts")
        if self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.experts} experts cannot form {self.groups} equal groups of which {self.keep} are kept")
        if self.top > self.keep * (self.experts // self.groups):
            raise ValueError(f"{self.keep} groups of {self.experts // self.groups} experts cannot give {self.top} choices")
        self.w_up = self.w_down = self.w_router = self.correction = self.shared_up = self.shared_down = None

    def param_specs(self):
        specs = {}
        for e in range(self.experts):
            specs[f"experts.{e}.up_proj"] = ParamSpec((self.inter, self.hidden))
            specs[f"experts.{e}.down_proj"] = ParamSpec((self.hidden, self.inter))
        specs["router"] = ParamSpec((self.experts, self.hidden))
        if self.has_correction:
            specs["correction"] = ParamSpec((self.experts,), role="vector", init="normal")
        if self.shared_size is not None:
            specs["shared.up_proj"] = ParamSpec((int(self.shared_size), self.hidden))
            specs["shared.down_proj"] = ParamSpec((self.hidden, int(self.shared_size)))
            if self.shared_gated:
                specs["shared.gate"] = ParamSpec((1, self.hidden))
        return specs

    def load(self, tensors, *, compute_dtype, device):
        ups = [tensors[f"experts.{e}.up_proj"] for e in range(self.experts)]
        downs = [tensors[f"experts.{e}.down_proj"] for e in range(self.experts)]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in ups + downs) else ups[0].dtype
        self.w_up = torch.stack([p.to(dtype) for p in ups]).contiguous()       # [E, ff, H]
        self.w_down = torch.stack([p.to(dtype) for p in downs]).contiguous()   # [E, H, ff]
        # The router's rows (and the shared expert's gate, one more row) keep the type they arrive in: bfloat16 weights
        # against bfloat16 rows multiply exactly and are summed in float32, and the logits leave the product as float32.
        rows = [tensors["router"]] + ([tensors["shared.gate"]] if self.shared_gated else [])
        dtype = torch.float32 if any(r.dtype == torch.float32 for r in rows) else rows[0].dtype
        self.w_router = torch.cat([r.to(dtype) for r in rows], dim=0).contiguous()
        if self.has_correction:
            self.correction = tensors["correction"].to(device=device, dtype=torch.float32).contiguous()
        if self.shared_size is not None:
            self.shared_up = tensors["shared.up_proj"].contiguous()
            self.shared_down = tensors["shared.down_proj"].contiguous()

    def forward(self, x, ctx: StepContext):
        z = ops.linear(x, self.w_router, out_dtype=torch.float32)  # [T, experts (+1: the shared expert's gate)]
        chosen, weight = ops.moe_route(z, self.correction, experts=self.experts, top=self.top, groups=self.groups,
                                       keep=self.keep, scale=self.scale)
        shared = gate = None
        if self.shared_size is not None:
            shared = ops.linear(ops.activation(ops.linear(x, self.shared_up), self.activation), self.shared_down)
            if self.shared_gated:
                gate = z[:, self.experts:]
        return ops.moe_experts(x, chosen, weight, self.w_up, self.w_down, activation=self.activation, shared=shared,
                               shared_gate=gate)


register_ffn("routed_experts", RoutedExperts, replace=True)
