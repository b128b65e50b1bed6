"""A gated linear recurrence behind a short causal convolution (the recurrent block of Griffin-like models).

Two branches of ``width`` channels read x: g = gelu_tanh(W_y x + b_y) and
u = conv(W_x x + b_x), a causal convolution per channel over the last ``taps``
inputs.  The channels are cut into ``blocks`` equal parts; in each part two
gates come from square matrices, r = sigmoid(A_b u_b + a_b) and
i = sigmoid(B_b u_b + b_b).  Then, per channel and in float32,

    a = exp(-decay * r * softplus(lam)),  S_t = a S_(t-1) + sqrt(1 - a^2) * i * u,

from S = 0, and the result is W_o (S * g).  S and the convolution's last
``taps - 1`` inputs are carried from step to step in the request's slot (one
float32 state [taps, width]: the inputs, oldest first, then S).  The two
branches are one product, the two gates one batched product.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, CacheView, FixedState, Mixer, ParamSpec, StepContext
from .registry import register_mixer


class GatedLinearRecurrence(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])
        self.blocks = int(params["blocks"])
        self.taps = int(params["taps"])
        self.decay = float(params.get("decay", 8.0))
        if self.width % self.blocks:
            raise ValueError(f"{self.width} channels cannot be cut into {self.blocks} equal blocks")
        self.w_in = self.w_gates = self.w_o = None
        self.bias_y = self.bias_x = self.bias_r = self.bias_i = self.conv_w = self.conv_b = self.lam = None

    def param_specs(self):
        w, bw = self.width, self.width // self.blocks
        return {
            "gate_proj": ParamSpec((w, self.hidden)), "gate_bias": ParamSpec((w,), role="vector", init="normal"),
            "in_proj": ParamSpec((w, self.hidden)), "in_bias": ParamSpec((w,), role="vector", init="normal"),
            "conv_weight": ParamSpec((w, self.taps), role="vector", init="normal"),
            "conv_bias": ParamSpec((w,), role="vector", init="normal"),
            "recurrence_gate": ParamSpec((self.blocks, bw, bw)),
            "recurrence_gate_bias": ParamSpec((self.blocks, bw), role="vector", init="normal"),
            "input_gate": ParamSpec((self.blocks, bw, bw)),
            "input_gate_bias": ParamSpec((self.blocks, bw), role="vector", init="normal"),
            "decay_param": ParamSpec((w,), role="vector", init="normal"),
            "o_proj": ParamSpec((self.hidden, w)),
        }

    def cache_need(self):
        return CacheNeed(state=FixedState((self.taps, self.width), torch.float32))

    def load(self, tensors, *, compute_dtype, device):
        f32 = dict(device=device, dtype=torch.float32)
        y, x = tensors["gate_proj"], tensors["in_proj"]
        dtype = torch.float32 if torch.float32 in (y.dtype, x.dtype) else y.dtype
        self.w_in = torch.cat([y.to(dtype), x.to(dtype)], dim=0).contiguous()
        r, i = tensors["recurrence_gate"], tensors["input_gate"]
        dtype = torch.float32 if torch.float32 in (r.dtype, i.dtype) else r.dtype
        self.w_gates = torch.cat([r.to(dtype), i.to(dtype)], dim=1).contiguous()  # [blocks, 2 * bw, bw]
        self.w_o = tensors["o_proj"].contiguous()
        self.bias_y = tensors["gate_bias"].to(**f32).contiguous()
        self.bias_x = tensors["in_bias"].to(**f32).contiguous()
        self.bias_r = tensors["recurrence_gate_bias"].to(**f32).reshape(-1).contiguous()
        self.bias_i = tensors["input_gate_bias"].to(**f32).reshape(-1).contiguous()
        self.conv_w = tensors["conv_weight"].to(**f32).contiguous()
        self.conv_b = tensors["conv_bias"].to(**f32).contiguous()
        self.lam = tensors["decay_param"].to(**f32).contiguous()

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if cache.state is None or not cache.writes:
            raise RuntimeError("a recurrent part needs the state of its own cache entry")
        t, bw = x.shape[0], self.width // self.blocks
        proj = ops.linear(x, self.w_in)                                   # [T, 2W]: gate branch, convolution branch
        u = ops.causal_conv(proj, self.bias_x, self.conv_w, self.conv_b, cache.state, ctx)
        gates = ops.linear_per_head(u.view(t, self.blocks, bw), self.w_gates, out_dtype=torch.float32)
        mixed = ops.recurrence_scan(proj, u, gates, self.bias_y, self.bias_x, self.bias_r, self.bias_i, self.lam, cache.state,
                                    ctx, blocks=self.blocks, decay=self.decay)
        return ops.linear(mixed, self.w_o)


register_mixer("gated_linear_recurrence", GatedLinearRecurrence, replace=True)
