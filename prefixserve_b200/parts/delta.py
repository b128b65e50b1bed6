"""The gated delta rule: a linear-attention mixer with a matrix state per head.

From the input x: q = W_q x and k = W_k x (``groups`` heads of ``dim``), v = W_v x (``heads`` heads of ``vdim``; head h
reads q/k group h // (heads / groups)), an output gate W_g x, and per head a write strength and a decay.  q, k and v
each pass a short causal convolution per channel (``taps`` inputs, no bias) and SiLU; q and k are then made unit
vectors per group (x / sqrt(sum x^2 + 1e-6)) and q is multiplied by dim^-1/2.  With beta = sigmoid(W_b x) and
decay = exp(-exp(A_log) * softplus(W_a x + dt_bias)), per head and token, in float32:

    S <- decay S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q

The read-out o is divided by its root mean square over vdim, multiplied by a gain shared by the heads and by
silu(W_g x), and projected by W_o.  A request carries S and the convolution's last taps - 1 inputs in its slot (one
float32 state: the inputs [taps - 1, channels], oldest first, then S [heads, dim, vdim]); a fresh slot is zeros.
The four wide projections are one product; the two narrow ones another, kept in float32.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, CacheView, FixedState, Mixer, ParamSpec, StepContext
from .registry import register_mixer


class GatedDeltaRule(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.groups = int(params["num_kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.taps = int(params["taps"])
        self.eps = float(params["eps"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads cannot share {self.groups} query/key groups")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.channels = 2 * self.groups * self.dim + self.heads * self.vdim
        self.w_in = self.w_gates = self.w_o = self.conv = self.a_log = self.dt_bias = self.gain = None

    def param_specs(self):
        qk, v = self.groups * self.dim, self.heads * self.vdim
        return {
            "q_proj": ParamSpec((qk, self.hidden)), "q_conv": ParamSpec((qk, self.taps), role="vector", init="normal"),
            "k_proj": ParamSpec((qk, self.hidden)), "k_conv": ParamSpec((qk, self.taps), role="vector", init="normal"),
            "v_proj": ParamSpec((v, self.hidden)), "v_conv": ParamSpec((v, self.taps), role="vector", init="normal"),
            "beta_proj": ParamSpec((self.heads, self.hidden)),
            "decay_rate": ParamSpec((self.heads,), role="vector", init="normal"),
            "out_norm": ParamSpec((self.vdim,), role="vector", init="ones"),
            "decay_proj": ParamSpec((self.heads, self.hidden)),
            "decay_bias": ParamSpec((self.heads,), role="vector", init="normal"),
            "gate_proj": ParamSpec((v, self.hidden)),
            "o_proj": ParamSpec((self.hidden, v)),
        }

    def cache_need(self):
        return CacheNeed(state=FixedState(((self.taps - 1) * self.channels + self.heads * self.dim * self.vdim,), torch.float32))

    def load(self, tensors, *, compute_dtype, device):
        f32 = dict(device=device, dtype=torch.float32)
        wide = [tensors["q_proj"], tensors["k_proj"], tensors["v_proj"], tensors["gate_proj"]]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in wide) else wide[0].dtype
        self.w_in = torch.cat([p.to(dtype) for p in wide], dim=0).contiguous()
        narrow = [tensors["beta_proj"], tensors["decay_proj"]]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in narrow) else narrow[0].dtype
        self.w_gates = torch.cat([p.to(dtype) for p in narrow], dim=0).contiguous()  # [2 * heads, hidden]
        self.w_o = tensors["o_proj"].contiguous()
        self.conv = torch.cat([tensors["q_conv"].to(**f32), tensors["k_conv"].to(**f32), tensors["v_conv"].to(**f32)], dim=0).contiguous()
        self.a_log = tensors["decay_rate"].to(**f32).contiguous()
        self.dt_bias = tensors["decay_bias"].to(**f32).contiguous()
        self.gain = tensors["out_norm"].to(**f32).contiguous()

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if cache.state is None or not cache.writes:
            raise RuntimeError("a recurrent part needs the state of its own cache entry")
        proj = ops.linear(x, self.w_in)                                   # [T, q | k | v | gate]
        gates = ops.linear(x, self.w_gates, out_dtype=torch.float32)      # [T, beta | decay] pre-activations, float32
        mixed = ops.delta_rule(proj, gates, self.conv, self.a_log, self.dt_bias, self.gain, cache.state, ctx,
                               groups=self.groups, heads=self.heads, dim=self.dim, vdim=self.vdim, eps=self.eps)
        return ops.linear(mixed, self.w_o)


register_mixer("gated_delta_rule", GatedDeltaRule, replace=True)
