"""Grouped-query attention whose scores carry a learned bias by distance, with an optional chunk mask, window and sink.

q, k, v come from one fused projection (no biases, no rotation); keys and values may have different sizes and are
appended to the request's pages as one row per token and key/value head.  Per query head h at position i and a key
at position j <= i:

    score = (q . k) * scale + rel[bucket(i - j), h]
    bucket(n) = n                                                       for n < B/2
              = min(B - 1, B/2 + floor(log(n / (B/2)) / log(D / (B/2)) * (B - B/2)))   otherwise

with B rows in the table ``rel`` and D = ``bias_reach``; the scale does not multiply the bias.  ``chunk``: i sees j
only if both lie in the same run of ``chunk`` positions counted from the start of the sequence.  ``window``: only
the last ``window`` keys.  ``sink``: a learned number per head whose exponential joins the softmax denominator once,
without a key or a value.  Softmax and the weighted sum are float32.

The bucket function is applied once, when the weights arrive: the kernels read a table of biases by distance,
[heads, reach], whose last column stands for every distance of reach - 1 and more.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from .base import CacheNeed, CacheView, Mixer, PagedKV, ParamSpec, StepContext
from .registry import register_mixer


def distance_bucket(n: int, rows: int, reach: int) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(reach / half) * (rows - half))))


class BiasedAttention(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.hq = int(params["num_heads"])
        self.hkv = int(params["num_kv_heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params.get("vdim") or self.dim)
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.dim))
        self.window = params.get("window")
        self.chunk = params.get("chunk")
        self.bias_rows = params.get("bias_rows")      # rows of the learned table; None: no distance bias
        self.bias_reach = params.get("bias_reach")    # the distance from which every key shares the last row
        self.has_sink = bool(params.get("sink", False))
        if self.hq % self.hkv:
            raise ValueError(f"{self.hq} query heads cannot share {self.hkv} key/value heads")
        if self.bias_rows is not None:
            self.bias_rows, self.bias_reach = int(self.bias_rows), int(self.bias_reach)
            if self.bias_rows < 2 or self.bias_reach <= self.bias_rows // 2:
                raise ValueError(f"a distance bias of {self.bias_rows} rows needs a reach beyond {self.bias_rows // 2}, not {self.bias_reach}")
        self.w_qkv = self.w_o = self.bias = self.sink = None

    def param_specs(self):
        specs = {"q_proj": ParamSpec((self.hq * self.dim, self.hidden)), "k_proj": ParamSpec((self.hkv * self.dim, self.hidden)),
                 "v_proj": ParamSpec((self.hkv * self.vdim, self.hidden))}
        if self.bias_rows is not None:
            specs["rel_bias"] = ParamSpec((self.bias_rows, self.hq), role="vector", init="normal")
        if self.has_sink:
            specs["sink"] = ParamSpec((self.hq,), role="vector", init="normal")
        specs["o_proj"] = ParamSpec((self.hidden, self.hq * self.vdim))
        return specs

    def cache_need(self):
        return CacheNeed(paged=PagedKV(self.hkv, self.dim + self.vdim, self.window, "natural", planes=1, chunk=self.chunk))

    def load(self, tensors, *, compute_dtype, device):
        pieces = [tensors["q_proj"], tensors["k_proj"], tensors["v_proj"]]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in pieces) else pieces[0].dtype
        self.w_qkv = torch.cat([p.to(dtype) for p in pieces], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()
        if self.bias_rows is not None:
            # by distance: every distance up to the one whose bucket is the last row, which then stands for all beyond
            reach = 1
            while distance_bucket(reach - 1, self.bias_rows, self.bias_reach) < self.bias_rows - 1:
                reach += 1
            rows = torch.tensor([distance_bucket(n, self.bias_rows, self.bias_reach) for n in range(reach)], device=device)
            rel = tensors["rel_bias"].to(device=device, dtype=torch.float32)
            self.bias = rel[rows].t().contiguous()  # [heads, reach]
        if self.has_sink:
            self.sink = tensors["sink"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if not cache.writes or cache.kv is None:
            raise RuntimeError("this attention part appends its own keys and values and needs its cache entry")
        qkv = ops.linear(x, self.w_qkv)
        o = ops.biased_attention(qkv, cache.kv, ctx.block_tables[cache.group], ctx, num_heads=self.hq, num_kv_heads=self.hkv,
                                 dim=self.dim, vdim=self.vdim, page_size=cache.page_size, scale=self.scale, window=self.window,
                                 chunk=self.chunk, bias=self.bias, sink=self.sink)
        return ops.linear(o, self.w_o)


register_mixer("biased_attention", BiasedAttention, replace=True)
