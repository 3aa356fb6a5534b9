"""minGRU: a gated recurrence whose gates read only the current token.

Three projections of the input, ``width`` channels each: z = sigmoid(W_z x + b_z), u = W_x x + b_x, g = W_g x.  The
candidate is u + 1/2 where u >= 0 and sigmoid(u) where u < 0 (a positive function with a continuous slope).  Per
channel and in float32,

    S_t = (1 - z_t) S_(t-1) + z_t candidate_t,        from S = 0,

and the result is W_o (S_t * silu(g_t)).  S is carried from step to step in the request's slot (float32 [width]).
The three projections are one product; gates, candidate and state are float32 whatever the products' type.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, CacheView, FixedState, Mixer, ParamSpec, StepContext
from .registry import register_mixer


class MinGRU(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.width = int(params["width"])
        self.w_in = self.w_o = self.bias_z = self.bias_x = None

    def param_specs(self):
        w = self.width
        return {
            "update_proj": ParamSpec((w, self.hidden)), "update_bias": ParamSpec((w,), role="vector", init="normal"),
            "candidate_proj": ParamSpec((w, self.hidden)), "candidate_bias": ParamSpec((w,), role="vector", init="normal"),
            "gate_proj": ParamSpec((w, self.hidden)),
            "o_proj": ParamSpec((self.hidden, w)),
        }

    def cache_need(self):
        return CacheNeed(state=FixedState((self.width,), torch.float32))

    def load(self, tensors, *, compute_dtype, device):
        pieces = [tensors["update_proj"], tensors["candidate_proj"], tensors["gate_proj"]]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in pieces) else pieces[0].dtype
        self.w_in = torch.cat([p.to(dtype) for p in pieces], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()
        self.bias_z = tensors["update_bias"].to(device=device, dtype=torch.float32).contiguous()
        self.bias_x = tensors["candidate_bias"].to(device=device, dtype=torch.float32).contiguous()

    def input_weight(self) -> torch.Tensor:
        """The one matrix this mixer applies to its input first (see ``side_by_side``)."""
        return self.w_in

    def forward_projected(self, proj, ctx: StepContext, cache: CacheView):
        if cache.state is None or not cache.writes:
            raise RuntimeError("a recurrent part needs the state of its own cache entry")
        mixed = ops.min_gru(proj, self.bias_z, self.bias_x, cache.state, ctx, width=self.width)
        return ops.last_product(mixed, self.w_o, ctx)

    def forward(self, x, ctx: StepContext, cache: CacheView):
        return self.forward_projected(ops.linear(x, self.w_in), ctx, cache)


register_mixer("min_gru", MinGRU, replace=True)
