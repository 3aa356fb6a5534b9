"""A routed feed-forward: ``experts`` small feed-forwards down_e(act(up_e x)), of which each token uses ``top``.

Router: z = W_r x in float32, scores s = sigmoid(z).  The choice is made on s + correction (a learned offset per
expert), the weights on s.  With ``groups`` > 1 the experts form that many equal groups of neighbours; a group's score
is the sum of its two largest choice scores and only experts of the ``keep`` best groups can be chosen.  The weights
of the chosen experts are their s divided by the sum of those (+ 1e-20), times ``scale``.  A shared expert of the same
form (``shared_size``) may run for every token; its output is multiplied by sigmoid(w_sg . x), one number per token.

Options, each a parameter: ``scores`` "softmax" (s = softmax(z) over all experts) instead of "sigmoid";
``group_score`` "max" (a group counts by its largest choice score) instead of "top2"; ``normalize`` False (the weights
are the chosen s as they are, times ``scale``); ``activation`` "clipped_swiglu": gated experts (and shared expert),
y = g * sigmoid(alpha g) * (u + offset) with g = min(gate_e x, limit), u = clamp(up_e x, -limit, limit) and tensors
``gate_proj`` beside ``up_proj`` (``limit``, ``shared_limit``, ``gate_alpha``, ``up_offset``); ``shared_gate`` False: the
shared expert's output is added as it is.

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
        self.gated = self.activation == "clipped_swiglu"
        if self.gated:
            self.limit = float(params["limit"])
            self.shared_limit = float(params.get("shared_limit") or self.limit)
            self.gate_alpha = float(params.get("gate_alpha", 1.702))
            self.up_offset = float(params.get("up_offset", 1.0))
            if not (self.limit > 0 and self.shared_limit > 0):
                raise ValueError("clipped_swiglu needs positive limits")
        elif self.activation not in ops.UNARY_ACTIVATIONS or self.activation not in ops.MOE_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not built for routed experts")
        self.scores = str(params.get("scores", "sigmoid"))
        self.group_score = str(params.get("group_score", "top2"))
        self.normalize = bool(params.get("normalize", True))
        if self.scores not in ("sigmoid", "softmax") or self.group_score not in ("top2", "max"):
            raise ValueError(f"router scores {self.scores!r} / group score {self.group_score!r} are not built")
        if self.experts % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"{self.experts} experts cannot form {self.groups} equal groups of which {self.keep} are kept")
        if self.top > self.keep * (self.experts // self.groups):
            raise ValueError(f"{self.keep} groups of {self.experts // self.groups} experts cannot give {self.top} choices")
        self.w_up = self.w_down = self.w_router = self.correction = self.shared_up = self.shared_down = None

    def param_specs(self):
        specs = {}
        for e in range(self.experts):
            if self.gated:
                specs[f"experts.{e}.gate_proj"] = ParamSpec((self.inter, self.hidden))
            specs[f"experts.{e}.up_proj"] = ParamSpec((self.inter, self.hidden))
            specs[f"experts.{e}.down_proj"] = ParamSpec((self.hidden, self.inter))
        specs["router"] = ParamSpec((self.experts, self.hidden))
        if self.has_correction:
            specs["correction"] = ParamSpec((self.experts,), role="vector", init="normal")
        if self.shared_size is not None:
            if self.gated:
                specs["shared.gate_proj"] = ParamSpec((int(self.shared_size), self.hidden))
            specs["shared.up_proj"] = ParamSpec((int(self.shared_size), self.hidden))
            specs["shared.down_proj"] = ParamSpec((self.hidden, int(self.shared_size)))
            if self.shared_gated:
                specs["shared.gate"] = ParamSpec((1, self.hidden))
        return specs

    def load(self, tensors, *, compute_dtype, device):
        ups = [tensors[f"experts.{e}.up_proj"] for e in range(self.experts)]
        downs = [tensors[f"experts.{e}.down_proj"] for e in range(self.experts)]
        gates = [tensors[f"experts.{e}.gate_proj"] for e in range(self.experts)] if self.gated else []
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in ups + downs + gates) else ups[0].dtype
        if self.gated:  # an expert's gate rows, then its up rows: one product gives both branches
            ups = [torch.cat([g.to(dtype), u.to(dtype)], dim=0) for g, u in zip(gates, ups)]
        self.w_up = torch.stack([p.to(dtype) for p in ups]).contiguous()       # [E, ff (or 2 ff), H]
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
            if self.gated:
                g, u = tensors["shared.gate_proj"], self.shared_up
                dtype = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
                self.shared_up = torch.cat([g.to(dtype), u.to(dtype)], dim=0).contiguous()
            self.shared_down = tensors["shared.down_proj"].contiguous()

    def forward(self, x, ctx: StepContext):
        z = ops.linear(x, self.w_router, out_dtype=torch.float32)  # [T, experts (+1: the shared expert's gate)]
        chosen, weight = ops.moe_route(z, self.correction, experts=self.experts, top=self.top, groups=self.groups,
                                       keep=self.keep, scale=self.scale, scores=self.scores, group_score=self.group_score,
                                       normalize=self.normalize)
        shared = gate = None
        if self.shared_size is not None:
            if self.gated:
                act = ops.clipped_gated_linear(x, self.shared_up, self.shared_limit, self.gate_alpha, self.up_offset)
            else:
                act = ops.activation(ops.linear(x, self.shared_up), self.activation)
            shared = ops.linear(act, self.shared_down)
            if self.shared_gated:
                gate = z[:, self.experts:]
        if self.gated:
            return ops.moe_experts(x, chosen, weight, self.w_up, self.w_down, activation=None, shared=shared, shared_gate=gate,
                                   glu=(self.limit, self.gate_alpha, self.up_offset))
        return ops.moe_experts(x, chosen, weight, self.w_up, self.w_down, activation=self.activation, shared=shared,
                               shared_gate=gate)


register_ffn("routed_experts", RoutedExperts, replace=True)
