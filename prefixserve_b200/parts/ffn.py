"""Gated feed-forward: down(act(gate(x)) * up(x)), gate and up fused into one
matrix (prefixserve/model/llama.py:120-121, prefixserve/model/weights.py:120-123).

``activation``: ``silu``, ``gelu_tanh``, or ``clipped_swiglu``, in which both branches are clipped before they meet:
g = min(gate, limit), u = clamp(up, -limit, limit), and the product is g * sigmoid(alpha * g) * (u + offset)
(``limit`` required; ``gate_alpha`` defaults to 1.702 and ``up_offset`` to 1)."""

from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, ParamSpec, StepContext
from .registry import register_ffn


class GatedMLP(FeedForward):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_deferred_input = True  # x goes to one product only, which may do the norm in front of it itself

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        self.clipped = self.activation == "clipped_swiglu"
        if self.clipped:
            self.limit = float(params["limit"])
            self.gate_alpha = float(params.get("gate_alpha", 1.702))
            self.up_offset = float(params.get("up_offset", 1.0))
            if not self.limit > 0:
                raise ValueError(f"clipped_swiglu needs a positive limit, not {self.limit}")
        elif self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not built (one of {sorted(ops.ACTIVATIONS) + ['clipped_swiglu']})")
        self.w_gate_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None

    def param_specs(self):
        return {
            "gate_proj": ParamSpec((self.inter, self.hidden)),
            "up_proj": ParamSpec((self.inter, self.hidden)),
            "down_proj": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors, *, compute_dtype, device):
        g, u = tensors["gate_proj"], tensors["up_proj"]
        dtype = torch.float32 if torch.float32 in (g.dtype, u.dtype) else g.dtype
        self.w_gate_up = torch.cat([g.to(dtype), u.to(dtype)], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def forward(self, x, ctx: StepContext):
        if self.clipped:
            act = ops.clipped_gated_linear(x, self.w_gate_up, self.limit, self.gate_alpha, self.up_offset)
            return ops.last_product(act, self.w_down, ctx)
        return ops.last_product(ops.gated_linear(x, self.w_gate_up, self.activation), self.w_down, ctx)


class DenseMLP(FeedForward):
    """Feed-forward without a gate branch: down(act(up(x))).  ``activation``: silu, gelu_tanh, or xielu, which brings
    two learned numbers of its own (tensor ``act`` [2])."""

    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "gelu_tanh"))
        if self.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"activation {self.activation!r} is not built (one of {sorted(ops.UNARY_ACTIVATIONS)})")
        self.w_up: torch.Tensor | None = None
        self.w_down: torch.Tensor | None = None
        self.act_params: torch.Tensor | None = None

    def param_specs(self):
        specs = {"up_proj": ParamSpec((self.inter, self.hidden)), "down_proj": ParamSpec((self.hidden, self.inter))}
        if self.activation == "xielu":
            specs["act"] = ParamSpec((2,), role="vector", init="normal")
        return specs

    def load(self, tensors, *, compute_dtype, device):
        self.w_up = tensors["up_proj"].contiguous()
        self.w_down = tensors["down_proj"].contiguous()
        if self.activation == "xielu":
            self.act_params = tensors["act"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, ctx: StepContext):
        return ops.linear(ops.activation(ops.linear(x, self.w_up), self.activation, self.act_params), self.w_down)


register_ffn("gated_mlp", GatedMLP, replace=True)
register_ffn("mlp", DenseMLP, replace=True)
