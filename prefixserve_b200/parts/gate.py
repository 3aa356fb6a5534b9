"""Gates on a sublayer's result.

``sigmoid_linear``: the result is multiplied, element by element, by
sigmoid(W x + b) of the sublayer's input x.  The part computes W x; the bias
and the sigmoid are applied by the kernel that also norms the gated result and
adds it to the stream (``Norm.add_normed``).

``channel_scale``: a learned factor per channel on a sublayer's result (``weight`` [size]), applied in float32 where
the result joins the stream.  It has no input of its own: the block reads ``weight`` and wraps the sublayer's result
(``ops.Affine``).
"""

from __future__ import annotations

import torch

from .. import ops
from .base import Gate, ParamSpec, StepContext
from .registry import register_gate


class SigmoidLinearGate(Gate):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.has_bias = bool(params.get("bias", True))
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def param_specs(self):
        specs = {"weight": ParamSpec((self.size, self.size))}
        if self.has_bias:
            specs["bias"] = ParamSpec((self.size,), role="vector", init="normal")
        return specs

    def load(self, tensors, *, compute_dtype, device):
        self.weight = tensors["weight"].contiguous()
        if self.has_bias:
            self.bias = tensors["bias"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, ctx: StepContext):
        return ops.linear(x, self.weight)


class ChannelScale(Gate):
    graph_safe = True  # no device work of its own

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.size,), role="vector", init="ones")}

    def load(self, tensors, *, compute_dtype, device):
        self.weight = tensors["weight"].to(device=device, dtype=torch.float32).contiguous()

    def forward(self, x, ctx: StepContext):
        raise RuntimeError("a channel scale is applied by the block where the sublayer's result joins the stream")


register_gate("sigmoid_linear", SigmoidLinearGate, replace=True)
register_gate("channel_scale", ChannelScale, replace=True)
