"""Mixers made of other mixers.

``token_shift``: what the inner mixer reads is moved toward the row the mixer in front of the previous token read,
channel by channel by a learned vector: y_t = x_t + (x_(t-1) - x_t) * mix, with zeros before a sequence's first token.
The unshifted row of a portion's last token is carried in the request's slot, so a prompt may be cut anywhere.

``side_by_side``: several mixers read the same input; their results are each RMS-normed over the model width with a
learned gain and added, times ``weight`` (one half: the mean of two).  Branches that start with one matrix product of
their input (they offer ``input_weight`` / ``forward_projected``) share a single product over the stacked matrices.

Both hand their inner mixers' tensors, paged cache need and graph-safety through.  Fixed states are float32 vectors
laid one after the other in the slot's state (the combinator's own first); an inner mixer sees its run of columns,
so its kernels must take a state whose rows are part of wider ones (the row stride is the tensor's).
"""

from __future__ import annotations

import math

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import CacheNeed, CacheView, FixedState, Mixer, ParamSpec, StepContext
from .registry import make, register_mixer


def _as_spec(value) -> PartSpec:
    if isinstance(value, PartSpec):
        return value
    return PartSpec(str(value["kind"]), {k: v for k, v in value.items() if k != "kind"})


def _state_floats(need: CacheNeed, who: str) -> int:
    if need.state is None:
        return 0
    if need.state.dtype != torch.float32:
        raise ValueError(f"{who}: a state of {need.state.dtype} cannot share a slot's float32 state")
    return math.prod(need.state.shape)


def _inner_view(cache: CacheView, need: CacheNeed, at: int, count: int, alone: bool) -> CacheView:
    """The cache entry as an inner mixer sees it: the pages as they are, its own columns of the state."""
    state = None
    if need.state is not None:
        state = cache.state if alone else cache.state[:, at: at + count].view(cache.state.shape[0], *need.state.shape)
    return CacheView(group=cache.group if need.paged is not None else None, kv=cache.kv if need.paged is not None else None,
                     state=state, page_size=cache.page_size, writes=cache.writes)


class TokenShifted(Mixer):
    takes_deferred_input = True  # x goes to the shift only, which may do the sum and the norm in front of it itself

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.inner = make("mixer", _as_spec(params["inner"]))
        self.inner_need = self.inner.cache_need()
        self.inner_floats = _state_floats(self.inner_need, "token_shift")
        self.mix: torch.Tensor | None = None

    @property
    def graph_safe(self) -> bool:
        return bool(getattr(self.inner, "graph_safe", False))

    def param_specs(self):
        specs = {"mix": ParamSpec((self.size,), role="vector", init="normal")}
        specs.update({f"inner.{name}": ps for name, ps in self.inner.param_specs().items()})
        return specs

    def cache_need(self):
        return CacheNeed(paged=self.inner_need.paged, state=FixedState((self.size + self.inner_floats,), torch.float32))

    def load(self, tensors, *, compute_dtype, device):
        self.mix = tensors["mix"].to(device=device, dtype=torch.float32).contiguous()
        self.inner.load({name[len("inner."):]: t for name, t in tensors.items() if name.startswith("inner.")},
                        compute_dtype=compute_dtype, device=device)

    def prepare(self, *, max_positions, compute_dtype, device):
        self.inner.prepare(max_positions=max_positions, compute_dtype=compute_dtype, device=device)

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if cache.state is None or not cache.writes:
            raise RuntimeError("token shift carries a row per request and needs the state of its own cache entry")
        shifted = ops.token_shift(x, self.mix, cache.state[:, : self.size], ctx)
        return self.inner.forward(shifted, ctx, _inner_view(cache, self.inner_need, self.size, self.inner_floats, alone=False))


class SideBySide(Mixer):
    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.names = tuple(str(n) for n in params.get("names") or ("left", "right"))
        self.branches = [make("mixer", _as_spec(s)) for s in params["branches"]]
        if len(self.branches) != 2 or len(self.names) != 2:
            raise ValueError("side_by_side is built for two branches")  # the kernel that norms and adds takes a pair
        self.weight = float(params.get("weight", 1.0 / len(self.branches)))
        self.needs = [b.cache_need() for b in self.branches]
        if sum(n.paged is not None for n in self.needs) > 1:
            raise ValueError("side_by_side: at most one branch may keep keys and values (a cache entry has one set of pages)")
        self.floats = [_state_floats(n, "side_by_side") for n in self.needs]
        self.alone = sum(f > 0 for f in self.floats) == 1  # a single state passes through in its own shape
        self.gains: list[torch.Tensor] = []
        self.w_in: torch.Tensor | None = None
        self.columns: list[tuple[int, int]] = []

    @property
    def graph_safe(self) -> bool:
        return all(getattr(b, "graph_safe", False) for b in self.branches)

    def param_specs(self):
        specs = {}
        for name, b in zip(self.names, self.branches):
            specs.update({f"{name}.{local}": ps for local, ps in b.param_specs().items()})
        for name in self.names:
            specs[f"{name}_gain"] = ParamSpec((self.hidden,), role="vector", init="ones")
        return specs

    def cache_need(self):
        paged = next((n.paged for n in self.needs if n.paged is not None), None)
        if self.alone:
            state = next(n.state for n in self.needs if n.state is not None)
        else:
            state = FixedState((sum(self.floats),), torch.float32) if sum(self.floats) else None
        return CacheNeed(paged=paged, state=state)

    def load(self, tensors, *, compute_dtype, device):
        for name, b in zip(self.names, self.branches):
            b.load({k[len(name) + 1:]: t for k, t in tensors.items() if k.startswith(name + ".")}, compute_dtype=compute_dtype, device=device)
        self.gains = [tensors[f"{name}_gain"].to(device=device, dtype=torch.float32).contiguous() for name in self.names]
        # one product for every branch that starts with a matrix of its own on the shared input
        if all(hasattr(b, "input_weight") and hasattr(b, "forward_projected") for b in self.branches):
            pieces = [b.input_weight() for b in self.branches]
            if len({p.dtype for p in pieces}) == 1:
                self.w_in = torch.cat(pieces, dim=0).contiguous()
                at = 0
                for p in pieces:
                    self.columns.append((at, at + p.shape[0]))
                    at += p.shape[0]

    def prepare(self, *, max_positions, compute_dtype, device):
        for b in self.branches:
            b.prepare(max_positions=max_positions, compute_dtype=compute_dtype, device=device)

    def forward(self, x, ctx: StepContext, cache: CacheView):
        proj = ops.linear(x, self.w_in) if self.w_in is not None else None
        results, at = [], 0
        for i, (b, need) in enumerate(zip(self.branches, self.needs)):
            view = _inner_view(cache, need, at, self.floats[i], alone=self.alone)
            at += self.floats[i]
            if proj is not None:
                lo, hi = self.columns[i]
                y = b.forward_projected(proj[:, lo:hi], ctx, view)
            else:
                y = b.forward(x, ctx, view)
            results.append(y.tensor() if isinstance(y, ops.PendingProduct) else y)
        return ops.normed_pair_sum(results[0], results[1], self.gains[0], self.gains[1], self.eps, self.weight)


register_mixer("token_shift", TokenShifted, replace=True)
register_mixer("side_by_side", SideBySide, replace=True)
