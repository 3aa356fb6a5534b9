"""One block: how a mixer, a feed-forward and their norms are arranged.

The arrangement is chosen by name per layer.  Built in:

``pre_norm``: x = norm(h); h += mixer(x); x = norm(h); h += ffn(x)
(prefixserve/model/llama.py:112-121, the only one that architecture uses).  With ``mixer_scale`` / ``ffn_scale`` in
the layer's description the sublayer's result is multiplied by a learned vector, channel by channel, before the sum:
h += scale_1 * mixer(x); h += scale_2 * ffn(x).
``parallel``: both sublayers read the same stream, h += mixer(norm_a(h)) + ffn(norm_b(h)).
``gated_post_norm``: the sublayers read the stream itself and the norm sits on their result, behind a gate computed
from the same input: h += scale * norm_a(mixer(h) * sigmoid(gate_a(h))); then the same with the feed-forward.

``sandwich_norm``: a norm on both sides of each sublayer, h += norm_1b(mixer(norm_1(h))); h += norm_2b(ffn(norm_2(h))).

The residual stream h is float32.  A block takes and returns (h, pending):
``pending`` is a sublayer output that has not been added yet, because the sum
is done inside the next norm's kernel.  An arrangement is a function
``(block, h, pending, ctx, cache) -> (h, pending)`` over the block's parts
(``mixer_norm``, ``mixer``, ``ffn_norm``, ``ffn``; the last two are None in a
layer without feed-forward) and is added with ``register_arrangement``.
"""

from __future__ import annotations

from typing import Callable

from .. import ops
from ..config.spec import LayerSpec
from .base import CacheView, StepContext
from .registry import make

_ARRANGEMENTS: dict[str, Callable] = {}


def register_arrangement(name: str, run: Callable, *, replace: bool = False) -> None:
    if name in _ARRANGEMENTS and not replace:
        raise ValueError(f"block arrangement {name!r} is already registered")
    _ARRANGEMENTS[name] = run


class Block:
    def __init__(self, spec: LayerSpec):
        try:
            self.run = _ARRANGEMENTS[spec.arrangement]
        except KeyError:
            raise ValueError(f"block arrangement {spec.arrangement!r} is not registered (known: {sorted(_ARRANGEMENTS)})") from None
        self.mixer_norm = make("norm", spec.mixer_norm)
        self.mixer = make("mixer", spec.mixer)
        self.ffn_norm = make("norm", spec.ffn_norm) if spec.ffn_norm is not None else None
        self.ffn = make("ffn", spec.ffn) if spec.ffn is not None else None
        self.mixer_gate = make("gate", spec.mixer_gate) if spec.mixer_gate is not None else None
        self.ffn_gate = make("gate", spec.ffn_gate) if spec.ffn_gate is not None and spec.ffn is not None else None
        self.residual_scale = float(spec.residual_scale)
        self.mixer_post_norm = make("norm", spec.mixer_post_norm) if spec.mixer_post_norm is not None else None
        self.ffn_post_norm = make("norm", spec.ffn_post_norm) if spec.ffn_post_norm is not None and spec.ffn is not None else None
        self.mixer_scale = make("gate", spec.mixer_scale) if spec.mixer_scale is not None else None
        self.ffn_scale = make("gate", spec.ffn_scale) if spec.ffn_scale is not None and spec.ffn is not None else None
        if (self.mixer_scale is not None or self.ffn_scale is not None) and spec.arrangement != "pre_norm":
            raise ValueError("a channel scale on a sublayer's result goes with the pre_norm arrangement")

    def named_parts(self):
        parts = [("mixer_norm", self.mixer_norm), ("mixer", self.mixer)]
        if self.mixer_post_norm is not None:
            parts.append(("mixer_post_norm", self.mixer_post_norm))
        if self.mixer_gate is not None:
            parts.append(("mixer_gate", self.mixer_gate))
        if self.mixer_scale is not None:
            parts.append(("mixer_scale", self.mixer_scale))
        if self.ffn is not None:
            parts += [("ffn_norm", self.ffn_norm), ("ffn", self.ffn)]
            if self.ffn_post_norm is not None:
                parts.append(("ffn_post_norm", self.ffn_post_norm))
            if self.ffn_gate is not None:
                parts.append(("ffn_gate", self.ffn_gate))
            if self.ffn_scale is not None:
                parts.append(("ffn_scale", self.ffn_scale))
        return tuple(parts)

    def forward(self, h, pending, ctx: StepContext, cache: CacheView):
        return self.run(self, h, pending, ctx, cache)


def _sublayer(norm, part, h, pending, ctx, *more):
    """(stream after adding ``pending``, the part's output).  A part that takes a deferred input may have the sum
    and the norm done inside its first product, which then writes the summed stream to a new tensor."""
    if part.takes_deferred_input:
        x = norm.defer(h, pending, ctx)
        out = part.forward(x, ctx, *more)
        return x.residual(), out
    return h, part.forward(norm.forward(h, pending, ctx), ctx, *more)


def pre_norm(block: Block, h, pending, ctx: StepContext, cache: CacheView):
    h, pending = _sublayer(block.mixer_norm, block.mixer, h, pending, ctx, cache)
    if block.mixer_scale is not None:  # joins the stream as pending * scale, in the next norm's kernel
        pending = ops.Affine(pending, scale=block.mixer_scale.weight)
    if block.ffn is not None:
        h, pending = _sublayer(block.ffn_norm, block.ffn, h, pending, ctx)
        if block.ffn_scale is not None:
            pending = ops.Affine(pending, scale=block.ffn_scale.weight)
    return h, pending


def parallel(block: Block, h, pending, ctx: StepContext, cache: CacheView):
    """Both sublayers see the stream as it entered the block (after ``pending``); their outputs are added together."""
    x = block.mixer_norm.forward(h, pending, ctx)       # h now holds the sum
    mixed = block.mixer.forward(x, ctx, cache)
    if block.ffn is None:
        return h, mixed
    fed = block.ffn.forward(block.ffn_norm.forward(h, None, ctx), ctx)
    ops.residual_add(h, mixed)
    return h, fed


STREAM_COPY = "stream_in_compute_type"  # ctx.extras: (the stream tensor, its current value in the compute type)


def _stream_as_input(h, ctx):
    """The stream in the type the products take: h itself on the float32 path, else the copy its last writer left
    (the embedding, or the kernel that added the previous sublayer), made now if there is none."""
    if ctx.compute_dtype == h.dtype:
        return h
    held = ctx.extras.get(STREAM_COPY)
    if held is not None and held[0] is h:
        return held[1]
    return h.to(ctx.compute_dtype)


def gated_post_norm(block: Block, h, pending, ctx: StepContext, cache: CacheView):
    """Sublayers read the stream; each result is gated by its input, normed and added with the block's factor."""
    if pending is not None:
        ops.residual_add(h, pending)
        ctx.extras.pop(STREAM_COPY, None)
    x = _stream_as_input(h, ctx)
    for part, gate, norm, more in ((block.mixer, block.mixer_gate, block.mixer_norm, (cache,)),
                                   (block.ffn, block.ffn_gate, block.ffn_norm, ())):
        if part is None:
            continue
        y = part.forward(x, ctx, *more)
        g = gate.forward(x, ctx) if gate is not None else None
        x = norm.add_normed(h, y, ctx, gate=g, gate_bias=gate.bias if gate is not None else None, scale=block.residual_scale)
    ctx.extras[STREAM_COPY] = (h, x)
    return h, None


def sandwich_norm(block: Block, h, pending, ctx: StepContext, cache: CacheView):
    """A norm in front of each sublayer and one on its result.  The result travels on as ``pending`` with its norm
    (``Norm.post``); the next norm in front of a sublayer (this block's, the next block's, or the model's last) adds
    it to the stream and norms the sum in one kernel."""
    if block.mixer_post_norm is None or (block.ffn is not None and block.ffn_post_norm is None):
        raise ValueError("the sandwich_norm arrangement needs a norm for every sublayer's result")
    y = block.mixer.forward(block.mixer_norm.forward(h, pending, ctx), ctx, cache)
    pending = block.mixer_post_norm.post(y)
    if block.ffn is not None:
        y = block.ffn.forward(block.ffn_norm.forward(h, pending, ctx), ctx)
        pending = block.ffn_post_norm.post(y)
    return h, pending


register_arrangement("pre_norm", pre_norm)
register_arrangement("sandwich_norm", sandwich_norm)
register_arrangement("gated_post_norm", gated_post_norm)
register_arrangement("parallel", parallel)
