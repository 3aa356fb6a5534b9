"""Grouped-query softmax attention whose queries and keys are brought to unit root mean square, with the options that
come with it in designs of that kind.

q, k (and v) come from one fused projection without biases; per head and in float32,

    rotation of the first ``rotary_dim`` elements by absolute position (``position``: any registered encoding, or none);
    q <- q / sqrt(mean(q^2) + eps),  k <- k / sqrt(mean(k^2) + eps)      (``eps`` None: left out);
    score(i, j) = (q_i . k_j) * scale * temperature[h]                      (``head_temperature``: a learned number per head);
    weights = exp(score) / (sum over visible j + exp(sink))                  (``sink``: a fixed score that joins the
                                                                             denominator without a key or a value; None: plain softmax).

Query head h reads key/value head h // (heads / kv_heads).  ``values``: "projected" (a projection of their own, size
``vdim``) or "keys" (the projected key, before rotation and norm, is also the value; no v_proj).  Optional ``window``
and ``chunk`` masks; with a window, ``keep_first``: the first so many keys of a sequence stay visible to every later
query (at their true positions).  ``bias``: the projections (q, k, v and the output) have biases, added in float32.
``own_kv`` False: the layer has no key and value projections; it reads the cache entry another layer writes (keys as
that layer stored them, after its rotation) with queries, scale and mask of its own.

Only the pass between projection and scores is this part's own; the attention kernels are those of the other
attention parts.  With keys and values of one size that the tensor-core kernels take (64 or 128) and no chunk mask,
the cache entry has a plane of keys and a plane of values and ``ops.attention`` reads it (the kernels of the plain
``attention`` part, which take the sink at the end of a row's sum); any other sizes, or a chunk mask, keep one row per
token and key/value head (key, then value) and the kernels of ``biased_attention``.
"""

from __future__ import annotations

import math

import torch

from .. import ops
from ..config.spec import PartSpec
from .base import CacheNeed, CacheView, Mixer, PagedKV, ParamSpec, StepContext
from .registry import make, register_mixer


SPLIT_PLANE_SIZES = (64, 128)  # head sizes of the kernels behind ``ops.attention``


class UnitNormAttention(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.hq = int(params["num_heads"])
        self.hkv = int(params["num_kv_heads"])
        self.dim = int(params["dim"])
        self.values = str(params.get("values", "projected"))
        if self.values not in ("projected", "keys"):
            raise ValueError(f"values {self.values!r}: one of 'projected', 'keys'")
        self.vdim = self.dim if self.values == "keys" else int(params.get("vdim") or self.dim)
        self.scale = float(params.get("scale") or 1.0 / math.sqrt(self.dim))
        self.eps = None if params.get("eps") is None else float(params["eps"])
        self.window = params.get("window")
        self.chunk = params.get("chunk")
        self.keep_first = int(params.get("keep_first") or 0) if self.window is not None else 0
        self.has_bias = bool(params.get("bias", False))
        self.own_kv = bool(params.get("own_kv", True))
        if self.keep_first and self.chunk is not None:
            raise ValueError("kept first keys go with a window, not with a chunk mask")
        if not self.own_kv and self.values == "keys":
            raise ValueError("a layer without projections of its own reads another layer's keys and values as they are")
        self.head_temperature = bool(params.get("head_temperature", False))
        self.sink_score = None if params.get("sink") is None else float(params["sink"])
        if self.hq % self.hkv:
            raise ValueError(f"{self.hq} query heads cannot share {self.hkv} key/value heads")
        self.position = make("position", params.get("position") or PartSpec("none"))
        self.rotary_dim = int(getattr(self.position, "rotary_dim", None) or self.dim)
        self.interleaved = getattr(self.position, "layout", "half") == "interleaved"
        # the layout is a matter of the sizes only (a layer that reads another's entry must arrive at the same one);
        # masks the plane kernels do not know (kept first keys) ask for ``rows`` through the ``layout`` parameter
        self.split_planes = (self.chunk is None and self.vdim == self.dim and self.dim in SPLIT_PLANE_SIZES
                             and params.get("layout", "auto") != "rows")
        if self.keep_first and self.split_planes:
            raise ValueError("kept first keys need the row layout of the cache entry (layout='rows')")
        self.w_in = self.w_o = self.temperature = self.sink = self.b_in = self.b_o = None

    def param_specs(self):
        specs = {"q_proj": ParamSpec((self.hq * self.dim, self.hidden))}
        if self.has_bias:
            specs["q_bias"] = ParamSpec((self.hq * self.dim,), role="vector", init="normal")
        if self.own_kv:
            specs["k_proj"] = ParamSpec((self.hkv * self.dim, self.hidden))
            if self.has_bias:
                specs["k_bias"] = ParamSpec((self.hkv * self.dim,), role="vector", init="normal")
            if self.values == "projected":
                specs["v_proj"] = ParamSpec((self.hkv * self.vdim, self.hidden))
                if self.has_bias:
                    specs["v_bias"] = ParamSpec((self.hkv * self.vdim,), role="vector", init="normal")
        if self.head_temperature:
            specs["temperature"] = ParamSpec((self.hq,), role="vector", init="ones")
        specs["o_proj"] = ParamSpec((self.hidden, self.hq * self.vdim))
        if self.has_bias:
            specs["o_bias"] = ParamSpec((self.hidden,), role="vector", init="normal")
        return specs

    def cache_need(self):
        if self.split_planes:
            return CacheNeed(paged=PagedKV(self.hkv, self.dim, self.window, "natural"))
        return CacheNeed(paged=PagedKV(self.hkv, self.dim + self.vdim, self.window, "natural", planes=1, chunk=self.chunk,
                                       keep_first=self.keep_first))

    def load(self, tensors, *, compute_dtype, device):
        names = ["q"] + ((["k"] + (["v"] if self.values == "projected" else [])) if self.own_kv else [])
        pieces = [tensors[f"{n}_proj"] for n in names]
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in pieces) else pieces[0].dtype
        self.w_in = torch.cat([p.to(dtype) for p in pieces], dim=0).contiguous()
        self.w_o = tensors["o_proj"].contiguous()
        if self.has_bias:
            self.b_in = torch.cat([tensors[f"{n}_bias"].to(device=device, dtype=torch.float32) for n in names]).contiguous()
            self.b_o = tensors["o_bias"].to(device=device, dtype=torch.float32).contiguous()
        if self.head_temperature:
            self.temperature = tensors["temperature"].to(device=device, dtype=torch.float32).contiguous()
        if self.sink_score is not None:
            self.sink = torch.full((self.hq,), self.sink_score, dtype=torch.float32, device=device)

    def prepare(self, *, max_positions, compute_dtype, device):
        self.position.prepare(max_positions=max_positions, compute_dtype=compute_dtype, device=device)

    # A mixer that applies one matrix to its input before anything else may say so: whoever runs several such mixers
    # on the same input (``side_by_side``) then multiplies once by the stacked matrices and hands each its columns.
    def input_weight(self) -> torch.Tensor:
        return self.w_in

    def forward_projected(self, proj, ctx: StepContext, cache: CacheView):
        if cache.writes != self.own_kv or cache.kv is None:
            raise RuntimeError("an attention part with projections of its own must write its cache entry, and only such a part may")
        table = ctx.block_tables[cache.group]
        q = ops.attention_prepare(proj, cache.kv, table, ctx, num_heads=self.hq, num_kv_heads=self.hkv, dim=self.dim,
                                  vdim=self.vdim, page_size=cache.page_size, cos=self.position.cos, sin=self.position.sin,
                                  rotary_dim=self.rotary_dim, interleaved=self.interleaved, unit_norm_eps=self.eps,
                                  head_factor=self.temperature, values_are_keys=self.values == "keys",
                                  split_planes=self.split_planes, bias=self.b_in, write_kv=self.own_kv)
        if self.split_planes:
            o = ops.attention(q, cache.kv, table, ctx.positions, ctx.token_item, window=self.window, scale=self.scale, ctx=ctx,
                              sink=self.sink)
        else:
            o = ops.attention_over_rows(q, cache.kv, table, ctx, num_heads=self.hq, num_kv_heads=self.hkv, dim=self.dim,
                                        vdim=self.vdim, page_size=cache.page_size, scale=self.scale, window=self.window,
                                        chunk=self.chunk, sink=self.sink, keep_first=self.keep_first)
        if self.b_o is not None:  # the output bias joins the stream with the product, in float32 (``ops.Affine``)
            return ops.Affine(ops.linear(o, self.w_o), shift=self.b_o)
        return ops.last_product(o, self.w_o, ctx)  # may be handed on unrun: the next norm's kernels take it from there

    def forward(self, x, ctx: StepContext, cache: CacheView):
        return self.forward_projected(ops.linear(x, self.w_in), ctx, cache)


register_mixer("unit_norm_attention", UnitNormAttention, replace=True)
