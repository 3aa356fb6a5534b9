"""Attention through low-rank latents over the paged cache, with a sliding window and a gate per head.

Queries: c_q = norm(W_dq x), q = W_uq c_q, laid out head by head as
[``dim`` unrotated | ``rot_dim`` rotated].  Keys and values: W_dkv x gives a
latent of ``kv_rank`` numbers (normed) and one rotated key part of ``rot_dim``
numbers that all heads share; head h's unrotated key is U_k[h] c and its value
U_v[h] c.  Only the latent and the rotated key part are cached: one row of
``kv_rank + rot_dim`` numbers per token, a cache entry with a single plane and
a single head.  Instead of expanding every cached latent into per-head keys,
the query is carried into the latent space (q' = U_k[h]^T q_unrotated), the
attention runs there, and U_v[h] is applied once to its result:

    score = (q' . c + q_rot . k_rot) * scale,  out_h = sigmoid(w_g[h] . x) * U_v[h] (sum_j p_j c_j)

The rotation pairs dimension 2i with 2i+1 over the first ``rot_dims`` of the
rotated part; position i sees position j when 0 <= i - j < window (no window:
every j <= i).  The input projections that read x (query latent, key/value
latent with the rotated key part, gates) are one product.

Options: ``q_rank`` None: no query latent, q = W_q x directly (tensor
``q_proj``).  ``sink``: a learned score per head whose exponential joins the
softmax denominator once, without a key or a value.  ``gate``: "head" (one
sigmoid gate per head, as above), "channel" (the concatenated heads' values
are multiplied element by element by sigmoid(W_g x), tensor ``out_gate``
[heads * vdim, hidden]) or None.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import CacheNeed, CacheView, Mixer, PagedKV, ParamSpec, StepContext
from .registry import make, register_mixer


class LatentAttention(Mixer):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["dim"])
        self.rot = int(params["rot_dim"])
        self.vdim = int(params["vdim"])
        self.q_rank = None if params.get("q_rank") is None else int(params["q_rank"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.window = params.get("window")
        self.eps = float(params["eps"])
        self.gate_kind = params.get("gate", "head" if params.get("head_gate", True) else None)
        if self.gate_kind not in (None, "head", "channel"):
            raise ValueError(f"gate {self.gate_kind!r}: one of None, 'head', 'channel'")
        self.head_gate = self.gate_kind == "head"
        self.has_sink = bool(params.get("sink", False))
        self.position = make("position", params["position"])
        self.rot_dims = int(getattr(self.position, "rotary_dim", None) or 0)
        if self.rot_dims and getattr(self.position, "layout", "half") != "interleaved":
            raise ValueError("the latent attention kernels rotate neighbouring pairs (layout 'interleaved') only")
        if self.rot_dims > self.rot:
            raise ValueError(f"{self.rot_dims} rotated dimensions do not fit a rotated part of {self.rot}")
        self.w_in = self.w_uq = self.w_ukt = self.w_uv = self.w_o = None
        self.gain_q = self.gain_kv = self.sink = None

    def param_specs(self):
        if self.q_rank is None:
            specs = {"q_proj": ParamSpec((self.heads * (self.dim + self.rot), self.hidden))}
        else:
            specs = {
                "q_down": ParamSpec((self.q_rank, self.hidden)),
                "q_down_norm": ParamSpec((self.q_rank,), role="vector", init="ones"),
                "q_up": ParamSpec((self.heads * (self.dim + self.rot), self.q_rank)),
            }
        specs.update({
            "kv_down": ParamSpec((self.rank + self.rot, self.hidden)),
            "kv_down_norm": ParamSpec((self.rank,), role="vector", init="ones"),
            "k_up": ParamSpec((self.heads * self.dim, self.rank)),
            "v_up": ParamSpec((self.heads * self.vdim, self.rank)),
        })
        if self.has_sink:
            specs["sink"] = ParamSpec((self.heads,), role="vector", init="normal")
        if self.head_gate:
            specs["head_gate"] = ParamSpec((self.heads, self.hidden))
        elif self.gate_kind == "channel":
            specs["out_gate"] = ParamSpec((self.heads * self.vdim, self.hidden))
        specs["o_proj"] = ParamSpec((self.hidden, self.heads * self.vdim))
        return specs

    def cache_need(self):
        return CacheNeed(paged=PagedKV(1, self.rank + self.rot, self.window, "latent", planes=1))

    def load(self, tensors, *, compute_dtype, device):
        # one product for everything that reads x; a direct query projection comes first in it and is read from there
        pieces = [tensors["q_proj"] if self.q_rank is None else tensors["q_down"], tensors["kv_down"]]
        if self.head_gate:
            pieces.append(tensors["head_gate"])
        elif self.gate_kind == "channel":
            pieces.append(tensors["out_gate"])
        dtype = torch.float32 if any(p.dtype == torch.float32 for p in pieces) else pieces[0].dtype
        self.w_in = torch.cat([p.to(dtype) for p in pieces], dim=0).contiguous()
        self.w_uq = None if self.q_rank is None else tensors["q_up"].contiguous()
        # per head [rank, dim]: the transpose of the key expansion, which carries a query into the latent space
        self.w_ukt = tensors["k_up"].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.w_uv = tensors["v_up"].view(self.heads, self.vdim, self.rank).contiguous()
        self.w_o = tensors["o_proj"].contiguous()
        if self.q_rank is not None:
            self.gain_q = tensors["q_down_norm"].to(device=device, dtype=torch.float32).contiguous()
        self.gain_kv = tensors["kv_down_norm"].to(device=device, dtype=torch.float32).contiguous()
        if self.has_sink:
            self.sink = tensors["sink"].to(device=device, dtype=torch.float32).contiguous()

    def prepare(self, *, max_positions, compute_dtype, device):
        self.position.prepare(max_positions=max_positions, compute_dtype=compute_dtype, device=device)

    def forward(self, x, ctx: StepContext, cache: CacheView):
        if not cache.writes:
            raise RuntimeError("a latent attention part writes its own cache entry")
        table = ctx.block_tables[cache.group]
        t, heads = x.shape[0], self.heads
        proj = ops.linear(x, self.w_in)
        gates = heads if self.head_gate else (heads * self.vdim if self.gate_kind == "channel" else 0)
        if self.q_rank is None:
            # the row is [queries | key/value latent | rotated key part | gates]: the queries are read where they lie, the
            # rest goes through the pass that norms, rotates, appends and takes the gates' sigmoids (both kernels, and the
            # per-head product, take rows that are runs of columns of a wider product)
            qw = heads * (self.dim + self.rot)
            q = proj[:, :qw]
            _, gate = ops.latent_prepare(proj[:, qw:], ctx.positions, ctx.token_item, table, self.position.cos,
                                         self.position.sin, None, self.gain_kv, cache.kv, q_rank=0, rank=self.rank, rot=self.rot,
                                         rot_dims=self.rot_dims, heads=gates, page_size=cache.page_size, eps=self.eps)
        else:
            cq, gate = ops.latent_prepare(proj, ctx.positions, ctx.token_item, table, self.position.cos, self.position.sin,
                                          self.gain_q, self.gain_kv, cache.kv, q_rank=self.q_rank, rank=self.rank, rot=self.rot,
                                          rot_dims=self.rot_dims, heads=gates, page_size=cache.page_size, eps=self.eps)
            q = ops.linear(cq, self.w_uq)
        q_lat = torch.empty((t, heads, self.rank + self.rot), dtype=torch.float32, device=x.device)
        ops.linear_per_head(q.view(t, heads, self.dim + self.rot)[:, :, : self.dim], self.w_ukt, out=q_lat[:, :, : self.rank])
        ops.latent_query_rotate(q, ctx.positions, self.position.cos, self.position.sin, q_lat, heads=heads, plain=self.dim,
                                rot=self.rot, rot_dims=self.rot_dims, rank=self.rank)
        mixed = ops.latent_attention(q_lat, cache.kv, table, ctx.positions, ctx.token_item, gate if self.head_gate else None, rank=self.rank,
                                     page_size=cache.page_size, window=self.window, scale=self.scale, out_dtype=x.dtype,
                                     items=ctx.items, key_hint=int(ctx.extras.get("static_kv_len") or ctx.max_kv_len),
                                     sink=self.sink, static_shapes=bool(ctx.extras.get("static_kv_len")))
        if self.gate_kind == "channel":  # the values leave their product in float32, meet the gate there, and are rounded once
            values = ops.gate_mul(ops.linear_per_head(mixed, self.w_uv, out_dtype=torch.float32), gate, out_dtype=x.dtype)
        else:
            values = ops.linear_per_head(mixed, self.w_uv)
        return ops.linear(values.view(t, heads * self.vdim), self.w_o)


register_mixer("latent_attention", LatentAttention, replace=True)
