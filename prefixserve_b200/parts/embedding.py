"""Token embedding and LM head (prefixserve/model/llama.py:109, :125-126).

The embedding gathers rows straight into the float32 residual stream.  The
head multiplies the normalised, selected rows by [vocab, hidden]^T and returns
float32 logits; when tied it uses the embedding's tensor.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import ParamSpec, Part
from .registry import register_embedding, register_head


class TokenEmbedding(Part):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.scale = float(params.get("scale", 1.0))  # the rows are multiplied by this on their way into the float32 stream
        self.table: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors, *, compute_dtype, device):
        self.table = tensors["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.table, scale=self.scale)


class HashedPairEmbedding(Part):
    """Token embedding plus a row of a second table chosen by a hash of (previous token, token):
    row (previous * mul_prev + token * mul_cur) mod buckets, and the table's last row (number ``buckets``) for the
    first token of a sequence.  The previous token of a portion's first token is not in the step: it is carried per
    request in a one-word state, which makes this an embedding with a cache entry of its own (``uses_step``)."""

    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    uses_step = True   # forward_step(ctx, cache) instead of forward(token_ids)

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.buckets = int(params["buckets"])
        self.mul_prev = int(params["mul_prev"])
        self.mul_cur = int(params["mul_cur"])
        self.table: torch.Tensor | None = None
        self.pair_table: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab, self.hidden)), "pair_weight": ParamSpec((self.buckets + 1, self.hidden))}

    def cache_need(self):
        from .base import CacheNeed, FixedState
        return CacheNeed(state=FixedState((1,), torch.int32))

    def load(self, tensors, *, compute_dtype, device):
        self.table = tensors["weight"].contiguous()
        self.pair_table = tensors["pair_weight"].to(self.table.dtype).contiguous()

    def forward_step(self, ctx, cache):
        """(float32 stream [T, H], the same in the compute type or None on the float32 path)."""
        return ops.hashed_embedding(ctx.token_ids, ctx.positions, ctx.token_item, ctx.item_start, ctx.slots,
                                    cache.state.view(-1), self.table, self.pair_table, mul_prev=self.mul_prev,
                                    mul_cur=self.mul_cur, copy_dtype=ctx.compute_dtype)


class TokenPositionEmbedding(Part):
    """Token rows times a constant plus a learned row per absolute position: h = table[token] * scale + positions[p].
    It reads the step's positions (``uses_step``) but carries nothing from step to step."""

    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    uses_step = True   # forward_step(ctx, cache) instead of forward(token_ids)

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.max_positions = int(params["max_positions"])
        self.scale = float(params.get("scale", 1.0))
        self.table: torch.Tensor | None = None
        self.position_table: torch.Tensor | None = None

    def param_specs(self):
        return {"weight": ParamSpec((self.vocab, self.hidden)), "position_weight": ParamSpec((self.max_positions, self.hidden))}

    def cache_need(self):
        from .base import CacheNeed
        return CacheNeed()

    def load(self, tensors, *, compute_dtype, device):
        self.table = tensors["weight"].contiguous()
        self.position_table = tensors["position_weight"].to(self.table.dtype).contiguous()

    def forward_step(self, ctx, cache):
        return ops.embedding_positions(ctx.token_ids, ctx.positions, self.table, self.position_table, self.scale), None


class LMHead(Part):
    graph_safe = True  # device work depends only on tensor shapes and device-side inputs
    takes_deferred_input = True  # x goes to one product only, which may do the norm in front of it itself

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab_size"])
        self.hidden = int(params["hidden_size"])
        self.tied = bool(params.get("tied", False))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {} if self.tied else {"weight": ParamSpec((self.vocab, self.hidden))}

    def load(self, tensors, *, compute_dtype, device):
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, table: torch.Tensor) -> None:
        self.weight = table

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)


register_embedding("token_embedding", TokenEmbedding, replace=True)
register_embedding("hashed_pair_embedding", HashedPairEmbedding, replace=True)
register_embedding("token_position_embedding", TokenPositionEmbedding, replace=True)
register_head("lm_head", LMHead, replace=True)
