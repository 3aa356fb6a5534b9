"""Goganex as a list of parts.

Embedding: token row times a constant.  Layers in the order config.json lists them, pre-norm blocks with RMS norms;
what a layer's mixer reads passes a token shift first (the ``token_shift`` mixer around the layer's own).  Mixers:
``attention`` is the ``unit_norm_attention`` part with an interleaved rotation of the leading elements (frequencies
scaled by wavelength), a learned factor per head and a sink of score zero; ``parallel`` is ``side_by_side`` over a
``unit_norm_attention`` whose projected keys are its values (no rotation, plain softmax) and a ``min_gru``, each
result normed with a gain of its own and the two averaged.  Feed-forward: the gated one with the ``clipped_swiglu``
activation.  Final norm, untied head.

``loop``: a run of the layers is repeated with the same weights.  The run list names those layers several times, every
call with a cache entry of its own (pages, shifted row and recurrent state per pass).

The design has no position limit of its own: ``max_positions`` is only the bound up to which the engine may be asked
to build angle tables.
"""

from __future__ import annotations

import re

from ..config.goganex import ARCHITECTURE, AttentionConfig, GoganexConfig, ParallelConfig
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, part

MAX_POSITIONS = 1 << 20
SINK_SCORE = 0.0        # the softmax denominator of an attention layer holds one more term, exp(0)
GATE_ALPHA = 1.702      # g * sigmoid(1.702 g): the feed-forward's gate
UP_OFFSET = 1.0         # ... times (u + 1)
BRANCH_WEIGHT = 0.5     # a parallel mixer is the mean of its two normed branches


def _attention_spec(cfg: GoganexConfig, m: AttentionConfig, *, plain: bool):
    position = None
    if m.rot is not None and not plain:
        scaling = None if m.rot.factor is None else {"kind": "llama3", "factor": m.rot.factor, "low_freq_factor": m.rot.low,
                                                     "high_freq_factor": m.rot.high, "original_max_positions": m.rot.original}
        position = part("rope", head_dim=m.dim, rotary_dim=m.rot.dims, theta=m.rot.base, scaling=scaling, layout="interleaved")
    return part("unit_norm_attention", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                scale=m.scale, eps=cfg.norm_eps, position=position, head_temperature=not plain,
                sink=None if plain else SINK_SCORE, values="keys" if plain else "projected")


def _mixer_spec(cfg: GoganexConfig, m):
    if isinstance(m, AttentionConfig):
        inner = _attention_spec(cfg, m, plain=False)
    elif isinstance(m, ParallelConfig):
        inner = part("side_by_side", hidden_size=cfg.width, eps=cfg.norm_eps, names=("left", "right"), weight=BRANCH_WEIGHT,
                     branches=(_attention_spec(cfg, m.left, plain=True), part("min_gru", hidden_size=cfg.width, width=m.right_width)))
    else:
        raise TypeError(f"no mixer for {type(m).__name__}")
    return part("token_shift", size=cfg.width, inner=inner)


def goganex_spec(cfg: GoganexConfig) -> ModelSpec:
    norm = part("rms", size=cfg.width, eps=cfg.norm_eps)
    layers = []
    for layer in cfg.layers:
        ffn = None if layer.mlp is None else part("gated_mlp", hidden_size=cfg.width, intermediate_size=layer.mlp.ff,
                                                 activation="clipped_swiglu", limit=layer.mlp.limit, gate_alpha=GATE_ALPHA,
                                                 up_offset=UP_OFFSET)
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, layer.mixer), ffn=ffn, mixer_norm=norm,
                                ffn_norm=None if ffn is None else norm, arrangement="pre_norm"))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=MAX_POSITIONS,
        embedding=part("token_embedding", vocab_size=cfg.vocab, hidden_size=cfg.width, scale=cfg.embedding_scale),
        layers=tuple(layers),
        schedule=tuple(LayerCall(layer=i, cache=at) for at, i in enumerate(cfg.run_order())),
        final_norm=norm,
        head=part("lm_head", vocab_size=cfg.vocab, hidden_size=cfg.width, tied=False),
        stop_token_ids=cfg.stop_token_ids,
    )


_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
_ATTENTION = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "temperature": "temp", "o_proj": "o"}
_RECURRENCE = {"update_proj": "z", "update_bias": "z.b", "candidate_proj": "x", "candidate_bias": "x.b", "gate_proj": "g", "o_proj": "o"}
_IN_LAYER = {
    "mixer_norm.weight": "norm1",
    "ffn_norm.weight": "norm2",
    "mixer.mix": "shift",
    "mixer.inner.left_gain": "mix.left.out",
    "mixer.inner.right_gain": "mix.right.out",
    "ffn.gate_proj": "mlp.gate",
    "ffn.up_proj": "mlp.up",
    "ffn.down_proj": "mlp.down",
}
_IN_LAYER.update({f"mixer.inner.{local}": f"mix.{name}" for local, name in _ATTENTION.items()})
_IN_LAYER.update({f"mixer.inner.left.{local}": f"mix.left.{name}" for local, name in _ATTENTION.items()})
_IN_LAYER.update({f"mixer.inner.right.{local}": f"mix.right.{name}" for local, name in _RECURRENCE.items()})
_TOP = {"embedding.weight": "embed", "final_norm.weight": "final.norm", "head.weight": "head"}


def goganex_tensor_name(path: str) -> str:
    if path in _TOP:
        return _TOP[path]
    m = _LAYER.match(path)
    if m and m.group(2) in _IN_LAYER:
        return f"l{m.group(1)}.{_IN_LAYER[m.group(2)]}"
    raise KeyError(f"{ARCHITECTURE} has no tensor for part path {path!r}")


GOGANEX = Architecture(
    name=ARCHITECTURE,
    model_types=("goganex",),
    read_config=GoganexConfig.from_dicts,
    to_spec=goganex_spec,
    tensor_name=goganex_tensor_name,
)

register_architecture(GOGANEX, replace=True)
