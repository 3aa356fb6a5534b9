"""Zomolix as a list of parts.

Embedding: token row times a constant.  Layers in the order config.json lists them, pre-norm blocks with RMS norms and
a learned factor per channel on every sublayer's result (``channel_scale``).  Mixers: ``attention`` is the
``unit_norm_attention`` part without its unit norm: biases on the four projections, a split-half rotation of the
leading elements with ramped frequency scaling (``yarn``), the configured score scale, a sliding window that keeps a
sequence's first keys, and optionally no key/value projections of its own (the run list then lets the layer read the
cache entry of the layer it names); ``latent_attention`` is the part of that name with a direct query projection, a
learned sink per head, a sigmoid gate per channel on the concatenated heads, the interleaved rotation of the rotated
part and no window.  Feed-forward: ``routed_experts`` with softmax scores, groups that count by their best expert,
weights that are the chosen scores as they are, gated experts with both branches clipped, and a shared expert of the
same form that is simply added.  Final norm, untied head.

The design has no position limit of its own: ``max_positions`` is only the bound up to which the engine may be asked
to build angle tables.
"""

from __future__ import annotations

import re

from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, part
from ..config.zomolix import ARCHITECTURE, AttentionConfig, LatentAttentionConfig, RotationConfig, ZomolixConfig

MAX_POSITIONS = 1 << 20
GATE_ALPHA = 1.702      # an expert's gate: g * sigmoid(1.702 g) ...
UP_OFFSET = 1.0         # ... times (u + 1)


def _position(rot: RotationConfig | None, size: int, layout: str):
    if rot is None:
        return None
    scaling = None
    if rot.factor is not None:
        scaling = {"kind": "yarn", "factor": rot.factor, "original_max_positions": rot.original, "fast": rot.fast, "slow": rot.slow}
    return part("rope", head_dim=size, rotary_dim=rot.dims, theta=rot.base, scaling=scaling, layout=layout)


def _writer_of(cfg: ZomolixConfig, i: int) -> int:
    m = cfg.layers[i].mixer
    return m.kv_from if isinstance(m, AttentionConfig) and m.kv_from is not None else i


def _mixer_spec(cfg: ZomolixConfig, i: int):
    m = cfg.layers[i].mixer
    if isinstance(m, AttentionConfig):
        # Layers that share a cache entry agree on its layout: a row per token as soon as one of them has a window.  The
        # kernels that read planes of keys and values know no kept first keys, and behind a window they multiply
        # whatever a page that has gone back to the pool holds by a weight of zero, which the kernels over rows never read.
        sharing = [l.mixer for j, l in enumerate(cfg.layers) if isinstance(l.mixer, AttentionConfig) and _writer_of(cfg, j) == _writer_of(cfg, i)]
        rows = any(s.window is not None for s in sharing)
        return part("unit_norm_attention", hidden_size=cfg.width, num_heads=m.heads, num_kv_heads=m.kv_heads, dim=m.dim, vdim=m.vdim,
                    scale=m.scale, eps=None, position=_position(m.rot, m.dim, "half"), head_temperature=False, sink=None,
                    values="projected", window=m.window, keep_first=m.keep_first, bias=True, own_kv=m.kv_from is None,
                    layout="rows" if rows else "auto")
    if isinstance(m, LatentAttentionConfig):
        return part("latent_attention", hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim,
                    q_rank=None, kv_rank=m.kv_rank, scale=m.scale, window=None, eps=cfg.norm_eps, gate="channel", sink=True,
                    position=_position(m.rot, m.rot_dim, "interleaved") or part("none"))
    raise TypeError(f"no mixer for {type(m).__name__}")


def zomolix_spec(cfg: ZomolixConfig) -> ModelSpec:
    norm = part("rms", size=cfg.width, eps=cfg.norm_eps)
    scale = part("channel_scale", size=cfg.width)
    layers = []
    for i, layer in enumerate(cfg.layers):
        f = layer.mlp
        ffn = None if f is None else part(
            "routed_experts", hidden_size=cfg.width, experts=f.experts, expert_size=f.ff, top=f.top, groups=f.groups, keep=f.keep,
            scale=1.0, correction=False, scores="softmax", group_score="max", normalize=False, activation="clipped_swiglu",
            limit=f.limit, gate_alpha=GATE_ALPHA, up_offset=UP_OFFSET, shared_size=f.shared_ff, shared_limit=f.shared_limit,
            shared_gate=False)
        layers.append(LayerSpec(mixer=_mixer_spec(cfg, i), ffn=ffn, mixer_norm=norm, ffn_norm=None if ffn is None else norm,
                                arrangement="pre_norm", mixer_scale=scale, ffn_scale=None if ffn is None else scale))
    return ModelSpec(
        architecture=ARCHITECTURE,
        vocab_size=cfg.vocab,
        hidden_size=cfg.width,
        max_positions=MAX_POSITIONS,
        embedding=part("token_embedding", vocab_size=cfg.vocab, hidden_size=cfg.width, scale=cfg.embedding_scale),
        layers=tuple(layers),
        # a layer that names another layer's keys and values reads that layer's cache entry and writes none
        schedule=tuple(LayerCall(layer=i, cache=_writer_of(cfg, i), writes_cache=_writer_of(cfg, i) == i) for i in range(len(layers))),
        final_norm=norm,
        head=part("lm_head", vocab_size=cfg.vocab, hidden_size=cfg.width, tied=False),
        stop_token_ids=cfg.stop_token_ids,
    )


_LAYER = re.compile(r"^layers\.(\d+)\.(.+)$")
_EXPERT = re.compile(r"^ffn\.experts\.(\d+)\.(gate|up|down)_proj$")
_IN_LAYER = {
    "mixer_norm.weight": "norm1",
    "ffn_norm.weight": "norm2",
    "mixer_scale.weight": "ls1",
    "ffn_scale.weight": "ls2",
    # attention
    "mixer.q_proj": "mix.q", "mixer.q_bias": "mix.q.b",
    "mixer.k_proj": "mix.k", "mixer.k_bias": "mix.k.b",
    "mixer.v_proj": "mix.v", "mixer.v_bias": "mix.v.b",
    "mixer.o_proj": "mix.o", "mixer.o_bias": "mix.o.b",
    # latent attention (its query projection is mix.q as well)
    "mixer.kv_down": "mix.dkv",
    "mixer.kv_down_norm": "mix.dkv.norm",
    "mixer.k_up": "mix.uk",
    "mixer.v_up": "mix.uv",
    "mixer.sink": "mix.sink",
    "mixer.out_gate": "mix.g",
    # feed-forward
    "ffn.router": "mlp.router",
    "ffn.shared.gate_proj": "mlp.shared.gate",
    "ffn.shared.up_proj": "mlp.shared.up",
    "ffn.shared.down_proj": "mlp.shared.down",
}
_TOP = {"embedding.weight": "embed", "final_norm.weight": "final.norm", "head.weight": "head"}


def zomolix_tensor_name(path: str) -> str:
    if path in _TOP:
        return _TOP[path]
    m = _LAYER.match(path)
    if m:
        if m.group(2) in _IN_LAYER:
            return f"l{m.group(1)}.{_IN_LAYER[m.group(2)]}"
        e = _EXPERT.match(m.group(2))
        if e:
            return f"l{m.group(1)}.mlp.e{e.group(1)}.{e.group(2)}"
    raise KeyError(f"{ARCHITECTURE} has no tensor for part path {path!r}")


ZOMOLIX = Architecture(
    name=ARCHITECTURE,
    model_types=("zomolix",),
    read_config=ZomolixConfig.from_dicts,
    to_spec=zomolix_spec,
    tensor_name=zomolix_tensor_name,
)

register_architecture(ZOMOLIX, replace=True)
