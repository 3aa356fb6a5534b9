"""Named configurations for the random-weights mode (benchmarks and tests).

These are config.json contents, i.e. data: the engine reads sizes only from a
configuration, never from this file directly.
"""

from __future__ import annotations

from .llama import LlamaConfig
from .registry import architecture_of

_LLAMA3_ROPE = {"rope_type": "llama3", "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                "original_max_position_embeddings": 8192}

PRESETS: dict[str, dict] = {
    "tiny-a": {
        "model_type": "llama", "vocab_size": 256, "hidden_size": 64, "intermediate_size": 128, "num_hidden_layers": 2,
        "num_attention_heads": 4, "num_key_value_heads": 2, "head_dim": 16, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
        "max_position_embeddings": 256, "tie_word_embeddings": True,
    },
    "tiny-b": {
        "model_type": "llama", "vocab_size": 384, "hidden_size": 96, "intermediate_size": 256, "num_hidden_layers": 3,
        "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "rms_norm_eps": 1e-6, "rope_theta": 500000.0,
        "rope_scaling": {"rope_type": "llama3", "factor": 4.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                         "original_max_position_embeddings": 64},
        "max_position_embeddings": 512, "tie_word_embeddings": False,
    },
    "llama-3.2-1b": {
        "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048, "intermediate_size": 8192,
        "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 64,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_ROPE, factor=32.0),
        "max_position_embeddings": 131072, "tie_word_embeddings": True,
    },
    "llama-3.2-3b": {
        "model_type": "llama", "vocab_size": 128256, "hidden_size": 3072, "intermediate_size": 8192,
        "num_hidden_layers": 28, "num_attention_heads": 24, "num_key_value_heads": 8, "head_dim": 128,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_ROPE, factor=32.0),
        "max_position_embeddings": 131072, "tie_word_embeddings": True,
    },
    "llama-3.1-8b": {
        "model_type": "llama", "vocab_size": 128256, "hidden_size": 4096, "intermediate_size": 14336,
        "num_hidden_layers": 32, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
        "rms_norm_eps": 1e-5, "rope_theta": 500000.0, "rope_scaling": dict(_LLAMA3_ROPE, factor=8.0),
        "max_position_embeddings": 131072, "tie_word_embeddings": False,
    },
}


def _nerenex(width: int, vocab: int, groups: int, heads: int, ff: int, window: int, recurrent_width: int) -> dict:
    """``groups`` times (recurrence, recurrence, latent attention), every layer with a dense feed-forward."""
    attention = {"type": "latent_attention", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 3 * width // 4, "kv_rank": 512,
                           "scale": 192 ** -0.5, "mask": {"size": window}, "rot": {"base": 10000.0, "dims": 64}}}
    recurrent = {"type": "rglru", "mlp": {"kind": "dense", "ff": ff},
                 "mixer": {"width": recurrent_width, "blocks": heads, "conv": 4}}
    return {"architecture": "Nerenex", "vocab": vocab, "width": width, "residual_mult": 0.5, "norm": {"eps": 1e-6},
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 8191}},
            "layers": [recurrent, recurrent, attention] * groups}


PRESETS.update({
    "nerenex-tiny": {
        "architecture": "Nerenex", "vocab": 256, "width": 64, "residual_mult": 0.5, "norm": {"eps": 1e-6},
        "embedding": {"bigram": {"buckets": 251, "mul_prev": 31, "mul_cur": 7}},
        "layers": [
            {"type": "rglru", "mixer": {"width": 96, "blocks": 3, "conv": 4}, "mlp": {"kind": "dense", "ff": 128}},
            {"type": "latent_attention", "mlp": None,
             "mixer": {"heads": 4, "dim": 16, "rot_dim": 8, "vdim": 24, "q_rank": 48, "kv_rank": 32, "scale": 0.2,
                       "mask": {"size": 24}, "rot": {"base": 10000.0, "dims": 8}}},
        ],
    },
    # layer sizes of a 1B- and an 8B-class decoder (width, heads, feed-forward), for the benchmarks
    "nerenex-2048": _nerenex(2048, 32768, 4, 16, 8192, 1024, 2560),
    "nerenex-4096": _nerenex(4096, 32768, 2, 32, 14336, 2048, 4096),
})


def _gekopel(width: int, vocab: int, groups: int, heads: int, ff: int, chunk: int, experts: int, expert_ff: int) -> dict:
    """A dense first layer, then ``groups`` times (delta rule, delta rule, chunked attention) with routed experts."""
    moe = {"kind": "moe", "expert": {"ff": expert_ff}, "shared": {"ff": expert_ff},
           "router": {"experts": experts, "top": 4, "scale": 2.5, "groups": {"count": 8, "keep": 4}}}
    attention = {"type": "attention", "mlp": moe,
                 "mixer": {"heads": heads, "kv_heads": heads // 4, "dim": 128, "vdim": 128, "scale": 128 ** -0.5,
                           "bias_max": chunk, "mask": {"size": chunk}}}
    delta = {"type": "delta", "mlp": moe, "mixer": {"heads": heads, "kv_heads": heads // 2, "dim": 128, "vdim": 128, "conv": 4}}
    layers = [delta, delta, attention] * groups
    layers[0] = dict(delta, mlp={"kind": "dense", "ff": ff})
    return {"architecture": "Gekopel", "vocab": vocab, "width": width, "max_positions": 8192, "norm": {"eps": 1e-6},
            "embedding": {"scale": 1.0}, "layers": layers}


PRESETS.update({
    "gekopel-tiny": {
        "architecture": "Gekopel", "vocab": 256, "width": 64, "max_positions": 512, "norm": {"eps": 1e-6}, "embedding": {"scale": 4.0},
        "layers": [
            {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "conv": 4}, "mlp": {"kind": "dense", "ff": 128}},
            {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "bias_max": 48, "mask": {"size": 40}},
             "mlp": {"kind": "moe", "expert": {"ff": 32}, "shared": {"ff": 48},
                     "router": {"experts": 8, "top": 2, "scale": 1.25, "groups": {"count": 4, "keep": 2}}}},
        ],
    },
    # layer sizes of a 1B- and an 8B-class decoder (width, heads), for the benchmarks: per token 4 of 32 experts and a shared one
    "gekopel-2048": _gekopel(2048, 32768, 4, 16, 8192, 1024, 32, 1024),
    "gekopel-4096": _gekopel(4096, 32768, 2, 32, 14336, 2048, 32, 2048),
})


def _goganex(width: int, vocab: int, groups: int, heads: int, kv_heads: int, dim: int, ff: int, recurrent_width: int) -> dict:
    """``groups`` times (attention, attention, attention, parallel), every layer with a feed-forward."""
    rot = {"base": 500000.0, "dims": dim, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    mlp = {"kind": "dense", "ff": ff, "limit": 7.0}
    attention = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": rot}}
    parallel = {"type": "parallel", "mlp": mlp,
                "mixer": {"left": {"heads": heads // 2, "kv_heads": kv_heads // 2, "dim": dim, "vdim": dim, "scale": dim ** -0.5},
                          "right": {"width": recurrent_width}}}
    return {"architecture": "Goganex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0},
            "layers": [attention, attention, attention, parallel] * groups}


PRESETS.update({
    "goganex-tiny": {
        "architecture": "Goganex", "vocab": 256, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
        "loop": {"start": 0, "stop": 2, "times": 2},
        "layers": [
            {"type": "attention", "mlp": {"kind": "dense", "ff": 128, "limit": 2.0},
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25,
                       "rot": {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}}},
            {"type": "parallel", "mlp": None,
             "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 16, "vdim": 16, "scale": 0.25}, "right": {"width": 48}}},
        ],
    },
    # layer sizes of a 1B- and an 8B-class decoder (width, heads, feed-forward), for the benchmarks
    "goganex-2048": _goganex(2048, 32768, 3, 32, 8, 64, 8192, 2048),
    "goganex-4096": _goganex(4096, 32768, 2, 32, 8, 128, 14336, 4096),
})


def _zomolix(width: int, vocab: int, groups: int, heads: int, kv_heads: int, dim: int, latent_heads: int, kv_rank: int,
             window: int, experts: int, top: int, ff: int, shared_ff: int) -> dict:
    """``groups`` times (latent attention, windowed attention, latent attention, windowed attention reading the keys and
    values of the one before it), every layer with routed experts and a shared one."""
    rot = {"base": 500000.0, "dims": dim // 2, "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    lrot = {"base": 10000.0, "dims": 64, "scaling": {"factor": 4.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    mlp = {"kind": "moe", "expert": {"ff": ff, "limit": 7.0}, "router": {"experts": experts, "top": top, "groups": {"count": 8, "keep": 4}},
           "shared": {"ff": shared_ff, "limit": 7.0}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": latent_heads, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": kv_rank, "scale": 192 ** -0.5, "rot": lrot}}
    layers = []
    for g in range(groups):
        attention = {"type": "attention", "mlp": mlp,
                     "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": rot,
                               "mask": {"size": window, "keep_first": 4}}}
        reader = {"type": "attention", "mlp": mlp, "mixer": dict(attention["mixer"], kv_from=4 * g + 1)}
        layers += [latent, attention, latent, reader]
    return {"architecture": "Zomolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.0}, "layers": layers}


PRESETS.update({
    "zomolix-tiny": {
        "architecture": "Zomolix", "vocab": 256, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
        "layers": [
            {"type": "latent_attention",
             "mlp": {"kind": "moe", "expert": {"ff": 32, "limit": 2.0}, "router": {"experts": 8, "top": 2, "groups": {"count": 4, "keep": 2}},
                     "shared": {"ff": 48, "limit": 1.5}},
             "mixer": {"heads": 2, "dim": 16, "rot_dim": 8, "vdim": 24, "kv_rank": 32, "scale": 0.2,
                       "rot": {"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}}},
            {"type": "attention", "mlp": None,
             "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "mask": {"size": 24, "keep_first": 3},
                       "rot": {"base": 10000.0, "dims": 8}}},
            {"type": "attention",
             "mlp": {"kind": "moe", "expert": {"ff": 16, "limit": 3.0}, "router": {"experts": 4, "top": 1, "groups": {"count": 1, "keep": 1}}},
             "mixer": {"heads": 2, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.25, "mask": {"size": 40, "keep_first": 0},
                       "rot": {"base": 10000.0, "dims": 8}, "kv_from": 1}},
        ],
    },
    # layer sizes of a 1B- and an 8B-class decoder (width, heads), for the benchmarks: per token 4 of 32 experts and a shared one
    "zomolix-2048": _zomolix(2048, 32768, 3, 16, 4, 128, 16, 512, 1024, 32, 4, 1024, 1024),
    "zomolix-4096": _zomolix(4096, 32768, 2, 32, 8, 128, 32, 512, 2048, 32, 4, 2048, 2048),
})


def preset(name: str):
    """The typed configuration of a preset, read by its architecture's own reader."""
    try:
        raw = PRESETS[name]
    except KeyError:
        raise ValueError(f"no preset {name!r}; known: {sorted(PRESETS)}") from None
    if "architecture" not in raw and "architectures" not in raw:
        return LlamaConfig.from_dicts(raw)
    return architecture_of(raw).read_config(raw, None)
