"""Small Goganex configurations and random weights of the tests' own making (no code of the package is used to draw or
name a tensor): config.json contents, a tensor dictionary by checkpoint name, and a folder writer."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file


def rot(dims, base=10000.0, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        factor, low, high, original = scaling
        out["scaling"] = {"factor": factor, "low": low, "high": high, "original": original}
    return out


def attention(heads=3, kv_heads=1, dim=8, vdim=6, scale=0.3, rotation=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rotation is not None:
        m["rot"] = rotation
    return m


def parallel(heads=2, kv_heads=1, dim=8, scale=0.25, width=12):
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}, "right": {"width": width}}


def dense(ff, limit=2.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=61, width=24, eps=2e-5, scale=2.5, loop=None):
    out = {"architecture": "Goganex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
           "layers": layers}
    if loop is not None:
        out["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return out


# Frequencies of every kind for the scaling by wavelength: with base 10,000 over 16 elements the wavelengths run from 6
# to 20,000 positions; original 64 with low 1 and high 4 keeps those below 16, slows those above 64 and blends between.
SCALED = (4.0, 1.0, 4.0, 64)

# Sizes that differ wherever a model could happen to make them equal or 1: key and value sizes, query heads per
# key/value head (1, 2, 3), rotations of the whole head and of a part, with and without scaling, layers without a
# feed-forward, both mixers first and last, no loop, a loop over the middle, a loop over everything, a loop that runs once.
CONFIGS = {
    "attn_only": config([layer("attention", attention(rotation=rot(4)), None)]),
    "parallel_only": config([layer("parallel", parallel(), None)], vocab=47, width=16),
    "mixed": config([
        layer("parallel", parallel(heads=4, kv_heads=2, dim=6, scale=0.4, width=20), dense(28, limit=0.7)),
        layer("attention", attention(heads=4, kv_heads=2, dim=16, vdim=10, scale=0.21, rotation=rot(16, scaling=SCALED)), dense(36, limit=3.0)),
        layer("attention", attention(heads=2, kv_heads=2, dim=12, vdim=24, scale=0.3, rotation=rot(6, base=500.0)), None),
        layer("parallel", parallel(heads=3, kv_heads=3, dim=10, scale=0.2, width=7), dense(50, limit=1.2)),
        layer("attention", attention(heads=6, kv_heads=1, dim=4, vdim=3, scale=0.5), None),
    ], vocab=131, width=40, eps=3e-6, scale=5.5, loop=(1, 4, 3)),
    "whole_loop": config([
        layer("attention", attention(heads=6, kv_heads=3, dim=10, vdim=9, scale=0.35, rotation=rot(8, base=300.0, scaling=(8.0, 1.0, 2.0, 32))), dense(40, limit=1.0)),
        layer("parallel", parallel(heads=2, kv_heads=1, dim=24, scale=0.15, width=33), dense(33, limit=5.0)),
    ], vocab=97, width=48, eps=1e-5, scale=2.0, loop=(0, 2, 2)),
    "loop_once": config([
        layer("parallel", parallel(heads=1, kv_heads=1, dim=5, scale=0.6, width=9), None),
        layer("attention", attention(heads=1, kv_heads=1, dim=6, vdim=6, scale=0.4, rotation=rot(6)), dense(20, limit=0.9)),
    ], vocab=53, width=20, eps=1e-6, scale=1.0, loop=(1, 2, 1)),
    # sizes in the multiples the tensor-core products and the tensor-core attention kernel take
    "wide": config([
        layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=32, scale=0.05, rotation=rot(32, scaling=SCALED)), dense(192, limit=1.5)),
        layer("parallel", parallel(heads=4, kv_heads=1, dim=32, scale=0.08, width=96), dense(256, limit=2.5)),
        layer("attention", attention(heads=8, kv_heads=8, dim=16, vdim=40, scale=0.12, rotation=rot(16)), None),
    ], vocab=512, width=128, scale=3.5, loop=(0, 2, 2)),
    # keys and values of one size, 64 or 128: the cache entry with a plane of keys and a plane of values, and the
    # attention kernels that the plain attention part uses (here with the sink, the factors and keys that are values)
    "planes": config([
        layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.06, rotation=rot(32, scaling=SCALED)), dense(160, limit=1.5)),
        layer("parallel", parallel(heads=2, kv_heads=1, dim=128, scale=0.05, width=72), None),
        layer("attention", attention(heads=3, kv_heads=3, dim=128, vdim=128, scale=0.04, rotation=rot(128, base=5000.0)), dense(96, limit=2.0)),
        layer("parallel", parallel(heads=6, kv_heads=2, dim=64, scale=0.07, width=40), dense(128, limit=1.0)),
    ], vocab=300, width=96, eps=1e-5, scale=3.0, loop=(1, 3, 2)),
}


def tensors(cfg, seed=0, dtype=torch.float32, std=0.5):
    """Checkpoint name -> tensor.  Matrices scaled so that activations stay of order one; norm gains around one; shift
    weights between 0 and 1; head factors around one; gate biases that give the recurrence a memory of several tokens."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    def attn(p, m, own_values, temp):
        h, kv = m["heads"], m["kv_heads"]
        out[p + "q"] = rnd(h * m["dim"], w, s=2 * std / w ** 0.5)
        out[p + "k"] = rnd(kv * m["dim"], w, s=2 * std / w ** 0.5)
        if own_values:
            out[p + "v"] = rnd(kv * m["vdim"], w, s=std / w ** 0.5)
        if temp:
            out[p + "temp"] = 1.5 + rnd(h, s=0.5)
        out[p + "o"] = rnd(w, h * m["vdim"], s=std)

    w = cfg["width"]
    out = {"embed": rnd(cfg["vocab"], w, s=0.3), "final.norm": 1 + rnd(w, s=0.1), "head": rnd(cfg["vocab"], w, s=1.0 / w ** 0.5)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = 1 + rnd(w, s=0.1)
        out[p + "shift"] = torch.rand(w, generator=g)
        if lay["type"] == "attention":
            attn(p + "mix.", m, True, True)
        else:
            attn(p + "mix.left.", m["left"], False, False)
            r = m["right"]["width"]
            out[p + "mix.right.z"] = rnd(r, w, s=2 * std / w ** 0.5)
            out[p + "mix.right.z.b"] = rnd(r, s=0.5) - 1.0
            out[p + "mix.right.x"] = rnd(r, w, s=2 * std / w ** 0.5)
            out[p + "mix.right.x.b"] = rnd(r, s=0.5)
            out[p + "mix.right.g"] = rnd(r, w, s=2 * std / w ** 0.5)
            out[p + "mix.right.o"] = rnd(w, r, s=std)
            out[p + "mix.left.out"] = 1 + rnd(w, s=0.1)
            out[p + "mix.right.out"] = 1 + rnd(w, s=0.1)
        mlp = lay["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = 1 + rnd(w, s=0.1)
        out[p + "mlp.gate"] = rnd(mlp["ff"], w, s=3 * std / w ** 0.5)   # wide enough to reach the limit now and then
        out[p + "mlp.up"] = rnd(mlp["ff"], w, s=3 * std / w ** 0.5)
        out[p + "mlp.down"] = rnd(w, mlp["ff"], s=std / mlp["ff"] ** 0.5)
    return {k: v.to(dtype).contiguous() for k, v in out.items()}


def write_folder(folder, cfg, weights) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
