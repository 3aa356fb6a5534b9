"""Small Zomolix configurations and random weights of the tests' own making (no code of the package is used to draw or
name a tensor): config.json contents, a tensor dictionary by checkpoint name, and a folder writer."""

from __future__ import annotations

import json
from pathlib import Path

import torch
from safetensors.torch import save_file


def rot(dims, base=10000.0, scaling=None):
    out = {"base": base, "dims": dims}
    if scaling is not None:
        factor, original, fast, slow = scaling
        out["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return out


def attention(heads=3, kv_heads=1, dim=8, vdim=6, scale=0.3, rotation=None, mask=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rotation or rot(4)}
    if mask is not None:
        m["mask"] = {"size": mask[0], "keep_first": mask[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def latent(heads=2, dim=8, rot_dim=4, vdim=6, kv_rank=12, scale=0.3, rotation=None):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
            "rot": rotation or rot(rot_dim)}


def moe(experts=6, top=2, ff=10, limit=1.5, groups=(3, 2), shared=(14, 1.0)):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit},
           "router": {"experts": experts, "top": top, "groups": {"count": groups[0], "keep": groups[1]}}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


def config(layers, vocab=61, width=24, eps=2e-5, scale=2.5):
    return {"architecture": "Zomolix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": scale},
            "layers": layers}


# With base 10,000 over 16 elements the wavelengths run from 6 to 20,000 positions; an original length of 64 with
# fast 8 and slow 1 leaves the shortest as they are, stretches the longest and ramps between.
SCALED = (4.0, 64, 8.0, 1.0)

# Sizes that differ wherever a model could happen to make them equal or 1: key and value sizes, query heads per
# key/value head (1, 2, 3), rotations of the whole head and of a part, with and without scaling, windows with and
# without kept first keys, no window, a reader whose mask differs from its writer's, layers without a feed-forward,
# one group (nothing dropped), every group kept, one choice, no shared expert, both mixers first and last.
CONFIGS = {
    "attn_only": config([layer("attention", attention(mask=(9, 2)), None)]),
    "latent_only": config([layer("latent_attention", latent(), None)], vocab=47, width=16),
    "mixed": config([
        layer("latent_attention", latent(heads=3, dim=6, rot_dim=8, vdim=10, kv_rank=20, scale=0.4, rotation=rot(6, base=300.0, scaling=(2.0, 32, 4.0, 1.0))),
              moe(experts=8, top=3, ff=12, limit=0.7, groups=(4, 3), shared=(20, 2.0))),
        layer("attention", attention(heads=4, kv_heads=2, dim=16, vdim=10, scale=0.21, rotation=rot(16, scaling=SCALED), mask=(21, 5)),
              moe(experts=4, top=1, ff=9, limit=3.0, groups=(1, 1), shared=None)),
        layer("attention", attention(heads=2, kv_heads=2, dim=16, vdim=10, scale=0.3, rotation=rot(16, scaling=SCALED), mask=(33, 0), kv_from=1), None),
        layer("latent_attention", latent(heads=1, dim=5, rot_dim=2, vdim=7, kv_rank=9, scale=0.5), moe(experts=6, top=2, ff=8, limit=1.2, groups=(2, 2))),
        layer("attention", attention(heads=6, kv_heads=2, dim=16, vdim=10, scale=0.25, rotation=rot(16, scaling=SCALED), mask=(7, 18), kv_from=1),
              moe(experts=6, top=4, ff=5, limit=2.0, groups=(3, 2), shared=(7, 0.5))),
        layer("attention", attention(heads=6, kv_heads=1, dim=4, vdim=3, scale=0.5, rotation=rot(2, base=50.0)), None),
    ], vocab=131, width=40, eps=3e-6, scale=5.5),
    # a window on the writer only, none on the reader: nothing of the entry may be let go
    "reader_sees_all": config([
        layer("attention", attention(heads=2, kv_heads=1, dim=12, vdim=12, scale=0.3, rotation=rot(8, base=500.0), mask=(10, 3)), moe()),
        layer("attention", attention(heads=3, kv_heads=1, dim=12, vdim=12, scale=0.2, rotation=rot(8, base=500.0), kv_from=0), moe(groups=(2, 1), top=3)),
    ], vocab=97, width=48, eps=1e-5, scale=2.0),
    # sizes in the multiples the tensor-core products and the tensor-core attention kernels take; heads of 64 and 128
    # with keys and values of one size: without kept keys such a layer keeps planes of keys and values
    "wide": config([
        layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.06, rotation=rot(32, scaling=SCALED), mask=(50, 0)),
              moe(experts=8, top=2, ff=64, limit=1.5, groups=(4, 2), shared=(96, 1.0))),
        layer("latent_attention", latent(heads=2, dim=40, rot_dim=24, vdim=24, kv_rank=72, scale=0.1, rotation=rot(16, scaling=(3.0, 64, 8.0, 1.0))),
              moe(experts=12, top=3, ff=32, limit=2.5, groups=(3, 2), shared=(64, 1.25))),
        layer("attention", attention(heads=4, kv_heads=2, dim=96, vdim=40, scale=0.07, rotation=rot(32, base=30000.0, scaling=(6.0, 64, 8.0, 1.0)), mask=(44, 5)), None),
        layer("attention", attention(heads=2, kv_heads=2, dim=96, vdim=40, scale=0.07, rotation=rot(32, base=30000.0, scaling=(6.0, 64, 8.0, 1.0)), mask=(70, 1), kv_from=2),
              moe(experts=4, top=2, ff=128, limit=1.0, groups=(2, 1), shared=None)),
        layer("attention", attention(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.04, rotation=rot(128, base=5000.0)), None),
        layer("attention", attention(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.06, rotation=rot(64), mask=(30, 4)), moe(experts=4, top=2, ff=16, groups=(2, 2))),
    ], vocab=300, width=128, eps=1e-5, scale=3.0),
}


def tensors(cfg, seed=0, dtype=torch.float32, std=0.5):
    """Checkpoint name -> tensor.  Matrices scaled so that activations stay of order one; norm gains and layer scales
    around one; biases, sinks and router rows large enough to matter."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0):
        return torch.randn(*shape, generator=g) * s

    def expert(p, ff):
        out[p + "gate"] = rnd(ff, w, s=3 * std / w ** 0.5)   # wide enough to reach the limit now and then
        out[p + "up"] = rnd(ff, w, s=3 * std / w ** 0.5)
        out[p + "down"] = rnd(w, ff, s=std / ff ** 0.5)

    w = cfg["width"]
    out = {"embed": rnd(cfg["vocab"], w, s=0.3), "final.norm": 1 + rnd(w, s=0.1), "head": rnd(cfg["vocab"], w, s=1.0 / w ** 0.5)}
    for i, lay in enumerate(cfg["layers"]):
        p, m = f"l{i}.", lay["mixer"]
        out[p + "norm1"] = 1 + rnd(w, s=0.1)
        out[p + "ls1"] = 1 + rnd(w, s=0.3)
        if lay["type"] == "attention":
            h, kv = m["heads"], m["kv_heads"]
            out[p + "mix.q"] = rnd(h * m["dim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.q.b"] = rnd(h * m["dim"], s=0.3)
            if m.get("kv_from") is None:
                out[p + "mix.k"] = rnd(kv * m["dim"], w, s=2 * std / w ** 0.5)
                out[p + "mix.k.b"] = rnd(kv * m["dim"], s=0.3)
                out[p + "mix.v"] = rnd(kv * m["vdim"], w, s=std / w ** 0.5)
                out[p + "mix.v.b"] = rnd(kv * m["vdim"], s=0.3)
            out[p + "mix.o"] = rnd(w, h * m["vdim"], s=std)
            out[p + "mix.o.b"] = rnd(w, s=0.3)
        else:
            h = m["heads"]
            out[p + "mix.q"] = rnd(h * (m["dim"] + m["rot_dim"]), w, s=2 * std / w ** 0.5)
            out[p + "mix.dkv"] = rnd(m["kv_rank"] + m["rot_dim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.dkv.norm"] = 1 + rnd(m["kv_rank"], s=0.1)
            out[p + "mix.uk"] = rnd(h * m["dim"], m["kv_rank"], s=1.0 / m["kv_rank"] ** 0.5)
            out[p + "mix.uv"] = rnd(h * m["vdim"], m["kv_rank"], s=1.0 / m["kv_rank"] ** 0.5)
            out[p + "mix.sink"] = rnd(h, s=1.0)
            out[p + "mix.g"] = rnd(h * m["vdim"], w, s=2 * std / w ** 0.5)
            out[p + "mix.o"] = rnd(w, h * m["vdim"], s=std)
        mlp = lay["mlp"]
        if mlp is None:
            continue
        out[p + "norm2"] = 1 + rnd(w, s=0.1)
        out[p + "ls2"] = 1 + rnd(w, s=0.3)
        for e in range(mlp["router"]["experts"]):
            expert(f"{p}mlp.e{e}.", mlp["expert"]["ff"])
        out[p + "mlp.router"] = rnd(mlp["router"]["experts"], w, s=2.0 / w ** 0.5)
        if mlp.get("shared"):
            expert(p + "mlp.shared.", mlp["shared"]["ff"])
    return {k: v.to(dtype).contiguous() for k, v in out.items()}


def write_folder(folder, cfg, weights) -> Path:
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(folder / "model.safetensors"))
    return folder
