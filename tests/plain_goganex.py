"""A plain, slow implementation of the Goganex decoder, one function per mechanism, written from the design's
equations in whatever precision the given tensors have (the tests use float64).  It shares no code with the engine:
no cache, no pages, no batching; a sequence is run whole, token by token where the design is a recurrence.

Notation: x is the stream [T, width]; weights are looked up in ``w`` by their checkpoint names (``l3.mix.q`` ...);
``cfg`` is the parsed config.json.
"""

from __future__ import annotations

import math

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (its mean square + eps), along the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * gain


def token_shift(h: torch.Tensor, mix: torch.Tensor) -> torch.Tensor:
    """Every row moves toward the row before it (as that row was before it moved), channel by channel by ``mix``; the
    row before the first one is zero."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (before - h) * mix


def rotary_frequencies(rot, dtype=torch.float64) -> torch.Tensor:
    """One frequency per pair of rotated elements: base^(-2i/n), then stretched by wavelength: short waves stay, long
    ones are slowed by ``factor``, those between are blended linearly in original/wavelength."""
    n = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / n) for i in range(n // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if sc:
        out = []
        for fi in f.tolist():
            wave = 2 * math.pi / fi
            if wave < sc["original"] / sc["high"]:
                out.append(fi)
            elif wave > sc["original"] / sc["low"]:
                out.append(fi / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1 - s) * fi / sc["factor"] + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(dtype)


def rotate(x: torch.Tensor, rot, first_position: int = 0) -> torch.Tensor:
    """x [T, heads, dim]: elements 2i and 2i+1 of the first ``dims`` turn together by position * frequency_i."""
    t, n = x.shape[0], rot["dims"]
    places = torch.arange(first_position, first_position + t, dtype=torch.float64)
    angle = (places[:, None] * rotary_frequencies(rot)[None, :]).to(x.dtype)          # [T, n/2]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., 0:n:2], x[..., 1:n:2]
    out = x.clone()
    out[..., 0:n:2] = a * c - b * s
    out[..., 1:n:2] = b * c + a * s
    return out


def softmax_attention(q, k, v, scale, temp=None, sink=False):
    """Causal attention, q [T, heads, dim], k [T, groups, dim], v [T, groups, vdim]; query head a reads group
    a // (heads / groups).  ``temp``: a factor on every score of a head.  ``sink``: one is added to the sum of the
    exponentials (a key with score zero and no value)."""
    t, heads, _ = q.shape
    groups = k.shape[1]
    out = torch.zeros(t, heads, v.shape[2], dtype=q.dtype)
    for i in range(t):
        for a in range(heads):
            g = a // (heads // groups)
            s = (k[: i + 1, g] @ q[i, a]) * scale
            if temp is not None:
                s = s * temp[a]
            top = s.max().clamp_min(0) if sink else s.max()
            e = torch.exp(s - top)
            total = e.sum() + (torch.exp(-top) if sink else 0)
            out[i, a] = (e[:, None] * v[: i + 1, g]).sum(0) / total
    return out


def attention(m, w, pre, h, eps):
    """Rotated, unit-normed queries and keys, a factor per head, a sink in the denominator."""
    t = h.shape[0]
    heads, groups, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).view(t, heads, dim)
    k = (h @ w[pre + "k"].T).view(t, groups, dim)
    v = (h @ w[pre + "v"].T).view(t, groups, vdim)
    if m.get("rot"):
        q, k = rotate(q, m["rot"]), rotate(k, m["rot"])
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    o = softmax_attention(q, k, v, m["scale"], temp=w[pre + "temp"], sink=True)
    return o.reshape(t, heads * vdim) @ w[pre + "o"].T


def key_value_attention(m, w, pre, h, eps):
    """The left half of a parallel mixer: no rotation, the projected keys serve as values, plain softmax."""
    t = h.shape[0]
    heads, groups, dim = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[pre + "q"].T).view(t, heads, dim)
    k = (h @ w[pre + "k"].T).view(t, groups, dim)
    o = softmax_attention(unit_rms(q, eps), unit_rms(k, eps), k, m["scale"])
    return o.reshape(t, heads * dim) @ w[pre + "o"].T


def min_gru(m, w, pre, h):
    """S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0, gates and candidate from the current token only."""
    z = torch.sigmoid(h @ w[pre + "z"].T + w[pre + "z.b"])
    u = h @ w[pre + "x"].T + w[pre + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    gate = h @ w[pre + "g"].T
    state = torch.zeros(m["width"], dtype=h.dtype)
    rows = []
    for i in range(h.shape[0]):
        state = (1 - z[i]) * state + z[i] * cand[i]
        rows.append(state * gate[i] * torch.sigmoid(gate[i]))
    return torch.stack(rows) @ w[pre + "o"].T


def parallel(m, w, pre, h, eps):
    left = key_value_attention(m["left"], w, pre + "left.", h, eps)
    right = min_gru(m["right"], w, pre + "right.", h)
    return 0.5 * (norm(left, w[pre + "left.out"], eps) + norm(right, w[pre + "right.out"], eps))


def feed_forward(f, w, pre, h):
    lim = f["limit"]
    g = (h @ w[pre + "gate"].T).clamp(max=lim)
    u = (h @ w[pre + "up"].T).clamp(-lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[pre + "down"].T


def layer_order(cfg) -> list[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer run, if asked)."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    seen = []
    for i in layer_order(cfg):
        lay, pre = cfg["layers"][i], f"l{i}."
        h = token_shift(norm(x, w[pre + "norm1"], eps), w[pre + "shift"])
        if lay["type"] == "attention":
            x = x + attention(lay["mixer"], w, pre + "mix.", h, eps)
        elif lay["type"] == "parallel":
            x = x + parallel(lay["mixer"], w, pre + "mix.", h, eps)
        else:
            raise ValueError(lay["type"])
        if lay.get("mlp"):
            x = x + feed_forward(lay["mlp"], w, pre + "mlp.", norm(x, w[pre + "norm2"], eps))
        seen.append(x)
    logits = norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(seen)) if return_layers else logits
