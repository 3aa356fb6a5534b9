"""Zomolix restated plainly: float64 torch on the CPU, one function per mechanism, whole sequences at a time, no cache.

Shares no code with the package.  A model is a dict ``config`` in the shape of the design's config.json and a dict of
tensors by checkpoint name; ``forward`` returns the logits of every position (and, on request, the stream after every
layer).

Notation: x is a [tokens, width] stream, positions count from 0, W applies as x @ W.T.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight, the mean over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotary_frequencies(rot):
    """(angular frequency per pair [dims / 2], amplitude) of a rotation described by ``rot`` = {base, dims, scaling}.

    Plain: f_i = base^(-2i / dims).  With ``scaling`` = {factor, original, fast, slow}: the pair index at which a
    wavelength makes t turns over the original length is d(t) = dims * ln(original / (2 pi t)) / (2 ln base); pairs
    below lo = floor(d(fast)) keep f_i, pairs above hi = ceil(d(slow)) get f_i / factor, a linear ramp between; the
    amplitude of cos and sin becomes 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(original / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0, 1)
    return f / factor * ramp + f * (1 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, positions, rot, layout):
    """v [tokens, heads, size]: the first rot.dims elements of every head turned by the token's position.
    layout "half": element i pairs with i + dims/2; "interleaved": 2i with 2i + 1."""
    dims = int(rot["dims"])
    f, amplitude = rotary_frequencies(rot)
    a = positions.to(F64)[:, None] * f[None, :]
    cos, sin = (a.cos() * amplitude)[:, None, :], (a.sin() * amplitude)[:, None, :]
    out = v.clone()
    if layout == "half":
        u, w = v[..., : dims // 2], v[..., dims // 2: dims]
        out[..., : dims // 2] = u * cos - w * sin
        out[..., dims // 2: dims] = w * cos + u * sin
    else:
        u, w = v[..., 0:dims:2], v[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - w * sin
        out[..., 1:dims:2] = w * cos + u * sin
    return out


def visible(n, window=None, keep_first=0):
    """[n, n] bool: query i sees key j when j <= i and (no window, or i - j < window, or j < keep_first)."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if window is not None:
        ok = ok & ((i - j < window) | (j < keep_first))
    return ok


def softmax_attention(q, k, v, scale, mask, sink=None):
    """q [n, H, d], k [n, H, d], v [n, H, dv] -> [n, H, dv].  ``sink`` [H]: exp(sink) joins every row's denominator."""
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    s = s.masked_fill(~mask[None], -math.inf)
    top = s.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.to(F64)[:, None, None])
    e = (s - top).exp()
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + (sink.to(F64)[:, None, None] - top).exp()
    return torch.einsum("hij,jhd->ihd", e / den, v)


def attention_keys_values(h, m, w, name, positions):
    """The rotated keys [n, G, dim] and the values [n, G, vdim] of an attention layer that has projections."""
    n, G, dim, vdim = h.shape[0], int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    k = (h @ w[f"{name}.k"].to(F64).T + w[f"{name}.k.b"].to(F64)).view(n, G, dim)
    v = (h @ w[f"{name}.v"].to(F64).T + w[f"{name}.v.b"].to(F64)).view(n, G, vdim)
    return rotate(k, positions, m["rot"], "half"), v


def attention_mixer(h, m, w, name, positions, kv):
    """Grouped-query attention with biases, a partial rotation (half layout) and a sliding window that keeps the first
    tokens.  ``kv``: (rotated keys, values) this layer uses (its own, or another layer's)."""
    n, H, G, dim = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    q = (h @ w[f"{name}.q"].to(F64).T + w[f"{name}.q.b"].to(F64)).view(n, H, dim)
    q = rotate(q, positions, m["rot"], "half")
    k, v = kv
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    mask_cfg = m.get("mask") or {}
    mask = visible(n, mask_cfg.get("size"), int(mask_cfg.get("keep_first", 0)))
    o = softmax_attention(q, k, v, float(m["scale"]), mask)
    return o.reshape(n, -1) @ w[f"{name}.o"].to(F64).T + w[f"{name}.o.b"].to(F64)


def latent_attention_mixer(h, m, w, name, positions, eps):
    """Attention through a shared latent: per token a normed latent c and one rotated key part; per head an unrotated
    key W_uk c and a value W_uv c; a sink in the denominator; an output gate sigmoid(W_g h)."""
    n, H, dim, rot_dim, vdim, rank = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = (h @ w[f"{name}.q"].to(F64).T).view(n, H, dim + rot_dim)
    q_plain, q_rot = q[..., :dim], rotate(q[..., dim:], positions, m["rot"], "interleaved")
    down = h @ w[f"{name}.dkv"].to(F64).T
    c = rms_norm(down[:, :rank], w[f"{name}.dkv.norm"].to(F64), eps)
    k_rot = rotate(down[:, None, rank:], positions, m["rot"], "interleaved")          # [n, 1, rot_dim]
    k_plain = (c @ w[f"{name}.uk"].to(F64).T).view(n, H, dim)
    v = (c @ w[f"{name}.uv"].to(F64).T).view(n, H, vdim)
    qq = torch.cat([q_plain, q_rot], -1)
    kk = torch.cat([k_plain, k_rot.expand(n, H, rot_dim)], -1)
    o = softmax_attention(qq, kk, v, float(m["scale"]), visible(n), sink=w[f"{name}.sink"])
    o = o.reshape(n, -1) * torch.sigmoid(h @ w[f"{name}.g"].to(F64).T)
    return o @ w[f"{name}.o"].to(F64).T


def clipped_expert(h, w, name, limit):
    """down(g * sigmoid(1.702 g) * (u + 1)), g = min(gate h, limit), u = clamp(up h, +-limit)."""
    g = (h @ w[f"{name}.gate"].to(F64).T).clamp(max=limit)
    u = (h @ w[f"{name}.up"].to(F64).T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ w[f"{name}.down"].to(F64).T


def route(z, top, groups, keep):
    """Router logits [n, E] -> (chosen [n, top], weights [n, top]): softmax scores; a group's score is its largest; only
    experts of the ``keep`` best groups can be chosen; the weights are the chosen scores as they are."""
    n, E = z.shape
    s = torch.softmax(z, -1)
    allowed = s.clone()
    if groups > 1 and keep < groups:
        per = E // groups
        gscore = s.view(n, groups, per).max(-1).values
        kept = gscore.topk(keep, dim=-1).indices
        ok = torch.zeros(n, groups, dtype=torch.bool)
        ok.scatter_(1, kept, True)
        allowed = s.masked_fill(~ok.repeat_interleave(per, dim=1), -math.inf)
    chosen = allowed.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def moe_feed_forward(h, f, w, name):
    """The routed experts' weighted sum plus the shared expert."""
    r = f["router"]
    E, top = int(r["experts"]), int(r["top"])
    groups = r.get("groups") or {}
    z = h @ w[f"{name}.router"].to(F64).T
    chosen, weight = route(z, top, int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1))))
    out = torch.zeros_like(h)
    limit = float(f["expert"]["limit"])
    for e in range(E):
        hit = chosen == e
        rows = hit.any(-1).nonzero().flatten()
        if rows.numel():
            y = clipped_expert(h[rows], w, f"{name}.e{e}", limit)
            out[rows] += y * (weight[rows] * hit[rows]).sum(-1, keepdim=True)
    if f.get("shared"):
        out = out + clipped_expert(h, w, f"{name}.shared", float(f["shared"]["limit"]))
    return out


def forward(config, w, tokens, *, return_layers=False):
    """tokens: a list of ids of one sequence -> float64 logits [n, vocab] (and the stream after every layer)."""
    eps = float(config["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["embed"].to(F64)[ids] * float(config["embedding"]["scale"])
    kept_kv = {}
    after = []
    for i, layer in enumerate(config["layers"]):
        name, m = f"l{i}", layer["mixer"]
        h = rms_norm(x, w[f"{name}.norm1"].to(F64), eps)
        if layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kept_kv[i] = attention_keys_values(h, m, w, f"{name}.mix", positions)
                src = i
            y = attention_mixer(h, m, w, f"{name}.mix", positions, kept_kv[src])
        elif layer["type"] == "latent_attention":
            y = latent_attention_mixer(h, m, w, f"{name}.mix", positions, eps)
        else:
            raise ValueError(f"layer type {layer['type']!r}")
        x = x + y * w[f"{name}.ls1"].to(F64)
        if layer.get("mlp") is not None:
            h = rms_norm(x, w[f"{name}.norm2"].to(F64), eps)
            x = x + moe_feed_forward(h, layer["mlp"], w, f"{name}.mlp") * w[f"{name}.ls2"].to(F64)
        after.append(x.clone())
    logits = rms_norm(x, w["final.norm"].to(F64), eps) @ w["head"].to(F64).T
    return (logits, torch.stack(after)) if return_layers else logits
