"""Zomolix through the engine against the plain implementation (tests/plain_zomolix.py): every mechanism alone, every
cutting of the work, reused pages and slots, keys far back, at page borders and at the edges of the window and of the
kept first keys, the first tokens, long decoding, generation through the scheduler.  Models and weights are made here
(tests/zomolix_models.py)."""

import math
import types

import numpy as np
import pytest
import torch

import helpers
import plain_zomolix as plain
import zomolix_models as zm

pytestmark = pytest.mark.gpu

LIMIT = {"float32": 2e-5, "bfloat16": 4e-2}
TRACES = {"whole": helpers.trace_whole, "tail_decode": helpers.trace_tail_decode, "portions": helpers.trace_portions,
          "mixed": helpers.trace_mixed}
LENGTHS = [1, 2, 19, 53, 97, 140]


def row_error(got, want):
    """Root mean square of the difference (its mean taken off) over that of the wanted row."""
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    d = got - want
    d = d - d.mean()
    w = want - want.mean()
    return float(np.sqrt((d * d).mean()) / max(np.sqrt((w * w).mean()), 1e-30))


def sequences(vocab, lengths=LENGTHS, seed=100):
    return {f"r{i}": helpers.random_tokens(vocab, n, seed=seed + i) for i, n in enumerate(lengths)}


def stored(weights, dtype):
    """The weights as a checkpoint of ``dtype`` holds them, and their exact values in float64 for the oracle."""
    held = {k: v.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in weights.items()}
    return held, {k: v.double() for k, v in held.items()}


def replay(folder, dtype, steps, *, max_tokens=None, max_live=64, page_size=16, poison=True, graphs=True):
    from prefixserve_b200.engine.replay import Replayer
    rp = Replayer(folder, dtype, max_tokens or helpers.peak_tokens(steps), max_live=max_live, page_size=page_size,
                  use_graphs=graphs)
    rp.cache.poison_freed = poison
    if poison:  # pages nobody has written yet are as void as pages given back
        for kv in rp.cache.kv:
            if kv is not None:
                kv.fill_(float("nan"))
    outputs = {}
    for st in steps:
        out = rp.run_step(st)
        if out is not None:
            outputs[st["step"]] = out
    rp.cache.check()
    return helpers.collect(steps, outputs)


def errors(rows, truth):
    out = []
    for (rid, pos), got in rows.items():
        assert np.isfinite(got).all(), f"{rid} position {pos}: not finite"
        out.append(row_error(got, truth[rid][pos].numpy()))
    return np.asarray(out)


def assert_close(rows, truth, dtype, routed=True):
    """float32: every row within the limit.  bfloat16 with a router: rounding moves a score by a few thousandths, so now
    and then a token goes to another expert than in the float64 oracle; nine rows of ten are held to the limit, the
    rest to ten times it.  Without routing every row is held to it."""
    e = errors(rows, truth)
    if dtype == "float32" or not routed:
        assert e.max() < LIMIT[dtype], e.max()
    else:
        assert np.quantile(e, 0.9) < LIMIT[dtype] and e.max() < 10 * LIMIT[dtype], (np.quantile(e, 0.9), e.max())


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    """(configuration name, dtype) -> (folder, float64 logits of every test sequence)."""
    out = {}
    for which, cfg in zm.CONFIGS.items():
        weights = zm.tensors(cfg, seed=sorted(zm.CONFIGS).index(which))
        for dtype in ("float32", "bfloat16"):
            held, exact = stored(weights, dtype)
            folder = zm.write_folder(tmp_path_factory.mktemp(f"{which}-{dtype}"), cfg, held)
            truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in sequences(cfg["vocab"]).items()}
            out[which, dtype] = (folder, truth)
    return out


def routed(which):
    return any(l["mlp"] is not None for l in zm.CONFIGS[which]["layers"])


@pytest.mark.parametrize("trace", sorted(TRACES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(zm.CONFIGS))
def test_every_cutting_matches_the_plain_model(made, which, dtype, trace):
    """Whole prompts, a decoded tail, portions down to two tokens, and up to four requests at once over a pool that
    only holds what is live (pages and slots are used again; freed pages are filled with NaN)."""
    folder, truth = made[which, dtype]
    seqs = sequences(zm.CONFIGS[which]["vocab"])
    steps = TRACES[trace](seqs)
    rows = replay(folder, dtype, steps, max_live=4 if trace == "mixed" else 64)
    assert len(rows) == sum(len(t) for t in seqs.values())
    assert_close(rows, truth, dtype, routed(which))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [1, 4, 64])
@pytest.mark.parametrize("which", ["mixed", "wide"])
def test_token_by_token_through_small_and_large_pages(made, which, dtype, page_size):
    """Every token decoded alone from the first on, over many page borders: prefill against token-by-token decoding.
    With pages of one and four tokens the kept first keys end inside a page or fill several."""
    folder, truth = made[which, dtype]
    seqs = {rid: toks for rid, toks in sequences(zm.CONFIGS[which]["vocab"]).items() if len(toks) in (2, 140)}
    steps = helpers.trace_tail_decode(seqs, tail=10 ** 6)
    rows = replay(folder, dtype, steps, page_size=page_size, max_tokens=helpers.peak_tokens(steps, page=max(page_size, 64)))
    assert_close(rows, truth, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_slots_and_an_exact_pool_serve_six_requests(made, dtype):
    folder, truth = made["mixed", dtype]
    seqs = sequences(131)
    steps = helpers.trace_mixed(seqs, max_live=2, seed=7)
    rows = replay(folder, dtype, steps, max_live=2, page_size=4, max_tokens=helpers.peak_tokens(steps, page=4))
    assert_close(rows, truth, dtype)


def test_a_batch_gives_each_request_what_it_gets_alone(made):
    """float32: the same kernels run either way, so the rows agree to the last bits, not only within the limit."""
    folder, _ = made["mixed", "float32"]
    seqs = sequences(131)
    together = replay(folder, "float32", helpers.trace_mixed(seqs, max_live=4, seed=3), max_live=4)
    alone = replay(folder, "float32", helpers.trace_whole(seqs))
    for key, row in alone.items():
        assert row_error(together[key], row) < 2e-6


def test_captured_steps_give_what_uncaptured_ones_give(made):
    folder, _ = made["mixed", "bfloat16"]
    seqs = sequences(131)
    steps = helpers.trace_tail_decode(seqs, tail=20)
    a, b = replay(folder, "bfloat16", steps, graphs=True), replay(folder, "bfloat16", steps, graphs=False)
    assert all(np.array_equal(a[k], b[k]) for k in a)


def test_pages_behind_the_window_go_back_and_the_kept_ones_stay(made):
    """A windowed layer with kept first keys holds the pages of those keys and of its window, not of everything."""
    from prefixserve_b200.engine.replay import Replayer
    folder, _ = made["attn_only", "float32"]   # window 9, two kept keys
    rp = Replayer(folder, "float32", 1024, page_size=4)
    toks = helpers.random_tokens(61, 200, seed=3)
    rp.run_step({"step": 0, "entries": [{"id": "a", "tokens": toks[:150], "want": []}], "end": []})
    for i in range(150, 200):
        rp.run_step({"step": i, "entries": [{"id": "a", "tokens": toks[i: i + 1], "want": [0]}], "end": []})
    held = [p for p in rp.cache.page_ids(rp.slot_of["a"], 0) if p >= 0]
    assert rp.cache.page_ids(rp.slot_of["a"], 0)[0] >= 0          # the page of the kept keys
    assert len(held) <= 1 + (9 + 3) // 4 + 2                      # it, the window's pages and the one being filled
    rp.cache.check()


# ---- keys that must not be lost --------------------------------------------------------------------------------

MARK, ASK = 62, 63


def echo_model(dtype, window, keep, dim=16):
    """One attention layer that answers the token ASK with the key of the token MARK wherever that lies and is visible:
    the key matrix is the first query head's behind a fixed permutation of the width, and ASK's embedding is MARK's
    under the same permutation, so ASK's query is MARK's key (up to the few rotated elements) and its score stands out
    among hundreds of random ones.  Whoever loses that one key, or sees it where the mask hides it, gives a visibly
    different row."""
    mixer = zm.attention(heads=2, kv_heads=1, dim=dim, vdim=8 if dim == 16 else dim, scale=12.8 / dim, rotation=zm.rot(4, base=100.0),
                         mask=None if window is None else (window, keep))
    cfg = zm.config([zm.layer("attention", mixer, None)], vocab=64, width=32)
    w = zm.tensors(cfg, seed=11)
    turn = torch.eye(32)[torch.roll(torch.arange(32), 1)]
    w["l0.mix.k"] = w["l0.mix.q"][:dim] @ turn
    w["embed"][ASK] = turn @ w["embed"][MARK]
    w["l0.norm1"] = torch.ones(32)
    for b in ("q", "k"):
        w[f"l0.mix.{b}.b"] *= 0.0
    return cfg, *stored(w, dtype)


CUTTINGS = (
    (16, lambda s, n, m: helpers.trace_whole(s)),
    (64, lambda s, n, m: helpers.trace_tail_decode(s, tail=140)),
    (16, lambda s, n, m: helpers.trace_tail_decode(s, tail=n - m - 1)),
    (64, lambda s, n, m: helpers.trace_portions(s, sizes=(3, 2, 59, 2, 40, 7, 2, 31, 64))),
    (16, lambda s, n, m: helpers.trace_portions(s, sizes=(64, 1, 35, 100, 2))),
)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("marked", [0, 3, 63, 64])
@pytest.mark.parametrize("dim", [16, 64])
def test_one_key_far_back_or_at_a_page_border_is_found(tmp_path, dim, dtype, marked):
    """No window: the marked key is a sequence's first, an early one, a page's last or a page's first (pages of 16 and
    of 64); it is asked for right behind it and hundreds of tokens later, in prompts, in portions and in single tokens.
    Heads of 16: the cache entry with a row per token; of 64: planes of keys and values."""
    cfg, held, exact = echo_model(dtype, None, 0, dim)
    folder = zm.write_folder(tmp_path / "m", cfg, held)
    n = 330
    toks = helpers.random_tokens(62, n, seed=5)
    toks[marked] = MARK
    asks = [marked + 1, 100, 200, n - 1]
    for a in asks:
        toks[a] = ASK
    truth = {"a": plain.forward(cfg, exact, toks)}
    quiet = list(toks)
    quiet[marked] = 1
    hidden = plain.forward(cfg, exact, quiet)
    seen = [row_error(truth["a"][i].numpy(), hidden[i].numpy()) for i in asks]
    assert seen[0] > 0.25 and max(seen[1:]) > 0.25 and row_error(truth["a"][150].numpy(), hidden[150].numpy()) < 0.02
    seqs = {"a": toks}
    for page_size, cut in CUTTINGS:
        steps = cut(seqs, n, marked)
        rows = replay(folder, dtype, steps, page_size=page_size, max_tokens=helpers.peak_tokens(steps, page=64))
        assert_close(rows, truth, dtype, routed=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dim", [16, 64])
@pytest.mark.parametrize("window,keep,marked", [(40, 6, 100), (40, 6, 5), (40, 6, 6), (64, 17, 16), (64, 17, 17), (33, 0, 70), (16, 1, 0)])
def test_a_key_just_inside_and_just_outside_the_window_and_the_kept_keys(tmp_path, dim, dtype, window, keep, marked):
    """The marked key is asked for by the last query that sees it through the window and by the first that does not,
    and again far behind, where only a kept key is still seen.  The oracle says which of the asking rows depend on it;
    the engine must agree with the oracle in prompts, in portions (whose tiles straddle the edges) and in single tokens."""
    cfg, held, exact = echo_model(dtype, window, keep, dim)
    folder = zm.write_folder(tmp_path / "m", cfg, held)
    n = 330
    toks = helpers.random_tokens(62, n, seed=9)
    toks[marked] = MARK
    asks = [marked + window - 1, marked + window, n - 1]
    for a in asks:
        toks[a] = ASK
    truth = {"a": plain.forward(cfg, exact, toks)}
    quiet = list(toks)
    quiet[marked] = 1
    hidden = plain.forward(cfg, exact, quiet)
    seen = [row_error(truth["a"][i].numpy(), hidden[i].numpy()) for i in asks]
    kept = marked < keep
    assert seen[0] > 0.15                                    # just inside the window
    assert (seen[1] > 0.15) == kept and (seen[2] > 0.15) == kept   # outside it: only a kept key is still there
    if not kept:
        assert max(seen[1:]) < 1e-9                          # a key behind the window does not exist for the row
    seqs = {"a": toks}
    for page_size, cut in CUTTINGS:
        steps = cut(seqs, n, marked)
        rows = replay(folder, dtype, steps, page_size=page_size, max_tokens=helpers.peak_tokens(steps, page=64))
        assert_close(rows, truth, dtype, routed=False)


@pytest.mark.parametrize("which", ["mixed", "wide"])
def test_long_decoding(made, which):
    """Hundreds of single tokens behind a short prompt, several requests side by side in captured steps."""
    cfg = zm.CONFIGS[which]
    for dtype in ("float32", "bfloat16"):
        folder, _ = made[which, dtype]
        _, exact = stored(zm.tensors(cfg, seed=sorted(zm.CONFIGS).index(which)), dtype)
        seqs = sequences(cfg["vocab"], lengths=[400, 260, 333], seed=60)
        truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in seqs.items()}
        steps = helpers.trace_many_live(seqs, tail=250, portion_beside=False)
        assert_close(replay(folder, dtype, steps, max_live=3), truth, dtype)


# ---- mechanisms alone -------------------------------------------------------------------------------------------

def dev(x, dtype=torch.int32):
    return torch.tensor(x, dtype=dtype).cuda()


def step_context(lengths, starts, slots=None):
    """What the ops read of a step: portions of the given lengths starting at the given absolute positions."""
    slots = slots or list(range(len(lengths)))
    positions, item_of, offsets = [], [], [0]
    for i, (n, s) in enumerate(zip(lengths, starts)):
        positions += list(range(s, s + n))
        item_of += [i] * n
        offsets.append(offsets[-1] + n)
    items = [types.SimpleNamespace(slot=sl, start=s, end=s + n, first_token=o) for sl, s, n, o in zip(slots, starts, lengths, offsets)]
    return types.SimpleNamespace(positions=dev(positions), token_item=dev(item_of), item_start=dev(offsets), slots=dev(slots),
                                 num_items=len(lengths), num_tokens=len(positions), max_new_tokens=max(lengths),
                                 kv_len=dev([n + s for n, s in zip(lengths, starts)]),
                                 max_kv_len=max(n + s for n, s in zip(lengths, starts)), extras={}, items=items)


def test_ramped_frequencies_and_amplitude_of_the_angle_tables():
    from prefixserve_b200.parts.registry import make
    from prefixserve_b200.config.spec import part
    for dims, base, sc in ((16, 10000.0, zm.SCALED), (6, 300.0, (2.0, 32, 4.0, 1.0)), (48, 30000.0, (6.0, 64, 8.0, 1.0)), (8, 500.0, None)):
        scaling = None if sc is None else {"kind": "yarn", "factor": sc[0], "original_max_positions": sc[1], "fast": sc[2], "slow": sc[3]}
        pos = make("position", part("rope", head_dim=dims + 4, rotary_dim=dims, theta=base, scaling=scaling, layout="half"))
        pos.prepare(max_positions=300, compute_dtype=torch.float32, device=torch.device("cuda"))
        f, amp = plain.rotary_frequencies(zm.rot(dims, base, sc))
        angles = torch.arange(300, dtype=torch.float64)[:, None] * f[None]
        assert pos.cos.shape[0] >= 300 and pos.cos.shape[1] == dims // 2   # (layers with the same constants share a table)
        assert torch.allclose(pos.cos[:300].cpu().double(), angles.cos() * amp, atol=2e-4)   # float32 angles up to position 300
        assert torch.allclose(pos.sin[:300].cpu().double(), angles.sin() * amp, atol=2e-4)
        assert torch.allclose(pos.cos[:4].cpu().double(), (angles.cos() * amp)[:4], atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [24, 1100, 2048])
def test_sum_with_shift_and_scale_in_front_of_a_norm(dtype, width):
    """h += (y + shift) * scale, then the norm: each of shift and scale alone, both, and rows picked out."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(width)
    h, y = torch.randn(7, width, generator=g), torch.randn(7, width, generator=g).to(dtype)
    gain, scale, shift, eps = 1 + 0.1 * torch.randn(width, generator=g), 1 + 0.3 * torch.randn(width, generator=g), torch.randn(width, generator=g), 1e-5
    for sc, sh in ((scale, None), (None, shift), (scale, shift)):
        want_h = h.double() + (y.double() + (0 if sh is None else sh.double())) * (1 if sc is None else sc.double())
        stream = h.clone().cuda()
        pending = ops.Affine(y.cuda(), scale=None if sc is None else sc.cuda(), shift=None if sh is None else sh.cuda())
        x = ops.add_rmsnorm(stream, pending, gain.cuda(), eps, dtype)
        tol = 1e-5 if dtype == torch.float32 else 3e-2
        assert torch.allclose(stream.cpu().double(), want_h, atol=1e-5)
        assert torch.allclose(x.cpu().double(), plain.rms_norm(want_h, gain.double(), eps), atol=tol)
        stream = h.clone().cuda()
        picked = ops.add_rmsnorm(stream, pending, gain.cuda(), eps, dtype, rows=dev([5, 0]))
        assert torch.equal(stream.cpu(), h) and torch.allclose(picked.cpu().double(), plain.rms_norm(want_h[[5, 0]], gain.double(), eps), atol=tol)
    wrapped = ops.Affine(ops.Affine(y.cuda(), shift=shift.cuda()), scale=scale.cuda())   # a block's scale around a mixer's bias
    assert wrapped.y.data_ptr() == pending.y.data_ptr() or torch.equal(wrapped.y, pending.y)
    assert torch.equal(wrapped.shift.cpu(), shift) and torch.equal(wrapped.scale.cpu(), scale)


def paged(rows, page_size, seed=0):
    """rows [items][n_i, heads, width] -> (cache [pages, 1, heads, page_size, width] with the pages in a shuffled order
    and NaN wherever nothing was written, page table [items, max pages])."""
    heads, width = rows[0].shape[1], rows[0].shape[2]
    need = [-(-r.shape[0] // page_size) for r in rows]
    order = np.random.RandomState(seed).permutation(sum(need) + 2)
    cache = torch.full((sum(need) + 2, 1, heads, page_size, width), float("nan"), dtype=rows[0].dtype)
    table = torch.full((len(rows), max(need)), -1, dtype=torch.int32)
    at = 0
    for i, r in enumerate(rows):
        for pi in range(need[i]):
            page = int(order[at]); at += 1
            table[i, pi] = page
            piece = r[pi * page_size: (pi + 1) * page_size]
            cache[page, 0, :, : piece.shape[0]] = piece.transpose(0, 1)
    return cache, table


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,vdim,hq,hkv", [(16, 10, 4, 2), (96, 40, 6, 2), (64, 64, 2, 1), (12, 20, 3, 3)])
@pytest.mark.parametrize("window,keep", [(20, 3), (64, 70), (5, 33), (37, 0), (130, 64)])
def test_attention_over_rows_with_kept_first_keys_alone(dtype, dim, vdim, hq, hkv, window, keep):
    """A long portion from the start, a long portion behind a cached prefix (its first tiles still reach the kept keys,
    its later ones have a gap), short portions and single tokens, against the plain softmax over the visible keys.  The
    keys between the kept ones and the window are NaN in the cache wherever no query of the step can see them."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(window * 100 + keep)
    lengths, starts = [150, 120, 1, 1, 3, 1], [0, 85, 0, 9, 40, 299]
    page = 16
    ctx = step_context(lengths, starts)
    total = [s + n for s, n in zip(starts, lengths)]
    kv_rows = [(torch.randn(t, hkv, dim + vdim, generator=g)).to(dtype) for t in total]
    q = torch.randn(sum(lengths), hq, dim, generator=g).to(dtype)
    hidden = []
    for rows, s, n in zip(kv_rows, starts, lengths):   # what no query of this step sees is void
        seen = torch.zeros(rows.shape[0], dtype=torch.bool)
        for p in range(s, s + n):
            seen[max(0, p - window + 1): p + 1] = True
            seen[: min(keep, p + 1)] = True
        hidden.append(seen)
    void = [r.clone() for r in kv_rows]
    for r, seen in zip(void, hidden):
        r[~seen] = float("nan")
    cache, table = paged(void, page)
    scale = 1.3 / math.sqrt(dim)
    out = ops.attention_over_rows(q.cuda(), cache.cuda(), table.cuda(), ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=vdim,
                                  page_size=page, scale=scale, window=window, keep_first=keep).cpu().double().view(-1, hq, vdim)
    at = 0
    for rows, s, n in zip(kv_rows, starts, lengths):
        k = rows[:, :, :dim].double().repeat_interleave(hq // hkv, dim=1)
        v = rows[:, :, dim:].double().repeat_interleave(hq // hkv, dim=1)
        mask = plain.visible(s + n, window, keep)[s:]
        qq = torch.zeros(s + n, hq, dim, dtype=torch.float64)
        qq[s:] = q[at: at + n].double()
        want = plain.softmax_attention(qq, k, v, scale, plain.visible(s + n, window, keep))[s:]
        assert mask.shape[0] == n
        assert torch.allclose(out[at: at + n], want, atol=1e-5 if dtype == torch.float32 else 2e-2), (s, n)
        at += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("dim,vdim,hq,hkv,rot_dims", [(16, 10, 4, 2, 16), (96, 40, 6, 2, 32), (12, 20, 3, 1, 6)])
def test_projection_bias_rotation_and_append_alone(dtype, dim, vdim, hq, hkv, rot_dims):
    """The pass between the projection and the scores: biases added in float32, the split-half rotation of the leading
    elements, queries out, keys and values into the token's cache row; and the same for a layer that only has queries."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(dim)
    lengths, starts = [5, 1, 40], [0, 17, 3]
    ctx = step_context(lengths, starts)
    page = 8
    width = hq * dim + hkv * (dim + vdim)
    proj = torch.randn(sum(lengths), width, generator=g).to(dtype)
    bias = torch.randn(width, generator=g)
    rot = zm.rot(rot_dims, 200.0, (2.0, 16, 4.0, 1.0))
    f, amp = plain.rotary_frequencies(rot)
    angles = torch.arange(64, dtype=torch.float64)[:, None] * f[None]
    cos, sin = (angles.cos() * amp).float().cuda(), (angles.sin() * amp).float().cuda()
    pages = sum(-(-(s + n) // page) for s, n in zip(starts, lengths))
    table = torch.full((3, 8), -1, dtype=torch.int32)
    nxt = 0
    for i, (s, n) in enumerate(zip(starts, lengths)):
        for pi in range(-(-(s + n) // page)):
            table[i, pi] = nxt; nxt += 1
    kv = torch.zeros(pages, 1, hkv, page, dim + vdim, dtype=dtype).cuda()
    q = ops.attention_prepare(proj.cuda(), kv, table.cuda(), ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=vdim, page_size=page,
                              cos=cos, sin=sin, rotary_dim=rot_dims, interleaved=False, bias=bias.cuda()).cpu().double()
    full = proj.double() + bias.double()
    positions = ctx.positions.cpu()
    want_q = plain.rotate(full[:, : hq * dim].view(-1, hq, dim), positions, rot, "half")
    want_k = plain.rotate(full[:, hq * dim: (hq + hkv) * dim].view(-1, hkv, dim), positions, rot, "half")
    want_v = full[:, (hq + hkv) * dim:].view(-1, hkv, vdim)
    tol = 1e-5 if dtype == torch.float32 else 3e-2
    assert torch.allclose(q, want_q, atol=tol)
    held = kv.cpu().double()
    for t in range(sum(lengths)):
        i, p = int(ctx.token_item[t]), int(positions[t])
        row = held[int(table[i, p // page]), 0, :, p % page]
        assert torch.allclose(row[:, :dim], want_k[t], atol=tol) and torch.allclose(row[:, dim:], want_v[t], atol=tol)
    only_q = ops.attention_prepare(proj[:, : hq * dim].contiguous().cuda(), None, None, ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=vdim,
                                   page_size=page, cos=cos, sin=sin, rotary_dim=rot_dims, interleaved=False, bias=bias[: hq * dim].contiguous().cuda(),
                                   write_kv=False).cpu().double()
    assert torch.allclose(only_q, want_q, atol=tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rank,rot,heads", [(64, 16, 4), (20, 8, 3), (72, 24, 2), (9, 2, 1)])
def test_latent_attention_with_a_sink_alone(dtype, rank, rot, heads):
    """Queries in the latent space over cached rows, the sink in the denominator: single tokens over hundreds of keys
    (the keys split among blocks and joined), short portions, a long one; one query is a cached row scaled up, so one
    key among hundreds carries the weight; one head's sink is so high that it takes nearly all of it."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(rank)
    lengths, starts = [1, 1, 4, 90, 1], [700, 0, 33, 20, 64]
    page = 16
    ctx = step_context(lengths, starts)
    rows = [torch.randn(s + n, 1, rank + rot, generator=g).to(dtype) for s, n in zip(starts, lengths)]
    cache, table = paged(rows, page, seed=1)
    q = torch.randn(sum(lengths), heads, rank + rot, generator=g) * 0.5
    q[0, 0] = rows[0][123, 0].float() * 3.0      # the first token's first head looks for key 123 of 701
    sink = torch.randn(heads, generator=g)
    sink[-1] = 9.0
    scale = 0.2
    out = ops.latent_attention(q.cuda(), cache.cuda(), table.cuda(), ctx.positions, ctx.token_item, None,
                               rank=rank, page_size=page, window=None, scale=scale, out_dtype=torch.float32, items=ctx.items,
                               key_hint=ctx.max_kv_len, sink=sink.cuda()).cpu().double()
    at = 0
    for r, s, n in zip(rows, starts, lengths):
        keys = r[:, 0].double()
        for t in range(n):
            p = s + t
            sc = torch.einsum("hd,jd->hj", q[at + t].double(), keys[: p + 1]) * scale
            top = torch.maximum(sc.max(-1).values, sink.double())
            e = (sc - top[:, None]).exp()
            w = e / (e.sum(-1) + (sink.double() - top).exp())[:, None]
            want = w @ keys[: p + 1, :rank]
            assert torch.allclose(out[at + t], want, atol=1e-5 if dtype == torch.float32 else 2e-2), (s, t)
            if at + t == 0 and heads > 1:   # (with one head the high sink is this head's)
                assert w[0, 123] > 0.5
        at += n


def test_router_alone():
    """Softmax scores, groups that count by their best expert, the kept groups' best experts, weights that are the
    scores as they are; sizes where nothing is dropped, where one group is kept, one choice, many experts."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(3)
    for experts, top, groups, keep in ((16, 4, 4, 3), (8, 3, 4, 3), (6, 2, 1, 1), (6, 3, 2, 1), (12, 1, 3, 2), (64, 6, 8, 3), (5, 5, 1, 1)):
        z = torch.randn(300, experts + 2, generator=g) * 2.0        # further columns of a wider product are ignored
        chosen, weight = ops.moe_route(z.cuda(), None, experts=experts, top=top, groups=groups, keep=keep, scale=1.0,
                                       scores="softmax", group_score="max", normalize=False)
        want_e, want_w = plain.route(z[:, :experts].double(), top, groups, keep)
        order = chosen.cpu().long().sort(-1)
        want_order = want_e.sort(-1)
        assert torch.equal(order.values, want_order.values), (experts, top, groups, keep)
        assert torch.allclose(weight.cpu().double().gather(1, order.indices), want_w.gather(1, want_order.indices), atol=1e-6)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("tokens", [3, 70, 600])
def test_gated_experts_alone(dtype, tokens):
    """The experts' weighted sum plus the shared expert, for a handful of rows, for some dozens and for enough pairs
    that the grouped tensor-core product takes them; limits low enough that both clips act."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(tokens)
    width, ff, experts, top, limit = 64, 40, 6, 2, 0.8
    x = torch.randn(tokens, width, generator=g).to(dtype)
    w = {}
    for e in range(experts):
        w[f"m.e{e}.gate"] = (torch.randn(ff, width, generator=g) * 0.2).to(dtype)
        w[f"m.e{e}.up"] = (torch.randn(ff, width, generator=g) * 0.2).to(dtype)
        w[f"m.e{e}.down"] = (torch.randn(width, ff, generator=g) * 0.2).to(dtype)
    chosen = torch.stack([torch.randperm(experts, generator=g)[:top] for _ in range(tokens)]).int()
    weight = torch.rand(tokens, top, generator=g)
    shared = torch.randn(tokens, width, generator=g).to(dtype)
    w_up = torch.stack([torch.cat([w[f"m.e{e}.gate"], w[f"m.e{e}.up"]]) for e in range(experts)]).cuda()
    w_down = torch.stack([w[f"m.e{e}.down"] for e in range(experts)]).cuda()
    out = ops.moe_experts(x.cuda(), chosen.cuda(), weight.cuda(), w_up, w_down, activation=None, shared=shared.cuda(),
                          glu=(limit, 1.702, 1.0), out_dtype=torch.float32).cpu().double()
    want = shared.double().clone()
    wd = {k: v.double() for k, v in w.items()}
    for e in range(experts):
        y = plain.clipped_expert(x.double(), wd, f"m.e{e}", limit)
        want += y * (weight.double() * (chosen == e)).sum(-1, keepdim=True)
    assert torch.allclose(out, want, atol=1e-5 if dtype == torch.float32 else 4e-2)


def test_gate_on_the_values_alone():
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(0)
    v, gate = torch.randn(9, 3, 7, generator=g), torch.rand(9, 21, generator=g)
    out = ops.gate_mul(v.cuda(), gate.cuda(), out_dtype=torch.bfloat16)
    assert out.dtype == torch.bfloat16 and torch.allclose(out.float().cpu(), (v.view(9, 21) * gate).view(9, 3, 7), atol=2e-2)
    assert torch.equal(ops.gate_mul(v.cuda(), gate.cuda()).cpu().view(9, 21), v.view(9, 21) * gate)


# ---- generation ---------------------------------------------------------------------------------------------------

def greedy(cfg, exact, prompt, n):
    toks = list(prompt)
    for _ in range(n):
        toks.append(int(plain.forward(cfg, exact, toks)[-1].argmax()))
    return toks[len(prompt):]


def test_greedy_generation_through_the_entry_point_and_scheduler(made):
    """Prompts longer than a portion, more requests than run at once, captured decode steps: the same tokens as the
    plain model's greedy continuation (float32: a tie would have to be exact to differ)."""
    from prefixserve_b200.engine.llm import LLM
    from prefixserve_b200.sampling import SamplingParams
    folder, _ = made["mixed", "float32"]
    cfg = zm.CONFIGS["mixed"]
    _, exact = stored(zm.tensors(cfg, seed=sorted(zm.CONFIGS).index("mixed")), "float32")
    prompts = [helpers.random_tokens(131, n, seed=70 + n) for n in (1, 5, 23, 40)]
    llm = LLM(folder, dtype="float32", max_seq_len=128, num_blocks=64, max_running_requests=3, chunked_prefill_size=16)
    got = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert got == [greedy(cfg, exact, p, 12) for p in prompts]
    assert llm.engine.runner.graph_replays > 0
    llm.engine.cache.check()
    # a second call on the same engine starts from clean slots
    assert llm.generate(prompts[:2], SamplingParams(max_tokens=5, ignore_eos=True)) == [greedy(cfg, exact, p, 5) for p in prompts[:2]]


def test_command_line_generates_from_a_zomolix_folder(made):
    import json
    import subprocess
    import sys
    folder, _ = made["reader_sees_all", "bfloat16"]
    out = subprocess.run([sys.executable, "-m", "prefixserve_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--max-tokens", "6",
                          "--num-blocks", "32", "--max-seq-len", "64", "--max-running-requests", "2"],
                         capture_output=True, text=True, timeout=600, cwd=str(helpers.__file__).rsplit("/tests/", 1)[0])
    assert out.returncode == 0, out.stderr[-2000:]
    first = json.loads(out.stdout.splitlines()[0])
    assert first["prompt_ids"] == [5, 17, 3] and len(first["output_ids"]) == 6


def test_a_preset_of_the_design_generates(tmp_path):
    from prefixserve_b200.config.presets import preset
    from prefixserve_b200.engine.llm import LLM
    from prefixserve_b200.sampling import SamplingParams
    from prefixserve_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "m", preset("zomolix-tiny"), 0, std=0.1, gain_noise=0.1, dtype=torch.bfloat16)
    llm = LLM(folder, dtype="bfloat16", max_seq_len=64, num_blocks=32, max_running_requests=2)
    got = llm.generate([[5, 6, 7], [9]], SamplingParams(max_tokens=4, ignore_eos=True))
    assert [len(g) for g in got] == [4, 4]
