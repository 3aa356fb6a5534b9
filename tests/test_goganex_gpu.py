"""Goganex through the engine against the plain implementation (tests/plain_goganex.py): every mechanism alone, every
cutting of the work, reused pages and slots, keys far back and at page borders, the first tokens, long decoding,
generation through the scheduler.  Models and weights are made here (tests/goganex_models.py)."""

import types

import numpy as np
import pytest
import torch

import goganex_models as gm
import helpers
import plain_goganex as plain

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


def worst_error(rows, truth):
    worst = 0.0
    for (rid, pos), got in rows.items():
        assert np.isfinite(got).all(), f"{rid} position {pos}: not finite"
        worst = max(worst, row_error(got, truth[rid][pos].numpy()))
    return worst


@pytest.fixture(scope="module")
def made(tmp_path_factory):
    """(configuration name, dtype) -> (folder, float64 logits of every test sequence)."""
    out = {}
    for which, cfg in gm.CONFIGS.items():
        weights = gm.tensors(cfg, seed=sorted(gm.CONFIGS).index(which))
        for dtype in ("float32", "bfloat16"):
            held, exact = stored(weights, dtype)
            folder = gm.write_folder(tmp_path_factory.mktemp(f"{which}-{dtype}"), cfg, held)
            truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in sequences(cfg["vocab"]).items()}
            out[which, dtype] = (folder, truth)
    return out


@pytest.mark.parametrize("trace", sorted(TRACES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", sorted(gm.CONFIGS))
def test_every_cutting_matches_the_plain_model(made, which, dtype, trace):
    """Whole prompts, a decoded tail, portions down to two tokens, and up to four requests at once over a pool that
    only holds what is live (pages and slots are used again; freed pages are filled with NaN)."""
    folder, truth = made[which, dtype]
    seqs = sequences(gm.CONFIGS[which]["vocab"])
    steps = TRACES[trace](seqs)
    rows = replay(folder, dtype, steps, max_live=4 if trace == "mixed" else 64)
    assert len(rows) == sum(len(t) for t in seqs.values())
    assert worst_error(rows, truth) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("page_size", [1, 4, 64])
@pytest.mark.parametrize("which", ["mixed", "planes"])
def test_token_by_token_through_small_and_large_pages(made, which, dtype, page_size):
    """Every token decoded alone from the first on, over many page borders: prefill against token-by-token decoding.
    (Pages below 16 tokens take the plane layout to the attention kernel that walks its keys.)"""
    folder, truth = made[which, dtype]
    seqs = {rid: toks for rid, toks in sequences(gm.CONFIGS[which]["vocab"]).items() if len(toks) in (2, 140)}
    steps = helpers.trace_tail_decode(seqs, tail=10 ** 6)
    rows = replay(folder, dtype, steps, page_size=page_size, max_tokens=helpers.peak_tokens(steps, page=max(page_size, 64)))
    assert worst_error(rows, truth) < LIMIT[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_two_slots_and_an_exact_pool_serve_six_requests(made, dtype):
    folder, truth = made["mixed", dtype]
    seqs = sequences(131)
    steps = helpers.trace_mixed(seqs, max_live=2, seed=7)
    rows = replay(folder, dtype, steps, max_live=2, page_size=4, max_tokens=helpers.peak_tokens(steps, page=4))
    assert worst_error(rows, truth) < LIMIT[dtype]


def test_a_batch_gives_each_request_what_it_gets_alone(made):
    """float32: the same kernels run either way, so the rows agree to the last bits, not only within the limit."""
    folder, _ = made["mixed", "float32"]
    seqs = sequences(131)
    together = replay(folder, "float32", helpers.trace_mixed(seqs, max_live=4, seed=3), max_live=4)
    alone = replay(folder, "float32", helpers.trace_whole(seqs))
    for key, row in alone.items():
        assert row_error(together[key], row) < 2e-6


def test_captured_steps_give_what_uncaptured_ones_give(made):
    folder, truth = made["whole_loop", "bfloat16"]
    seqs = sequences(97)
    steps = helpers.trace_tail_decode(seqs, tail=20)
    a, b = replay(folder, "bfloat16", steps, graphs=True), replay(folder, "bfloat16", steps, graphs=False)
    assert all(np.array_equal(a[k], b[k]) for k in a)


# ---- keys that must not be lost --------------------------------------------------------------------------------

MARK, ASK = 62, 63


def echo_model(kind, dtype, dim=16):
    """One layer whose attention answers the token ASK with the key of the token MARK, wherever that lies: the key
    matrix is the first query head's behind a fixed permutation of the width, and ASK's embedding is MARK's under the
    same permutation, so ASK's query is MARK's key (up to the few rotated elements and a weak token shift) and its
    score stands out among hundreds of random ones.  Whoever loses that one key gives a visibly different row.  The
    scale goes down as the head grows, so that the one score stands as high above the others whatever the size."""
    if kind == "attention":
        mixer, p = gm.attention(heads=2, kv_heads=1, dim=dim, vdim=8 if dim == 16 else dim, scale=12.8 / dim, rotation=gm.rot(4, base=100.0)), "l0.mix."
    else:
        mixer, p = gm.parallel(heads=2, kv_heads=1, dim=dim, scale=17.6 / dim, width=8), "l0.mix.left."
    cfg = gm.config([gm.layer(kind, mixer, None)], vocab=64, width=32)
    w = gm.tensors(cfg, seed=11)
    turn = torch.eye(32)[torch.roll(torch.arange(32), 1)]
    w[p + "k"] = w[p + "q"][:dim] @ turn
    w["embed"][ASK] = turn @ w["embed"][MARK]
    w["l0.norm1"] = torch.ones(32)
    w["l0.shift"] *= 0.05
    if kind == "attention":
        w[p + "temp"] = torch.tensor([1.6, 1.2])
    return cfg, *stored(w, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("marked", [0, 3, 63, 64])
@pytest.mark.parametrize("kind", ["attention", "parallel"])
@pytest.mark.parametrize("dim", [16, 64])
def test_one_key_far_back_or_at_a_page_border_is_found(tmp_path, dim, kind, dtype, marked):
    """The marked key is a sequence's first, an early one, a page's last or a page's first (pages of 16 and of 64);
    it is asked for right behind it and hundreds of tokens later, in prompts, in portions and in single tokens.  Heads
    of 16: the cache entry with a row per token; of 64: planes of keys and values and the kernels that read those."""
    cfg, held, exact = echo_model(kind, dtype, dim)
    folder = gm.write_folder(tmp_path / "m", cfg, held)
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
    # the oracle itself says that the marked key matters where it is asked for, and hardly elsewhere
    seen = [row_error(truth["a"][i].numpy(), hidden[i].numpy()) for i in asks]
    assert seen[0] > 0.25 and max(seen[1:]) > 0.25 and row_error(truth["a"][150].numpy(), hidden[150].numpy()) < 0.02
    seqs = {"a": toks}
    for page_size, steps in ((16, helpers.trace_whole(seqs)), (64, helpers.trace_tail_decode(seqs, tail=140)),
                             (16, helpers.trace_tail_decode(seqs, tail=n - marked - 1)),
                             (64, helpers.trace_portions(seqs, sizes=(3, 2, 59, 2, 40, 7, 2, 31, 64))),
                             (16, helpers.trace_portions(seqs, sizes=(64, 1, 35, 100, 2)))):
        rows = replay(folder, dtype, steps, page_size=page_size, max_tokens=helpers.peak_tokens(steps, page=64))
        assert worst_error(rows, truth) < LIMIT[dtype]


def test_a_long_memory_survives_portions_and_decoding(tmp_path):
    """A recurrence that forgets slowly (update gates near zero) and a strong token shift: a lost state or a lost
    previous row at a portion's start shows for long."""
    cfg = gm.CONFIGS["parallel_only"]
    weights = gm.tensors(cfg, seed=21)
    weights["l0.mix.right.z.b"] -= 4.0
    weights["l0.shift"] = 0.5 + 0.5 * weights["l0.shift"]
    held, exact = stored(weights, "float32")
    folder = gm.write_folder(tmp_path / "m", cfg, held)
    seqs = sequences(cfg["vocab"], lengths=[3, 64, 300], seed=40)
    truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in seqs.items()}
    # the oracle says so: without its first 100 tokens the long request's last row is another one
    cut = plain.forward(cfg, exact, seqs["r2"][100:])
    assert row_error(cut[-1].numpy(), truth["r2"][-1].numpy()) > 1e-3
    for steps in (helpers.trace_portions(seqs, sizes=(2, 2, 3, 1, 2, 50, 2, 140)), helpers.trace_tail_decode(seqs, tail=150),
                  helpers.trace_mixed(seqs, max_live=3, seed=1), helpers.trace_whole(seqs)):
        assert worst_error(replay(folder, "float32", steps), truth) < LIMIT["float32"]


@pytest.mark.parametrize("which", ["whole_loop", "planes"])
def test_long_decoding(made, which):
    """Hundreds of single tokens behind a short prompt, several requests side by side in captured steps."""
    cfg = gm.CONFIGS[which]
    for dtype in ("float32", "bfloat16"):
        folder, _ = made[which, dtype]
        _, exact = stored(gm.tensors(cfg, seed=sorted(gm.CONFIGS).index(which)), dtype)
        seqs = sequences(cfg["vocab"], lengths=[400, 260, 333], seed=60)
        truth = {rid: plain.forward(cfg, exact, toks) for rid, toks in seqs.items()}
        steps = helpers.trace_many_live(seqs, tail=250, portion_beside=False)
        assert worst_error(replay(folder, dtype, steps, max_live=3), truth) < LIMIT[dtype]


# ---- mechanisms alone -------------------------------------------------------------------------------------------

def dev(x, dtype=torch.int32):
    return torch.tensor(x, dtype=dtype).cuda()


def step_context(lengths, starts, slots):
    """What the ops read of a step: portions of the given lengths starting at the given absolute positions."""
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


def test_scaled_embedding_alone():
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(0)
    table = torch.randn(50, 24, generator=g)
    ids = [4, 9, 9, 49, 0]
    assert torch.allclose(ops.embedding(dev(ids), table.cuda(), scale=2.5).cpu(), table[ids] * 2.5, atol=1e-6)
    assert torch.equal(ops.embedding(dev(ids), table.cuda()).cpu(), table[ids])
    h = ops.embedding(dev(ids), table.bfloat16().cuda(), scale=7.0)
    assert h.dtype == torch.float32 and torch.allclose(h.cpu(), table.bfloat16().float()[ids] * 7.0, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [24, 1100])
def test_token_shift_alone(dtype, width):
    """Portions that start a sequence, portions that go on (the row before them comes from the slot), a single token;
    the slots' rows lie inside wider rows, as when an inner mixer's state follows."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(1)
    lengths, starts, slots = [5, 1, 3, 1], [0, 9, 4, 0], [2, 0, 3, 1]
    x = torch.randn(sum(lengths), width, generator=g).to(dtype)
    mix = torch.rand(width, generator=g)
    wide = torch.randn(5, width + 13, generator=g)
    before = wide.clone()
    state = wide.cuda()
    y = ops.token_shift(x.cuda(), mix.cuda(), state[:, :width], step_context(lengths, starts, slots)).cpu().double()
    at = 0
    for n, s, slot in zip(lengths, starts, slots):
        rows = x[at: at + n].double()
        first = torch.zeros(1, width, dtype=torch.float64) if s == 0 else before[slot, :width].double()[None]
        want = plain.token_shift(torch.cat([first, rows]), mix.double())[1:]
        assert torch.allclose(y[at: at + n], want, atol=1e-6 if dtype == torch.float32 else 2e-2)
        assert torch.equal(state[slot, :width].cpu(), x[at + n - 1].float())     # the unshifted last row is carried on
        at += n
    assert torch.equal(state[:, width:].cpu(), before[:, width:]) and torch.equal(state[4].cpu(), before[4])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [24, 2056])
@pytest.mark.parametrize("with_delta", [False, True])
def test_sum_norm_and_shift_in_one_kernel(dtype, width, with_delta):
    """A step of single tokens hands the shift a norm that has not run: stream += delta, norm and shift against the
    plain functions, the stream and the carried row left as the separate kernels leave them."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(width)
    starts, slots = [0, 9, 4, 0], [2, 0, 3, 1]
    lengths = [1] * len(starts)
    h = torch.randn(len(starts), width, generator=g)
    delta = torch.randn(len(starts), width, generator=g).to(dtype) if with_delta else None
    gain, mix, eps = 1 + 0.1 * torch.randn(width, generator=g), torch.rand(width, generator=g), 1e-5
    wide = torch.randn(5, width + 16, generator=g)
    ctx = step_context(lengths, starts, slots)
    results = []
    for fused in (True, False):
        ops.kernels.FUSE_NORM_SHIFT = fused
        try:
            stream, state = h.clone().cuda(), wide.clone().cuda()
            x = ops.NormedRows(stream, None if delta is None else delta.cuda(), gain.cuda(), eps, dtype)
            y = ops.token_shift(x, mix.cuda(), state[:, :width], ctx)
            assert x.residual() is stream
        finally:
            ops.kernels.FUSE_NORM_SHIFT = True
        results.append((y.cpu().double(), stream.cpu(), state.cpu()))
    summed = h.double() + (0 if delta is None else delta.double())
    normed = plain.norm(summed, gain.double(), eps)
    for y, stream, state in results:
        assert torch.allclose(stream.double(), summed, atol=1e-6)
        for i, (s, slot) in enumerate(zip(starts, slots)):
            first = torch.zeros(1, width, dtype=torch.float64) if s == 0 else wide[slot, :width].double()[None]
            want = plain.token_shift(torch.cat([first, normed[i: i + 1]]), mix.double())[1:]
            assert torch.allclose(y[i: i + 1], want, atol=1e-5 if dtype == torch.float32 else 3e-2)
            assert torch.allclose(state[slot, :width].double(), normed[i], atol=1e-5 if dtype == torch.float32 else 2e-2)
        assert torch.equal(state[:, width:], wide[:, width:]) and torch.equal(state[4], wide[4])
    # one kernel or two: the same rows up to the last bit of the norm's factor
    assert torch.allclose(results[0][0], results[1][0], atol=1e-6 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("lengths", [[1, 1, 1], [5, 1, 40], [300, 2, 129, 64, 1]])   # the last: chunks that run side by side
def test_min_gru_alone(dtype, lengths):
    from prefixserve_b200 import ops
    width = 20
    g = torch.Generator().manual_seed(len(lengths))
    t = sum(lengths)
    proj = torch.randn(t, 3 * width + 11, generator=g).to(dtype)      # the three runs of columns lie in a wider product
    bz, bx = torch.randn(width, generator=g) - 2.0, torch.randn(width, generator=g)
    slots = list(range(len(lengths)))[::-1]
    wide = torch.rand(len(lengths) + 1, 7 + width, generator=g)
    before = wide.clone()
    state = wide.cuda()
    ctx = step_context(lengths, [3] * len(lengths), slots)
    out = ops.min_gru(proj.cuda()[:, 4: 4 + 3 * width], bz.cuda(), bx.cuda(), state[:, 7:], ctx, width=width).cpu().double()
    at = 0
    for n, slot in zip(lengths, slots):
        p = proj[at: at + n, 4: 4 + 3 * width].double()
        s = before[slot, 7:].double()
        for i in range(n):   # the design's recurrence, from the state the slot held
            z = torch.sigmoid(p[i, :width] + bz.double())
            u = p[i, width: 2 * width] + bx.double()
            s = (1 - z) * s + z * torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
            gate = p[i, 2 * width:]
            want = s * gate * torch.sigmoid(gate)
            assert torch.allclose(out[at + i], want, atol=1e-5 if dtype == torch.float32 else 3e-2, rtol=1e-5 if dtype == torch.float32 else 1e-2)
        assert torch.allclose(state[slot, 7:].cpu().double(), s, atol=1e-5)    # float32 whatever the rows' type
        at += n
    assert torch.equal(state[:, :7].cpu(), before[:, :7]) and torch.equal(state[len(lengths)].cpu(), before[len(lengths)])


def paged_entry(hkv, row, page_size, tokens_per_item, dtype, seed=0, planes=1):
    """A pool of pages in shuffled order, filled with NaN, and each item's table."""
    per = [-(-n // page_size) for n in tokens_per_item]
    order = torch.randperm(sum(per) + 3, generator=torch.Generator().manual_seed(seed)).tolist()
    kv = torch.full((sum(per) + 3, planes, hkv, page_size, row), float("nan"), dtype=dtype).cuda()
    table = torch.full((len(per), max(per)), -1, dtype=torch.int32)
    for i, n in enumerate(per):
        table[i, :n] = torch.tensor([order.pop() for _ in range(n)], dtype=torch.int32)
    return kv, table.cuda()


ATTENTION_SHAPES = [
    # heads, kv heads, dim, vdim, rotated, interleaved, unit norm, factors, sink, keys as values
    (4, 2, 16, 24, 8, True, True, True, True, False),
    (3, 3, 8, 8, 8, True, True, False, False, True),
    (6, 1, 12, 5, None, False, True, True, True, False),
    (2, 1, 32, 32, 16, False, False, False, True, False),
    (8, 4, 64, 64, 32, True, True, True, True, False),     # sizes the tensor-core kernel takes
    (4, 1, 128, 128, 64, True, True, True, True, False),
    (4, 2, 64, 64, None, False, True, False, False, True),
    (2, 2, 128, 128, 128, False, False, True, True, False),  # a rotation of halves: the general pass in front
]
# (tokens already there, new tokens) per request: single tokens beside short and long portions; a long portion alone (the
# kernels that cut a portion's keys into ranges); single tokens only, far enough back for several key ranges
ATTENTION_STEPS = [([37, 0, 9], [1, 2, 70]), ([150], [300]), ([700, 3, 1100], [1, 1, 1])]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("planes", [1, 2])
@pytest.mark.parametrize("steps", range(len(ATTENTION_STEPS)))
@pytest.mark.parametrize("shape", ATTENTION_SHAPES)
def test_prepared_attention_alone(shape, steps, planes, dtype):
    """Two steps over the requests: their first tokens, then the new ones behind them; pages in shuffled order.  Against
    the plain rotation, unit norm and softmax with factors and a sink.  ``planes`` 1: a row per token (key, then value)
    and the kernels that read such rows; 2: a plane of keys and a plane of values and the kernels of ``ops.attention``."""
    from prefixserve_b200 import ops
    hq, hkv, dim, vdim, rotated, interleaved, unit, factors, sink, keys = shape
    if planes == 2 and dim != vdim:
        pytest.skip("planes of their own need keys and values of one size")
    if steps and (dim < 64 or planes == 1):
        pytest.skip("the long steps are for the kernels that cut keys into ranges")
    eps, scale, page = 1e-5, 0.37 if dim < 64 else 0.11, 8 if planes == 1 else 16
    g = torch.Generator().manual_seed(hq)
    had, new = ATTENTION_STEPS[steps]
    total = [a + b for a, b in zip(had, new)]
    width = (hq + hkv) * dim + (0 if keys else hkv * vdim)
    seqs = [torch.randn(n, width, generator=g).to(dtype) for n in total]
    temp = (1.5 + 0.5 * torch.randn(hq, generator=g)) if factors else None
    rot = None if rotated is None else gm.rot(rotated, base=300.0, scaling=(4.0, 1.0, 4.0, 32))
    cos = sin = None
    if rot is not None:
        angle = torch.arange(max(total) + 1, dtype=torch.float64)[:, None] * plain.rotary_frequencies(rot)[None, :]
        cos, sin = torch.cos(angle).float().cuda(), torch.sin(angle).float().cuda()
    kv, table = paged_entry(hkv, dim + vdim if planes == 1 else dim, page, total, dtype, planes=planes)
    outs = {}
    for step, (lengths, starts) in enumerate((([h for h in had if h], [0 for h in had if h]), (new, had))):
        items = [i for i, h in enumerate(had) if h] if step == 0 else list(range(len(had)))
        rows = torch.cat([seqs[i][s: s + n] for i, n, s in zip(items, lengths, starts)]).cuda()
        ctx = step_context(lengths, starts, items)
        tab = table.cpu()[items].contiguous().cuda()   # rows picked on the host: a wrong index raises here, not on the device
        q = ops.attention_prepare(rows, kv, tab, ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=vdim, page_size=page,
                                  cos=cos, sin=sin, rotary_dim=rotated, interleaved=interleaved, unit_norm_eps=eps if unit else None,
                                  head_factor=None if temp is None else temp.cuda(), values_are_keys=keys,
                                  split_planes=planes == 2)
        if planes == 2:
            o = ops.attention(q, kv, tab, ctx.positions, ctx.token_item, scale=scale, ctx=ctx,
                              sink=torch.zeros(hq).cuda() if sink else None)
        else:
            o = ops.attention_over_rows(q, kv, tab, ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=vdim, page_size=page,
                                        scale=scale, sink=torch.zeros(hq).cuda() if sink else None)
        at = 0
        for i, n, s in zip(items, lengths, starts):
            outs[i, step] = (s, o[at: at + n].cpu().double())
            at += n
    for i, n in enumerate(total):
        x = seqs[i].double()
        q = x[:, : hq * dim].view(n, hq, dim)
        k = x[:, hq * dim: (hq + hkv) * dim].view(n, hkv, dim)
        v = k if keys else x[:, (hq + hkv) * dim:].view(n, hkv, vdim)
        if rot is not None:
            if interleaved:
                q, k = plain.rotate(q, rot), plain.rotate(k, rot)
            else:   # element i turns with element i + rotated/2: the plain rotation on a reordered head
                order = [j // 2 + (j % 2) * (rotated // 2) for j in range(rotated)] + list(range(rotated, dim))
                back = torch.argsort(torch.tensor(order))
                q, k = plain.rotate(q[..., order], rot)[..., back], plain.rotate(k[..., order], rot)[..., back]
        if unit:
            q, k = plain.unit_rms(q, eps), plain.unit_rms(k, eps)
        want = plain.softmax_attention(q, k, v, scale, temp=None if temp is None else temp.double(), sink=sink).reshape(n, hq * vdim)
        for step in (0, 1):
            if (i, step) in outs:
                s, got = outs[i, step]
                assert torch.allclose(got, want[s: s + got.shape[0]], atol=1e-5 if dtype == torch.float32 else 4e-2), (i, step)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_sink_takes_the_weight_that_no_key_deserves(dtype):
    """Queries that point away from every key: all scores far below the sink's zero, so the result is almost nothing,
    where a softmax without the sink would return a mean of the values (of size one)."""
    from prefixserve_b200 import ops
    hq, hkv, dim, page, n = 2, 1, 16, 8, 90
    g = torch.Generator().manual_seed(3)
    way = torch.randn(dim, generator=g)
    k = way[None] + 0.1 * torch.randn(n, dim, generator=g)
    q = -way[None, None] + 0.1 * torch.randn(n, hq, dim, generator=g)
    rows = torch.cat([q.reshape(n, hq * dim), k, torch.ones(n, dim)], 1).to(dtype)
    kv, table = paged_entry(hkv, 2 * dim, page, [n], dtype)
    ctx = step_context([n], [0], [0])
    qd = ops.attention_prepare(rows.cuda(), kv, table, ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=dim, page_size=page,
                               unit_norm_eps=1e-6)
    for sink, least, most in ((torch.zeros(hq).cuda(), 0.0, 0.05), (None, 0.99, 1.01)):
        o = ops.attention_over_rows(qd, kv, table, ctx, num_heads=hq, num_kv_heads=hkv, dim=dim, vdim=dim, page_size=page,
                                    scale=0.5, sink=sink).float()
        assert least <= float(o.min()) and float(o.max()) <= most


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width", [40, 1500])
def test_pair_of_normed_results_alone(dtype, width):
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(4)
    a, b = (3 * torch.randn(7, width, generator=g)).to(dtype), (0.2 * torch.randn(7, width, generator=g)).to(dtype)
    ga, gb = 1 + 0.1 * torch.randn(width, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
    got = ops.normed_pair_sum(a.cuda(), b.cuda(), ga.cuda(), gb.cuda(), 3e-6, 0.5)
    want = 0.5 * (plain.norm(a.double(), ga.double(), 3e-6) + plain.norm(b.double(), gb.double(), 3e-6))
    assert got.dtype == torch.float32 and torch.allclose(got.cpu().double(), want, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clipped_gate_alone(dtype):
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(5)
    z = (2 * torch.randn(33, 2 * 50, generator=g)).to(dtype)
    z[0, :4] = torch.tensor([9.0, -9.0, 0.7, -0.7]).to(dtype)
    z[0, 50:54] = torch.tensor([9.0, -9.0, -9.0, 0.7]).to(dtype)
    eye = torch.eye(50, dtype=torch.float64)
    x = z.double()
    for limit in (0.7, 7.0):
        got = ops.clipped_glu(z.cuda(), limit).cpu().double()
        want = plain.feed_forward({"limit": limit}, {"f.gate": torch.cat([eye, 0 * eye], 1), "f.up": torch.cat([0 * eye, eye], 1), "f.down": eye}, "f.", x)
        assert torch.allclose(got, want, atol=1e-5 if dtype == torch.float32 else 3e-2, rtol=0 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("rows", [5, 40, 1024])
def test_clipped_gated_product_alone(rows):
    """Both products and the clipped gate as one op (a few bfloat16 rows: in the streaming product's epilogue, also with
    the norm in front; many: in the tcgen05 product's; between: product, then gate) against the plain feed-forward
    with an identity behind it."""
    from prefixserve_b200 import ops
    g = torch.Generator().manual_seed(rows)
    width, ff = 256, 2048
    x = torch.randn(rows, width, generator=g).to(torch.bfloat16)
    w = (1.5 * torch.randn(2 * ff, width, generator=g) / width ** 0.5).to(torch.bfloat16)
    eye = torch.eye(ff, dtype=torch.float64)
    for limit in (0.7, 7.0):
        got = ops.clipped_gated_linear(x.cuda(), w.cuda(), limit).cpu().double()
        want = plain.feed_forward({"limit": limit}, {"f.gate": w[:ff].double(), "f.up": w[ff:].double(), "f.down": eye}, "f.", x.double())
        assert got.shape == want.shape and torch.allclose(got, want, atol=4e-2, rtol=2e-2)
    # the same behind a norm that has not run yet: stream + delta, norm, products, gate
    h, delta = torch.randn(rows, width, generator=g), torch.randn(rows, width, generator=g).to(torch.bfloat16)
    gain = 1 + 0.1 * torch.randn(width, generator=g)
    x = ops.NormedRows(h.cuda(), delta.cuda(), gain.cuda(), 1e-5, torch.bfloat16)
    got = ops.clipped_gated_linear(x, w.cuda(), 1.5).cpu().double()
    normed = plain.norm(h.double() + delta.double(), gain.double(), 1e-5)
    want = plain.feed_forward({"limit": 1.5}, {"f.gate": w[:ff].double(), "f.up": w[ff:].double(), "f.down": eye}, "f.", normed)
    assert torch.allclose(got, want, atol=5e-2, rtol=2e-2)
    assert torch.allclose(x.residual().cpu().double(), h.double() + delta.double(), atol=1e-6)


# ---- generation through the scheduler --------------------------------------------------------------------------

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
    cfg = gm.CONFIGS["mixed"]
    _, exact = stored(gm.tensors(cfg, seed=sorted(gm.CONFIGS).index("mixed")), "float32")
    prompts = [helpers.random_tokens(131, n, seed=70 + n) for n in (1, 5, 23, 40)]
    llm = LLM(folder, dtype="float32", max_seq_len=128, num_blocks=64, max_running_requests=3, chunked_prefill_size=16)
    got = llm.generate(prompts, SamplingParams(max_tokens=12, ignore_eos=True))
    assert got == [greedy(cfg, exact, p, 12) for p in prompts]
    assert llm.engine.runner.graph_replays > 0
    llm.engine.cache.check()
    # a second call on the same engine starts from clean slots
    assert llm.generate(prompts[:2], SamplingParams(max_tokens=5, ignore_eos=True)) == [greedy(cfg, exact, p, 5) for p in prompts[:2]]


def test_command_line_generates_from_a_goganex_folder(made):
    import json
    import subprocess
    import sys
    folder, _ = made["whole_loop", "bfloat16"]
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
    folder = write_random_model(tmp_path / "m", preset("goganex-tiny"), 0, std=0.1, gain_noise=0.1, dtype=torch.bfloat16)
    llm = LLM(folder, dtype="bfloat16", max_seq_len=64, num_blocks=32, max_running_requests=2)
    got = llm.generate([[5, 6, 7], [9]], SamplingParams(max_tokens=4, ignore_eos=True))
    assert [len(g) for g in got] == [4, 4]
