"""Goganex without a GPU: the configuration reader, the parts list, run list and tensor names, the cache needs of
nested mixers, the rotation's frequencies, and the plain implementation's own consistency where the design says two
forms are the same."""

import json
import math

import pytest
import torch

import goganex_models as gm
import plain_goganex as plain


def test_config_reader_takes_every_key_and_refuses_what_is_missing():
    from prefixserve_b200.config import GoganexConfig, ParallelConfig, UnsupportedModelError
    raw = gm.CONFIGS["mixed"]
    cfg = GoganexConfig.from_dicts(raw)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale) == (131, 40, 3e-6, 5.5)
    assert [l.mixer.kind for l in cfg.layers] == ["parallel", "attention", "attention", "parallel", "attention"]
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1, 4, 3)
    assert cfg.run_order() == (0, 1, 2, 3, 1, 2, 3, 1, 2, 3, 4)
    assert isinstance(cfg.layers[0].mixer, ParallelConfig) and cfg.layers[0].mixer.right_width == 20
    assert cfg.layers[1].mixer.rot.factor == 4.0 and cfg.layers[2].mixer.rot.factor is None and cfg.layers[4].mixer.rot is None
    assert cfg.layers[2].mlp is None and cfg.layers[0].mlp.limit == 0.7
    assert cfg.to_config_json() == raw  # what is written is what was read
    assert GoganexConfig.from_dicts(gm.CONFIGS["attn_only"]).run_order() == (0,)
    assert GoganexConfig.from_dicts(gm.CONFIGS["whole_loop"]).run_order() == (0, 1, 0, 1)
    for drop in (("vocab",), ("norm", "eps"), ("layers", 0, "mixer", "right"), ("layers", 1, "mixer", "scale"),
                 ("layers", 1, "mixer", "rot", "scaling", "original"), ("layers", 0, "mlp", "limit"), ("loop", "times")):
        broken = json.loads(json.dumps(raw))
        at = broken
        for k in drop[:-1]:
            at = at[k]
        del at[drop[-1]]
        with pytest.raises(UnsupportedModelError):
            GoganexConfig.from_dicts(broken)
    for path, value in ((("loop", "stop"), 9), (("layers", 1, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "left", "vdim"), 7),
                        (("layers", 2, "mixer", "rot", "dims"), 14), (("layers", 1, "type"), "other")):
        broken = json.loads(json.dumps(raw))
        at = broken
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(UnsupportedModelError):
            GoganexConfig.from_dicts(broken)


def test_every_tensor_of_a_checkpoint_has_a_part_and_every_pass_of_a_loop_its_own_cache_entry(tmp_path):
    from prefixserve_b200.config.registry import read_model_folder
    from prefixserve_b200 import architectures  # noqa: F401
    from prefixserve_b200.parts.model import build_model
    for which, cfg in gm.CONFIGS.items():
        weights = gm.tensors(cfg, seed=1)
        folder = gm.write_folder(tmp_path / which, cfg, weights)
        arch, typed = read_model_folder(folder)
        spec = arch.to_spec(typed)
        model = build_model(spec)
        wanted = {arch.tensor_name(path): tuple(ps.shape) for path, ps in model.param_table().items()}
        assert wanted == {k: tuple(v.shape) for k, v in weights.items()}, which
        assert [c.layer for c in spec.schedule] == plain.layer_order(cfg)
        assert [c.cache for c in spec.schedule] == list(range(len(spec.schedule))) and all(c.writes_cache for c in spec.schedule)


def test_cache_needs_of_nested_mixers(tmp_path):
    from prefixserve_b200.config.registry import read_model_folder
    from prefixserve_b200 import architectures  # noqa: F401
    from prefixserve_b200.parts.model import build_model
    from prefixserve_b200.cache.manager import CacheManager
    cfg = gm.CONFIGS["mixed"]
    arch, typed = read_model_folder(gm.write_folder(tmp_path, cfg, gm.tensors(cfg)))
    model = build_model(arch.to_spec(typed))
    needs = model.cache_needs()
    assert len(needs) == 11
    # a row per token and key/value head: the key, then the value (the key again where keys are the values)
    assert [(n.paged.num_kv_heads, n.paged.head_dim) for n in needs[:4]] == [(2, 12), (2, 26), (2, 36), (3, 20)]
    assert all(n.paged.planes == 1 and n.paged.window is None and n.paged.chunk is None for n in needs)
    # the slot's state: the shifted row, then the recurrence's channels where the layer has one
    assert [n.state.shape for n in needs[:4]] == [(40 + 20,), (40,), (40,), (40 + 7,)]
    assert needs[4] == needs[1] and needs[9] == needs[3] and needs[10].state.shape == (40,)
    cache = CacheManager(needs, num_pages=10, num_slots=2, max_seq_len=64, page_size=8, device=None)
    assert len(cache.groups) == 1 and not cache.prefix_cache_possible   # a carried state cannot be restored from a prefix


@pytest.mark.parametrize("dims, base, scaling", [(16, 10000.0, gm.SCALED), (8, 300.0, (8.0, 1.0, 2.0, 32)), (6, 500.0, None),
                                                 (32, 10000.0, gm.SCALED)])
def test_rotation_frequencies_of_the_engine_and_the_plain_model(dims, base, scaling):
    from prefixserve_b200.parts.position import rope_inverse_frequencies
    r = gm.rot(dims, base, scaling)
    want = plain.rotary_frequencies(r)
    sc = None if scaling is None else {"kind": "llama3", "factor": scaling[0], "low_freq_factor": scaling[1],
                                       "high_freq_factor": scaling[2], "original_max_positions": scaling[3]}
    got = rope_inverse_frequencies(dims, base, sc).double()
    assert torch.allclose(got, want, rtol=1e-6, atol=0)
    if scaling is not None:  # the test's constants meet every branch: kept, slowed and blended frequencies
        plain_f = plain.rotary_frequencies(gm.rot(dims, base))
        ratio = (want / plain_f).tolist()
        assert any(abs(x - 1) < 1e-12 for x in ratio) and any(abs(x - 1 / scaling[0]) < 1e-12 for x in ratio)
        assert any(1 / scaling[0] + 1e-6 < x < 1 - 1e-6 for x in ratio)


def test_plain_rotation_keeps_lengths_and_depends_on_distance_only():
    r = gm.rot(6, 500.0)
    g = torch.Generator().manual_seed(0)
    q, k = torch.randn(1, 1, 10, generator=g).double(), torch.randn(1, 1, 10, generator=g).double()
    a = (plain.rotate(q, r, 7) * plain.rotate(k, r, 3)).sum()
    b = (plain.rotate(q, r, 104) * plain.rotate(k, r, 100)).sum()
    assert abs(a - b) < 1e-9
    assert torch.allclose(plain.rotate(q, r, 50)[..., 6:], q[..., 6:])   # the elements beyond ``dims`` pass unchanged
    assert abs(plain.rotate(q, r, 50).norm() - q.norm()) < 1e-12


def test_plain_softmax_sink_and_first_token():
    """The first token sees itself only: without a sink its output is its own value, with one it is that value times
    e^s / (1 + e^s)."""
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(5, 2, 4, generator=g).double() for _ in range(3))
    plain_out = plain.softmax_attention(q, k[:, :1], v[:, :1], 0.5)
    assert torch.allclose(plain_out[0], v[0, :1].expand(2, 4))
    temp = torch.tensor([2.0, 0.5], dtype=torch.float64)
    out = plain.softmax_attention(q, k[:, :1], v[:, :1], 0.5, temp=temp, sink=True)
    for a in range(2):
        s = (q[0, a] @ k[0, 0]) * 0.5 * temp[a]
        assert torch.allclose(out[0, a], v[0, 0] * torch.exp(s) / (1 + torch.exp(s)))
    # every row's weights add up to less than one with a sink: values of all ones come out below one
    ones = torch.ones(5, 1, 3, dtype=torch.float64)
    assert (plain.softmax_attention(q, k[:, :1], ones, 0.5, sink=True) < 1).all()
    assert torch.allclose(plain.softmax_attention(q, k[:, :1], ones, 0.5), torch.ones(5, 2, 3, dtype=torch.float64))


def test_plain_recurrence_is_a_running_mean_of_candidates():
    m = {"width": 3}
    eye = torch.eye(3, dtype=torch.float64)
    w = {"r.z": torch.zeros(3, 3, dtype=torch.float64), "r.z.b": torch.zeros(3, dtype=torch.float64), "r.x": eye,
         "r.x.b": torch.zeros(3, dtype=torch.float64), "r.g": torch.zeros(3, 3, dtype=torch.float64), "r.o": eye}
    h = torch.tensor([[1.0, -1.0, 0.0], [2.0, -3.0, 0.5]], dtype=torch.float64)
    assert torch.equal(plain.min_gru(m, w, "r.", h), torch.zeros(2, 3, dtype=torch.float64))   # silu(0) = 0 closes the output
    w["r.g"] = 50 * eye      # silu(50 h) ~ 50 h for h > 0
    out = plain.min_gru(m, w, "r.", h)
    cand = torch.where(h >= 0, h + 0.5, torch.sigmoid(h))
    s0 = 0.5 * cand[0]
    s1 = 0.5 * s0 + 0.5 * cand[1]
    assert torch.allclose(out[0, 0], s0[0] * 50.0) and torch.allclose(out[1, 0], s1[0] * 100.0)
    assert abs(cand[0, 2] - 0.5) < 1e-15 and abs(float(torch.sigmoid(torch.tensor(0.0))) - 0.5) < 1e-15   # both forms meet at zero


def test_plain_token_shift_and_feed_forward():
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 0.0]], dtype=torch.float64)
    mix = torch.tensor([0.0, 0.5], dtype=torch.float64)
    assert torch.equal(plain.token_shift(h, mix), torch.tensor([[1.0, 1.0], [3.0, 4.0], [5.0, 3.0]], dtype=torch.float64))
    f = {"limit": 1.5}
    eye = torch.eye(2, dtype=torch.float64)
    w = {"f.gate": eye, "f.up": eye, "f.down": eye}
    x = torch.tensor([[4.0, -4.0], [0.5, 1.0]], dtype=torch.float64)
    got = plain.feed_forward(f, w, "f.", x)
    sig = lambda z: 1 / (1 + math.exp(-z))  # noqa: E731
    assert abs(got[0, 0] - 1.5 * sig(1.702 * 1.5) * 2.5) < 1e-12      # both branches at the upper limit
    assert abs(got[0, 1] - (-4.0) * sig(1.702 * -4.0) * (-0.5)) < 1e-12  # the gate has no lower limit, the other branch has
    assert abs(got[1, 1] - 1.0 * sig(1.702) * 2.0) < 1e-12


def test_plain_model_is_causal_and_loops_share_weights():
    cfg = gm.CONFIGS["mixed"]
    w = {k: v.double() for k, v in gm.tensors(cfg, seed=4).items()}
    toks = [5, 9, 100, 3, 77, 8, 41]
    whole, layers = plain.forward(cfg, w, toks, return_layers=True)
    assert layers.shape[0] == 11
    assert torch.allclose(plain.forward(cfg, w, toks[:4]), whole[:4], atol=1e-12)
    once = json.loads(json.dumps(cfg))
    once["loop"]["times"] = 1
    assert not torch.allclose(plain.forward(once, w, toks), whole, atol=1e-3)


def test_presets_of_the_design_read_back():
    from prefixserve_b200.config.presets import PRESETS, preset
    names = [n for n in PRESETS if n.startswith("goganex")]
    assert "goganex-tiny" in names and len(names) >= 3
    for n in names:
        cfg = preset(n)
        assert cfg.architecture == "Goganex" and cfg.to_config_json()["layers"]
