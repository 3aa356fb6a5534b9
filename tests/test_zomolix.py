"""Zomolix without a GPU: the configuration reader, the parts list, run list and tensor names, the cache needs of
layers that share keys and values, pages that stay for the kept first keys, and the plain implementation's own
consistency where the design says two forms are the same."""

import json
import math

import numpy as np
import pytest
import torch

import plain_zomolix as plain
import zomolix_models as zm


def test_config_reader_takes_every_key_and_refuses_what_is_missing():
    from prefixserve_b200.config import UnsupportedModelError, ZomolixConfig
    raw = zm.CONFIGS["mixed"]
    cfg = ZomolixConfig.from_dicts(raw)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale) == (131, 40, 3e-6, 5.5)
    assert [l.mixer.kind for l in cfg.layers] == ["latent_attention", "attention", "attention", "latent_attention", "attention", "attention"]
    a = cfg.layers[1].mixer
    assert (a.heads, a.kv_heads, a.dim, a.vdim, a.window, a.keep_first, a.kv_from) == (4, 2, 16, 10, 21, 5, None)
    assert (a.rot.factor, a.rot.original, a.rot.fast, a.rot.slow) == (4.0, 64, 8.0, 1.0)
    assert cfg.layers[2].mixer.kv_from == 1 and cfg.layers[4].mixer.kv_from == 1 and cfg.layers[5].mixer.window is None
    assert cfg.layers[5].mixer.rot.factor is None
    l0 = cfg.layers[0]
    assert (l0.mixer.heads, l0.mixer.dim, l0.mixer.rot_dim, l0.mixer.vdim, l0.mixer.kv_rank) == (3, 6, 8, 10, 20)
    assert (l0.mlp.experts, l0.mlp.top, l0.mlp.groups, l0.mlp.keep, l0.mlp.ff, l0.mlp.limit, l0.mlp.shared_ff, l0.mlp.shared_limit) == (8, 3, 4, 3, 12, 0.7, 20, 2.0)
    assert cfg.layers[1].mlp.shared_ff is None and cfg.layers[2].mlp is None
    assert cfg.to_config_json() == raw  # what is written is what was read
    for drop in (("vocab",), ("norm", "eps"), ("layers", 0, "mixer", "kv_rank"), ("layers", 1, "mixer", "scale"),
                 ("layers", 1, "mixer", "rot", "scaling", "original"), ("layers", 0, "mlp", "expert", "limit"),
                 ("layers", 0, "mlp", "router", "top"), ("layers", 0, "mlp", "shared", "ff")):
        broken = json.loads(json.dumps(raw))
        at = broken
        for k in drop[:-1]:
            at = at[k]
        del at[drop[-1]]
        with pytest.raises(UnsupportedModelError):
            ZomolixConfig.from_dicts(broken)
    for path, value in ((("layers", 1, "mixer", "kv_heads"), 3), (("layers", 2, "mixer", "kv_from"), 0), (("layers", 2, "mixer", "kv_from"), 4),
                        (("layers", 4, "mixer", "vdim"), 12), (("layers", 5, "mixer", "rot", "dims"), 6), (("layers", 1, "type"), "other"),
                        (("layers", 0, "mlp", "router", "groups", "count"), 3), (("layers", 0, "mlp", "router", "top"), 7),
                        (("layers", 0, "mlp", "kind"), "dense")):
        broken = json.loads(json.dumps(raw))
        at = broken
        for k in path[:-1]:
            at = at[k]
        at[path[-1]] = value
        with pytest.raises(UnsupportedModelError):
            ZomolixConfig.from_dicts(broken)


def test_every_tensor_of_a_checkpoint_has_a_part_and_a_reader_shares_its_writers_cache_entry(tmp_path):
    from prefixserve_b200 import architectures  # noqa: F401
    from prefixserve_b200.config.registry import read_model_folder
    from prefixserve_b200.parts.model import build_model
    for which, cfg in zm.CONFIGS.items():
        weights = zm.tensors(cfg, seed=1)
        folder = zm.write_folder(tmp_path / which, cfg, weights)
        arch, typed = read_model_folder(folder)
        spec = arch.to_spec(typed)
        model = build_model(spec)
        wanted = {arch.tensor_name(path): tuple(ps.shape) for path, ps in model.param_table().items()}
        assert wanted == {k: tuple(v.shape) for k, v in weights.items()}, which
        for i, (call, lay) in enumerate(zip(spec.schedule, cfg["layers"])):
            src = lay["mixer"].get("kv_from")
            assert call.layer == i and call.cache == (i if src is None else src) and call.writes_cache == (src is None)
    # an entry that several layers read keeps whatever any of them can still see
    spec = arch.to_spec(read_model_folder(tmp_path / "mixed")[1])
    needs = build_model(spec).cache_needs()
    assert (needs[1].paged.window, needs[1].paged.keep_first) == (33, 18) and needs[2].paged is None and needs[4].paged is None
    needs = build_model(arch.to_spec(read_model_folder(tmp_path / "reader_sees_all")[1])).cache_needs()
    assert needs[0].paged.window is None and needs[0].paged.keep_first == 0
    wide = build_model(arch.to_spec(read_model_folder(tmp_path / "wide")[1])).cache_needs()
    assert [n.paged.planes if n.paged else None for n in wide] == [1, 1, 1, None, 2, 1]   # planes only without a mask, 64 or 128


def test_kept_first_pages_stay_and_the_gap_goes_back():
    from prefixserve_b200.cache.manager import CacheManager
    from prefixserve_b200.parts.base import CacheNeed, PagedKV
    needs = [CacheNeed(paged=PagedKV(1, 8, window=10, planes=1, keep_first=6)), CacheNeed(paged=PagedKV(1, 8, window=10, planes=1)),
             CacheNeed(paged=PagedKV(1, 8, window=10, planes=1, keep_first=6))]
    cm = CacheManager(needs, num_pages=40, num_slots=2, max_seq_len=160, page_size=4, device=None)
    assert len(cm.groups) == 2 and cm.entry_group == [0, 1, 0]
    slot = cm.open()
    assert cm.reserve(slot, 100)
    first = cm.page_ids(slot, 0)[:2]
    cm.advance(slot, 100)
    kept, plain_window = cm.page_ids(slot, 0), cm.page_ids(slot, 1)
    low = (100 - 10 + 1) // 4
    assert kept[:2] == first and all(p < 0 for p in kept[2:low]) and all(p >= 0 for p in kept[low:25])
    assert all(p < 0 for p in plain_window[:low]) and all(p >= 0 for p in plain_window[low:25])
    assert cm.free_pages(0) == 40 - 2 - (25 - low) and cm.free_pages(1) == 40 - (25 - low)
    cm.check()
    cm.advance(slot, 100)   # again: nothing more to give back, nothing given back twice
    cm.check()
    cm.close(slot)
    assert cm.free_pages(0) == 40 and cm.free_pages(1) == 40
    cm.check()
    # a short sequence that has not left its kept keys yet lets nothing go
    slot = cm.open()
    cm.reserve(slot, 7)
    cm.advance(slot, 7)
    assert all(p >= 0 for p in cm.page_ids(slot, 0)[:2])
    cm.close(slot)
    cm.check()


def test_rotation_forms_agree_and_the_ramp_has_its_ends():
    g = torch.Generator().manual_seed(0)
    v = torch.randn(7, 2, 12, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 5, 40, 41, 300, 7])
    r = zm.rot(8, 300.0, (4.0, 32, 4.0, 1.0))
    half = plain.rotate(v, pos, r, "half")
    # the interleaved form is the half form on a head whose leading elements are shuffled (0,4,1,5,...)
    order = torch.tensor([0, 2, 4, 6, 1, 3, 5, 7, 8, 9, 10, 11])
    inv = torch.argsort(order)
    assert torch.allclose(plain.rotate(v[..., inv], pos, r, "interleaved")[..., order], half, atol=1e-12)
    assert torch.equal(half[..., 8:], v[..., 8:])   # what lies behind the rotated elements passes unchanged
    # a rotation keeps a pair's length up to the amplitude
    f, amp = plain.rotary_frequencies(r)
    assert amp == pytest.approx(0.1 * math.log(4.0) + 1)
    assert torch.allclose((half[..., :4] ** 2 + half[..., 4:8] ** 2), (v[..., :4] ** 2 + v[..., 4:8] ** 2) * amp ** 2, atol=1e-12)
    # pairs that turn fast keep their frequency, pairs that turn slowly have it divided by the factor
    plain_f, _ = plain.rotary_frequencies(zm.rot(64, 10000.0))
    f, _ = plain.rotary_frequencies(zm.rot(64, 10000.0, (8.0, 512, 32.0, 1.0)))
    assert f[0] == plain_f[0] and f[-1] == pytest.approx(float(plain_f[-1]) / 8.0) and bool((f[1:] < f[:-1]).all())


def test_mask_sink_and_router_of_the_plain_model():
    m = plain.visible(12, 4, 2)
    assert m[11].tolist() == [True, True] + [False] * 6 + [True] * 4
    assert m[3].tolist() == [True] * 4 + [False] * 8 and m[5].tolist() == [True, True, True, True, True, True] + [False] * 6
    assert plain.visible(5).tolist() == torch.tril(torch.ones(5, 5, dtype=torch.bool)).tolist()
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(6, 2, 4, generator=g, dtype=torch.float64) for _ in range(3))
    no_sink = plain.softmax_attention(q, k, v, 0.5, plain.visible(6))
    low = plain.softmax_attention(q, k, v, 0.5, plain.visible(6), sink=torch.tensor([-60.0, -60.0]))
    high = plain.softmax_attention(q, k, v, 0.5, plain.visible(6), sink=torch.tensor([60.0, -60.0]))
    assert torch.allclose(low, no_sink, atol=1e-12) and high[:, 0].abs().max() < 1e-20 and torch.allclose(high[:, 1], no_sink[:, 1], atol=1e-12)
    z = torch.tensor([[0.0, 5.0, 1.0, 1.1, 4.0, 0.2, 3.0, 3.1]], dtype=torch.float64)
    chosen, weight = plain.route(z, 3, 4, 2)            # groups (0,1) (2,3) (4,5) (6,7): the best two are the first and the third
    assert sorted(chosen[0].tolist()) == [1, 4, 5] and torch.allclose(weight[0].sort().values, torch.softmax(z, -1)[0, [5, 4, 1]])
    chosen, _ = plain.route(z, 3, 1, 1)
    assert sorted(chosen[0].tolist()) == [1, 4, 7]


def test_release_front_keeps_the_first_entries():
    from prefixserve_b200.cache.core import SeqTables
    t = SeqTables(2, 16)
    t.append(0, np.arange(100, 112, dtype=np.int32))
    assert t.release_front(0, 1, 2) == [] and t.release_front(0, 2, 2) == []
    assert t.release_front(0, 5, 2) == [102, 103, 104]
    assert t.row(0)[:6] == [100, 101, -1, -1, -1, 105]
    assert t.release_front(0, 5, 2) == [] and t.release_front(0, 7) == [105, 106]
    assert sorted(t.clear(0)) == [100, 101, 107, 108, 109, 110, 111]
    t.append(1, np.arange(5, dtype=np.int32))
    assert t.release_front(1, 3) == [0, 1, 2] and t.clear(1) == [3, 4]
