"""The Tizodra configuration, its model builder, cache needs and random weights, the cache manager's kept first pages,
and the plain implementation's own consistency, without a device."""
import copy

import numpy as np
import pytest
import torch

import plain_tizodra as pt
from tizodra_helpers import CONFIGS, ids_for, make_dir, read_tensors


def test_config_is_found_by_its_name_and_round_trips():
    import ai_engine_b200 as aie
    from ai_engine_b200.config import load_config

    for name, raw in CONFIGS.items():
        arch, cfg = load_config(raw)
        assert arch.name == "Tizodra" and isinstance(cfg, aie.TizodraConfig)
        assert aie.TizodraConfig.from_dict(cfg.to_dict()) == cfg
        assert cfg.width == raw["width"] and len(cfg.layers) == len(raw["layers"])
    a = aie.TizodraConfig.from_dict(CONFIGS["A"])
    assert a.logit_scale == 0.5 and (a.loop_start, a.loop_stop, a.loop_times) == (1, 3, 3)
    assert a.run_order() == [0, 1, 2, 1, 2, 1, 2, 3]
    assert (a.layers[1].mixer.window, a.layers[1].mixer.keep_first, a.layers[1].mixer.scale) == (37, 3, 0.3)
    assert a.layers[1].ff == 0 and a.layers[0].ff == 80 and a.layers[0].mixer.conv == 4
    b = aie.TizodraConfig.from_dict(CONFIGS["B"])
    assert b.layers[2].mixer.window == 0 and b.run_order() == [0, 1, 0, 1, 2, 3, 4]
    c = aie.TizodraConfig.from_dict(CONFIGS["C"])
    assert c.logit_scale == 1.0 and c.loop_times == 0 and c.run_order() == [0, 1, 2, 3]
    assert aie.TizodraConfig.from_dict(CONFIGS["D"]).run_order() == [0, 1, 2]


def test_a_missing_or_wrong_key_is_named():
    import ai_engine_b200 as aie

    def bad(name, change, match):
        raw = copy.deepcopy(CONFIGS[name])
        change(raw)
        with pytest.raises(aie.ConfigError, match=match):
            aie.TizodraConfig.from_dict(raw)

    bad("A", lambda r: r["layers"][0]["mixer"].pop("conv"), "conv")
    bad("A", lambda r: r["layers"][1]["mixer"].pop("scale"), "scale")
    bad("A", lambda r: r["layers"][1]["mixer"].update(kv_heads=4), "kv_heads")
    bad("A", lambda r: r["layers"][1]["mixer"].pop("vdim"), "vdim")
    bad("A", lambda r: r["layers"][2].update(type="mamba2"), "type")
    bad("A", lambda r: r["layers"][0]["mlp"].update(kind="moe"), "kind")
    bad("A", lambda r: r["loop"].update(stop=5), "loop")
    bad("A", lambda r: r["loop"].update(start=3), "loop")
    bad("A", lambda r: r["loop"].pop("times"), "times")
    bad("C", lambda r: r.pop("norm"), "norm")
    bad("C", lambda r: r.update(width="36"), "width")


def test_tensor_names_and_shapes_follow_the_configuration():
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts.model import tensor_specs_of

    arch, cfg = load_config(CONFIGS["A"])
    specs = {s.name: tuple(s.shape) for s in tensor_specs_of(arch.build_spec(cfg))}
    assert specs["embed"] == (211, 96) and specs["head"] == (211, 96) and specs["final.norm"] == (96,)
    assert specs["loop.in"] == (96, 192)
    assert specs["l0.mix.q"] == (48, 96) and specs["l0.mix.k.conv"] == (48, 4) and specs["l0.mix.v.conv"] == (80, 4)
    assert specs["l0.mix.b"] == (4, 96) and specs["l0.mix.a"] == (4, 96) and specs["l0.mix.A_log"] == (4,)
    assert specs["l0.mix.norm"] == (20,) and specs["l0.mix.g"] == (80, 96) and specs["l0.mix.o"] == (96, 80)
    assert specs["l1.mix.q"] == (96, 96) and specs["l1.mix.k.b"] == (32,) and specs["l1.mix.v"] == (48, 96)
    assert specs["l1.mix.temp"] == (6,) and specs["l1.mix.sink"] == (6,) and specs["l1.mix.g"] == (6, 96)
    assert specs["l1.mix.o"] == (96, 144) and "l1.mlp.up" not in specs and "l1.norm2" not in specs
    assert specs["l0.mlp.up"] == (80, 96) and specs["l0.mlp.down"] == (96, 80)
    _, c = load_config(CONFIGS["C"])
    assert "loop.in" not in {s.name for s in tensor_specs_of(arch.build_spec(c))}


def test_cache_needs_every_pass_of_the_loop_has_a_cache_of_its_own():
    from ai_engine_b200.cache.manager import group_requests
    from ai_engine_b200.config import load_config
    from ai_engine_b200.parts.model import Model

    arch, cfg = load_config(CONFIGS["A"])
    needs = Model(arch.build_spec(cfg), torch.float32, device="cpu").cache_requests()
    assert [n.run for n in needs] == list(range(8))
    kv = {n.run: n.kv for n in needs if n.kv is not None}
    assert sorted(kv) == [1, 3, 5, 7]
    assert (kv[1].kv_heads, kv[1].head_dim, kv[1].window, kv[1].keep_first, kv[1].planes) == (2, 40, 37, 3, 1)
    assert kv[1] == kv[3] == kv[5] and (kv[7].head_dim, kv[7].window, kv[7].keep_first) == (56, 21, 0)
    groups = group_requests(needs)
    assert sorted(len(e) for _, e in groups) == [1, 3]
    st = {n.run: n.state for n in needs if n.state is not None}
    assert sorted(st) == [0, 2, 4, 6]
    assert st[0]["tail"].shape == (3, 48 + 48 + 80) and st[0]["S"].shape == (4, 24, 20)
    assert st[2]["tail"].shape == (1, 120 + 120 + 24) and st[4]["S"].shape == (3, 40, 8)


def test_a_window_keeps_the_pages_of_its_first_tokens():
    from ai_engine_b200.cache.manager import host

    h = host()
    book = h.CacheManager([h.GroupSpec(4, 16, 8, 5), h.GroupSpec(4, 16, 8, 0)], 2, 64)
    s = book.admit()
    assert book.ensure(s, 40) and book.pages_in_use(0) == 10
    book.advance(s, 40)                  # later queries sit at 40 or beyond: keys from 33 on, and the first five
    assert book.kept_pages(0) == 2 and book.kept_pages(1) == 0
    p0, p1 = book.pages(0, s), book.pages(1, s)
    assert [p >= 0 for p in p0] == [True, True] + [False] * 6 + [True, True]
    assert [p >= 0 for p in p1] == [False] * 8 + [True, True]
    book.check_invariants()
    assert book.ensure(s, 64)
    book.advance(s, 64)
    assert sum(p >= 0 for p in book.pages(0, s)) == 2 + 2 and book.pages(0, s)[0] == p0[0]
    book.check_invariants()
    book.finish(s)
    assert book.pages_in_use(0) == 0 and book.pages_in_use(1) == 0
    s2 = book.admit()
    assert book.ensure(s2, 3)
    book.advance(s2, 3)                  # shorter than the kept run: nothing is given back
    assert book.pages_in_use(0) == 1
    book.check_invariants()


def test_sinusoid_frequencies_by_hand():
    from ai_engine_b200.parts.sinusoid import sinusoid_frequencies

    f = sinusoid_frequencies(8, 10000.0)
    assert np.allclose(f, [1.0, 0.1, 0.01, 0.001], rtol=1e-6)
    assert sinusoid_frequencies(5, 100.0).shape == (3,)
    v = pt.sinusoid(torch.tensor([0, 3]), 8)
    assert np.allclose(v[0].numpy(), [0, 1] * 4)
    assert np.allclose(v[1].numpy()[:4], [np.sin(3.0), np.cos(3.0), np.sin(0.3), np.cos(0.3)])


def test_distance_slopes_by_hand():
    from ai_engine_b200.parts.sink_attention import distance_slopes

    assert distance_slopes(4, 8.0) == [0.25, 0.0625, 0.015625, 0.00390625]
    assert pt.head_slopes(8)[0] == 0.5 and pt.head_slopes(8)[-1] == 2.0 ** -8


def test_random_weights_are_written_and_read_back(tmp_path):
    d = make_dir(tmp_path, "A")
    t = read_tensors(d)
    assert t["l1.mix.sink"].shape == (6,) and t["loop.in"].shape == (96, 192)
    assert abs(float(t["l0.norm1"].float().mean()) - 1.0) < 0.2
    assert float(t["l1.mix.temp"].float().min()) > 0.0


def test_the_oracle_window_and_sink_by_hand():
    """One head, scores of zero: with a window of two keys and one kept token, the weights are 1 / (n + e^sink)."""
    z = torch.zeros
    w = {"q": z(4, 4, dtype=torch.float64), "q.b": z(4, dtype=torch.float64), "k": z(4, 4, dtype=torch.float64),
         "k.b": z(4, dtype=torch.float64), "v": torch.eye(4, dtype=torch.float64), "v.b": z(4, dtype=torch.float64),
         "temp": torch.ones(1, dtype=torch.float64), "sink": torch.tensor([0.0], dtype=torch.float64),
         "g": z(1, 4, dtype=torch.float64), "o": torch.eye(4, dtype=torch.float64)}
    m = dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=1.0, mask=dict(size=2, keep_first=1))
    h = torch.eye(4, dtype=torch.float64) * 3.0
    out = pt.sink_attention(h, w, m, 0.0)
    # values are unit rows times 2 (rms of a one-hot row of four is 1/2); the distance bias of the only head is 2^-8
    s = 2.0 ** -8
    w3 = np.exp([-3 * s, -s, 0.0])              # token 3 reads tokens 0 (kept), 2 and 3
    assert np.allclose(out[3].numpy(), 0.5 * 2.0 * np.array([w3[0], 0.0, w3[1], w3[2]]) / (w3.sum() + 1.0))
    assert np.allclose(out[0].numpy(), 0.5 * 2.0 * np.array([1.0, 0, 0, 0]) / 2.0)


def test_the_oracle_delta_rule_by_hand():
    """One head of one key channel: S is a row; with beta = 1 and no decay the state takes each value whole."""
    keep = []
    one = lambda *s: torch.ones(*s, dtype=torch.float64)
    w = {"q": one(1, 2), "k": one(1, 2), "v": torch.eye(2, dtype=torch.float64), "q.conv": one(1, 1), "k.conv": one(1, 1),
         "v.conv": one(2, 1), "b": one(1, 2) * 50.0, "a": one(1, 2) * -50.0, "A_log": torch.zeros(1, dtype=torch.float64),
         "dt_bias": torch.zeros(1, dtype=torch.float64), "norm": one(2), "g": torch.eye(2, dtype=torch.float64),
         "o": torch.eye(2, dtype=torch.float64)}
    m = dict(heads=1, kv_heads=1, dim=1, vdim=2, conv=1)
    h = torch.tensor([[2.0, 0.0], [0.0, 2.0]], dtype=torch.float64)
    pt.delta_mixer(h, w, m, 1e-6, keep_states=keep)
    k = float(pt.unit(pt.silu(torch.tensor([2.0], dtype=torch.float64))))
    v = pt.silu(torch.tensor([0.0, 2.0], dtype=torch.float64))
    # after the second token u = v_2 - k^2 S_1 and S_2 = S_1 + k u: with k nearly 1, S_2 k is nearly v_2
    assert np.allclose((keep[0][0] * k).numpy(), v.numpy(), atol=1e-5)


def test_the_oracle_does_not_depend_on_later_tokens(tmp_path):
    d = make_dir(tmp_path, "D")
    ids = ids_for(30, CONFIGS["D"]["vocab"], 3)
    t = read_tensors(d)
    a = pt.forward(t, CONFIGS["D"], ids)
    b = pt.forward(t, CONFIGS["D"], ids[:17])
    assert torch.allclose(a[:17], b, atol=1e-9)
