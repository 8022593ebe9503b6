"""Fokisun without a GPU: config.json keys and their defaults, rejections that name the key, the tensors a model of a
configuration reads, random weights written and read back, and the plain implementation's own mechanisms against
closed forms."""
import copy
import json
import os

import pytest
import torch

import ai_engine_b200 as aie
import plain_fokisun as pf
from ai_engine_b200.config import ConfigError, load_config
from ai_engine_b200.parts.model import tensor_specs_of
from fokisun_helpers import CONFIGS, ids_for, make_dir, read_tensors


def test_every_key_is_read_and_written_back():
    for name, raw in CONFIGS.items():
        arch, cfg = load_config(raw)
        assert arch.name == "Fokisun"
        again = aie.FokisunConfig.from_dict(cfg.to_dict())
        assert again == cfg, name
    cfg = aie.FokisunConfig.from_dict(CONFIGS["A"])
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.residual_mult, cfg.logit_scale) == (211, 96, 1e-4, 0.6, 0.5)
    a, h, l = cfg.layers[0], cfg.layers[1], cfg.layers[2]
    assert (a.type, a.mixer.heads, a.mixer.kv_heads, a.mixer.dim, a.mixer.vdim, a.mixer.window) == ("attention", 6, 2, 16, 24, 37)
    assert (a.mixer.rot_dims, a.mixer.rot_base, a.mixer.rot_factor, a.mixer.v_mix, a.mixer.scale) == (8, 5000.0, 2.0, True, 0.3)
    assert (h.type, h.mixer.heads, h.mixer.dim, h.mixer.vdim) == ("hgrn2", 3, 20, 24)
    assert (h.mlp.kind, h.mlp.ff, h.mlp.experts, h.mlp.top, h.mlp.group_count, h.mlp.group_keep, h.mlp.scale, h.mlp.shared_ff) \
        == ("moe", 40, 6, 2, 3, 2, 1.7, 24)
    assert (l.mixer.rot_dim, l.mixer.kv_rank, l.mixer.q_rank, l.mixer.rot_dims, l.mlp) == (8, 24, 40, 8, None)


def test_absent_keys_mean_none():
    cfg = aie.FokisunConfig.from_dict(CONFIGS["C"])
    assert cfg.residual_mult == 1.0 and cfg.logit_scale == 1.0
    plain = cfg.layers[4].mixer                  # no mask, no rot, no v_mix
    assert (plain.window, plain.rot_dims, plain.rot_factor, plain.v_mix) == (0, 0, 1.0, False)
    assert cfg.layers[0].mlp.group_count == 1 and cfg.layers[0].mlp.shared_ff == 0
    raw = copy.deepcopy(CONFIGS["C"])
    del raw["layers"][1]["mixer"]["kv_heads"]    # as many key/value heads as query heads
    assert aie.FokisunConfig.from_dict(raw).layers[1].mixer.kv_heads == 1


@pytest.mark.parametrize("edit,needle", [
    (lambda r: r.pop("vocab"), "vocab"),
    (lambda r: r["norm"].pop("eps"), "eps"),
    (lambda r: r["layers"][0].__setitem__("type", "conv"), "conv"),
    (lambda r: r["layers"][0]["mixer"].__setitem__("kv_heads", 4), "kv_heads"),
    (lambda r: r["layers"][0]["mixer"]["rot"].__setitem__("dims", 7), "rot.dims"),
    (lambda r: r["layers"][0]["mixer"]["rot"].__setitem__("dims", 18), "rot.dims"),
    (lambda r: r["layers"][1]["mlp"]["router"].__setitem__("top", 5), "choices"),
    (lambda r: r["layers"][1]["mlp"].__setitem__("kind", "sparse"), "sparse"),
    (lambda r: r["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda r: r["layers"][3]["mixer"].__setitem__("vdim", 12), "mix values"),
    (lambda r: r["layers"][4]["mixer"].__setitem__("heads", "four"), "heads"),
])
def test_rejections_name_the_key(edit, needle):
    raw = copy.deepcopy(CONFIGS["A"])
    edit(raw)
    with pytest.raises(ConfigError) as e:
        aie.FokisunConfig.from_dict(raw)
    assert needle in str(e.value), str(e.value)


def test_tensors_of_a_configuration():
    arch, cfg = load_config(CONFIGS["A"])
    specs = {s.name: tuple(s.shape) for s in tensor_specs_of(arch.build_spec(cfg)) if s.stored}
    assert specs["embed"] == (211, 96) and specs["final.norm.alpha"] == () and specs["final.norm.b"] == (96,)
    assert specs["l0.mix.q.norm"] == (96,) and specs["l0.mix.k.norm"] == (32,) and specs["l0.mix.g"] == (144, 96)
    assert specs["l0.mix.vmix"] == () and specs["l0.mix.o.b"] == (96,) and specs["l0.dwa"] == (2,) and specs["l5.dwa"] == (7,)
    assert specs["l1.mix.lower"] == (60,) and specs["l1.mix.f.b"] == (60,) and specs["l1.mix.norm"] == (24,)
    assert specs["l1.mlp.router"] == (6, 96) and specs["l1.mlp.e5.down"] == (96, 40) and specs["l1.mlp.shared.up"] == (24, 96)
    assert specs["l2.mix.dq"] == (40, 96) and specs["l2.mix.uq"] == (100, 40) and specs["l2.mix.dkv"] == (32, 96)
    assert specs["l2.mix.g"] == (5, 96) and specs["l2.mix.uk"] == (60, 24) and specs["l2.mix.uv"] == (100, 24)
    assert "l2.mlp.router" not in specs and "l3.mlp.shared.up" not in specs and "head" not in specs


def test_random_weights_are_written_and_read_back(tmp_path):
    d = make_dir(tmp_path, "D")
    with open(os.path.join(d, "config.json")) as f:
        raw = json.load(f)
    assert raw["architecture"] == "Fokisun" and len(raw["layers"]) == 4
    t = read_tensors(d)
    arch, cfg = load_config(d)
    assert set(t) == {s.name for s in tensor_specs_of(arch.build_spec(cfg)) if s.stored}
    logits, streams = pf.forward(CONFIGS["D"], t, ids_for(12, 97, 3))
    assert logits.shape == (12, 97) and streams.shape == (4, 12, 48) and bool(torch.isfinite(logits).all())


# ---------------------------------------------------------------------------------------------------
def test_plain_rotations_turn_pairs_and_keep_lengths():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(5, 2, 12, generator=g, dtype=torch.float64)
    pos = torch.tensor([0, 1, 7, 100, 1000])
    for fn in (pf.rotate_halves, pf.rotate_interleaved):
        y = fn(x, pos, 100.0, 8, 2.0)
        assert torch.equal(y[0], x[0]) and torch.equal(y[..., 8:], x[..., 8:])
        assert torch.allclose(y[..., :8].norm(dim=-1), x[..., :8].norm(dim=-1))
    # position 1, first pair: the angle is 1 / factor
    c, s = torch.cos(torch.tensor(0.5, dtype=torch.float64)), torch.sin(torch.tensor(0.5, dtype=torch.float64))
    y = pf.rotate_interleaved(x, pos, 100.0, 8, 2.0)
    assert torch.allclose(y[1, :, 0], x[1, :, 0] * c - x[1, :, 1] * s) and torch.allclose(y[1, :, 1], x[1, :, 1] * c + x[1, :, 0] * s)
    y = pf.rotate_halves(x, pos, 100.0, 8, 2.0)
    assert torch.allclose(y[1, :, 0], x[1, :, 0] * c - x[1, :, 4] * s) and torch.allclose(y[1, :, 4], x[1, :, 4] * c + x[1, :, 0] * s)
    # the dot product of two rotated vectors depends on the distance only
    a, b = x[:1].expand(5, 2, 12), x[1:2].expand(5, 2, 12)
    d1 = (pf.rotate_interleaved(a, pos, 100.0, 12) * pf.rotate_interleaved(b, pos - 0, 100.0, 12)).sum(-1)
    assert torch.allclose(d1, (x[0] * x[1]).sum(-1).expand(5, 2))


def test_plain_hgrn2_with_a_constant_gate_is_a_geometric_average():
    H, d, e, D, T = 1, 4, 3, 4, 30
    W = {"q": torch.eye(d, dtype=torch.float64) * 50, "f": torch.zeros(d, D, dtype=torch.float64), "f.b": torch.zeros(d, dtype=torch.float64),
         "lower": torch.full((d,), 0.5, dtype=torch.float64), "v": torch.randn(e, D, dtype=torch.float64),
         "norm": torch.ones(e, dtype=torch.float64), "o": torch.eye(e, dtype=torch.float64)}
    h = torch.randn(T, D, dtype=torch.float64).abs() + 0.5       # silu(50 x) = 50 x for x well above zero
    got = pf.hgrn2(h, W, "", dict(heads=H, dim=d, vdim=e), 0.0)
    f = 0.5 + 0.5 * 0.5                                           # lower + (1 - lower) sigmoid(0)
    v = h @ W["v"].T
    S = torch.zeros(d, e, dtype=torch.float64)
    for t in range(T):
        S = f * S + (1 - f) * v[t][None, :].expand(d, e)
        o = (S * (50 * h[t])[:, None]).sum(0)
        assert torch.allclose(got[t], o / o.pow(2).mean().sqrt(), atol=1e-9)


def test_plain_attention_window_and_sink():
    torch.manual_seed(0)
    D, T = 8, 12
    m = dict(heads=1, kv_heads=1, dim=4, vdim=4, scale=0.0, mask=dict(size=3))
    W = {k: torch.randn(*s, dtype=torch.float64) for k, s in dict(q=(4, D), k=(4, D), v=(4, D), g=(4, D), o=(D, 4)).items()}
    W.update({"q.b": torch.zeros(4, dtype=torch.float64), "k.b": torch.zeros(4, dtype=torch.float64), "v.b": torch.zeros(4, dtype=torch.float64),
              "o.b": torch.zeros(D, dtype=torch.float64), "q.norm": torch.ones(4, dtype=torch.float64), "k.norm": torch.ones(4, dtype=torch.float64)})
    W["g"].zero_()
    W["o"] = torch.eye(D, 4, dtype=torch.float64)
    h = torch.randn(T, D, dtype=torch.float64)
    out, v = pf.attention(h, W, "", m, 1e-6, None)
    # all scores are zero: every visible key weighs 1 / (1 + visible keys); the gate is one half
    for i in range(T):
        seen = list(range(max(0, i - 2), i + 1))
        want = 0.5 * v[seen, 0].sum(0) / (1 + len(seen))
        assert torch.allclose(out[i, :4], want, atol=1e-12)


def test_plain_router_groups_by_the_sum_of_two():
    # scores in two groups of three: the first has the single best score, the second the better pair
    z = torch.tensor([[3.0, -3.0, -3.0, 2.0, 2.0, -3.0]], dtype=torch.float64)
    W = {"router": torch.eye(6, dtype=torch.float64)}
    ids, w = pf.route(z, W, "", dict(experts=6, top=2, scale=2.0, groups=dict(count=2, keep=1)))
    assert sorted(ids[0].tolist()) == [3, 4]
    assert torch.allclose(w, torch.tensor([[1.0, 1.0]], dtype=torch.float64))
    ids, w = pf.route(z, W, "", dict(experts=6, top=2, scale=1.0, groups=dict(count=2, keep=2)))
    assert ids[0, 0] == 0 and ids[0, 1] in (3, 4)
    assert torch.allclose(w.sum(), torch.tensor(1.0, dtype=torch.float64))
