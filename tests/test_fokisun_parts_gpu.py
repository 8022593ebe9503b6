"""Each mechanism of the Fokisun design alone, on a real cache and step context, against the plain implementation:
the norm without statistics, the kernel that joins two branches to the stream and averages over depth, the router,
the experts with their shared one, HGRN2 (odd sizes, portions, long memory, a slot used again), latent attention with
a query latent and head gates, and the normed attention (three requests in unequal portions; keys planted just
inside and just outside the window, at a page's edges and far back, as one prompt, decoded token by token and in
portions of two; the sink; values mixed from another layer)."""
import numpy as np
import pytest
import torch

import plain_fokisun as pf
from fokisun_helpers import DEV, Rig, env, load

pytestmark = pytest.mark.gpu
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def near(got, ref, dtype, what):
    ref = ref.double()
    spread = max(float(ref.std()), 1e-6)
    diff = (got.double() - ref).abs()
    # bfloat16 against the oracle on the same inputs: single elements up to 0.12 of the spread, 0.015 on average
    tol = (2e-4 if dtype == "float32" else 0.12) * spread
    assert float(diff.max()) <= tol, f"{what}: {float(diff.max()):.3e} above {tol:.3e} at row {int(diff.max(dim=-1).values.argmax())}"
    if dtype != "float32":
        assert float(diff.mean()) <= 0.015 * spread, f"{what}: mean difference {float(diff.mean()):.3e}"


def rnd(gen, *shape, std=1.0, mean=0.0):
    return (torch.randn(*shape, generator=gen) * std + mean).to(torch.bfloat16).float()      # exact in both dtypes


def f64(t):
    return {k: v.double() for k, v in t.items()}


# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_norm_without_statistics(dtype):
    from ai_engine_b200.parts import DynamicTanh, PartSpec
    gen = torch.Generator().manual_seed(1)
    for D, T in ((36, 5), (97, 1), (128, 300)):
        t = {"w": rnd(gen, D, std=0.3, mean=1.0), "w.b": rnd(gen, D, std=0.3), "w.alpha": rnd(gen, 1, std=0.1, mean=0.7).reshape(())}
        part = load(DynamicTanh(PartSpec("dynamic_tanh", dict(size=D), dict(weight="w", bias="w.b", alpha="w.alpha")),
                                env(DT[dtype], D)), t, DT[dtype])
        x, delta = rnd(gen, T, D, std=2.0), rnd(gen, 3, T, D)
        ref = pf.dyt(x.double(), t["w"].double(), t["w.b"].double(), t["w.alpha"].double())
        xd = x.to(DEV)
        near(part.forward(xd).cpu(), ref, dtype, "norm of the stream")
        assert torch.equal(xd.cpu(), x)
        # a pending branch in three parts joins the stream first and is stored
        ref2 = pf.dyt((x + delta.sum(0)).double(), t["w"].double(), t["w.b"].double(), t["w.alpha"].double())
        near(part.forward(xd, delta.to(DEV)).cpu(), ref2, dtype, "norm with a pending branch")
        assert float((xd.cpu() - (x + delta.sum(0))).abs().max()) < 1e-5
        rows = torch.tensor([T - 1, 0], dtype=torch.int32, device=DEV)
        near(part.forward(xd, None, rows=rows, write_back=False).cpu(), ref2[[T - 1, 0]], dtype, "norm of chosen rows")


def test_two_branches_join_the_stream_and_the_layers_are_averaged():
    from ai_engine_b200.kernels import ops
    gen = torch.Generator().manual_seed(2)
    T, D, levels = 37, 44, 4
    x0 = rnd(gen, T, D)
    coefs = [rnd(gen, i + 2, std=0.3, mean=0.4) for i in range(levels - 1)]
    w, b, al = rnd(gen, D, mean=1.0, std=0.2), rnd(gen, D, std=0.2), torch.tensor([0.6])
    hist = torch.zeros(levels, T, D, device=DEV)
    hist[0] = x0.to(DEV)
    x, ref_hist, ref_x = x0.to(DEV).clone(), [x0.double()], x0.double()
    for i in range(levels - 1):
        a, bb = rnd(gen, 3, T, D), (rnd(gen, T, D) if i != 1 else None)
        made = ops.parallel_residual(x, a.to(DEV), bb.to(DEV) if bb is not None else None, 0.65, hist, coefs[i].to(DEV),
                                     i + 1, norm_ahead=(w.to(DEV), b.to(DEV), al.to(DEV)), out_dtype=torch.float32)
        X = ref_x + 0.65 * (a.double().sum(0) + (bb.double() if bb is not None else 0))
        ref_hist.append(X)
        ref_x = sum(coefs[i][j].double() * ref_hist[j] for j in range(i + 2))
        assert float((x.cpu().double() - ref_x).abs().max()) < 1e-5
        assert float((made.cpu().double() - pf.dyt(ref_x, w.double(), b.double(), al.double())).abs().max()) < 1e-5
    # without averaging: the sum alone
    y = x0.to(DEV).clone()
    a = rnd(gen, T, D)
    assert ops.parallel_residual(y, a.to(DEV), None, 1.5) is None
    assert float((y.cpu() - (x0 + 1.5 * a)).abs().max()) < 1e-5


@pytest.mark.parametrize("E,count,keep,top", [(8, 4, 2, 3), (6, 3, 2, 2), (4, 4, 2, 2), (5, 1, 1, 3), (1, 1, 1, 1),
                                              (12, 3, 3, 12), (9, 3, 1, 1)])
def test_router_choices_and_weights(E, count, keep, top):
    from ai_engine_b200.kernels import ops
    gen = torch.Generator().manual_seed(E * 100 + count)
    T, D = 200, 24
    h, w = rnd(gen, T, D), rnd(gen, E, D, std=0.4)
    router = dict(experts=E, top=top, scale=1.7, groups=dict(count=count, keep=keep))
    ids, weights = pf.route(h.double(), {"router": w.double()}, "", router)
    z = (h @ w.T).to(DEV).contiguous()
    got_ids, got_w = ops.route_topk(z, None, count, keep, top, score="sigmoid", group_top=2, normalise=True,
                                    weight_scale=1.7)
    order = got_ids.cpu().long().sort(dim=1)
    ref_order = ids.sort(dim=1)
    assert torch.equal(order.values, ref_order.values)
    assert float((got_w.cpu().double().gather(1, order.indices) - weights.gather(1, ref_order.indices)).abs().max()) < 1e-5
    assert float((got_w.sum(dim=1).cpu() - 1.7).abs().max()) < 1e-5


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D,F,E,top,count,keep,Fs,T", [(40, 24, 6, 2, 3, 2, 16, 70), (128, 64, 4, 2, 2, 1, 64, 150),
                                                       (36, 20, 1, 1, 1, 1, 0, 5), (64, 128, 8, 3, 4, 2, 32, 1)])
def test_experts_with_a_shared_one(dtype, D, F, E, top, count, keep, Fs, T):
    from ai_engine_b200.parts import PartSpec, RoutedMoE
    gen = torch.Generator().manual_seed(D + F)
    t = {"router": rnd(gen, E, D, std=0.5)}
    for e in range(E):
        t.update({f"e{e}.gate": rnd(gen, F, D, std=0.2), f"e{e}.up": rnd(gen, F, D, std=0.2), f"e{e}.down": rnd(gen, D, F, std=0.2)})
    if Fs:
        t.update({"shared.gate": rnd(gen, Fs, D, std=0.2), "shared.up": rnd(gen, Fs, D, std=0.2), "shared.down": rnd(gen, D, Fs, std=0.2)})
    part = load(RoutedMoE(PartSpec("routed_moe", dict(
        hidden_size=D, num_experts=E, top=top, intermediate_size=F, groups=count, keep=keep, score="sigmoid", group_top=2,
        normalise=True, route_scale=1.9, shared_intermediate_size=Fs),
        dict(router="router", gate="e{e}.gate", up="e{e}.up", down="e{e}.down", shared_gate="shared.gate",
             shared_up="shared.up", shared_down="shared.down")), env(DT[dtype], D)), t, DT[dtype])
    h = rnd(gen, T, D)
    f = dict(router=dict(experts=E, top=top, scale=1.9, groups=dict(count=count, keep=keep)), shared=dict(ff=Fs) if Fs else None)
    margins = []
    ref = pf.moe_ff(h.double(), f64(t), "", f, margins)
    ctx = type("C", (), {"err": torch.zeros(1, dtype=torch.int32, device=DEV)})()
    out = part.forward(h.to(DEV).to(DT[dtype]), ctx).double().cpu()
    clear = margins[0] > 1e-3                          # a close call may turn either way under rounding
    near(out[clear], ref[clear], dtype, "experts")


# ---------------------------------------------------------------------------------------------------
def hgrn_part(m, hidden, eps, dtype, gen, lower_mean=0.3):
    from ai_engine_b200.parts import ForgetGateLinearAttention, PartSpec
    H, d, e = m["heads"], m["dim"], m["vdim"]
    t = {"q": rnd(gen, H * d, hidden, std=0.3), "f": rnd(gen, H * d, hidden, std=0.3), "f.b": rnd(gen, H * d, std=1.0, mean=1.0),
         "lower": rnd(gen, H * d, std=0.02, mean=lower_mean).clamp(0.0, 0.995), "v": rnd(gen, H * e, hidden, std=0.3),
         "norm": rnd(gen, e, std=0.1, mean=1.0), "o": rnd(gen, hidden, H * e, std=0.2)}
    spec = PartSpec("forget_gate_linear_attention", dict(hidden_size=hidden, num_heads=H, key_dim=d, value_dim=e, eps=eps),
                    dict(q="q", f="f", f_bias="f.b", lower="lower", v="v", norm="norm", o="o"))
    return load(ForgetGateLinearAttention(spec, env(DT[dtype], hidden)), t, DT[dtype]), t


HGRN_SHAPES = [(dict(heads=4, dim=56, vdim=72), 96), (dict(heads=3, dim=20, vdim=24), 40), (dict(heads=1, dim=12, vdim=44), 36),
               (dict(heads=2, dim=128, vdim=128), 64), (dict(heads=5, dim=8, vdim=12), 40), (dict(heads=2, dim=136, vdim=8), 48)]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", range(len(HGRN_SHAPES)))
def test_hgrn2_portions_long_decoding_and_a_slot_used_again(dtype, shape):
    m, hidden = HGRN_SHAPES[shape]
    gen = torch.Generator().manual_seed(80 + shape)
    part, t = hgrn_part(m, hidden, 1e-5, dtype, gen)
    seqs = [rnd(gen, n, hidden) for n in (120, 33, 90)]
    refs = [pf.hgrn2(s.double(), f64(t), "", m, 1e-5) for s in seqs]
    rig = Rig(part, DT[dtype], page=8, pages=8, max_seqs=3)
    cuts = [[50] + [1] * 70, [16, 17], [2, 3, 1, 1, 31, 2, 33, 15, 2]]
    for got, ref, n in zip(rig.run([s.to(DT[dtype]) for s in seqs], cuts), refs, (120, 33, 90)):
        near(got, ref, dtype, f"hgrn2 shape {shape}, request of {n}")
    # the same slots again: their states start from zero
    for got, ref in zip(rig.run([s.to(DT[dtype]) for s in seqs[::-1]], [[90], [2] * 16 + [1], [120]]), refs[::-1]):
        near(got, ref, dtype, f"hgrn2 shape {shape}, slots used again")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_hgrn2_remembers_far_tokens(dtype):
    """A lower bound near one: what the first tokens wrote is still most of the state 250 tokens later, so a state that
    is lost or written twice on the way (between portions, at the single tokens) moves the last rows by the whole output."""
    m, hidden = dict(heads=2, dim=32, vdim=16), 64
    gen = torch.Generator().manual_seed(7)
    part, t = hgrn_part(m, hidden, 1e-5, dtype, gen, lower_mean=0.99)
    h = rnd(gen, 260, hidden)
    h[:6] *= 6.0
    ref = pf.hgrn2(h.double(), f64(t), "", m, 1e-5)
    forgot = pf.hgrn2(h[6:].double(), f64(t), "", m, 1e-5)
    assert float((forgot[-10:] - ref[-10:]).abs().max()) > 0.3 * float(ref.std())
    for cuts in ([260], [100] + [1] * 160, [2] * 130, [17, 16, 15, 64, 65, 83]):
        got = Rig(part, DT[dtype], page=8, pages=8).run([h.to(DT[dtype])], [cuts])[0]
        near(got, ref, dtype, f"hgrn2 far memory, portions {cuts[:2]}")


# ---------------------------------------------------------------------------------------------------
def latent_part(m, hidden, eps, dtype, gen):
    from ai_engine_b200.parts import LatentAttention, PartSpec, RotaryEncoding
    H, d, r, e, rank, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
    t = {"dq": rnd(gen, qr, hidden, std=0.3), "dq.norm": rnd(gen, qr, std=0.1, mean=1.0), "uq": rnd(gen, H * (d + r), qr, std=0.6),
         "dkv": rnd(gen, rank + r, hidden, std=0.3), "dkv.norm": rnd(gen, rank, std=0.1, mean=1.0),
         "uk": rnd(gen, H * d, rank, std=0.3), "uv": rnd(gen, H * e, rank, std=0.3), "g": rnd(gen, H, hidden, std=0.3),
         "o": rnd(gen, hidden, H * e, std=0.2)}
    e_ = env(DT[dtype], hidden)
    rope = RotaryEncoding(PartSpec("rotary", dict(rot_dim=m["rot"]["dims"], theta=m["rot"]["base"], layout="halves")), e_)
    rope.load(None)
    e_.position_encodings["r"] = rope
    spec = PartSpec("latent_attention", dict(hidden_size=hidden, num_heads=H, head_dim=d, rot_dim=r, value_dim=e, kv_rank=rank,
                                             q_rank=qr, scale=m["scale"], window=0, eps=eps, head_gate=True, position_encoding="r"),
                    dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o", g="g"))
    return load(LatentAttention(spec, e_), t, DT[dtype]), t


LATENT_SHAPES = [
    (dict(heads=4, dim=48, rot_dim=16, vdim=40, kv_rank=64, q_rank=72, scale=0.12, rot=dict(base=20000.0, dims=16)), 96),
    (dict(heads=5, dim=12, rot_dim=8, vdim=20, kv_rank=24, q_rank=40, scale=0.22, rot=dict(base=3000.0, dims=8)), 40),
    (dict(heads=1, dim=8, rot_dim=2, vdim=12, kv_rank=6, q_rank=10, scale=0.3, rot=dict(base=10000.0, dims=2)), 36),
    (dict(heads=2, dim=64, rot_dim=32, vdim=64, kv_rank=128, q_rank=64, scale=0.04, rot=dict(base=100.0, dims=32)), 128),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", range(len(LATENT_SHAPES)))
def test_latent_attention_three_requests_in_unequal_portions(dtype, shape):
    m, hidden = LATENT_SHAPES[shape]
    gen = torch.Generator().manual_seed(30 + shape)
    part, t = latent_part(m, hidden, 1e-5, dtype, gen)
    seqs = [rnd(gen, n, hidden) for n in (300, 41, 150)]
    refs = [pf.latent_attention(s.double(), f64(t), "", m, 1e-5) for s in seqs]
    rig = Rig(part, DT[dtype], page=8, pages=128)
    cuts = [[129, 2, 127, 1, 1, 40], [1, 2, 3, 35], [64, 1, 1, 1, 1, 1, 1, 80]]
    for got, ref, n in zip(rig.run([s.to(DT[dtype]) for s in seqs], cuts), refs, (300, 41, 150)):
        near(got, ref, dtype, f"latent attention shape {shape}, request of {n}")
    for got, ref in zip(rig.run([s.to(DT[dtype]) for s in seqs[:2]], [[300], [41]]), refs):
        near(got, ref, dtype, f"latent attention shape {shape}, pages used again")
    rig.cache.book.check_invariants()


# ---------------------------------------------------------------------------------------------------
def attention_part(m, hidden, eps, dtype, gen, tie_keys=False, value_mix=None):
    from ai_engine_b200.parts import NormedGatedAttention, PartSpec, RotaryEncoding
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    t = {"q": rnd(gen, H * d, hidden, std=0.25), "k": rnd(gen, G * d, hidden, std=0.25), "v": rnd(gen, G * e, hidden, std=0.25),
         "q.b": rnd(gen, H * d, std=0.2), "k.b": rnd(gen, G * d, std=0.2), "v.b": rnd(gen, G * e, std=0.2),
         "q.norm": rnd(gen, H * d, std=0.2, mean=3.0), "k.norm": rnd(gen, G * d, std=0.2, mean=1.0),
         "g": rnd(gen, H * e, hidden, std=0.3), "o": rnd(gen, hidden, H * e, std=0.2), "o.b": rnd(gen, hidden, std=0.2)}
    if value_mix:
        t["vmix"] = torch.tensor(0.35)
    if tie_keys:                    # k reads the second half of the input as q reads the first: q_i . k_j is large
        t["k"] = torch.roll(t["q"][:G * d], hidden // 2, dims=1).contiguous()      # when h_j is h_i moved by half the width
        t["q.b"].zero_()
        t["k.b"].zero_()
        t["q.norm"].fill_(3.0)
        t["k.norm"].fill_(1.0)
    e_ = env(DT[dtype], hidden)
    pe = None
    if m.get("rot"):
        sc = (m["rot"].get("scaling") or {}).get("factor")
        rope = RotaryEncoding(PartSpec("rotary", dict(rot_dim=m["rot"]["dims"], theta=m["rot"]["base"], layout="interleaved",
                                                      scaling=dict(type="linear", factor=sc) if sc else None)), e_)
        rope.load(None)
        e_.position_encodings["r"] = rope
        pe = "r"
    spec = PartSpec("normed_gated_attention", dict(
        hidden_size=hidden, num_heads=H, num_kv_heads=G, head_dim=d, value_dim=e, scale=m["scale"],
        window=(m.get("mask") or {}).get("size", 0), eps=eps, sink=0.0, position_encoding=pe, value_mix=value_mix),
        dict(q="q", k="k", v="v", g="g", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", o_bias="o.b", q_norm="q.norm",
             k_norm="k.norm", **{"lambda": "vmix"}))
    return load(NormedGatedAttention(spec, e_), t, DT[dtype]), t


def rot(base, dims, factor=None):
    r = dict(base=base, dims=dims)
    if factor:
        r["scaling"] = dict(factor=factor)
    return r


SHAPES = [
    (dict(heads=8, kv_heads=2, dim=64, vdim=40, scale=0.11, mask=dict(size=100), rot=rot(30000.0, 48, 3.0)), 96),
    (dict(heads=6, kv_heads=2, dim=16, vdim=24, scale=0.3, mask=dict(size=37), rot=rot(5000.0, 8, 2.0)), 96),
    (dict(heads=4, kv_heads=1, dim=64, vdim=32, scale=0.2, mask=dict(size=130), rot=rot(10000.0, 64)), 128),
    (dict(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09, rot=rot(100.0, 32)), 64),
    (dict(heads=1, kv_heads=1, dim=12, vdim=44, scale=0.4, mask=dict(size=2)), 36),
    (dict(heads=4, kv_heads=2, dim=64, vdim=128, scale=0.15, mask=dict(size=64), rot=rot(777.0, 2)), 64),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", range(len(SHAPES)))
def test_attention_three_requests_in_unequal_portions(dtype, shape):
    m, hidden = SHAPES[shape]
    gen = torch.Generator().manual_seed(10 + shape)
    part, t = attention_part(m, hidden, 1e-5, dtype, gen)
    seqs = [rnd(gen, n, hidden) for n in (300, 41, 150)]
    refs = [pf.attention(s.double(), f64(t), "", m, 1e-5, None)[0] for s in seqs]
    rig = Rig(part, DT[dtype], page=8, pages=128)
    cuts = [[129, 2, 127, 1, 1, 40], [1, 2, 3, 35], [64, 1, 1, 1, 1, 1, 1, 80]]
    for got, ref, n in zip(rig.run([s.to(DT[dtype]) for s in seqs], cuts), refs, (300, 41, 150)):
        near(got, ref, dtype, f"attention shape {shape}, request of {n}")
    # once more on the pages and slots the first three gave back
    for got, ref in zip(rig.run([s.to(DT[dtype]) for s in seqs[:2]], [[300], [41]]), refs):
        near(got, ref, dtype, f"attention shape {shape}, pages used again")
    rig.cache.book.check_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("sizes", [(32, 16), (32, 64)])        # the second pair takes the tensor-core kernels in bfloat16
@pytest.mark.parametrize("window,page", [(40, 8), (90, 16), (130, 32), (0, 8)])
def test_attention_planted_keys_at_every_edge(dtype, window, page, sizes):
    """Pairs of tokens with a strong input that the later one's query and the earlier one's key read alike, so that
    the later one's weight goes to the earlier one when it reads it: just inside the window and just outside, at a
    page's first and last place, and 250 tokens back.  A window one key off or a lost page moves those rows by the
    whole output; a sink that is left out moves every row."""
    hidden, n = 128, 300
    m = dict(heads=4, kv_heads=4, dim=sizes[0], vdim=sizes[1], scale=0.25)
    if window:
        m["mask"] = dict(size=window)
    gen = torch.Generator().manual_seed(50 + window)
    part, t = attention_part(m, hidden, 1e-5, dtype, gen, tie_keys=True)
    h = rnd(gen, n, hidden, std=0.3)
    w = window or 10 ** 6
    pairs = [(200, 200 - w + 1), (210, 210 - w), (180 + page, 180 + page - w + 1),        # the window's two sides
             (299, 49), (290, 5 * page), (280, 5 * page - 1), (270, 0)]                    # far back; a page's edges
    pairs = [(i, j) for i, j in pairs if 0 <= j < i]
    for p, (i, j) in enumerate(pairs):
        h[i, 5 * p:5 * p + 5] = 8.0
        h[j, hidden // 2 + 5 * p:hidden // 2 + 5 * p + 5] = 8.0
    tw = f64(t)
    ref = pf.attention(h.double(), tw, "", m, 1e-5, None)[0]
    if window:           # the planted rows do tell a window that is one key longer or shorter
        for other in (window + 1, window - 1):
            alt = pf.attention(h.double(), tw, "", dict(m, mask=dict(size=other)), 1e-5, None)[0]
            assert float((alt - ref).abs().max()) > 0.3 * float(ref.std())
    first = min(j for _, j in pairs)
    for cuts in ([n], [150] + [1] * 150, [2] * 150, [max(first, 1)] + [1] * (n - max(first, 1))):
        rig = Rig(part, DT[dtype], page=page, pages=max(16, 2 * n // page))
        got = rig.run([h.to(DT[dtype])], [cuts])[0]
        near(got, ref, dtype, f"planted keys, window {window}, portions {cuts[:2]}")


def test_the_sink_takes_its_share_at_the_first_tokens():
    """With one key the softmax alone would give the weight 1; the sink of score 0 leaves exp(s) / (1 + exp(s))."""
    m, hidden = dict(heads=2, kv_heads=1, dim=16, vdim=8, scale=0.2), 32
    gen = torch.Generator().manual_seed(5)
    part, t = attention_part(m, hidden, 1e-5, "float32", gen)
    h = rnd(gen, 3, hidden)
    ref = pf.attention(h.double(), f64(t), "", m, 1e-5, None)[0]
    got = Rig(part, torch.float32, page=8, pages=8).run([h], [[1, 1, 1]])[0]
    near(got, ref, "float32", "the first tokens one by one")
    # the oracle without a sink differs at the very first token
    T = 1
    q = pf.rms(h[:T].double() @ t["q"].double().T + t["q.b"].double(), t["q.norm"].double(), 1e-5)
    assert q.abs().max() > 0
    v = (h[:1].double() @ t["v"].double().T + t["v.b"].double()).view(1, 1, 8).repeat_interleave(2, dim=1).reshape(1, 16)
    no_sink = (v * torch.sigmoid(h[:1].double() @ t["g"].double().T)) @ t["o"].double().T + t["o.b"].double()
    assert float((no_sink - ref[:1]).abs().max()) > 0.05 * float(ref.std())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_values_mixed_with_another_layers(dtype):
    """The prepare kernel alone: v <- (1 - lambda) v + lambda v_src goes into the cache row and comes back as the
    values to keep; keys are normed over the whole projection and rotated in neighbouring pairs."""
    from ai_engine_b200.kernels import ops
    gen = torch.Generator().manual_seed(6)
    m, hidden = dict(heads=4, kv_heads=2, dim=20, vdim=12, scale=0.2, rot=rot(300.0, 12, 1.5), v_mix=True), 48
    part, t = attention_part(m, hidden, 1e-5, dtype, gen, value_mix="source")
    rig = Rig(part, DT[dtype], page=8, pages=16)
    slot = rig.admit()
    T = 21
    ctx, lc = rig.step([(slot, T)])
    H, G, d, e = 4, 2, 20, 12
    proj = rnd(gen, T, H * d + G * (d + e) + 5)
    src = rnd(gen, T, G * e)
    lam = torch.tensor([0.35], device=DEV)
    q, kept = ops.normed_attn_prepare(proj.to(DEV), part.bias, part.q_w, part.k_w, 1e-5, part.rope.inv_freq, 12, False,
                                      lc.k_pages, ctx, lc.block_table, H, G, d, e, mix_from=src.to(DEV), mix_lambda=lam,
                                      keep_values=True)
    pos = torch.arange(T)
    pd = proj.double()
    bias = part.bias.cpu().double()
    k = pf.rms(pd[:, H * d:H * d + G * d] + bias[H * d:H * d + G * d], t["k.norm"].double(), 1e-5).view(T, G, d)
    k = pf.rotate_interleaved(k, pos, 300.0, 12, 1.5)
    v = pd[:, H * d + G * d:H * d + G * (d + e)] + bias[H * d + G * d:]
    v = 0.65 * v + 0.35 * src.double()
    tol = 1e-5 if dtype == "float32" else 2e-2
    assert float((kept.cpu().double() - v).abs().max()) < 1e-5
    rows = lc.k_pages[lc.block_table[0, :3].long()].permute(1, 0, 2, 3).reshape(G, 24, d + e)[:, :T].cpu().double()
    assert float((rows[..., :d] - k.transpose(0, 1)).abs().max()) < tol * max(1.0, float(k.abs().max()))
    assert float((rows[..., d:] - v.view(T, G, e).transpose(0, 1)).abs().max()) < tol * max(1.0, float(v.abs().max()))
    qr = pf.rotate_interleaved(pf.rms(pd[:, :H * d] + bias[:H * d], t["q.norm"].double(), 1e-5).view(T, H, d), pos, 300.0, 12, 1.5)
    assert float((q.cpu().double() - qr).abs().max()) < tol * max(1.0, float(qr.abs().max()))
