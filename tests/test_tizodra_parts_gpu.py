"""Each mechanism of the Tizodra design alone, on a real cache and step context, against the plain implementation:
position vectors, the feed-forward without a gate, scaled logits, the attention (three requests in unequal portions;
keys planted just inside and just outside the window, among the kept first tokens and right behind them, as one
prompt, decoded token by token and in portions of two), the delta rule (odd sizes, portions, long decoding, a slot
used again)."""
import numpy as np
import pytest
import torch

import plain_tizodra as pt
from tizodra_helpers import DEV, Rig, env, load

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


# ---------------------------------------------------------------------------------------------------
def test_position_vectors():
    from ai_engine_b200.kernels import ops
    from ai_engine_b200.parts import PartSpec, SinusoidalPositions
    for width in (8, 36, 97):
        part = SinusoidalPositions(PartSpec("sinusoidal", dict(size=width)), env(torch.float32, width))
        part.load(None)
        pos = torch.tensor([0, 1, 2, 17, 255, 256, 1999], dtype=torch.int32, device=DEV)
        x = torch.zeros(pos.shape[0], width, device=DEV)
        ops.add_sinusoid(x, pos, part.freq)
        ref = pt.sinusoid(pos.cpu(), width)
        assert float((x.cpu().double() - ref).abs().max()) < 3e-4
        ops.add_sinusoid(x, pos, part.freq)              # it adds
        assert float((x.cpu().double() - 2 * ref).abs().max()) < 6e-4


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_feed_forward_without_a_gate(dtype):
    from ai_engine_b200.parts import DenseFF, PartSpec
    gen = torch.Generator().manual_seed(3)
    acts = {"relu_squared": pt.relu_squared, "relu": torch.relu, "silu": pt.silu,
            "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}
    for (D, F, T), (name, act) in zip(((40, 56, 5), (128, 256, 70), (36, 52, 1), (64, 24, 9)), acts.items()):
        t = {"up": rnd(gen, F, D, std=0.2), "down": rnd(gen, D, F, std=0.2)}
        part = load(DenseFF(PartSpec("dense_ff", dict(hidden_size=D, intermediate_size=F, activation=name),
                                     dict(up="up", down="down")), env(DT[dtype], D)), t, DT[dtype])
        h = rnd(gen, T, D)
        err = torch.zeros(1, dtype=torch.int32, device=DEV)
        ctx = type("C", (), {"err": err})()
        out = part.forward(h.to(DEV).to(DT[dtype]), ctx).double()
        out = (out.sum(0) if out.dim() == 3 else out).cpu()
        near(out, act(h.double() @ t["up"].double().T) @ t["down"].double().T, dtype, f"feed-forward {name}")


def test_scaled_logits():
    from ai_engine_b200.parts import LMHead, PartSpec
    gen = torch.Generator().manual_seed(4)
    t = {"head": rnd(gen, 50, 24)}
    for scale in (None, 1.0, 0.25, 3.0):
        part = load(LMHead(PartSpec("lm_head", dict(vocab_size=50, hidden_size=24, scale=scale), dict(weight="head")),
                           env(torch.float32, 24)), t, torch.float32)
        h = rnd(gen, 3, 24)
        out = part.forward(h.to(DEV)).cpu().double()
        assert torch.allclose(out, (h.double() @ t["head"].double().T) * (scale or 1.0), atol=1e-5)


# ---------------------------------------------------------------------------------------------------
def attention_part(m, hidden, eps, dtype, gen, tie_keys=False):
    from ai_engine_b200.parts import PartSpec, SinkWindowAttention
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    mask = m.get("mask") or {}
    t = {"q": rnd(gen, H * d, hidden, std=0.25), "k": rnd(gen, G * d, hidden, std=0.25), "v": rnd(gen, G * e, hidden, std=0.25),
         "q.b": rnd(gen, H * d, std=0.2), "k.b": rnd(gen, G * d, std=0.2), "v.b": rnd(gen, G * e, std=0.2),
         "temp": rnd(gen, H, std=0.2, mean=1.0), "sink": rnd(gen, H, std=1.0), "g": rnd(gen, H, hidden, std=0.3),
         "o": rnd(gen, hidden, H * e, std=0.2)}
    if tie_keys:                    # k reads the second half of the input as q reads the first: q_i . k_j is large
        t["k"] = torch.roll(t["q"], hidden // 2, dims=1).contiguous()        # when h_j is h_i moved by half the width
        t["q.b"].zero_()
        t["k.b"].zero_()
    spec = PartSpec("sink_window_attention", dict(
        hidden_size=hidden, num_heads=H, num_kv_heads=G, head_dim=d, value_dim=e, scale=m["scale"],
        window=mask.get("size", 0), keep_first=mask.get("keep_first", 0), eps=eps, slope_bits=8.0),
        dict(q="q", k="k", v="v", o="o", q_bias="q.b", k_bias="k.b", v_bias="v.b", temp="temp", sink="sink", g="g"))
    return load(SinkWindowAttention(spec, env(DT[dtype], hidden)), t, DT[dtype]), t


SHAPES = [
    (dict(heads=6, kv_heads=2, dim=16, vdim=24, scale=0.3, mask=dict(size=37, keep_first=3)), 96),
    (dict(heads=4, kv_heads=1, dim=64, vdim=32, scale=0.2, mask=dict(size=130, keep_first=17)), 128),
    (dict(heads=2, kv_heads=2, dim=128, vdim=128, scale=0.09), 64),
    (dict(heads=1, kv_heads=1, dim=12, vdim=44, scale=0.4, mask=dict(size=2, keep_first=1)), 36),
    (dict(heads=4, kv_heads=2, dim=64, vdim=128, scale=0.15, mask=dict(size=64, keep_first=64)), 64),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", range(len(SHAPES)))
def test_attention_three_requests_in_unequal_portions(dtype, shape):
    m, hidden = SHAPES[shape]
    gen = torch.Generator().manual_seed(10 + shape)
    part, t = attention_part(m, hidden, 1e-5, dtype, gen)
    seqs = [rnd(gen, n, hidden) for n in (300, 41, 150)]
    refs = [pt.sink_attention(s.double(), {k: v.double() for k, v in t.items()}, m, 1e-5) for s in seqs]
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
@pytest.mark.parametrize("window,keep,page", [(40, 3, 8), (96, 8, 16), (130, 1, 32), (0, 0, 8)])
def test_attention_planted_keys_at_every_edge(dtype, window, keep, page, sizes):
    """Pairs of tokens with a strong input that the later one's query and the earlier one's key read alike, so that
    the later one's weight goes to the earlier one when it reads it: just inside the window and just outside, the last kept token and the first one behind the kept run, at
    a page's first and last place, and 250 tokens back.  A window one key off, a lost page or a kept token that is
    not read moves those rows by the whole output."""
    hidden, n = 128, 300
    m = dict(heads=4, kv_heads=4, dim=sizes[0], vdim=sizes[1], scale=0.05)
    if window:
        m["mask"] = dict(size=window, keep_first=keep)
    gen = torch.Generator().manual_seed(50 + window)
    part, t = attention_part(m, hidden, 1e-5, dtype, gen, tie_keys=True)
    h = rnd(gen, n, hidden, std=0.3)
    w = window or 10 ** 6
    pairs = [(200, 200 - w + 1), (210, 210 - w), (180 + page, 180 + page - w + 1),        # the window's two sides
             (250, keep - 1), (260, keep), (270, 0),                                        # the kept run's two sides
             (299, 49), (290, 5 * page), (280, 5 * page - 1)]                               # far back; a page's edges
    pairs = [(i, j) for i, j in pairs if 0 <= j < i]
    for p, (i, j) in enumerate(pairs):
        h[i, 5 * p:5 * p + 5] = 8.0
        h[j, hidden // 2 + 5 * p:hidden // 2 + 5 * p + 5] = 8.0
    tw = {k: v.double() for k, v in t.items()}
    ref = pt.sink_attention(h.double(), tw, m, 1e-5)
    if window:           # the planted rows do tell a window that is one key longer or shorter, or one more kept token
        for other in (dict(size=window + 1, keep_first=keep), dict(size=window - 1, keep_first=keep),
                      dict(size=window, keep_first=keep + 1)):
            alt = pt.sink_attention(h.double(), tw, dict(m, mask=other), 1e-5)
            assert float((alt - ref).abs().max()) > 0.3 * float(ref.std())
    first = min(j for _, j in pairs)
    for cuts in ([n], [150] + [1] * 150, [2] * 150, [max(first, 1)] + [1] * (n - max(first, 1))):
        rig = Rig(part, DT[dtype], page=page, pages=max(16, 2 * n // page))
        got = rig.run([h.to(DT[dtype])], [cuts])[0]
        near(got, ref, dtype, f"planted keys, window {window}, portions {cuts[:2]}")


# ---------------------------------------------------------------------------------------------------
def delta_part(m, hidden, eps, dtype, gen):
    from ai_engine_b200.parts import GatedDeltaRule, PartSpec
    H, G, d, e, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    t = {"q": rnd(gen, G * d, hidden, std=0.3), "k": rnd(gen, G * d, hidden, std=0.3), "v": rnd(gen, H * e, hidden, std=0.3),
         "g": rnd(gen, H * e, hidden, std=0.3), "b": rnd(gen, H, hidden, std=0.3), "a": rnd(gen, H, hidden, std=0.3),
         "q.conv": rnd(gen, G * d, taps, std=0.5), "k.conv": rnd(gen, G * d, taps, std=0.5),
         "v.conv": rnd(gen, H * e, taps, std=0.5), "A_log": rnd(gen, H, std=0.5, mean=-1.0),
         "dt_bias": rnd(gen, H, std=0.5, mean=-1.0), "norm": rnd(gen, e, std=0.1, mean=1.0),
         "o": rnd(gen, hidden, H * e, std=0.2)}
    spec = PartSpec("gated_delta_rule", dict(hidden_size=hidden, num_heads=H, num_qk_heads=G, key_dim=d, value_dim=e,
                                             taps=taps, eps=eps),
                    dict(q="q", k="k", v="v", g="g", b="b", a="a", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv",
                         a_log="A_log", dt_bias="dt_bias", norm="norm", o="o"))
    return load(GatedDeltaRule(spec, env(DT[dtype], hidden)), t, DT[dtype]), t


DELTA_SHAPES = [
    (dict(heads=4, kv_heads=2, dim=24, vdim=20, conv=4), 96),
    (dict(heads=2, kv_heads=1, dim=64, vdim=64, conv=3), 128),
    (dict(heads=1, kv_heads=1, dim=12, vdim=36, conv=1), 36),
    (dict(heads=5, kv_heads=1, dim=8, vdim=12, conv=5), 40),
    (dict(heads=3, kv_heads=3, dim=130, vdim=8, conv=2), 48),
    (dict(heads=2, kv_heads=2, dim=128, vdim=72, conv=2), 64),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", range(len(DELTA_SHAPES)))
def test_delta_rule_portions_long_decoding_and_a_slot_used_again(dtype, shape):
    m, hidden = DELTA_SHAPES[shape]
    gen = torch.Generator().manual_seed(80 + shape)
    part, t = delta_part(m, hidden, 1e-5, dtype, gen)
    seqs = [rnd(gen, n, hidden) for n in (120, 33, 90)]
    tw = {k: v.double() for k, v in t.items()}
    refs = [pt.delta_mixer(s.double(), tw, m, 1e-5) for s in seqs]
    rig = Rig(part, DT[dtype], page=8, pages=8, max_seqs=3)
    cuts = [[50] + [1] * 70, [16, 17], [2, 3, 1, 1, 31, 2, 33, 15, 2]]
    for got, ref, n in zip(rig.run([s.to(DT[dtype]) for s in seqs], cuts), refs, (120, 33, 90)):
        near(got, ref, dtype, f"delta rule shape {shape}, request of {n}")
    # the same slots again: their states and tails start from zero
    for got, ref in zip(rig.run([s.to(DT[dtype]) for s in seqs[::-1]], [[90], [2] * 16 + [1], [120]]), refs[::-1]):
        near(got, ref, dtype, f"delta rule shape {shape}, slots used again")


def test_delta_rule_state_against_the_oracle():
    """The state the kernel leaves in the slot is the oracle's S after the last token."""
    m, hidden = DELTA_SHAPES[0]
    gen = torch.Generator().manual_seed(99)
    part, t = delta_part(m, hidden, 1e-5, "float32", gen)
    h = rnd(gen, 37, hidden)
    keep = []
    pt.delta_mixer(h.double(), {k: v.double() for k, v in t.items()}, m, 1e-5, keep_states=keep)
    rig = Rig(part, torch.float32, page=8, pages=8)
    slot = rig.admit()
    for n in (20, 1, 16):
        ctx, lc = rig.step([(slot, n)])
        part.forward(h[rig.have[slot]:rig.have[slot] + n].to(DEV), ctx, lc)
        rig.done([(slot, n)])
    S = lc.state["S"][slot].double().cpu()
    for a in range(m["heads"]):
        assert float((S[a] - keep[a]).abs().max()) < 1e-5


# heads and sizes that between them reach every pair of (padded rows of the state, value columns a CTA) the launcher picks
@pytest.mark.parametrize("sizes", [(4, 2, 24, 20), (2, 1, 64, 64), (2, 2, 128, 72), (3, 1, 40, 100), (1, 1, 32, 32),
                                   (148, 4, 16, 40), (40, 4, 64, 64), (20, 5, 128, 64), (20, 2, 48, 64), (20, 20, 20, 64),
                                   (2, 1, 126, 30)])
def test_delta_rule_in_chunks_against_token_by_token(sizes):
    """The chunked kernel and the token-by-token kernel on the same float32 inputs, from the same non-zero state,
    agree to float32 rounding times the chunk's length: a portion of several chunks with a ragged end, a portion of
    one short chunk, and beside them a single token and a portion too short for chunks, all in one step.  Decays
    from near one to strong, corrections from weak to full."""
    from ai_engine_b200.kernels import ops
    H, G, d, e = sizes
    gen = torch.Generator().manual_seed(H * 1000 + d)
    part, _ = delta_part(dict(heads=H, kv_heads=G, dim=d, vdim=e, conv=2), 16, 1e-5, "bfloat16", gen)
    rig = Rig(part, torch.bfloat16, page=8, pages=64, max_seqs=4)
    lens = [150, 1, 40, 31] if H < 100 else [70, 1]
    slots = [rig.admit() for _ in lens]
    portions = list(zip(slots, lens))
    ctx, lc = rig.step(portions)
    T = sum(lens)
    qkv = (torch.randn(T, 2 * G * d + H * e, generator=gen) * 1.5).to(DEV)
    b_raw = (torch.randn(T, H, generator=gen) * 2.0).to(DEV)
    a_raw = (torch.randn(T, H, generator=gen) * 3.0).to(DEV)
    a_log = (torch.randn(H, generator=gen) * 0.7 - 0.5).to(DEV)
    dt_bias = (torch.randn(H, generator=gen) * 0.5 - 1.0).to(DEV)
    S0 = (torch.randn(lc.state["S"].shape, generator=gen) * 0.5).to(DEV)
    res = []
    for chunked in (False, True):
        S = S0.clone()
        o = ops.delta_rule(qkv[:, :G * d], qkv[:, G * d:2 * G * d], qkv[:, 2 * G * d:], b_raw, a_raw, a_log, dt_bias,
                           d ** -0.5, 1e-6, S, ctx, H, G, d, e, chunked=chunked)
        torch.cuda.synchronize()
        res.append((o.double().cpu(), S.double().cpu()))
    assert int(rig.err.item()) == 0
    (o0, s0), (o1, s1) = res
    for what, a, b in (("output", o0, o1), ("state", s0, s1)):
        spread = float(a.std())
        diff = (a - b).abs()
        assert float(diff.max()) <= 3e-4 * spread, f"{what} {sizes}: {float(diff.max()):.3e} of spread {spread:.3e} at {int(diff.flatten().argmax())}"
    assert float((s1 - S0.double().cpu()).abs().max()) > 1e-3       # the states did move


@pytest.mark.parametrize("chunked", [False, True])
def test_delta_rule_recalls_a_pair_written_hundreds_of_tokens_back(chunked):
    """Closed form: with decays of one and full write strength, a value written along a key that no later key
    touches is read back whole by a query along that key, 285 tokens and several chunks later and across two steps;
    a query orthogonal to every key reads nothing.  A state that is lost between chunks or steps, or decayed once
    too often, shows at once."""
    from ai_engine_b200.kernels import ops
    H, G, d, e, T, at, ask = 2, 1, 64, 48, 300, 5, 290
    gen = torch.Generator().manual_seed(7)
    part, _ = delta_part(dict(heads=H, kv_heads=G, dim=d, vdim=e, conv=2), 16, 1e-5, "bfloat16", gen)
    rig = Rig(part, torch.bfloat16, page=8, pages=64, max_seqs=2)
    star = torch.zeros(d)
    star[3] = 1.0
    spare = torch.zeros(d)
    spare[4] = 1.0
    k = torch.randn(T, d, generator=gen)
    k[:, 3] = 0.0                                        # no other key has a share along the planted one
    k[:, 4] = 0.0                                        # ... nor along the spare direction
    k[at] = star * 3.0                                   # any length: the kernel makes it a unit vector
    q = torch.randn(T, d, generator=gen)
    q[ask] = star * 0.5
    q[ask + 1] = spare
    v = torch.randn(T, H * e, generator=gen)
    qkv = torch.cat([q, k, v], dim=1).to(DEV)
    b_raw = torch.full((T, H), 30.0, device=DEV)         # beta = 1
    a_raw = torch.full((T, H), -60.0, device=DEV)        # softplus = 0: no decay
    a_log, dt_bias = torch.zeros(H, device=DEV), torch.zeros(H, device=DEV)
    slot = rig.admit()
    outs = []
    for n0, n in ((0, 100), (100, 200)):
        ctx, lc = rig.step([(slot, n)])
        rows = qkv[n0:n0 + n]
        outs.append(ops.delta_rule(rows[:, :d], rows[:, d:2 * d], rows[:, 2 * d:], b_raw[n0:n0 + n], a_raw[n0:n0 + n],
                                   a_log, dt_bias, d ** -0.5, 1e-6, lc.state["S"], ctx, H, G, d, e, chunked=chunked))
        rig.done([(slot, n)])
    o = torch.cat(outs).cpu().double().reshape(T, H * e)
    want = v[at].double() * d ** -0.5
    assert float((o[ask] - want).abs().max()) < 2e-4 * float(want.abs().max())
    assert float(o[ask + 1].abs().max()) < 2e-4 * float(want.abs().max())
