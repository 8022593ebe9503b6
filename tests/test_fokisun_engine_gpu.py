"""Fokisun models through the engine's own loader, step function, cache and scheduler against the plain
implementation: whole prompts, prompts then tokens one by one, portions down to two tokens, mixed batches on a pool
so small that pages and slots are used again, long decoding behind windows, greedy generation through
Engine.generate, and the trace program.  In float32 (against the float64 oracle) and bfloat16 (against the float32
oracle on the same weights), at four small configurations that differ in every size, and at configurations drawn at
random."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_fokisun as pf
from fokisun_helpers import (CONFIGS, attn, close, dense, hgrn, ids_for, latent, layer, make_dir, moe, oracle_dtype,
                             plain_logits, read_tensors)
from test_zupitar_engine_gpu import feed, mixed_schedule, replayer

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CASES = [(n, d) for n in ("A", "B", "C", "D") for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_prompts_and_the_first_tokens(tmp_path, name, dtype):
    d = make_dir(tmp_path, name)
    vocab = CONFIGS[name]["vocab"]
    rep = replayer(d, dtype, 320)
    for n, seed in ((1, 1), (2, 2), (3, 3), (29, 4), (131, 5), (290, 6)):
        ids = ids_for(n, vocab, seed)
        close(feed(rep, f"w{n}", ids, [n]), plain_logits(d, name, ids, oracle_dtype(dtype)), dtype, f"{name} whole {n}")
    rep.cache.book.check_invariants()


@pytest.mark.parametrize("name", ["A", "D"])
def test_the_residual_stream_behind_every_layer(tmp_path, name):
    """Layer by layer: the float32 engine's stream behind every layer against the oracle's."""
    from ai_engine_b200.engine.step import StepContext, StepEntry
    d = make_dir(tmp_path, name)
    ids = ids_for(45, CONFIGS[name]["vocab"], 8)
    rep = replayer(d, "float32", 64)
    slot = rep.cache.admit()
    assert rep.cache.ensure(slot, len(ids))
    ctx = StepContext([StepEntry(slot, 0, ids, [])], rep.cache, rep.model.device, rep.runner.err,
                      planners=rep.runner.planners)
    got = []
    rep.model.forward(ctx, rep.cache, streams=got)
    ref = pf.forward(CONFIGS[name], read_tensors(d), ids)[1]
    assert len(got) == len(ref) == len(CONFIGS[name]["layers"])
    for i, (g, r) in enumerate(zip(got, ref)):
        err = float((g.double().cpu() - r).abs().max())
        assert err <= 2e-5 * float(r.abs().max()), (i, err)


@pytest.mark.parametrize("name,dtype", CASES)
def test_a_prompt_then_its_tokens_one_by_one(tmp_path, name, dtype):
    """Prefill against token-by-token decoding: 40 tokens at once, then 140 single tokens (bfloat16: replayed from a
    captured graph from the second on), which carries every state through its updates, walks every window over
    decoded tokens and the attention over page borders; then 150 single tokens from an empty state."""
    d = make_dir(tmp_path, name)
    ids = ids_for(180, CONFIGS[name]["vocab"], 11)
    rep = replayer(d, dtype, 192)
    ref = plain_logits(d, name, ids, oracle_dtype(dtype))
    close(feed(rep, "a", ids, [40] + [1] * 140), ref, dtype, f"{name} prompt then single tokens")
    close(feed(rep, "b", ids[:150], [1] * 150), ref[:150], dtype, f"{name} single tokens from the start")


@pytest.mark.parametrize("name,dtype", CASES)
def test_portions_of_several_sizes(tmp_path, name, dtype):
    d = make_dir(tmp_path, name)
    ids = ids_for(280, CONFIGS[name]["vocab"], 12)
    ref = plain_logits(d, name, ids, oracle_dtype(dtype))
    rep = replayer(d, dtype, 320)
    # 128 / 129 / 127: the edges of the attention kernels' query tiles; 16 / 17: of the recurrence's staged tokens;
    # 64 / 65: where the products change kernels
    for cuts in ([2] * 140, [7, 2, 3, 64, 2, 9, 1, 1, 17, 2, 33, 9, 128, 2], [129, 2, 127, 22], [3] * 93 + [1],
                 [16, 17, 15, 65, 65, 102]):
        close(feed(rep, "p", ids, cuts), ref, dtype, f"{name} portions {cuts[:4]}")
    if dtype == "float32":       # one schedule against another of the same engine: far closer than to the oracle
        a, b = feed(rep, "p", ids, [280]), feed(rep, "p", ids, [2] * 140)
        assert np.abs(a - b).max() <= 5e-5 * max(1.0, np.abs(a).max())


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_batches_with_pages_and_slots_used_again(tmp_path, name, dtype):
    d = make_dir(tmp_path, name)
    steps, seqs = mixed_schedule([44, 9, 150, 1, 70, 33, 64, 18, 97], CONFIGS[name]["vocab"], 21)
    held, peak = {}, 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = e["at"] + len(e["tokens"])
        peak = max(peak, sum((v + 63) // 64 * 64 for v in held.values()))
        for rid in s["end"]:
            held.pop(rid)
    rep = replayer(d, dtype, peak)
    refs = {rid: plain_logits(d, name, ids, oracle_dtype(dtype)) for rid, ids in seqs.items()}
    for k, s in enumerate(steps):
        out = rep.run_step(s["entries"], s["end"]).numpy().astype(np.float64)
        row = 0
        for e in s["entries"]:
            n = len(e["tokens"])
            close(out[row:row + n], refs[e["id"]][e["at"]:e["at"] + n], dtype, f"{name} step {k} request {e['id']} at {e['at']}")
            row += n
        rep.cache.book.check_invariants()
    assert rep.cache.book.free_slots == 4
    for g in range(len(rep.cache.groups)):
        assert rep.cache.book.pages_in_use(g) == 0
        assert rep.cache.book.total_allocations(g) > rep.cache.groups[g].num_pages      # pages were used again


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_request_does_not_depend_on_what_is_beside_it(tmp_path, dtype):
    d = make_dir(tmp_path, "A")
    vocab = CONFIGS["A"]["vocab"]
    a, b, c = ids_for(50, vocab, 31), ids_for(23, vocab, 32), ids_for(9, vocab, 33)
    alone = feed(replayer(d, dtype, 128), "a", a, [20, 30])
    rep = replayer(d, dtype, 256)
    o1 = rep.run_step([dict(id="b", tokens=b[:22], want=[]), dict(id="a", tokens=a[:20], want=list(range(20))),
                       dict(id="c", tokens=c[:2], want=[])]).numpy()
    o2 = rep.run_step([dict(id="c", tokens=c[2:3], want=[0]), dict(id="a", tokens=a[20:], want=list(range(30))),
                       dict(id="b", tokens=b[22:], want=[0])]).numpy()
    beside = np.concatenate([o1, o2[1:31]]).astype(np.float64)
    lim = (1e-5 if dtype == "float32" else 3e-2) * max(1.0, np.abs(alone).max())
    assert np.abs(beside - alone).max() <= lim


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_windows_give_pages_back_while_a_request_decodes(tmp_path, dtype):
    """A long request on pages of 8: the windows (37, 21 and 70 keys) pass over the prompt and the pages behind them
    return to the pool, the latent attention keeps every page, and the logits stay the oracle's."""
    d = make_dir(tmp_path, "A")
    ids = ids_for(260, CONFIGS["A"]["vocab"], 44)
    rep = replayer(d, dtype, 320)
    ref = plain_logits(d, "A", ids, oracle_dtype(dtype))
    got = feed(rep, "r", ids, [100, 60] + [1] * 100, end=False)
    close(got, ref, dtype, "decoding behind the windows")
    book = rep.cache.book
    assert sorted(grp.request.window for grp in rep.cache.groups) == [0, 21, 37, 70]
    for g, grp in enumerate(rep.cache.groups):
        w = grp.request.window
        assert book.pages_in_use(g) <= ((w + 7) // 8 + 1 if w else (260 + 7) // 8)
    rep.run_step([], end=["r"])
    book.check_invariants()


def greedy_matches(raw, t, prompt, got, n_new):
    toks = list(prompt)
    for k in range(n_new):
        logits = pf.forward(raw, t, toks)[0][-1]
        top = torch.topk(logits, 2).values
        if float(top[0] - top[1]) < 1e-3 * float(logits.std()):
            return                                      # a close call: either token is right; stop comparing
        assert got[k] == int(torch.argmax(logits)), (len(prompt), k)
        toks.append(got[k])


@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_engine(tmp_path, name):
    """Engine.generate: the scheduler cuts the prompts into portions under a small token budget, batches them
    with decoded tokens and runs a step ahead of the device; the tokens are the plain implementation's wherever
    its best logit leads the second by more than rounding can turn."""
    import ai_engine_b200 as aie
    d = make_dir(tmp_path, name)
    raw, t = CONFIGS[name], read_tensors(d)
    prompts = [ids_for(n, raw["vocab"], 40 + n) for n in (5, 37, 1, 18)]
    n_new = 24
    eng = aie.Engine(d, dtype="fp32", block_size=8, kv_cache_blocks=64, max_num_seqs=3, max_num_batched_tokens=16)
    outs = eng.generate(prompts, aie.SamplingParams(max_tokens=n_new, temperature=0.0, ignore_eos=True))
    for prompt, got in zip(prompts, outs):
        assert len(got) == n_new
        greedy_matches(raw, t, prompt, got, n_new)
    assert eng.stats()["running"] == 0


def test_generation_in_bfloat16_replays_graphs_and_matches_eager_steps(tmp_path):
    """Decode steps of one layout are captured into a CUDA graph at their second use; the states in the slots must
    advance exactly once per step, captured or not, and what a block hands ahead to the next must be made inside
    the graph too."""
    import ai_engine_b200 as aie
    d = make_dir(tmp_path, "B")
    prompts = [ids_for(n, CONFIGS["B"]["vocab"], 60 + n) for n in (9, 30)]
    sp = aie.SamplingParams(max_tokens=40, temperature=0.0, ignore_eos=True)
    eng = aie.Engine(d, dtype="bf16", block_size=8, kv_cache_blocks=64, max_num_seqs=2, max_num_batched_tokens=64)
    with_graphs = eng.generate(prompts, sp)
    assert eng.runner.graphs_captured >= 1 and eng.runner.graph_launches > 0
    os.environ["AI_ENGINE_B200_NO_GRAPHS"] = "1"
    try:
        eng2 = aie.Engine(d, dtype="bf16", block_size=8, kv_cache_blocks=64, max_num_seqs=2, max_num_batched_tokens=64)
        eager = eng2.generate(prompts, sp)
    finally:
        del os.environ["AI_ENGINE_B200_NO_GRAPHS"]
    assert eng2.runner.graphs_captured == 0
    assert with_graphs == eager


def test_the_trace_program_and_the_command_line_on_a_fokisun_folder(tmp_path):
    d = make_dir(tmp_path, "A")
    ids = ids_for(30, CONFIGS["A"]["vocab"], 77)
    out_dir = os.path.join(str(tmp_path), "out")
    steps = [dict(step=0, entries=[dict(id="r", tokens=ids[:21], want=[0, 20])], end=[]),
             dict(step=1, entries=[dict(id="r", tokens=ids[21:23], want=[])], end=[]),
             dict(step=2, entries=[dict(id="r", tokens=ids[23:], want=[6])], end=["r"])]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
                        "--out", out_dir, "--max-tokens", "64"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.split("\n") if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    assert not os.path.exists(os.path.join(out_dir, "1.f32"))
    ref = plain_logits(d, "A", ids)
    got0 = np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(2, -1)
    got2 = np.fromfile(os.path.join(out_dir, "2.f32"), dtype="<f4").reshape(1, -1)
    close(got0, ref[[0, 20]], "float32", "trace step 0")
    close(got2, ref[[29]], "float32", "trace step 2")
    exe = [sys.executable, os.path.join(ROOT, "bin", "ai-engine")]
    assert subprocess.run(exe + ["--model", d, "--check"], capture_output=True, text=True).stdout.strip() == "ok"
    p = subprocess.run(exe + ["--model", d, "--dtype", "fp32", "--prompt-ids", "5,17,3,200", "--prompt-ids", "9",
                              "--max-tokens", "5", "--ignore-eos", "--profile"], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-1500:]
    lines = [[int(t) for t in l.split(",")] for l in p.stdout.strip().splitlines()]
    assert len(lines) == 2 and all(len(l) == 5 for l in lines)
    for cls in ("add_dyt", "parallel_residual", "normed_attn_prepare", "sink_attention", "sigmoid_gate_mul",
                "linear_recurrence", "head_norm_gate", "latent_prepare", "slice_rmsnorm", "route_topk", "expert_combine"):
        assert cls in p.stderr, cls
    greedy_matches(CONFIGS["A"], read_tensors(d), [5, 17, 3, 200], lines[0], 5)


def drawn_config(seed):
    """A configuration drawn at random: 2-6 layers of any kind in any order, any sizes (also ones the tensor-core
    kernels do not take), windows shorter than a page or none, rotations over a part of a head or none, layers that
    mix values anywhere, feed-forwards of either kind or none."""
    import random
    r = random.Random(seed)
    width = r.choice([32, 44, 64, 72, 100, 128, 160])
    mix_shape = (r.choice([1, 2]), r.choice([4, 16, 32, 36, 64]))          # the layers that mix values share it
    layers = []
    for _ in range(r.randint(2, 6)):
        kind = r.choice(["attention", "hgrn2", "latent_attention"])
        u = r.random()
        if u < 0.25:
            mlp = None
        elif u < 0.55:
            mlp = dense(r.choice([24, 40, 96, 200]))
        else:
            count = r.choice([1, 2, 3, 4])
            per = r.choice([1, 2, 3])
            keep = r.randint(1, count)
            mlp = moe(r.choice([16, 24, 64, 96]), count * per, r.randint(1, per * keep), count, keep,
                      r.choice([0.5, 1.0, 2.0]), r.choice([None, 16, 64]))
        if kind == "attention":
            v_mix = r.random() < 0.6
            kv, vdim = mix_shape if v_mix else (r.choice([1, 2, 3, 4]), r.choice([4, 16, 32, 36, 64, 128]))
            heads = kv * r.choice([1, 2, 3])
            dim = r.choice([8, 12, 32, 40, 64, 96, 128])
            rot = None
            if r.random() < 0.8:
                rot = (r.choice([100.0, 10000.0, 200000.0]), r.choice([x for x in (2, 4, 8, 12, 32, 64, 128) if x <= dim]),
                       r.choice([None, 2.0, 4.0]))
            layers.append(layer(attn(heads, kv, dim, vdim, r.uniform(0.05, 0.4), r.choice([None, 1, 3, 17, 40, 64, 100]),
                                     rot, v_mix), mlp))
        elif kind == "hgrn2":
            layers.append(layer(hgrn(r.choice([1, 2, 3, 4]), r.choice([8, 20, 32, 48, 64, 128, 136]),
                                     r.choice([8, 16, 24, 64, 80, 128])), mlp))
        else:
            layers.append(layer(latent(r.choice([1, 2, 3, 6]), r.choice([8, 16, 32, 48, 64]), r.choice([2, 4, 16, 32]),
                                       r.choice([8, 16, 32, 40]), r.choice([8, 24, 64, 128]), r.choice([8, 20, 64, 128]),
                                       r.uniform(0.05, 0.3), r.choice([100.0, 50000.0])), mlp))
    return dict(architecture="Fokisun", vocab=r.choice([61, 128, 300]), width=width,
                norm=dict(eps=r.choice([1e-6, 1e-5, 1e-3])), residual_mult=r.choice([0.5, 0.75, 1.0, 1.4]),
                logit_scale=r.choice([0.25, 1.0, 2.5]), layers=layers)


@pytest.mark.parametrize("seed", range(24))
def test_configurations_drawn_at_random(tmp_path, seed):
    """float32 against the float64 oracle at every row; bfloat16 against the float32 oracle: whole, and in portions
    beside a second request that decodes."""
    name = f"R{seed}"
    CONFIGS[name] = drawn_config(seed)
    d = make_dir(tmp_path, name, seed=seed)
    vocab = CONFIGS[name]["vocab"]
    ids, other = ids_for(170, vocab, 100 + seed), ids_for(60, vocab, 200 + seed)
    for dtype in ("float32", "bfloat16"):
        ref, ref_o = (plain_logits(d, name, x, oracle_dtype(dtype)) for x in (ids, other))
        rep = replayer(d, dtype, 320)
        close(feed(rep, "w", ids, [170]), ref, dtype, f"drawn {seed} {dtype} whole")
        cuts, got, got_o, at, at_o = [40, 2, 33, 1, 1, 64, 29], [], [], 0, 0
        for k, n in enumerate(cuts):                 # portions of one request beside a prompt, then single tokens, of another
            m = 20 if k == 0 else (1 if at_o < 60 else 0)
            entries = [dict(id="p", tokens=ids[at:at + n], want=list(range(n)))]
            if m:
                entries.append(dict(id="o", tokens=other[at_o:at_o + m], want=list(range(m))))
            out = rep.run_step(entries, []).numpy().astype(np.float64)
            got.append(out[:n])
            got_o.append(out[n:n + m])
            at, at_o = at + n, at_o + m
        rep.run_step([], ["p", "o"])
        close(np.concatenate(got), ref, dtype, f"drawn {seed} {dtype} in portions")
        close(np.concatenate(got_o), ref_o[:at_o], dtype, f"drawn {seed} {dtype} the request beside")
        rep.cache.book.check_invariants()
