"""Shared by the Fokisun tests: small configurations (between them every size, count and constant differs, some are 1
or equal where the others differ), model folders with random weights, the plain implementation as oracle, and
tolerances relative to the spread of the logits."""
from __future__ import annotations

import os

import numpy as np
import torch

import plain_fokisun as pf
from zupitar_helpers import AFTER, DEV, Ref, Rig, close, env, ids_for, load, oracle_dtype, read_tensors  # noqa: F401


def attn(heads, kv_heads, dim, vdim, scale, size=None, rot=None, v_mix=False):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if size is not None:
        m["mask"] = dict(size=size)
    if rot is not None:
        base, dims, factor = rot
        m["rot"] = dict(base=base, dims=dims)
        if factor is not None:
            m["rot"]["scaling"] = dict(factor=factor)
    if v_mix:
        m["v_mix"] = True
    return dict(type="attention", mixer=m)


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, scale, base=10000.0):
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank,
                                                    q_rank=q_rank, scale=scale, rot=dict(base=base, dims=rot_dim)))


def hgrn(heads, dim, vdim):
    return dict(type="hgrn2", mixer=dict(heads=heads, dim=dim, vdim=vdim))


def dense(ff):
    return dict(kind="dense", ff=ff)


def moe(ff, experts, top, count=None, keep=None, scale=1.0, shared=None):
    r = dict(experts=experts, top=top, scale=scale)
    if count is not None:
        r["groups"] = dict(count=count, keep=keep)
    f = dict(kind="moe", expert=dict(ff=ff), router=r)
    if shared:
        f["shared"] = dict(ff=shared)
    return f


def layer(l, mlp=None):
    return dict(l, mlp=mlp)


# odd sizes; every mixer; three layers that mix values (the first only provides them); windows shorter than a prompt;
# a rotation over a part of a head; a layer without feed-forward; experts in three groups of which two stay open
CFG_A = dict(architecture="Fokisun", vocab=211, width=96, norm=dict(eps=1e-4), residual_mult=0.6, logit_scale=0.5, layers=[
    layer(attn(6, 2, 16, 24, 0.3, 37, (5000.0, 8, 2.0), v_mix=True), dense(80)),
    layer(hgrn(3, 20, 24), moe(40, 6, 2, 3, 2, 1.7, shared=24)),
    layer(latent(5, 12, 8, 20, 24, 40, 0.22, 3000.0)),
    layer(attn(2, 2, 40, 24, 0.11, 21, (100.0, 40, None), v_mix=True), moe(24, 4, 1, 2, 1, 0.8)),
    layer(hgrn(4, 8, 12), dense(56)),
    layer(attn(4, 2, 20, 24, 0.2, 70, (777.0, 12, 8.0), v_mix=True), moe(32, 5, 3, shared=40)),
])

# the sizes the tensor-core kernels take in bfloat16 (keys and values of 64 and 128, a value of 32; a latent of 64 and
# of 128; experts whose width is a multiple of 64), a window that a 128-token tile crosses, an attention without a window
CFG_B = dict(architecture="Fokisun", vocab=257, width=128, norm=dict(eps=1e-5), residual_mult=0.8, logit_scale=3.0, layers=[
    layer(attn(4, 2, 64, 64, 0.13, 70, (40000.0, 64, 3.0), v_mix=True), moe(64, 4, 2, 2, 1, 1.5, shared=64)),
    layer(hgrn(2, 64, 64), dense(256)),
    layer(latent(4, 32, 16, 48, 64, 96, 0.15)),
    layer(attn(2, 2, 128, 64, 0.09, None, (10000.0, 32, None), v_mix=True), dense(192)),
    layer(latent(2, 64, 32, 64, 128, 64, 0.1, 50000.0), moe(128, 2, 1)),
    layer(attn(4, 1, 64, 32, 0.2, 130, (10000.0, 64, None)), dense(128)),
    layer(hgrn(1, 128, 128)),
])

# sizes of 1: one head, one expert, one choice, a window of one and of two keys; no rotation and no window in one
# attention; a width that is no multiple of 8; no logit scale and no multiplier in the file; one layer alone mixes values
CFG_C = dict(architecture="Fokisun", vocab=130, width=36, norm=dict(eps=1e-6), layers=[
    layer(hgrn(1, 12, 44), moe(20, 1, 1)),
    layer(attn(1, 1, 12, 44, 0.4, 2), dense(52)),
    layer(latent(1, 8, 2, 12, 6, 10, 0.3), moe(12, 3, 3, 3, 3)),
    layer(attn(3, 3, 20, 4, 0.25, 1, (10000.0, 2, None), v_mix=True)),
    layer(attn(2, 1, 10, 6, 0.35), dense(24)),
])

# latent attention first and last; no attention at all before a layer that mixes values from nobody
CFG_D = dict(architecture="Fokisun", vocab=97, width=48, norm=dict(eps=1e-5), residual_mult=1.3, logit_scale=1.5, layers=[
    layer(latent(3, 16, 4, 8, 16, 24, 0.2), dense(32)),
    layer(hgrn(2, 16, 16), moe(16, 8, 2, 4, 2, 2.0, shared=16)),
    layer(attn(4, 2, 24, 12, 0.2, 5, (300.0, 24, 1.5), v_mix=True), dense(64)),
    layer(latent(2, 8, 8, 24, 32, 8, 0.3)),
])

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


def make_dir(tmp_path, name, seed=0, gain=3.0):
    """A model folder for configuration `name`: random weights N(0, 0.07) written by the engine's random-weights
    mode, norm weights 1 + N(0, 0.1), and what sets the size of the queries (the weight of attention's query norm,
    the up-projection of latent attention's queries) multiplied by `gain` so that scores spread and single keys
    stand out.  The embedding is scaled up to a stream of order one and the routers to scores that spread."""
    import ai_engine_b200 as aie
    from safetensors import safe_open
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"fokisun_{name}_{seed}_{gain}")
    if os.path.exists(os.path.join(d, "model.safetensors")):
        return d
    aie.write_random_model(aie.FokisunConfig.from_dict(CONFIGS[name]), d, seed=seed, std=0.07, norm_std=0.1)
    path = os.path.join(d, "model.safetensors")
    tensors = {}
    with safe_open(path, "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if (k.endswith("mix.q.norm") or k.endswith("mix.uq")) and gain != 1.0:
                t = (t.float() * gain).to(t.dtype)
            if k == "embed":                          # a stream of order one, so that the norm's tanh bends
                t = (t.float() * 10.0).to(t.dtype)
            if k.endswith("mlp.router"):              # scores that spread, so that few choices are close calls
                t = (t.float() * 2.5).to(t.dtype)
            tensors[k] = t.clone().contiguous()          # a copy: the file is written again below
    save_file(tensors, path)
    return d


_REFS = {}
CLEAR = 0.012    # a router's choice stands when it leads what it left out by this much (scores are sigmoids)


def plain_logits(d, name, ids, dtype=torch.float64):
    """[len(ids), vocab] from the plain implementation, with the rows whose routing is clear (cached per folder and
    sequence)."""
    key = (d, tuple(ids), dtype)
    if key not in _REFS:
        margins = []
        logits = pf.forward(CONFIGS[name], read_tensors(d), ids, dtype=dtype, margins_out=margins)[0].to(torch.float64).numpy()
        m = torch.stack(margins).min(dim=0).values.double().numpy() if margins else np.full(len(ids), np.inf)
        ok = m >= CLEAR
        clear = np.array([bool(ok[max(0, i - AFTER):i + 1].all()) for i in range(len(ids))])
        _REFS[key] = Ref(logits, clear)
    return _REFS[key]
