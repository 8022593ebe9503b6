"""Shared by the Tizodra tests: small configurations (between them every size, count and constant differs, some are 1
or equal where the others differ), model folders with random weights, the plain implementation as oracle, and
tolerances relative to the spread of the logits."""
from __future__ import annotations

import os

import numpy as np
import torch

import plain_tizodra as pt
from zupitar_helpers import DEV, Rig, env, ids_for, load, oracle_dtype, read_tensors  # noqa: F401  (shared rig)


def attn(heads, kv_heads, dim, vdim, scale, size=None, keep=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if size is not None:
        m["mask"] = dict(size=size, keep_first=keep or 0)
    return dict(type="attention", mixer=m)


def delta(heads, kv_heads, dim, vdim, conv):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv))


def layer(l, ff=None):
    return dict(l, mlp=dict(kind="dense", ff=ff) if ff else None)


# a loop that starts behind the first layer and runs three times; odd sizes; windows shorter than a prompt with and
# without kept tokens; a layer without feed-forward; key and value sizes that differ both ways
CFG_A = dict(architecture="Tizodra", vocab=211, width=96, norm=dict(eps=1e-4), logit_scale=0.5,
             loop=dict(start=1, stop=3, times=3), layers=[
    layer(delta(4, 2, 24, 20, 4), 80),
    layer(attn(6, 2, 16, 24, 0.3, 37, 3)),
    layer(delta(3, 3, 40, 8, 2), 56),
    layer(attn(2, 1, 40, 16, 0.11, 21, 0), 64),
])

# the sizes the tensor-core kernels take in bfloat16 (keys and values of 64 and 128, a value of 32), a window that a
# 128-token tile crosses, an attention without a window, the loop from the first layer on
CFG_B = dict(architecture="Tizodra", vocab=257, width=128, norm=dict(eps=1e-5), logit_scale=3.0,
             loop=dict(start=0, stop=2, times=2), layers=[
    layer(attn(4, 2, 64, 64, 0.125, 70, 5), 256),
    layer(delta(2, 1, 64, 64, 3), 128),
    layer(attn(2, 2, 128, 128, 0.09), 192),
    layer(delta(4, 4, 128, 32, 2)),
    layer(attn(4, 1, 64, 32, 0.2, 130, 17), 128),
])

# no loop; sizes of 1: one head, one tap (no tail to carry), a window of two keys, one kept token; a width that is no
# multiple of 8; no logit scale in the file
CFG_C = dict(architecture="Tizodra", vocab=130, width=36, norm=dict(eps=1e-6), layers=[
    layer(attn(1, 1, 12, 44, 0.4, 2, 1), 52),
    layer(delta(1, 1, 12, 36, 1), 40),
    layer(delta(5, 1, 8, 12, 5)),
    layer(attn(3, 3, 20, 4, 0.25, 9, 9), 24),
])

# a loop of one layer that runs once and is the last layer
CFG_D = dict(architecture="Tizodra", vocab=97, width=48, norm=dict(eps=1e-5), logit_scale=1.5,
             loop=dict(start=2, stop=3, times=1), layers=[
    layer(attn(2, 2, 8, 8, 0.35, 16, 2), 32),
    layer(delta(2, 2, 16, 16, 3), 32),
    layer(attn(4, 2, 24, 12, 0.2, 5, 0), 64),
])

CONFIGS = {"A": CFG_A, "B": CFG_B, "C": CFG_C, "D": CFG_D}


def make_dir(tmp_path, name, seed=0, gain=3.0):
    """A model folder for configuration `name`: random weights N(0, 0.07) written by the engine's random-weights
    mode, norm weights 1 + N(0, 0.1), and the query projections of attention multiplied by `gain` so that scores
    spread and single keys stand out."""
    import ai_engine_b200 as aie
    from safetensors import safe_open
    from safetensors.torch import save_file

    d = os.path.join(str(tmp_path), f"tizodra_{name}_{seed}_{gain}")
    if os.path.exists(os.path.join(d, "model.safetensors")):
        return d
    aie.write_random_model(aie.TizodraConfig.from_dict(CONFIGS[name]), d, seed=seed, std=0.07, norm_std=0.1)
    path = os.path.join(d, "model.safetensors")
    kinds = [l["type"] for l in CONFIGS[name]["layers"]]
    tensors = {}
    with safe_open(path, "pt") as f:
        for k in f.keys():
            t = f.get_tensor(k)
            if k.endswith("mix.q") and kinds[int(k.split(".")[0][1:])] == "attention" and gain != 1.0:
                t = (t.float() * gain).to(t.dtype)
            tensors[k] = t.clone().contiguous()          # a copy: the file is written again below
    save_file(tensors, path)
    return d


_REFS = {}


def plain_logits(d, name, ids, dtype=torch.float64):
    """[len(ids), vocab] from the plain implementation (cached per folder and sequence)."""
    key = (d, tuple(ids), dtype)
    if key not in _REFS:
        _REFS[key] = pt.forward(read_tensors(d), CONFIGS[name], ids, dtype=dtype).to(torch.float64).numpy()
    return _REFS[key]


def close(got, ref, dtype, what=""):
    """Logits agree within rounding.  The float32 engine against the float64 oracle: 2e-4 of the logits' spread at
    every element.  bfloat16 against the float32 oracle on the same weights: the worst element within 0.2 of the
    spread and the mean difference under 0.03 of it (a wrong key, a lost state or a window one token off moves a
    row by the spread itself)."""
    spread = max(float(np.std(ref)), 1e-3)
    diff = np.abs(np.asarray(got, dtype=np.float64) - np.asarray(ref))
    err = float(diff.max())
    tol = (2e-4 if dtype == "float32" else 0.2) * spread
    assert err <= tol, f"{what}: max difference {err:.3e} above {tol:.3e} (row {int(diff.max(axis=-1).argmax())})"
    if dtype != "float32":
        assert float(diff.mean()) <= 0.03 * spread, f"{what}: mean difference {diff.mean():.3e} above {0.03 * spread:.3e}"
    return err
