"""Fokisun as a ModelSpec: a decoder whose layers run their mixer and their feed-forward side by side on one normed
input (a norm without statistics, tanh(alpha x) w + b), add both to the stream with one multiplier, and hand on a
learned average of all layers' streams.  A layer mixes with latent attention (queries through a latent of their own,
a gate per head), with HGRN2 (linear attention whose forget gate also decides what is written) or with windowed
grouped-query attention (queries and keys normed over the whole projection, rotated pairs of neighbours with evenly
stretched positions, a softmax with one added to its denominator, values mixed with those of the first such layer, a
gate per output element); it feeds forward through a dense gated layer (gelu) or a mixture of experts chosen by
sigmoid scores within the best groups, beside a shared expert.  The head is the embedding table; the logits are
multiplied by a constant.

Tensor names: `embed`, `final.norm|.b|.alpha`, and per layer i `l<i>.norm1|.b|.alpha`, `l<i>.dwa`, `l<i>.mix.*`,
`l<i>.mlp.gate|up|down`, or `l<i>.mlp.router`, experts `l<i>.mlp.e<k>.gate|up|down` and `l<i>.mlp.shared.*`.
"""
from __future__ import annotations

from ..config.fokisun import FokisunConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep

UNIT_SINK = 0.0          # the softmax's sink has the score 0: its weight in the denominator is exp(0) = 1
GROUP_TOP = 2            # a group of experts counts as the sum of its two best scores


def _rotary(encodings: dict, m, layout: str):
    if not m.rot_dims:
        return None
    name = f"rotary_{layout}_{m.rot_dims}_{m.rot_base!r}_{m.rot_factor!r}"
    encodings[name] = PartSpec("rotary", dict(
        rot_dim=m.rot_dims, theta=m.rot_base, layout=layout,
        scaling=dict(type="linear", factor=m.rot_factor) if m.rot_factor != 1.0 else None))
    return name


def build_fokisun_spec(cfg: FokisunConfig) -> ModelSpec:
    D, V, eps = cfg.width, cfg.vocab, cfg.norm_eps
    n = len(cfg.layers)
    encodings = {}
    layers = []
    dyt = lambda name: PartSpec("dynamic_tanh", dict(size=D), dict(weight=name, bias=name + ".b", alpha=name + ".alpha"))
    mixes_seen = False
    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        q = p + "mix."
        parts = {"norm": dyt(p + "norm1")}
        if l.type == "latent_attention":
            parts["mixer"] = PartSpec("latent_attention", dict(
                hidden_size=D, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
                kv_rank=m.kv_rank, q_rank=m.q_rank, scale=m.scale, window=0, eps=eps, head_gate=True,
                position_encoding=_rotary(encodings, m, "halves")),
                dict(dq=q + "dq", dq_norm=q + "dq.norm", uq=q + "uq", dkv=q + "dkv", dkv_norm=q + "dkv.norm",
                     uk=q + "uk", uv=q + "uv", o=q + "o", g=q + "g"))
        elif l.type == "hgrn2":
            parts["mixer"] = PartSpec("forget_gate_linear_attention", dict(
                hidden_size=D, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, eps=eps),
                dict(q=q + "q", f=q + "f", f_bias=q + "f.b", lower=q + "lower", v=q + "v", norm=q + "norm", o=q + "o"))
        else:
            mix = None
            if m.v_mix:
                mix, mixes_seen = ("mix" if mixes_seen else "source"), True
            parts["mixer"] = PartSpec("normed_gated_attention", dict(
                hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                scale=m.scale, window=m.window, eps=eps, qk_norm=True, bias=True, sink=UNIT_SINK,
                position_encoding=_rotary(encodings, m, "interleaved"), value_mix=mix),
                dict(q=q + "q", k=q + "k", v=q + "v", g=q + "g", o=q + "o", q_bias=q + "q.b", k_bias=q + "k.b",
                     v_bias=q + "v.b", o_bias=q + "o.b", q_norm=q + "q.norm", k_norm=q + "k.norm", **{"lambda": q + "vmix"}))
        f = l.mlp
        if f is not None and f.kind == "dense":
            parts["ffn"] = PartSpec("swiglu", dict(hidden_size=D, intermediate_size=f.ff, activation="gelu_tanh"),
                                    dict(gate=p + "mlp.gate", up=p + "mlp.up", down=p + "mlp.down"))
        elif f is not None:
            parts["ffn"] = PartSpec("routed_moe", dict(
                hidden_size=D, num_experts=f.experts, top=f.top, intermediate_size=f.ff, groups=f.group_count,
                keep=f.group_keep, activation="silu", score="sigmoid", group_top=GROUP_TOP, normalise=True,
                route_scale=f.scale, shared_intermediate_size=f.shared_ff),
                dict(router=p + "mlp.router", gate=p + "mlp.e{e}.gate", up=p + "mlp.e{e}.up", down=p + "mlp.e{e}.down",
                     shared_gate=p + "mlp.shared.gate", shared_up=p + "mlp.shared.up", shared_down=p + "mlp.shared.down"))
        layers.append(LayerSpec("parallel_depth_average", parts, dict(mult=cfg.residual_mult, depth=i, levels=n + 1),
                                dict(coef=p + "dwa")))
    embedding = PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), dict(weight="embed"))
    head = PartSpec("lm_head", dict(vocab_size=V, hidden_size=D, stored=False, scale=cfg.logit_scale), dict(weight="embed"))
    # an attention layer that mixes values has the tensor `vmix` even where it is the first and reads none
    return ModelSpec(
        hidden_size=D, vocab_size=V, max_position=cfg.max_position_embeddings, embedding=embedding, layers=layers,
        order=[RunStep(i) for i in range(n)], final_norm=dyt("final.norm"), lm_head=head,
        position_encodings=encodings, eos_token_ids=cfg.eos_token_ids,
        ignored_tensors=tuple(f"l{i}.mix.vmix" for i, l in enumerate(cfg.layers)
                              if l.type == "attention" and not l.mixer.v_mix))


register_architecture(FokisunConfig.ARCHITECTURE, FokisunConfig, build_fokisun_spec)
