"""Tizodra as a ModelSpec: a pre-norm decoder without a rotation whose places enter as a sinusoidal vector added to
the embedding and as a distance bias in its attention.  Layers mix by softmax attention (biases on q, k, v, values
divided by their root mean square, a temperature, a sink and a gate per head, a window that keeps the first tokens)
or by the gated delta rule (short convolutions on q, k, v, unit-length q and k, a decay and a write strength per
token and head); the feed-forward is down(relu(up x)^2) or absent.  A group of neighbouring layers may run several
times in a row with the same weights, every pass with caches and states of its own; each pass opens with a
projection `loop.in` of the running stream and the embedding's output side by side.  The logits are multiplied
by `logit_scale`.

Tensor names: `embed`, `head`, `final.norm`, `loop.in`, and per layer i `l<i>.norm1|norm2`; attention
`l<i>.mix.q|k|v` (+ `.b`), `.temp`, `.sink`, `.g`, `.o`; delta `l<i>.mix.q|k|v` (+ `.conv`), `.b`, `.a`, `.A_log`,
`.dt_bias`, `.norm`, `.g`, `.o`; `l<i>.mlp.up|down`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tizodra import TizodraConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep

SLOPE_BITS = 8.0          # slope of head h's distance bias: 2^(-8 (h + 1) / heads)
UNIT_EPS = 1e-6           # under the root that makes q and k of the delta rule unit vectors
SINUSOID_BASE = 10000.0


def build_tizodra_spec(cfg: TizodraConfig) -> ModelSpec:
    D, V, eps = cfg.width, cfg.vocab, cfg.norm_eps
    layers = []

    def norm(name):
        return PartSpec("rmsnorm", dict(size=D, eps=eps), dict(weight=name))

    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        q = p + "mix."
        if l.type == "attention":
            mixer = PartSpec("sink_window_attention", dict(
                hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                scale=m.scale, window=m.window, keep_first=m.keep_first, eps=eps, slope_bits=SLOPE_BITS),
                dict(q=q + "q", k=q + "k", v=q + "v", o=q + "o", q_bias=q + "q.b", k_bias=q + "k.b", v_bias=q + "v.b",
                     temp=q + "temp", sink=q + "sink", g=q + "g"))
        else:
            mixer = PartSpec("gated_delta_rule", dict(
                hidden_size=D, num_heads=m.heads, num_qk_heads=m.kv_heads, key_dim=m.dim, value_dim=m.vdim,
                taps=m.conv, eps=eps, unit_eps=UNIT_EPS),
                dict(q=q + "q", k=q + "k", v=q + "v", g=q + "g", b=q + "b", a=q + "a", q_conv=q + "q.conv",
                     k_conv=q + "k.conv", v_conv=q + "v.conv", a_log=q + "A_log", dt_bias=q + "dt_bias",
                     norm=q + "norm", o=q + "o"))
        parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer}
        if l.ff:
            parts["ffn_norm"] = norm(p + "norm2")
            parts["ffn"] = PartSpec("dense_ff", dict(hidden_size=D, intermediate_size=l.ff, activation="relu_squared"),
                                    dict(up=p + "mlp.up", down=p + "mlp.down"))
        # the loop's first layer opens every pass: it mixes the stream with the embedding's output first
        opens = cfg.loop_times > 0 and i == cfg.loop_start
        layers.append(LayerSpec("prenorm", parts, tensors={"input_mix": "loop.in"} if opens else {}))
    return ModelSpec(
        hidden_size=D, vocab_size=V, max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), dict(weight="embed")),
        layers=layers, order=[RunStep(i) for i in cfg.run_order()],
        final_norm=norm("final.norm"),
        lm_head=PartSpec("lm_head", dict(vocab_size=V, hidden_size=D, scale=cfg.logit_scale), dict(weight="head")),
        position_encodings={"sinusoid": PartSpec("sinusoidal", dict(size=D, base=SINUSOID_BASE))},
        eos_token_ids=cfg.eos_token_ids,
        # a layer without a feed-forward has no use for its second norm; a file may still hold it
        ignored_tensors=tuple(f"l{i}.norm2" for i, l in enumerate(cfg.layers) if not l.ff)
        + (() if cfg.loop_times else ("loop.in",)))


register_architecture(TizodraConfig.ARCHITECTURE, TizodraConfig, build_tizodra_spec)
