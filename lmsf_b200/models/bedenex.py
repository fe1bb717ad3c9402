"""Bedenex: the description of the decoder as data, and its registry entry.

A plain embedding; layers of ONE norm whose output both branches read, x <- x + g1 * mixer(h) + g2 * ff(h) with a sigmoid
gate vector per branch (g = sigmoid(W h + b)); two mixers (grouped attention inside chunks of positions, with unit-RMS
queries, keys and values, a bias that grows with the logarithm of the distance and a sigmoid gate per head; attention over
a cached low-rank vector plus one rotated key part shared by all heads, with a sink in the softmax); a feed-forward that is
dense (tanh-GELU gate) or routed experts (sigmoid scores, the score multiplies the expert's input) or absent; a span of
layers that runs several times with the same weights (each run has a cache of its own; every pass starts with one
projection of [stream | embedding output] and a vector per pass); a final norm and a head.  Tensor names: `embed`,
`final.norm`, `head`, `loop.in`, `loop.step`, and `l<i>.` + `norm1`, `rg1`, `rg1.b`, `rg2`, `rg2.b`, `mix.*`, `mlp.*`.
"""
from __future__ import annotations

from ..config.bedenex_config import BedenexConfig
from ..config.registry import register_architecture
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def bedenex_spec(cfg: BedenexConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.eps), {"weight": name})
    layers, ignored = [], []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        if m.type == "attention":
            bias = PartSpec("log_distance_bias", dict(num_heads=m.heads), {"r1": p + "mix.r1", "r2": p + "mix.r2"})
            mixer = PartSpec("paged_attention",
                             dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                                  position_encoding=bias, scale=m.scale, qk_norm=True, qk_norm_eps=cfg.eps,
                                  qk_norm_weights=False, value_norm=True, chunk=m.chunk, head_gate=True),
                             {"qkv": [p + "mix.q", p + "mix.k", p + "mix.v", p + "mix.g"], "o": p + "mix.o"})
        else:
            mixer = PartSpec("latent_attention",
                             dict(hidden_size=D, num_heads=m.heads, head_dim=m.dim, value_dim=m.vdim, kv_rank=m.kv_rank,
                                  eps=cfg.eps, scale=m.scale, window=None, gate=False, rope_dim=m.rot_dim,
                                  rope_dims=m.rot_dims, rope_base=m.rot_base, sink=True),
                             {"qcg": [p + "mix.q", p + "mix.dkv"], "c_norm": p + "mix.dkv.norm", "uk": p + "mix.uk",
                              "uv": p + "mix.uv", "o": p + "mix.o", "sink": p + "mix.sink"})
        parts = {"norm": norm(p + "norm1"), "mixer": mixer}
        f = L.mlp
        if f is None:
            ignored += [rf"^l{i}\.rg2$", rf"^l{i}\.rg2\.b$"]
        elif f.kind == "dense":
            parts["feed_forward"] = PartSpec("gated_mlp", dict(hidden_size=D, intermediate_size=f.ff, activation="gelu_tanh"),
                                             {"gate_up": [p + "mlp.gate", p + "mlp.up"], "down": p + "mlp.down"})
        else:
            up = [p + f"mlp.e{e}.{w}" for e in range(f.experts) for w in ("gate", "up")]
            parts["feed_forward"] = PartSpec("routed_experts",
                                             dict(hidden_size=D, num_experts=f.experts, top_k=f.top, expert_size=f.ff,
                                                  activation="silu", router_bias=False, shared_gate=False,
                                                  routing="sigmoid_top", weight_on_input=True),
                                             {"up": up, "down": [p + f"mlp.e{e}.down" for e in range(f.experts)],
                                              "router": [p + "mlp.router"]})
        gates = ["rg1"] + (["rg2"] if f is not None else [])
        parts["gates"] = PartSpec("gate_logits", dict(in_features=D, out_features=[D] * len(gates), bias=True),
                                  {"weight": [p + g for g in gates], "bias": [p + g + ".b" for g in gates]})
        layers.append(LayerSpec("parallel_gated", parts))
    order, entries = [], []
    if cfg.has_loop:
        entries.append(PartSpec("loop_entry", dict(hidden_size=D, times=cfg.loop_times, mix_first=True, step_vector=True),
                                {"mix": "loop.in", "step": "loop.step"}))
        order += [LayerCall(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            for i in range(cfg.loop_start, cfg.loop_stop):
                order.append(LayerCall(i, entry=0, entry_pass=t) if i == cfg.loop_start else LayerCall(i))
        order += [LayerCall(i) for i in range(cfg.loop_stop, len(cfg.layers))]
    else:
        order = [LayerCall(i) for i in range(len(cfg.layers))]
        ignored += [r"^loop\.in$", r"^loop\.step$"]
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, max_model_len=cfg.max_model_len,
        embedding=PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=D, as_stream=True), {"weight": "embed"}),
        layers=layers, order=order, entries=entries,
        final_norm=norm("final.norm"),
        lm_head=PartSpec("dense", dict(in_features=D, out_features=cfg.vocab, out_dtype="float32"), {"weight": "head"}),
        eos_token_ids=list(cfg.eos_token_ids), ignored_weights=ignored,
    )


register_architecture("Bedenex", BedenexConfig.from_dict, bedenex_spec, aliases=("bedenex",))
