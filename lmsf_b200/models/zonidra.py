"""Zonidra: the description of the decoder as data, and its registry entry.

An embedding that adds to the token's scaled row a row chosen by the pair (token before, token); layers with a norm before and
after each branch and a layer scale on the branch, whose mixer reads the first norm's output mixed with the row of the token
before (token shift); one mixer: grouped attention with a partial rotation of the heads' front values (frequencies stretched
by wavelength), a sliding window that keeps the request's first tokens visible, weights sigmoid(score + bias of the head) that
are not normalised over the keys, and an element-wise sigmoid gate before the output projection; a layer may read the cached
keys and values of an earlier layer instead of projecting its own; a feed-forward that is dense (a polynomial activation whose
powers are normed), routed experts (a softmax over all router outputs, a correction for the choice only, outputs that return
the token's input, a gated shared expert) or absent; a final norm and a head.  Tensor names: `embed`, `bigram`, `final.norm`,
`head`, and `l<i>.` + `norm1`, `norm1b`, `ls1`, `norm2`, `norm2b`, `ls2`, `shift`, `mix.*`, `mlp.*`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zonidra_config import ZonidraConfig
from ..parts.base import LayerCall, LayerSpec, ModelSpec, PartSpec


def cache_needs(cfg: ZonidraConfig, owner: int):
    """(window, keep_first) that the cache of layer `owner` must hold: the widest mask among the layer and its readers."""
    masks = [(L.mixer.window, L.mixer.keep_first) for i, L in enumerate(cfg.layers) if i == owner or L.mixer.kv_from == owner]
    if any(w is None for w, _ in masks):
        return None, 0
    return max(w for w, _ in masks), max(k for _, k in masks)


def zonidra_spec(cfg: ZonidraConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.eps), {"weight": name})
    post = lambda name, ls: PartSpec("rmsnorm", dict(hidden_size=D, eps=cfg.eps, layer_scale=True), {"weight": name, "scale": ls})
    layers, order, ignored = [], [], []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}.", L.mixer
        rope = None
        if m.rot is not None:
            sc = m.rot.scaling
            rope = PartSpec("rotary", dict(rot_dim=m.rot.dims, theta=m.rot.base, is_neox=True,
                                           **(dict(scaling_type="llama3", factor=sc["factor"], low_freq_factor=sc["low"],
                                                   high_freq_factor=sc["high"],
                                                   original_max_position_embeddings=sc["original"]) if sc else {})))
        own = m.kv_from is None
        cache_window, cache_keep = cache_needs(cfg, i) if own else (m.window, m.keep_first)
        merged = [p + "mix.q"] + ([p + "mix.k", p + "mix.v"] if own else []) + [p + "mix.g"]
        mixer = PartSpec("paged_attention",
                         dict(hidden_size=D, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, value_dim=m.vdim,
                              position_encoding=rope, scale=m.scale, window=m.window, keep_first=m.keep_first,
                              score_weights="sigmoid", head_bias=True, value_gate=True, own_kv=own,
                              cache_window=cache_window, cache_keep_first=cache_keep),
                         {"qkv": merged, "o": p + "mix.o", "head_bias": p + "mix.pb"})
        parts = {"mixer_norm": norm(p + "norm1"), "mixer_shift": PartSpec("token_shift", dict(hidden_size=D), {"mix": p + "shift"}),
                 "mixer": mixer, "mixer_post_norm": post(p + "norm1b", p + "ls1")}
        f = L.mlp
        if f is None:
            ignored += [rf"^l{i}\.norm2$", rf"^l{i}\.norm2b$", rf"^l{i}\.ls2$"]
        else:
            if f.kind == "dense":
                ff = PartSpec("plain_mlp", dict(hidden_size=D, intermediate_size=f.ff, eps=cfg.eps, activation="poly_norm"),
                              {"up": p + "mlp.up", "down": p + "mlp.down", "act": p + "mlp.act"})
            else:
                w = {"up": [p + f"mlp.e{e}.{n}" for e in range(f.experts) for n in ("gate", "up")],
                     "down": [p + f"mlp.e{e}.down" for e in range(f.experts)],
                     "router": [p + "mlp.router"] + ([p + "mlp.shared.sg"] if f.shared_ff else []),
                     "router_bias": p + "mlp.correction"}
                if f.shared_ff:
                    w.update(shared_up=[p + "mlp.shared.gate", p + "mlp.shared.up"], shared_down=p + "mlp.shared.down")
                ff = PartSpec("routed_experts",
                              dict(hidden_size=D, num_experts=f.experts, top_k=f.top, expert_size=f.ff, shared_size=f.shared_ff,
                                   activation="silu", router_bias=True, shared_gate=True, routing="softmax_all",
                                   route_scale=f.route_scale, identity_experts=f.identity), w)
            parts.update(ffn_norm=norm(p + "norm2"), feed_forward=ff, ffn_post_norm=post(p + "norm2b", p + "ls2"))
        layers.append(LayerSpec("sandwich_norm", parts))
        order.append(LayerCall(i, cache_of=m.kv_from))
    if cfg.pair_buckets:
        embedding = PartSpec("pair_token_embedding",
                             dict(vocab_size=cfg.vocab, hidden_size=D, buckets=cfg.pair_buckets, mul_prev=cfg.pair_mul_prev,
                                  mul_cur=cfg.pair_mul_cur, scale=cfg.embed_scale), {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("token_embedding", dict(vocab_size=cfg.vocab, hidden_size=D, scale=cfg.embed_scale, as_stream=True),
                             {"weight": "embed"})
        ignored.append(r"^bigram$")
    return ModelSpec(
        hidden_size=D, vocab_size=cfg.vocab, max_model_len=cfg.max_model_len, embedding=embedding,
        layers=layers, order=order, final_norm=norm("final.norm"),
        lm_head=PartSpec("dense", dict(in_features=D, out_features=cfg.vocab, out_dtype="float32"), {"weight": "head"}),
        eos_token_ids=list(cfg.eos_token_ids), ignored_weights=ignored,
    )


register_architecture("Zonidra", ZonidraConfig.from_dict, zonidra_spec, aliases=("zonidra",))
