"""Prefill and decode throughput of the Zonidra design at layer sizes that resemble a real model's, beside the Vufolorn
design (the engine's other model of sandwich norms, a windowed mixer and routed experts with a shared expert) and the Llama
shape at equal width and layer count, and the design's kernels alone beside the like kernel of those models.

    python bench.py --design zonidra [--steps K] [--warmup W]

Random weights, seeded random token ids.  Timing as in bench.py: CUDA events on the launching stream after warm-up;
decode steps read weights and caches far larger than L2; prefill and the kernels alone start from a flushed L2.
"""
from __future__ import annotations

import json

import torch

from . import design_bench
from .design_bench import BLOCK_SIZE, CONTEXT, PREFILL_TOKENS, measure_model


def zonidra_config(width, heads, kv_heads, dim, window, keep, experts, top, ff, shared, dense_ff, vocab):
    rot = {"dims": dim // 2, "base": 1.0e6, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5, "rot": rot,
             "mask": {"size": window, "keep_first": keep}}
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": 2, "scale": 2.0},
           "shared": {"ff": shared}}
    own = lambda mlp: {"type": "attention", "mixer": dict(mixer), "mlp": mlp}
    reads = lambda j, mlp: {"type": "attention", "mixer": dict(mixer, kv_from=j), "mlp": mlp}
    # four layers, as the models beside it: two with keys and values of their own and a dense feed-forward, each followed
    # by a layer that reads them and routes to experts
    return {"architecture": "Zonidra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "embedding": {"scale": width ** 0.5, "bigram": {"buckets": 65521, "mul_prev": 33, "mul_cur": 5}},
            "layers": [own({"kind": "dense", "ff": dense_ff}), reads(0, moe), own({"kind": "dense", "ff": dense_ff}), reads(2, moe)]}


SIZES = {
    "width2048": zonidra_config(2048, 16, 4, 128, 1024, 4, 32, 4, 1024, 2048, 6144, 32000),
    "width4096": zonidra_config(4096, 32, 8, 128, 2048, 4, 64, 6, 1408, 2816, 11264, 32000),
}


def kernels_alone(pk, width=4096, heads=32, kv_heads=8, dim=128, window=1024, keep=4, experts=64, top=6, dense_ff=11264):
    """Each new kernel, or kernel that gained a branch, alone with the like kernel of the Vufolorn or Llama path beside it,
    and what each reaches of its roofline: the measured copy rate for kernels that stream, the measured bf16 product rate for
    the attention kernels (the products that the mask leaves, 4 x keys seen x head size per query and head)."""
    from lmsf_b200 import kernels
    from lmsf_b200.benchmarks.kernel_bench import Timer
    dev = torch.device("cuda:0")
    tm = Timer(dev)
    bf, f32, i32 = torch.bfloat16, torch.float32, torch.int32
    T = PREFILL_TOKENS
    hbm, tflops = pk["hbm_gbs"] * 1e9, pk["bf16_tflops"] * 1e12
    rows = {}

    def rec(name, sec, bytes_=None, flops=None, like=None):
        r = {"us": round(sec * 1e6, 1)}
        if bytes_ is not None:
            r["frac_of_copy_rate"] = round(bytes_ / sec / hbm, 3)
        if flops is not None:
            r["frac_of_bf16_peak"] = round(flops / sec / tflops, 4)
        if like:
            r["like"] = like
        rows[name] = r

    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s, dtype=bf, scale=1.0: (torch.randn(*s, generator=g, device=dev, dtype=f32) * scale).to(dtype)
    ones = lambda n: torch.ones(n, device=dev)
    H, G, bs = heads, kv_heads, BLOCK_SIZE
    pos, seq = torch.arange(T, dtype=i32, device=dev), torch.zeros(T, dtype=i32, device=dev)
    cu, ctxl = torch.tensor([0, T], dtype=i32, device=dev), torch.tensor([T], dtype=i32, device=dev)
    slot = torch.zeros(1, dtype=i32, device=dev)
    flag = torch.zeros(1, dtype=i32, device=dev)
    # ---- the embedding with its pair table against the plain gather
    vocab, buckets = 32000, 65521
    table, pairs = rnd(vocab, width), rnd(buckets + 1, width)
    ids = torch.randint(0, vocab, (T,), device=dev, generator=g).to(i32)
    last = torch.zeros(2, 1, dtype=i32, device=dev)
    res = torch.empty(T, width, dtype=f32, device=dev)
    rec("embedding_pairs (two rows gathered, scaled sum in float32) 2048 x 4096",
        tm.run(lambda: kernels.embedding_pairs(res, table, pairs, ids, pos, seq, cu, slot, last, buckets, 33, 5, 64.0, flag), 3, 10),
        bytes_=T * width * (2 + 2 + 4), like="embedding below")
    xb = torch.empty(T, width, dtype=bf, device=dev)
    rec("embedding (Llama: one row gathered) 2048 x 4096", tm.run(lambda: kernels.embedding(xb, table, ids, flag), 3, 10),
        bytes_=T * width * 4)
    # ---- token shift against the kernel between two branches
    h, hs, mix = rnd(T, width), torch.empty(T, width, dtype=bf, device=dev), torch.rand(width, device=dev, generator=g)
    state = torch.zeros(2, width, dtype=f32, device=dev)
    rec("token_shift (row and row before, mixed element by element) 2048 x 4096",
        tm.run(lambda: kernels.token_shift(hs, h, mix, state, pos, seq, cu, slot), 3, 10), bytes_=T * width * (2 + 2),
        like="stream_norm below")
    y1, w = rnd(T, width), ones(width)
    rec("stream_norm (Vufolorn: post norm, layer scale, add, next norm) 2048 x 4096",
        tm.run(lambda: kernels.stream_norm(res, y=y1, w_post=w, layer_scale=w, eps_post=1e-5, h=hs, w_next=w, eps_next=1e-5), 3, 10),
        bytes_=T * width * (4 + 4 + 2 + 2))
    # ---- the polynomial activation against the gated one
    z, act = rnd(T, dense_ff), torch.empty(T, dense_ff, dtype=bf, device=dev)
    coef = torch.tensor([0.7, -1.3, 0.4, 0.25], device=dev)
    rec(f"poly_norm (three sums and a polynomial per row) 2048 x {dense_ff}",
        tm.run(lambda: kernels.poly_norm(act, z, coef, 1e-5), 3, 10), bytes_=T * dense_ff * 4, like="gated_act below")
    gu = rnd(T, 2 * dense_ff)
    rec(f"gated_act (Llama, silu) 2048 x {dense_ff}", tm.run(lambda: kernels.gated_act(act, gu, "silu"), 3, 10), bytes_=T * dense_ff * 6)
    # ---- routing and combining
    R = experts + 2
    logits = rnd(T, R + 1, dtype=f32)
    rid, rw = torch.empty(T, top, dtype=i32, device=dev), torch.empty(T, top, dtype=f32, device=dev)
    corr = rnd(R, dtype=f32, scale=0.05)
    rec(f"moe_topk_softmax_all (softmax over {R} outputs, choice with a correction) 2048 tokens",
        tm.run(lambda: kernels.moe_topk_softmax_all(rid, rw, logits, corr, R, 2.0), 3, 10), bytes_=T * (R + 1) * 4 + T * top * 8,
        like="moe_topk below")
    rec(f"moe_topk (Vufolorn: top of {experts}, softmax over the chosen) 2048 tokens",
        tm.run(lambda: kernels.moe_topk(rid, rw, logits, corr[:experts].contiguous(), experts), 3, 10), bytes_=T * (R + 1) * 4 + T * top * 8)
    pairs_n = T * top
    down = rnd(pairs_n, width, dtype=f32)
    kernels.moe_topk_softmax_all(rid, rw, logits, corr, R, 2.0)
    pair_row = torch.randperm(pairs_n, device=dev, generator=g).to(i32).view(T, top)
    pair_row = torch.where(rid >= experts, torch.full_like(pair_row, -1), pair_row)
    shared, out = rnd(T, width), torch.empty(T, width, dtype=bf, device=dev)
    gate = logits[:, R]
    rec(f"moe_combine with outputs that return the input: 2048 tokens, {top} choices, width 4096",
        tm.run(lambda: kernels.moe_combine(out, down, pair_row, rw, shared, gate, identity=(rid, experts, h)), 3, 10),
        bytes_=T * width * (4 * top + 2 + 2 + 2), like="moe_combine below")
    rec(f"moe_combine (Vufolorn) 2048 tokens, {top} choices, width 4096",
        tm.run(lambda: kernels.moe_combine(out, down, pair_row, rw, shared, gate), 3, 10), bytes_=T * width * (4 * top + 2 + 2))
    # ---- the gate per element against the gate per head
    att, vg, hg = rnd(T, H * dim), rnd(T, H * dim), rnd(T, H)
    rec("value_gate_ (sigmoid gate per element of the heads) 2048 x 32 x 128",
        tm.run(lambda: kernels.value_gate_(att, vg, H, dim, dim), 3, 10), bytes_=T * H * dim * 6, like="head_gate_ below")
    rec("head_gate_ (Bedenex: sigmoid gate per head) 2048 x 32 x 128",
        tm.run(lambda: kernels.head_gate_(att, hg, H, dim), 3, 10), bytes_=T * H * dim * 4)
    # ---- attention of a prompt of 2048 tokens: sigmoid weights, a bias per head, a window that keeps the first keys
    qkv = rnd(T, (H + 2 * G) * dim)
    q = qkv[:, :H * dim]
    pages = T // bs
    cache = rnd(pages + 1, 2, G, bs, dim, scale=0.5)
    tab = torch.arange(pages, dtype=i32, device=dev).view(1, pages)
    o = torch.empty(T, H * dim, dtype=bf, device=dev)
    t128 = torch.arange(0, T, 128, dtype=i32, device=dev).flip(0).contiguous()
    s128 = torch.zeros_like(t128)
    t64 = torch.arange(0, T, 64, dtype=i32, device=dev).flip(0).contiguous()
    s64 = torch.zeros_like(t64)
    hb = rnd(H, dtype=f32) - 3.0
    seen = sum(min(p + 1, window) + (min(keep, max(0, p + 1 - window))) for p in range(T))
    fl = lambda seen_: 4.0 * seen_ * dim * H
    scale = dim ** -0.5
    ex = dict(keep_first=keep, sigmoid=True, head_bias=hb)
    rec(f"attention_prefill_tc, sigmoid weights, window {window} + {keep} kept: 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(o, q, cache, tab, bs, s128, t128, t128.numel(), cu, ctxl, scale, window, H, G, dim, flag, **ex), 3, 10),
        flops=fl(seen), like="the one below")
    rec(f"attention_prefill_tc (softmax, window {window}) 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(o, q, cache, tab, bs, s128, t128, t128.numel(), cu, ctxl, scale, window, H, G, dim, flag), 3, 10),
        flops=fl(seen))
    rec("attention_prefill_tc, sigmoid weights, no window: 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(o, q, cache, tab, bs, s128, t128, t128.numel(), cu, ctxl, scale, 0, H, G, dim, flag,
                                                    sigmoid=True, head_bias=hb), 3, 10), flops=fl(T * (T + 1) // 2), like="the one below")
    rec("attention_prefill_tc (Llama: causal softmax) 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(o, q, cache, tab, bs, s128, t128, t128.numel(), cu, ctxl, scale, 0, H, G, dim, flag), 3, 10),
        flops=fl(T * (T + 1) // 2))
    rec(f"attention_prefill (mma.sync), sigmoid weights, window {window} + {keep} kept: 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill(o, q, cache, tab, bs, s64, t64, t64.numel(), cu, ctxl, scale, window, H, G, dim, **ex), 3, 10),
        flops=fl(seen), like="the one below")
    rec(f"attention_prefill (mma.sync, softmax, window {window}) 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill(o, q, cache, tab, bs, s64, t64, t64.numel(), cu, ctxl, scale, window, H, G, dim), 3, 10),
        flops=fl(seen))
    # ---- decode: 64 requests of 2048 tokens
    B = 64
    pages = B * (CONTEXT // bs)
    cd = rnd(pages, 2, G, bs, dim, scale=0.5)
    tabd = torch.arange(pages, dtype=i32, device=dev).view(B, CONTEXT // bs)
    qd, od = rnd(B, H * dim), torch.empty(B, H * dim, dtype=bf, device=dev)
    cud, ctxd = torch.arange(B + 1, dtype=i32, device=dev), torch.full((B,), CONTEXT, dtype=i32, device=dev)

    def decode(visible, **extras):
        splits, warps = kernels.decode_plan(B, G, H // G, visible, dim, kernels.decode_widths(dim, H // G))
        need = kernels.attention_decode_scratch_floats(B, H, splits, dim)
        scratch = torch.zeros(max(need, 1), dtype=f32, device=dev)
        return tm.run(lambda: kernels.attention_decode(od, qd, cd, tabd, bs, None, B, cud, ctxd, scale, window, H, G, dim, splits,
                                                       scratch if need else None, warps, **extras), 3, 10)

    kv_bytes = lambda keys: B * keys * G * dim * 2 * 2
    rec(f"attention_decode, sigmoid weights, window {window} + {keep} kept: 64 requests at 2048, 32 heads of 128 over 8",
        decode(window + keep, **ex), bytes_=kv_bytes(window + keep), like="the one below")
    rec(f"attention_decode (softmax, window {window}) 64 requests at 2048, 32 heads of 128 over 8",
        decode(window), bytes_=kv_bytes(window))
    return rows


def run(bench, steps, warmup, pk):
    sampler = bench.ClockSampler()
    sampler.start()
    sizes = {}
    for name, cfg in SIZES.items():
        sizes[name] = {"zonidra": measure_model(cfg, [8, 64], steps, warmup, bench),
                       "vufolorn": measure_model(design_bench.SIZES[name][0], [8, 64], steps, warmup, bench),
                       "llama": measure_model(design_bench.SIZES[name][1], [8, 64], steps, warmup, bench)}
    alone = kernels_alone(pk)
    line = {"metric": "prefill and decode tokens/s of the Zonidra design beside the Vufolorn design and the Llama shape of equal width "
                      "(4 layers each, random weights)",
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
            "config": {"prefill_tokens": PREFILL_TOKENS, "context": CONTEXT, "block_size": BLOCK_SIZE, "sizes": SIZES,
                       "vufolorn": {k: v[0] for k, v in design_bench.SIZES.items()},
                       "llama": {k: v[1] for k, v in design_bench.SIZES.items()}, "peaks": pk.get("source", "measured")},
            "sizes": sizes, "kernels_alone": alone, "clocks": sampler.stop(), "impl": "ours"}
    print(json.dumps(line))
    return 0
