"""Prefill and decode throughput of the Bedenex design at layer sizes that resemble a real model's, beside the Vufolorn
design (the engine's other model of latent attention and routed experts) and the Llama shape at equal width and layer
count, and the design's kernels alone beside the like kernel of those models.

    python bench.py --design bedenex [--steps K] [--warmup W]

Random weights, seeded random token ids.  Timing as in bench.py: CUDA events on the launching stream after warm-up;
decode steps read weights and caches far larger than L2; prefill and the kernels alone start from a flushed L2.
"""
from __future__ import annotations

import json

import torch

from . import design_bench
from .design_bench import BLOCK_SIZE, CONTEXT, PREFILL_TOKENS, measure_model


def bedenex_config(width, heads, kv_heads, dim, chunk, rank, rot, experts, top, ff, dense_ff, vocab, times=2):
    moe = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    dense = {"kind": "dense", "ff": dense_ff}
    att = {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": dim ** -0.5,
                                          "mask": {"size": chunk}}}
    lat = {"type": "latent_attention",
           "mixer": {"heads": heads, "dim": dim, "rot_dim": rot, "vdim": dim, "kv_rank": rank, "scale": (dim + rot) ** -0.5,
                     "rot": {"dims": rot, "base": 10000.0}}}
    # four layer runs, as the models beside it: one layer, a span of one layer that runs twice, one layer
    return {"architecture": "Bedenex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [dict(att, mlp=dense), dict(lat, mlp=moe), dict(att, mlp=moe)],
            "loop": {"start": 1, "stop": 2, "times": times}}


SIZES = {
    # the cached row (rank + rotated part) is 128 wide: the tcgen05 prefill kernel takes it
    "width2048": bedenex_config(2048, 16, 4, 128, 1024, 96, 32, 32, 4, 1024, 4096, 32000),
    # 256 wide, the widest the attention kernels take: mma.sync prefill and decode
    "width4096": bedenex_config(4096, 32, 8, 128, 1024, 192, 64, 64, 6, 1408, 7552, 32000),
}


def _paged(dev, T, bs, G, hd, planes, g):
    pages = T // bs
    cache = (torch.randn(pages + 1, planes, G, bs, hd, generator=g, device=dev, dtype=torch.float32) * 0.5).to(torch.bfloat16)
    table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
    return cache, table


def kernels_alone(pk, width=4096, heads=32, kv_heads=8, dim=128, chunk=1024, experts=64, top=6, ff=1408):
    """Each new kernel, or kernel that gained a branch, alone with the like kernel of the Vufolorn or Llama path beside
    it, and what each reaches of its roofline: the measured copy rate for kernels that stream, the measured bf16 product
    rate for the attention kernels (the products that the mask leaves, 4 x keys seen x head size per query and head)."""
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
    # ---- the end of a layer: both gates, both branches, the sum, the next norm
    res, z = rnd(T, width, dtype=f32), rnd(T, 2 * width, dtype=f32)
    y1, y2, h = rnd(T, width), rnd(T, width), torch.empty(T, width, dtype=bf, device=dev)
    w, b2 = ones(width), rnd(2 * width, dtype=f32)
    rec("gated_branches (two gates, two branches, sum, next norm) 2048 x 4096",
        tm.run(lambda: kernels.gated_branches(res, z, b2, y1, y2, h=h, w_next=w, eps_next=1e-5), 3, 10),
        bytes_=T * width * (4 + 4 + 8 + 2 + 2 + 2), like="stream_norm below")
    rec("stream_norm (Vufolorn: post norm, layer scale, add, next norm) 2048 x 4096",
        tm.run(lambda: kernels.stream_norm(res, y=y1, w_post=w, layer_scale=w, eps_post=1e-5, h=h, w_next=w, eps_next=1e-5), 3, 10),
        bytes_=T * width * (4 + 4 + 2 + 2))
    both = torch.empty(T, 2 * width, dtype=bf, device=dev)
    first = rnd(T, width, dtype=f32)
    rec("stream_concat (stream | embedding output -> the span's entry product) 2048 x 2 x 4096",
        tm.run(lambda: kernels.stream_concat(both, res, first), 3, 10), bytes_=T * width * (4 + 4 + 4))
    # ---- unit-RMS q, k and v into the cache against norm with weights + rotation (Redarax) and rotation alone (Llama)
    qkv = rnd(T, (H + 2 * G) * dim)
    q, k, v = qkv[:, :H * dim], qkv[:, H * dim:(H + G) * dim], qkv[:, (H + G) * dim:]
    cache, table = _paged(dev, T, bs, G, dim, 2, g)
    moved = T * ((H + G) * dim * 2 * 2 + G * dim * 2 * 2)
    rec("qk_norm_rope_cache_write, no weights, no rotation, unit-RMS values: 2048 tokens, 32 + 8 heads of 128",
        tm.run(lambda: kernels.qk_norm_rope_cache_write(q, k, v, pos, seq, table, bs, cache, None, 0, True, H, G, dim, dim, None, None, 1e-5,
                                                        weightless=True, v_norm_dim=dim), 3, 10), bytes_=moved, like="the two below")
    inv = torch.tensor([1.0e6 ** (-2.0 * i / 64) for i in range(32)], dtype=f32, device=dev)
    rec("qk_norm_rope_cache_write (Redarax: weights, 64 rotated) 2048 tokens, 32 + 8 heads of 128",
        tm.run(lambda: kernels.qk_norm_rope_cache_write(q, k, v, pos, seq, table, bs, cache, inv, 64, False, H, G, dim, dim, ones(dim), ones(dim), 1e-5), 3, 10),
        bytes_=moved)
    inv_full = torch.tensor([1.0e6 ** (-2.0 * i / 128) for i in range(64)], dtype=f32, device=dev)
    rec("rope_cache_write (Llama) 2048 tokens, 32 + 8 heads of 128",
        tm.run(lambda: kernels.rope_cache_write(q, k, v, pos, seq, table, bs, cache, inv_full, 128, True, H, G, dim), 3, 10), bytes_=moved)
    # ---- attention of a prompt of 2048 tokens: chunks + logarithmic bias against the plain causal kernel
    out = torch.empty(T, H * dim, dtype=bf, device=dev)
    cu, ctxl = torch.tensor([0, T], dtype=i32, device=dev), torch.tensor([T], dtype=i32, device=dev)
    t128 = torch.arange(0, T, 128, dtype=i32, device=dev).flip(0).contiguous()
    s128 = torch.zeros_like(t128)
    flag = torch.zeros(1, dtype=i32, device=dev)
    r1, r2 = ones(H) * 0.5, ones(H) * 0.7
    seen_all = T * (T + 1) // 2
    seen_chunk = (T // chunk) * (chunk * (chunk + 1) // 2)
    fl = lambda seen, hd, heads_: 4.0 * seen * hd * heads_
    scale = dim ** -0.5
    rec(f"attention_prefill_tc, chunks of {chunk} + logarithmic bias: 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(out, q, cache, table, bs, s128, t128, t128.numel(), cu, ctxl, scale, 0, H, G, dim, flag,
                                                    chunk=chunk, log_bias=(r1, r2)), 3, 10), flops=fl(seen_chunk, dim, H), like="the two below")
    rec("attention_prefill_tc, logarithmic bias, no chunks: 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(out, q, cache, table, bs, s128, t128, t128.numel(), cu, ctxl, scale, 0, H, G, dim, flag,
                                                    log_bias=(r1, r2)), 3, 10), flops=fl(seen_all, dim, H))
    rec("attention_prefill_tc (Llama: causal) 2048 tokens, 32 heads of 128 over 8",
        tm.run(lambda: kernels.attention_prefill_tc(out, q, cache, table, bs, s128, t128, t128.numel(), cu, ctxl, scale, 0, H, G, dim, flag), 3, 10),
        flops=fl(seen_all, dim, H))
    # ---- attention over one cached row per token, with a sink: 128 wide (tcgen05) and 256 wide (mma.sync)
    t64 = torch.arange(0, T, 64, dtype=i32, device=dev).flip(0).contiguous()
    s64 = torch.zeros_like(t64)
    sinks = ones(H)
    for hd in (128, 256):
        c1, tb1 = _paged(dev, T, bs, 1, hd, 1, g)
        ql, ol = rnd(T, H * hd), torch.empty(T, H * hd, dtype=bf, device=dev)
        if hd == 128:
            rec("attention_prefill_tc, one cached row of 128 per token, sinks: 2048 tokens, 32 heads",
                tm.run(lambda: kernels.attention_prefill_tc(ol, ql, c1, tb1, bs, s128, t128, t128.numel(), cu, ctxl, 0.08, 0, H, 1, hd, flag,
                                                            kv_planes=1, sinks=sinks), 3, 10), flops=fl(seen_all, hd, H), like="the one below")
            rec("attention_prefill_tc (Vufolorn: one cached row of 128, no sink) 2048 tokens, 32 heads",
                tm.run(lambda: kernels.attention_prefill_tc(ol, ql, c1, tb1, bs, s128, t128, t128.numel(), cu, ctxl, 0.08, 0, H, 1, hd, flag,
                                                            kv_planes=1), 3, 10), flops=fl(seen_all, hd, H))
        else:
            rec("attention_prefill (mma.sync), one cached row of 256 per token, sinks: 2048 tokens, 32 heads",
                tm.run(lambda: kernels.attention_prefill(ol, ql, c1, tb1, bs, s64, t64, t64.numel(), cu, ctxl, 0.06, 0, H, 1, hd,
                                                         kv_planes=1, sinks=sinks), 3, 10), flops=fl(seen_all, hd, H),
                like="attention_prefill at 128 below (the same kernel at the width the Vufolorn model has)")
            c0, tb0 = _paged(dev, T, bs, 1, 128, 1, g)
            q0, o0 = rnd(T, H * 128), torch.empty(T, H * 128, dtype=bf, device=dev)
            rec("attention_prefill (mma.sync), one cached row of 128 per token, no sink: 2048 tokens, 32 heads",
                tm.run(lambda: kernels.attention_prefill(o0, q0, c0, tb0, bs, s64, t64, t64.numel(), cu, ctxl, 0.08, 0, H, 1, 128, kv_planes=1), 3, 10),
                flops=fl(seen_all, 128, H))
    # ---- decode: 64 requests of 2048 tokens
    B = 64
    pages = B * (CONTEXT // bs)
    cd = (torch.randn(pages, 2, G, bs, dim, generator=g, device=dev, dtype=f32) * 0.5).to(bf)
    tabd = torch.arange(pages, dtype=i32, device=dev).view(B, CONTEXT // bs)
    qd, od = rnd(B, H * dim), torch.empty(B, H * dim, dtype=bf, device=dev)
    cud, ctxd = torch.arange(B + 1, dtype=i32, device=dev), torch.full((B,), CONTEXT, dtype=i32, device=dev)

    def decode(cache_, table_, q_, o_, n_kv, hd, planes, visible, **extras):
        splits, warps = kernels.decode_plan(B, n_kv, H // n_kv, visible, hd, kernels.decode_widths(hd, H // n_kv))
        need = kernels.attention_decode_scratch_floats(B, H, splits, hd)
        scratch = torch.zeros(max(need, 1), dtype=f32, device=dev)
        return tm.run(lambda: kernels.attention_decode(o_, q_, cache_, table_, bs, None, B, cud, ctxd, 0.08, 0, H, n_kv, hd, splits,
                                                       scratch if need else None, warps, kv_planes=planes, **extras), 3, 10)

    kv_bytes = lambda keys, n_kv, hd, planes: B * keys * n_kv * hd * 2 * planes
    rec(f"attention_decode, chunks of {chunk} + logarithmic bias: 64 requests at 2048, 32 heads of 128 over 8",
        decode(cd, tabd, qd, od, G, dim, 2, chunk, chunk=chunk, log_bias=(r1, r2)), bytes_=kv_bytes(chunk, G, dim, 2), like="the one below")
    rec("attention_decode (Llama) 64 requests at 2048, 32 heads of 128 over 8",
        decode(cd, tabd, qd, od, G, dim, 2, CONTEXT), bytes_=kv_bytes(CONTEXT, G, dim, 2))
    for hd in (128, 256):
        c1 = (torch.randn(pages, 1, 1, bs, hd, generator=g, device=dev, dtype=f32) * 0.5).to(bf)
        ql, ol = rnd(B, H * hd), torch.empty(B, H * hd, dtype=bf, device=dev)
        rec(f"attention_decode, one cached row of {hd} per token, sinks: 64 requests at 2048, 32 heads",
            decode(c1, tabd, ql, ol, 1, hd, 1, CONTEXT, sinks=sinks), bytes_=kv_bytes(CONTEXT, 1, hd, 1))
        if hd == 128:
            rec("attention_decode (Vufolorn: one cached row of 128, no sink) 64 requests at 2048, 32 heads",
                decode(c1, tabd, ql, ol, 1, hd, 1, CONTEXT), bytes_=kv_bytes(CONTEXT, 1, hd, 1))
    # ---- the latent layer's small kernels
    for rank, rot in ((96, 32), (192, 64)):
        padded = rank + rot
        x = rnd(T, rank + rot)
        c1, tb1 = _paged(dev, T, bs, 1, padded, 1, g)
        invr = torch.tensor([10000.0 ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=f32, device=dev)
        rec(f"latent_norm_rope_cache_write, rank {rank} + {rot} rotated: 2048 tokens",
            tm.run(lambda: kernels.latent_norm_rope_cache_write(x, ones(rank), 1e-5, c1, pos, seq, tb1, bs, rank, rot, rot, invr, flag), 3, 10),
            bytes_=T * padded * 4, like="latent_norm_cache_write below")
        qh, qa = rnd(T, H * (dim + rot)), torch.empty(T, H * padded, dtype=bf, device=dev)
        rec(f"latent_query_rope, 32 heads, {rot} rotated values behind rank {rank}: 2048 tokens",
            tm.run(lambda: kernels.latent_query_rope(qa, qh, pos, H, dim, rot, rot, invr, rank, padded), 3, 10), bytes_=T * H * rot * 4)
    x = rnd(T, 128)
    c1, tb1 = _paged(dev, T, bs, 1, 128, 1, g)
    rec("latent_norm_cache_write (Vufolorn) rank 128: 2048 tokens",
        tm.run(lambda: kernels.latent_norm_cache_write(x, ones(128), 1e-5, c1, pos, seq, tb1, bs, 128, flag), 3, 10), bytes_=T * 128 * 4)
    gate = rnd(T, H)
    rec("head_gate_ (sigmoid gate per head after the fast attention kernels) 2048 x 32 x 128",
        tm.run(lambda: kernels.head_gate_(out, gate, H, dim), 3, 10), bytes_=T * H * dim * 4)
    # ---- the experts' activation with the routing weight inside
    pairs = T * top
    gu, act = rnd(pairs, 2 * ff), torch.empty(pairs, ff, dtype=bf, device=dev)
    pair_row = torch.randperm(pairs, device=dev, generator=g).to(i32).view(T, top)
    wts = torch.rand(T, top, device=dev, generator=g)
    rec(f"moe_weighted_glu (silu, weight on the input) {pairs} x {ff}",
        tm.run(lambda: kernels.moe_weighted_glu(act, gu, pair_row, wts, "silu"), 3, 10), bytes_=pairs * ff * 6, like="gated_act below")
    rec(f"gated_act (Llama, silu) {pairs} x {ff}", tm.run(lambda: kernels.gated_act(act, gu, "silu"), 3, 10), bytes_=pairs * ff * 6)
    return rows


def run(bench, steps, warmup, pk):
    sampler = bench.ClockSampler()
    sampler.start()
    sizes = {}
    for name, cfg in SIZES.items():
        sizes[name] = {"bedenex": measure_model(cfg, [8, 64], steps, warmup, bench),
                       "vufolorn": measure_model(design_bench.SIZES[name][0], [8, 64], steps, warmup, bench),
                       "llama": measure_model(design_bench.SIZES[name][1], [8, 64], steps, warmup, bench)}
    alone = kernels_alone(pk)
    line = {"metric": "prefill and decode tokens/s of the Bedenex design beside the Vufolorn design and the Llama shape of equal width "
                      "(4 layer runs each, random weights)",
            "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup, "dtype": "bf16", "data": "synthetic",
            "config": {"prefill_tokens": PREFILL_TOKENS, "context": CONTEXT, "block_size": BLOCK_SIZE, "sizes": SIZES,
                       "vufolorn": {k: v[0] for k, v in design_bench.SIZES.items()},
                       "llama": {k: v[1] for k, v in design_bench.SIZES.items()}, "peaks": pk.get("source", "measured")},
            "sizes": sizes, "kernels_alone": alone, "clocks": sampler.stop(), "impl": "ours"}
    print(json.dumps(line))
    return 0
