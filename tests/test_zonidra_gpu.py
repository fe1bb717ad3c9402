"""The Zonidra design on the GPU: every mechanism alone against the plain implementation (tests/plain_zonidra.py), then whole
models through the engine's step function in every way of cutting, long decoding, reuse of pages and slots, and generation."""
import math
import random

import numpy as np
import pytest
import torch

import plain_zonidra as P
import traces
import util
from test_bedenex_gpu import DEV, F32_TOL, TDT, _context, dev, i32, position_errors, worst_rel, write_model
from zonidra_configs import BLOCK, CONFIGS, attention, dense, embedding, moe, rotation, with_mlp

pytestmark = pytest.mark.gpu
_folders, _oracles = {}, {}


def folder_of(name, std=None):
    key = (name, std)
    if key not in _folders:
        w = P.random_weights(CONFIGS[name], seed=sum(map(ord, name)), std=std, dtype=torch.bfloat16)
        _folders[key] = (write_model(CONFIGS[name], w, f"lmsf_zon_{name}_"), w)
    return _folders[key]


def oracle(name, reqs, std=None):
    _, w = folder_of(name, std)
    out = {}
    for rid, toks in reqs.items():
        key = (name, std, tuple(toks))
        if key not in _oracles:
            _oracles[key] = P.forward(CONFIGS[name], w, toks, dtype=torch.float64).float().numpy()
        out[rid] = _oracles[key]
    return out


def requests_for(name, lengths, seed=0):
    return {f"q{i}": util.random_ids(n, CONFIGS[name]["vocab"], seed + 11 * i) for i, n in enumerate(lengths)}


def assert_close(rows, ref, dtype, what):
    """float32: every logit within 3e-5 of the largest.  bfloat16: a token whose rounded router scores choose another output
    moves far, in every way of cutting alike, so the bound is on the bulk of the positions; what bfloat16 could hide beyond
    that is tested on the mechanisms alone with inputs made to show it."""
    if dtype == "float32":
        assert worst_rel(rows, ref) <= F32_TOL, (what, worst_rel(rows, ref))
    else:
        e = position_errors(rows, ref)
        assert e[len(e) // 2] <= 3e-2 and e[int(0.9 * len(e))] <= 0.15, (what, e[len(e) // 2], e[int(0.9 * len(e))])


# ----------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("vocab,D,buckets,mp,mc", [(211, 72, 37, 5, 3), (130, 64, 1, 0, 1), (50000, 40, 4099, 1000003, 998244353),
                                                   (9, 10, 200, 1, 0)])
def test_the_pair_embedding_remembers_the_token_before_a_portion(dtype, vocab, D, buckets, mp, mc):
    """Two requests whose portions alternate, down to single tokens, in slots that a third request had used: the row of the
    pair table follows the token before, which is on the device between steps; a request's first token takes the last row."""
    from lmsf_b200.parts.embedding import PairTokenEmbedding
    g = torch.Generator().manual_seed(vocab)
    tdt = TDT[dtype]
    cfg = {"embedding": embedding(1.75, buckets, mp, mc)}
    W = {"embed": torch.randn(vocab, D, generator=g).to(tdt), "bigram": torch.randn(buckets + 1, D, generator=g).to(tdt)}
    part = PairTokenEmbedding(vocab, D, buckets, mp, mc, scale=1.75)
    part.set_weights({"weight": dev(W["embed"]), "pairs": dev(W["bigram"])})
    state = torch.full((4, 1), 7, dtype=torch.int32, device=DEV)              # stale tokens of whoever had the slots before
    toks = {0: util.random_ids(23, vocab, 1), 1: util.random_ids(17, vocab, 2)}
    want = {s: P.embed(t, {k: v.double() for k, v in W.items()}, cfg, torch.float64) for s, t in toks.items()}
    done = {0: 0, 1: 0}
    cuts = [(5, 1), (1, 1), (2, 7), (1, 0), (14, 1), (0, 7)]
    for a, b in cuts:
        seqs, ids = [], []
        for s, n in ((0, a), (1, b)):
            if n:
                seqs.append((s, done[s], n))
                ids += toks[s][done[s]:done[s] + n]
        ctx = _context([(d0, n) for _, d0, n in seqs], 16, 8, 0, tdt)
        ctx.token_ids = i32(ids)
        ctx.state_slot = i32([3 - s for s, _, _ in seqs])                     # the slots are not the batch's order
        ctx.embedding_state = state
        res, _ = part.forward_stream(ctx)
        assert int(ctx.error_flag.item()) == 0 and res.dtype == torch.float32
        at = 0
        for s, d0, n in seqs:
            got = res[at:at + n].cpu().double()
            assert float((got - want[s][d0:d0 + n]).abs().max()) <= 1e-6 * float(want[s].abs().max()), (s, d0, n)
            at += n
            done[s] += n
            assert int(state[3 - s, 0]) == toks[s][done[s] - 1]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("D", [72, 9, 256])
def test_the_shift_mixes_every_row_with_the_row_before_across_portions(dtype, D):
    """Whole, token by token, and in portions of two; two requests in one batch whose slots held another request's rows.  The
    state is exactly the rows' values, so no cut changes a bit."""
    from lmsf_b200.parts.shift import TokenShift
    g = torch.Generator().manual_seed(D)
    tdt = TDT[dtype]
    T = 31
    mix = torch.rand(D, generator=g).to(torch.bfloat16).float()
    part = TokenShift(D)
    part.set_weights({"mix": dev(mix)})
    part.prepare(tdt, torch.device(DEV))
    hs = [torch.randn(T, D, generator=g).to(tdt), torch.randn(T - 6, D, generator=g).to(tdt)]
    want = [P.token_shift(h.double(), mix.double()) for h in hs]
    outs = {}
    for cuts in ([(T, T - 6)], [(1, 1)] * (T - 6) + [(1, 0)] * 6, [(2, 3), (3, 2)] * 5 + [(6, 0)], [(T - 1, 0), (1, T - 6)]):
        state = torch.full((3, D), 5.0, dtype=torch.float32, device=DEV)
        done, got = [0, 0], [[], []]
        for cut in cuts:
            seqs = [(s, done[s], min(n, hs[s].shape[0] - done[s])) for s, n in enumerate(cut) if n and done[s] < hs[s].shape[0]]
            ctx = _context([(d0, n) for _, d0, n in seqs], 16, 8, 0, tdt)
            ctx.state_slot = i32([2 - s for s, _, _ in seqs])
            h = torch.cat([hs[s][d0:d0 + n] for s, d0, n in seqs])
            out = part.forward(ctx, dev(h), state).float().cpu()
            at = 0
            for s, d0, n in seqs:
                got[s].append(out[at:at + n])
                at += n
                done[s] += n
        outs[len(cuts)] = [torch.cat(x) for x in got]
        for s in range(2):
            assert outs[len(cuts)][s].shape[0] == hs[s].shape[0]
            tol = 1e-6 if dtype == "float32" else 8e-3
            assert float((outs[len(cuts)][s].double() - want[s]).abs().max()) <= tol * float(want[s].abs().max())
    first = outs[1]
    for other in outs.values():
        assert all(torch.equal(a, b) for a, b in zip(first, other))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,F", [(5, 100), (70, 384), (1, 7), (33, 1030)])
def test_the_polynomial_activation_norms_every_power(dtype, n, F):
    from lmsf_b200 import kernels
    g = torch.Generator().manual_seed(F)
    tdt = TDT[dtype]
    z = (torch.randn(n, F, generator=g) * 1.7).to(tdt)
    coef = torch.tensor([0.7, -1.3, 0.4, 0.25])
    out = torch.empty(n, F, dtype=tdt, device=DEV)
    kernels.poly_norm(out, dev(z), dev(coef), 1e-5)
    want = P.poly_norm(z.double(), coef.double(), 1e-5)
    # each power has its own norm: with one norm for the sum the result differs by far more than the bound
    one = P.rms_norm(0.7 * z.double() - 1.3 * z.double() ** 2 + 0.4 * z.double() ** 3, None, 1e-5) + 0.25
    tol = 2e-6 if dtype == "float32" else 8e-3
    assert float((one - want).abs().max()) > 0.2 * float(want.abs().max())
    assert float((out.float().cpu().double() - want).abs().max()) <= tol * float(want.abs().max())


def routed_part(f, D, W, tdt):
    from lmsf_b200.parts.moe import RoutedExperts
    r = f["router"]
    E, S = r["experts"], (f.get("shared") or {}).get("ff", 0)
    part = RoutedExperts(hidden_size=D, num_experts=E, top_k=r["top"], expert_size=f["expert"]["ff"], shared_size=S, activation="silu",
                         router_bias=True, shared_gate=True, routing="softmax_all", route_scale=r.get("scale", 1.0),
                         identity_experts=r.get("identity", 0))
    w = {"up": dev(torch.cat([W[f"e{e}.{n}"] for e in range(E) for n in ("gate", "up")]), tdt),
         "down": dev(torch.cat([W[f"e{e}.down"] for e in range(E)]), tdt),
         "router": dev(torch.cat([W["router"]] + ([W["shared.sg"]] if S else [])), tdt), "router_bias": dev(W["correction"].float())}
    if S:
        w.update(shared_up=dev(torch.cat([W["shared.gate"], W["shared.up"]]), tdt), shared_down=dev(W["shared.down"], tdt))
    part.set_weights(w)
    part.prepare(tdt, torch.device(DEV))
    return part


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,E,I,top,ff,shared", [(70, 5, 2, 2, 24, 20), (3, 1, 0, 1, 16, 0), (150, 3, 3, 6, 24, 8), (9, 12, 2, 3, 72, 0),
                                                 (1, 6, 1, 1, 8, 16), (40, 2, 5, 2, 32, 0)])
def test_routing_scores_all_outputs_and_some_return_the_input(dtype, n, E, I, top, ff, shared):
    """A softmax over experts and identity outputs together, a correction that changes the choice and not the weight, a
    constant on the weights, no renormalisation; the shared expert behind its own sigmoid.  The router's margins are wide, so
    bfloat16 chooses as the plain implementation does."""
    g = torch.Generator().manual_seed(n * 7 + E)
    D = 48
    tdt = TDT[dtype]
    f = moe(E, top, ff, I, 1.7, shared)
    W = {"router": torch.randn(E + I, D, generator=g) * 0.6, "correction": torch.randn(E + I, generator=g) * 0.15}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = (torch.randn(ff, D, generator=g) / 3, torch.randn(ff, D, generator=g) / 7,
                                                           torch.randn(D, ff, generator=g) / 6)
    if shared:
        W.update({"shared.gate": torch.randn(shared, D, generator=g) / 3, "shared.up": torch.randn(shared, D, generator=g) / 7,
                  "shared.down": torch.randn(D, shared, generator=g) / 6, "shared.sg": torch.randn(1, D, generator=g) / 4})
    W = {k: v.to(torch.bfloat16).float() for k, v in W.items()}
    h = torch.randn(n, D, generator=g).to(tdt)
    Wd = {k: v.double() for k, v in W.items()}
    want = P.routed_feed_forward(h.double(), Wd, f)
    if n > 8 and top < E + I:
        plain = P.routed_feed_forward(h.double(), dict(Wd, correction=torch.zeros(E + I, dtype=torch.float64)), f)
        assert float((plain - want).abs().max()) > 0.05 * float(want.abs().max())          # the correction changes choices
    got = routed_part(f, D, W, tdt).forward(None, dev(h)).float().cpu().double()
    err = (got - want).abs().max(dim=1).values / float(want.abs().max())
    if dtype == "float32":
        assert float(err.max()) <= 1e-5
    else:   # a token whose two best choice scores lie within bfloat16's rounding of the input may choose otherwise
        assert float(err.median()) <= 2e-2 and float((err > 3e-2).float().mean()) <= 0.1


def attention_parts(ms, D, Ws, tdt):
    """The parts of layers that share one cache: ms[0] owns it, the others read it."""
    from lmsf_b200.parts.attention import PagedAttention
    from lmsf_b200.parts.rope import RotaryEmbedding
    parts = []
    for i, (m, W) in enumerate(zip(ms, Ws)):
        rot, mask = m.get("rot"), m.get("mask") or {}
        rope = None
        if rot:
            sc = rot.get("scaling")
            rope = RotaryEmbedding(rot["dims"], rot["base"], True, **(dict(scaling_type="llama3", factor=sc["factor"], low_freq_factor=sc["low"],
                                                                        high_freq_factor=sc["high"],
                                                                        original_max_position_embeddings=sc["original"]) if sc else {}))
        wide = max((x.get("mask") or {}).get("size") or 10 ** 9 for x in ms)
        part = PagedAttention(D, m["heads"], m["kv_heads"], m["dim"], position_encoding=rope, window=mask.get("size"),
                              keep_first=mask.get("keep_first", 0), scale=m["scale"], value_dim=m["vdim"], score_weights="sigmoid",
                              head_bias=True, value_gate=True, own_kv=i == 0, cache_window=None if wide == 10 ** 9 else wide,
                              cache_keep_first=max((x.get("mask") or {}).get("keep_first", 0) for x in ms))
        merged = [W["q"]] + ([W["k"], W["v"]] if i == 0 else []) + [W["g"]]
        part.set_weights({"qkv": dev(torch.cat(merged), tdt), "o": dev(W["o"], tdt), "head_bias": dev(W["pb"].float())})
        part.prepare(tdt, torch.device(DEV))
        parts.append(part)
    return parts


def attention_weights(g, D, m, own=True, bias=-1.0):
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    W = {"q": torch.randn(H * dk, D, generator=g) / math.sqrt(D), "g": torch.randn(H * dv, D, generator=g) / math.sqrt(D),
         "o": torch.randn(D, H * dv, generator=g) / math.sqrt(H * dv), "pb": torch.randn(H, generator=g) + bias}
    if own:
        W.update(k=torch.randn(G * dk, D, generator=g) / math.sqrt(D), v=torch.randn(G * dv, D, generator=g) / math.sqrt(D))
    return {n: t.to(torch.bfloat16).float() for n, t in W.items()}


def run_in_cuts(parts, hs, cuts, bs, tdt, pages=40, seed=9):
    """The parts' outputs for a sequence run in portions `cuts` over one fresh cache that the first part owns."""
    from lmsf_b200.parts.base import LayerCache
    head_dim, G = parts[0].head_dim, parts[0].num_kv_heads
    kv = torch.zeros((pages, 2, G, bs, head_dim), dtype=tdt, device=DEV)
    outs, done = [[] for _ in parts], 0
    for c in cuts:
        ctx = _context([(done, c)], bs, pages, seed, tdt)
        for i, (part, h) in enumerate(zip(parts, hs)):
            outs[i].append(part.forward(ctx, dev(h[done:done + c]), LayerCache(kv=kv, group=0, owner=i == 0)).float().cpu())
        assert int(ctx.error_flag.item()) == 0
        done += c
    return [torch.cat(o).double() for o in outs]


SHAPES = [  # heads, kv heads, dim, vdim, window, keep_first, rotation, page size
    (4, 2, 24, 16, 21, 3, rotation(8, 300.0, (3.0, 1.0, 5.0, 40)), 8),
    (4, 1, 64, 48, 50, 0, rotation(64, 10000.0), 16),
    (2, 2, 128, 64, 150, 6, rotation(48, 5.0e5, (2.0, 1.0, 8.0, 512)), 16),
    (3, 3, 40, 24, None, 0, None, 16),
    (6, 2, 20, 80, 7, 1, rotation(2, 50.0), 16),
    (2, 1, 64, 64, 70, 130, rotation(16, 500.0), 32),
    (5, 5, 144, 130, 33, 40, rotation(144, 10000.0), 16),
    (8, 2, 128, 128, 200, 17, rotation(64, 10000.0), 16),
]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,G,dk,dv,window,keep,rot,bs", SHAPES)
def test_sigmoid_attention_in_portions_and_token_by_token(dtype, H, G, dk, dv, window, keep, rot, bs):
    """Sigmoid weights with a bias per head, a window that keeps the first tokens (shorter and longer than the window, than a
    page, than a tile of keys), a rotated front of the heads, the element-wise gate; and a second layer with a wider mask that
    reads the first one's keys and values.  Whole, with the last tokens one by one, and in portions that cut anywhere."""
    g = torch.Generator().manual_seed(H * 100 + dk)
    tdt = TDT[dtype]
    D, T = 56, 341
    m = attention(H, G, dk, dv, 1.5 / math.sqrt(dk), window, keep, rot)["mixer"]
    reader = attention(H, G, dk, dv, 1.0 / math.sqrt(dk), window and 2 * window + 3, keep and keep + 2, rot, kv_from=0)["mixer"]
    Ws = [attention_weights(g, D, m), attention_weights(g, D, reader, own=False)]
    hs = [torch.randn(T, D, generator=g).to(tdt) for _ in range(2)]
    Wd = [{n: t.double() for n, t in W.items()} for W in Ws]
    want0, kv = P.sigmoid_attention_mixer(hs[0].double(), Wd[0], m, None)
    want1, _ = P.sigmoid_attention_mixer(hs[1].double(), Wd[1], reader, kv)
    parts = attention_parts([m, reader], D, Ws, tdt)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for cuts in ([T], [T - 40] + [1] * 40, [2, 7, 64, 3, 129, 2, 50, 1, 1, 82]):
        got = run_in_cuts(parts, hs, cuts, bs, tdt, pages=64 if bs == 8 else 32)
        for which, (a, b) in enumerate(zip(got, (want0, want1))):
            err = (a - b).abs().max(dim=1).values
            assert float(err.max()) <= tol * float(b.abs().max()), (which, cuts[:3], int(err.argmax()), float(err.max()))


def standing_out(g, D, m, T, far):
    """Weights and inputs under which the token at `far` is the key that the last query prefers by far, with a value that only
    a tag column sets: queries and keys share their weights and the heads' biases silence every other key."""
    W = attention_weights(g, D, m, bias=-7.0)
    dk = m["dim"]
    W["q"][:, D - 1] = 0
    W["k"] = W["q"][:dk].clone()
    W["v"][:, D - 1] = 1.0
    W["pb"][:] = -7.0
    h = torch.randn(T, D, generator=g)
    h[far, :D - 1] = h[T - 1, :D - 1]
    h[:, D - 1] *= 3
    h[T - 1, D - 1], h[far, D - 1] = 4.0, -4.0             # opposite tags of one size
    return {n: t.to(torch.bfloat16).float() for n, t in W.items()}, h


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("dk", [64, 48])
@pytest.mark.parametrize("T,far,seen", [(237, 187, True), (237, 186, False), (237, 191, True), (237, 192, True), (237, 235, True),
                                        (237, 2, True), (237, 3, False), (237, 0, True), (237, 15, False), (237, 100, False),
                                        (30, 0, True), (51, 0, True), (52, 1, True), (54, 3, False), (54, 4, True)])
def test_a_key_stands_out_just_inside_the_window_or_the_kept_start_and_not_just_outside(dtype, dk, T, far, seen):
    """A window of 50 positions that keeps the first 3, over pages of 16: the key sits on the window's oldest position, on the
    one before it, at a page's edge, next to the query, on the last kept position, on the first that is not kept.  Run whole,
    with the last token alone, and cut right after the key."""
    g = torch.Generator().manual_seed(T + far)
    tdt = TDT[dtype]
    D, bs = 40, 16
    m = attention(2, 1, dk, 32, 16.0 / dk, 50, 3, rotation(4, 1.0e6))["mixer"]
    W, h = standing_out(g, D, m, T, far)
    h = h.to(tdt)
    Wd = {n: t.double() for n, t in W.items()}
    want = P.sigmoid_attention_mixer(h.double(), Wd, m, None)[0][T - 1]
    other = h.clone()
    other[far, :D - 1] = -other[far, :D - 1]
    miss = P.sigmoid_attention_mixer(other.double(), Wd, m, None)[0][T - 1]
    size = max(float(want.abs().max()), float(miss.abs().max()))
    moved = float((miss - want).abs().max()) / size
    assert (moved > 0.1) == seen, moved                # the key matters exactly when the design lets the query see it
    part = attention_parts([m], D, [W], tdt)
    tol = 2e-5 if dtype == "float32" else 3e-2
    for cuts in ([T], [T - 1, 1], [far + 1, T - far - 2, 1] if 0 < far < T - 3 else [3, T - 4, 1], [T - 20] + [1] * 20):
        got = run_in_cuts(part, [h], cuts, bs, tdt, pages=20)[0][-1]
        assert float((got - want).abs().max()) <= tol * size, (cuts[:3], float((got - want).abs().max()))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("far", [0, 1, 15, 16, 17, 255, 256, 300, 417])
def test_a_key_far_back_is_found_among_hundreds_at_and_around_page_borders(dtype, far):
    """No window: every earlier key is seen, and one of 420 carries the value."""
    g = torch.Generator().manual_seed(far)
    tdt = TDT[dtype]
    D, T, bs = 40, 420, 16
    m = attention(2, 1, 64, 24, 16.0 / 64, None, 0, rotation(4, 1.0e6))["mixer"]
    W, h = standing_out(g, D, m, T, far)
    h = h.to(tdt)
    Wd = {n: t.double() for n, t in W.items()}
    want = P.sigmoid_attention_mixer(h.double(), Wd, m, None)[0][T - 1]
    other = h.clone()
    other[far, :D - 1] = -other[far, :D - 1]
    miss = P.sigmoid_attention_mixer(other.double(), Wd, m, None)[0][T - 1]
    size = max(float(want.abs().max()), float(miss.abs().max()))
    assert float((want - miss).abs().max()) > 0.1 * size
    part = attention_parts([m], D, [W], tdt)
    tol = 5e-5 if dtype == "float32" else 3e-2
    for cuts in ([T], [T - 1, 1], [far + 1, T - far - 2, 1] if 0 < far < T - 3 else [3, T - 4, 1]):
        got = run_in_cuts(part, [h], cuts, bs, tdt, pages=30)[0][-1]
        assert float((got - want).abs().max()) <= tol * size, (cuts, float((got - want).abs().max()))


def test_the_stream_after_every_layer_is_the_plain_one():
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner, StepEntry
    folder, w = folder_of("X")
    toks = util.random_ids(67, CONFIGS["X"]["vocab"], 4)
    want = []
    P.forward(CONFIGS["X"], w, toks, dtype=torch.float64, layers_out=want)
    model, _, tdt = build_model(folder, "float32", DEV)
    runner = ModelRunner(model, tdt, torch.device(DEV), 8, num_blocks=32, max_num_seqs=2)
    mgr = runner.make_cache_manager()
    got = []
    model.layer_hook = lambda j, x, res: got.append(res.clone())
    mgr.add("a")
    runner.step([StepEntry("a", toks, [])], mgr)
    model.layer_hook = None
    assert len(got) == len(want) == 4
    for j, (a, b) in enumerate(zip(got, want)):
        assert float((a.cpu().double() - b).abs().max()) <= 2e-5 * float(b.abs().max()), j


# ----------------------------------------------------------------------------- whole models through the step function

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["X", "Y", "Z"])
def test_every_way_of_cutting_agrees_with_the_plain_implementation(name, dtype):
    """Whole prompts, prefill then token by token, portions of several sizes down to two tokens, and batches of unequal
    requests with few pages and three live requests (pages and slots are used again)."""
    folder, _ = folder_of(name)
    reqs = requests_for(name, [61, 5, 1, 130, 33, 18, 390 if name == "Z" else 77])
    ref = oracle(name, reqs)
    bs = BLOCK[name]
    modes = {"whole": traces.whole(reqs), "decode": traces.whole(reqs, tail=30), "portions": traces.portions(reqs, [2, 7, 3, 16, 2, 29]),
             "pairs": traces.portions(reqs, [2]), "mixed": traces.mixed(reqs, seed=4, max_live=3, tail=10)}
    got = {}
    for mode, steps in modes.items():
        out = traces.run_inprocess(folder, dtype, steps, bs, traces.max_live_tokens(steps, 64), max_live=3)
        got[mode] = traces.collect(steps, out)
        assert len(got[mode]) == sum(len(t) for t in reqs.values())
        assert_close(got[mode], ref, dtype, mode)
    if dtype == "float32":                            # a position's logits do not depend on the cut beyond rounding
        for mode in modes:
            for key, row in got[mode].items():
                assert np.abs(row - got["whole"][key]).max() <= 2e-5 * np.abs(got["whole"][key]).max(), (mode, key)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_passes_windows_and_pages_and_replays_graphs(dtype):
    """A short prompt, then 150 single tokens: every window passes over decoded tokens, pages behind them are given back, the
    kept first tokens stay; the decode steps are replayed from a CUDA graph and must equal the eager steps."""
    from lmsf_b200.engine.factory import build_model
    from lmsf_b200.engine.model_runner import ModelRunner, StepEntry
    folder, _ = folder_of("X")
    reqs = requests_for("X", [160, 158], seed=3)
    ref = oracle("X", reqs)
    model, _, tdt = build_model(folder, dtype, DEV)
    assert all(getattr(p, "graph_safe", False) for p, _ in model.parts_with_specs())
    rows = {}
    for eager in (False, True):
        runner = ModelRunner(model, tdt, torch.device(DEV), 8, num_blocks=48, max_num_seqs=3, enforce_eager=eager)
        mgr = runner.make_cache_manager()
        for rid in reqs:
            mgr.add(rid)
        runner.step([StepEntry(rid, reqs[rid][:8], []) for rid in reqs], mgr)
        got = {rid: [] for rid in reqs}
        for t in range(8, 158):
            lg = runner.step([StepEntry(rid, [reqs[rid][t]], [0]) for rid in reqs], mgr)
            for j, rid in enumerate(reqs):
                got[rid].append(lg[j].float().cpu().numpy())
        assert (len(runner._graphs) > 0) == (not eager)
        # the windows have let pages go, the kept first positions have not
        t0 = mgr.block_table("q0", 0)
        assert t0[0] >= 0 and -1 in t0
        rows[eager] = got
        for rid in reqs:
            mgr.free(rid)
    for rid in reqs:
        scale = float(np.abs(ref[rid]).max())
        for i, (a, b) in enumerate(zip(rows[False][rid], rows[True][rid])):
            if dtype == "float32":
                assert np.abs(a - ref[rid][8 + i]).max() <= F32_TOL * scale, (rid, i)
            assert np.abs(a - b).max() <= 1e-5 * scale
    if dtype == "bfloat16":
        e = position_errors({(rid, 8 + i): a for rid in reqs for i, a in enumerate(rows[False][rid])}, ref)
        assert e[len(e) // 2] <= 3e-2 and e[int(0.9 * len(e))] <= 0.15


def test_pages_and_slots_of_a_finished_request_serve_the_next():
    """One live request at a time, pages for one and ONE state slot: the second request gets the pages, the shift rows and the
    remembered token of the first, none of which it may see."""
    folder, _ = folder_of("Y")
    reqs = requests_for("Y", [40, 40, 33], seed=9)
    ref = oracle("Y", reqs)
    steps = traces.portions(reqs, [13, 2])
    out = traces.run_inprocess(folder, "float32", steps, 16, 64, max_live=1)
    assert worst_rel(traces.collect(steps, out), ref) <= F32_TOL


def test_a_request_that_is_dropped_starts_again_from_nothing():
    folder, _ = folder_of("X")
    reqs = requests_for("X", [70, 45], seed=6)
    ref = oracle("X", reqs)
    steps = traces.dropped_and_replayed(reqs, "q0", 31)
    out = traces.run_inprocess(folder, "float32", steps, 8, 2 * traces.max_live_tokens(steps, 64), max_live=2)
    rows = traces.collect(steps, out)
    assert worst_rel(rows, ref) <= F32_TOL


def test_larger_weights_keep_the_comparison_sharp():
    folder, _ = folder_of("Z", std=0.3)
    reqs = requests_for("Z", [190, 17], seed=5)
    ref = oracle("Z", reqs, std=0.3)
    steps = traces.mixed(reqs, seed=1, max_live=2, tail=6)
    out = traces.run_inprocess(folder, "float32", steps, 16, traces.max_live_tokens(steps, 64), max_live=2)
    assert worst_rel(traces.collect(steps, out), ref) <= 6e-5


def test_the_trace_program_runs_the_design():
    folder, _ = folder_of("Y")
    reqs = requests_for("Y", [30, 9], seed=2)
    ref = oracle("Y", reqs)
    steps = traces.mixed(reqs, seed=3, max_live=2, tail=4)
    out = traces.run_program(folder, "float32", steps, traces.max_live_tokens(steps, 64))
    assert worst_rel(traces.collect(steps, out), ref) <= F32_TOL


def test_greedy_generation_through_the_engine():
    """The generation entry point with its scheduler, continuous batching, steps launched before the last one's tokens are
    read (the token before a step's token is then known on the device alone) and sampler: greedy tokens in float32 equal those
    of the plain implementation fed its own tokens back."""
    from lmsf_b200 import LLM, SamplingParams
    folder, w = folder_of("X")
    cfg = CONFIGS["X"]
    prompts = [util.random_ids(n, cfg["vocab"], 50 + i) for i, n in enumerate([23, 4, 41])]
    llm = LLM(folder, dtype="float32", block_size=8, num_gpu_blocks=48, max_num_batched_tokens=24, max_num_seqs=3)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    for p, o in zip(prompts, outs):
        toks = list(p)
        for _ in range(12):
            lg = P.forward(cfg, w, toks, dtype=torch.float64)[-1]
            nxt = int(lg.argmax())
            got = o.outputs[0].token_ids[len(toks) - len(p)]
            if got != nxt:                             # only a near tie may be decided otherwise
                assert float(lg[nxt] - lg[got]) <= 1e-4 * float(lg.abs().max())
            toks.append(got)


def test_preemption_by_recompute_rebuilds_pages_and_state():
    """With few pages the youngest request is dropped and later recomputed from its prompt and its tokens so far: its pages,
    its shift rows and its remembered token start again from nothing.  Greedy and seeded sampling give the tokens of a run with
    room for all, synchronous or with steps launched ahead."""
    from lmsf_b200 import LLM, SamplingParams
    folder, _ = folder_of("X")
    cfg = CONFIGS["X"]
    prompts = [util.random_ids(n, cfg["vocab"], 20 + i) for i, n in enumerate([30, 25, 28, 20])]
    sp = [SamplingParams(temperature=0.7 if i % 2 else 0.0, seed=5 + i, max_tokens=40, ignore_eos=True) for i in range(4)]
    roomy = LLM(folder, dtype="float32", block_size=8, num_gpu_blocks=128, max_num_batched_tokens=32, max_num_seqs=4)
    want = [o.outputs[0].token_ids for o in roomy.generate(prompt_token_ids=prompts, sampling_params=sp)]
    assert roomy.engine.scheduler.num_preemptions == 0
    for ahead in (True, False):
        tight = LLM(folder, dtype="float32", block_size=8, num_gpu_blocks=14, max_num_batched_tokens=32, max_num_seqs=4,
                    async_scheduling=ahead)
        got = [o.outputs[0].token_ids for o in tight.generate(prompt_token_ids=prompts, sampling_params=sp)]
        assert tight.engine.scheduler.num_preemptions > 0
        assert got == want, ahead
        tight.engine.cache.check_invariants()
        assert all(tight.engine.cache.num_free_pages(g) == 14 for g in range(len(tight.engine.cache.groups)))


def test_the_example_program_generates_with_the_design():
    """bin/llm_engine_example as a process: a model folder and prompts in, one JSON line per request out; top-k sampling with a
    seed gives the same tokens twice, and greedy tokens are the plain implementation's."""
    import json
    import os
    import subprocess
    import sys
    folder, w = folder_of("Y")
    cfg = CONFIGS["Y"]
    prompts = [util.random_ids(n, cfg["vocab"], 90 + i) for i, n in enumerate([7, 33])]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(*options):
        cmd = [sys.executable, os.path.join(root, "bin", "llm_engine_example"), "--model", folder, "--dtype", "float32",
               "--block-size", "16", "--num-gpu-blocks", "32", "--max-num-seqs", "4", "--max-num-batched-tokens", "24",
               "--max-tokens", "8", "--ignore-eos", *options]
        for p in prompts:
            cmd += ["--prompt-ids", ",".join(str(t) for t in p)]
        proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, timeout=300)
        assert proc.returncode == 0, proc.stderr[-2000:]
        lines = [json.loads(ln) for ln in proc.stdout.splitlines() if ln.startswith("{")]
        return {d["request_id"]: d["token_ids"] for d in lines}

    greedy = run("--temperature", "0")
    for i, p in enumerate(prompts):
        toks = list(p)
        for got in greedy[i]:
            lg = P.forward(cfg, w, toks, dtype=torch.float64)[-1]
            nxt = int(lg.argmax())
            assert got == nxt or float(lg[nxt] - lg[got]) <= 1e-4 * float(lg.abs().max())
            toks.append(got)
    sampled = run("--temperature", "0.8", "--top-k", "5", "--seed", "3")
    assert sampled == run("--temperature", "0.8", "--top-k", "5", "--seed", "3") and sampled != greedy


# ----------------------------------------------------------------------------- random configurations

def random_config(seed):
    """Sizes that are no multiples of anything in particular, every optional piece present or absent by chance, readers of
    earlier layers with masks of their own, values that a hand-made configuration tends to make equal or 1."""
    rng = random.Random(seed)
    width = rng.choice([36, 50, 56, 72, 104, 140])
    layers, owners = [], []
    for i in range(rng.randint(1, 5)):
        window = rng.choice([None, 1, 5, 16, 31, 64, 100])
        keep = rng.choice([0, 1, 2, 9, 40]) if window else 0
        if owners and rng.random() < 0.4:
            j = rng.choice(owners)
            o = layers[j]["mixer"]
            mixer = attention(o["heads"], o["kv_heads"], o["dim"], o["vdim"], rng.choice([0.1, 0.3]), window, keep, o.get("rot"), kv_from=j)
        else:
            kv = rng.randint(1, 3)
            dim = rng.choice([8, 12, 16, 24, 40, 64, 128])
            rot = rng.choice([None, rotation(rng.choice([2, 4, 8]), rng.choice([50.0, 1.0e4, 1.0e6])),
                              rotation(dim - dim % 2, 1.0e4, (rng.choice([2.0, 8.0]), 1.0, rng.choice([2.0, 4.0]), rng.choice([16, 64, 1024])))])
            mixer = attention(kv * rng.randint(1, 3), kv, dim, rng.choice([8, 16, 20, 40, 64]), rng.choice([0.1, 0.3, dim ** -0.5]), window, keep, rot)
            owners.append(i)
        r = rng.random()
        if r < 0.2:
            mlp = None
        elif r < 0.5:
            mlp = dense(rng.choice([8, 20, 44, 100]))
        else:
            experts, identity = rng.randint(1, 7), rng.choice([0, 0, 1, 3])
            mlp = moe(experts, rng.randint(1, experts + identity), rng.choice([8, 16, 24, 40]), identity, rng.choice([1.0, 2.0, 0.5]),
                      rng.choice([0, 8, 24]))
        layers.append(with_mlp(mixer, mlp))
    vocab = rng.choice([61, 128, 257])
    return {"architecture": "Zonidra", "vocab": vocab, "width": width, "norm": {"eps": rng.choice([1e-6, 1e-5, 1e-3])},
            "embedding": embedding(rng.choice([1.0, 4.0, 12.0]), rng.choice([1, 7, 64, 521]), rng.randint(0, 40), rng.randint(0, 40)),
            "layers": layers}


@pytest.mark.parametrize("seed", range(12))
def test_random_configurations(seed):
    name = f"R{seed}"
    CONFIGS[name] = random_config(seed)
    folder, w = folder_of(name)
    rng = random.Random(seed)
    reqs = requests_for(name, [rng.randint(1, 150) for _ in range(4)], seed=seed)
    ref = oracle(name, reqs)
    # how far the plain implementation itself moves when it is run in float32
    scale = max(float(np.abs(r).max()) for r in ref.values())
    cond = max(float(np.abs(P.forward(CONFIGS[name], w, toks, dtype=torch.float32).numpy() - ref[rid]).max()) for rid, toks in reqs.items()) / scale
    bs = rng.choice([8, 16, 32])
    for dtype in ("float32", "bfloat16"):
        for steps in (traces.whole(reqs, tail=5), traces.mixed(reqs, seed=seed, max_live=2, tail=4)):
            out = traces.run_inprocess(folder, dtype, steps, bs, traces.max_live_tokens(steps, 64), max_live=2)
            rows = traces.collect(steps, out)
            if dtype == "float32":
                assert worst_rel(rows, ref) <= max(5e-5, 3 * cond), (CONFIGS[name], worst_rel(rows, ref), cond)
            else:
                e = position_errors(rows, ref)
                assert e[len(e) // 2] <= 4e-2, (CONFIGS[name], e[len(e) // 2])
