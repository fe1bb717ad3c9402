"""Host side of the Bedenex design: its configuration, its description as data, its tensor names, and the identities
that the engine's kernels rest on, checked on the plain implementation alone."""
import copy
import json
import math

import pytest
import torch

import plain_bedenex as P
from bedenex_configs import CONFIGS

CFG = CONFIGS["X"]


def build(cfg):
    from lmsf_b200.config.registry import resolve_architecture
    from lmsf_b200.parts.decoder import DecoderModel
    arch = resolve_architecture(cfg)
    typed = arch.parse_config(cfg)
    return typed, DecoderModel(arch.build_spec(typed))


def test_the_design_is_found_by_its_name_and_described_as_data():
    from lmsf_b200.cache.storage import plan_groups
    typed, model = build(CFG)
    assert typed.has_loop and (typed.loop_start, typed.loop_stop, typed.loop_times) == (1, 3, 2)
    # layer 0, then the span twice (each pass enters through the projection of [stream | embedding]), then layer 3
    assert [(c.layer, c.entry, c.entry_pass) for c in model.calls] == \
        [(0, None, 0), (1, 0, 0), (2, None, 0), (1, 0, 1), (2, None, 0), (3, None, 0)]
    groups, _ = plan_groups(model)
    # every run of a layer owns a cache (runs of one geometry share a block table); the latent layers cache one plane of
    # rank + rotated part, padded to 16; both attention layers pad their heads to 32 values
    by_calls = {tuple(g.calls): (g.spec.num_kv_heads, g.spec.head_dim, g.spec.planes) for g in groups}
    assert by_calls == {(0,): (1, 48, 1), (1, 2, 3, 4): (2, 32, 2), (5,): (1, 32, 1)}
    assert all(g.spec.window is None for g in groups)              # chunks keep their pages: a request may be cut anywhere
    assert model.blocks[2].feed_forward is None and model.blocks[0].feed_forward.weight_on_input
    assert [model.blocks[i]._mixer.chunk for i in (1, 2)] == [12, 7]


def test_tensor_names_and_shapes_are_those_of_the_design():
    from lmsf_b200.weights.loader import collect_requirements
    for name, cfg in CONFIGS.items():
        _, model = build(cfg)
        asked = {}
        for _, _, wspec, names in collect_requirements(model):
            asked.update(dict(zip(names, [tuple(s) for s in wspec.shapes])))
        want = {k: tuple(v) for k, v in P.tensor_shapes(cfg).items()}
        # a layer without feed-forward has no second gate; nothing of it is asked for
        assert asked == want, (name, set(asked) ^ set(want))


def test_without_a_span_nothing_is_projected_and_no_vector_is_asked_for():
    typed, model = build(CONFIGS["Y"])
    assert not typed.has_loop and model.entries == [] and [c.layer for c in model.calls] == [0, 1]
    cfg = copy.deepcopy(CFG)
    cfg["loop"] = {"start": 2, "stop": 2, "times": 5}             # an empty span is no span
    typed, model = build(cfg)
    assert not typed.has_loop and model.entries == []


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "kv heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=6), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "kind"),
    (lambda c: c.update(loop={"start": 2, "stop": 5, "times": 2}), "loop"),
    (lambda c: c.pop("width"), "width"),
    (lambda c: c["norm"].update(eps=0), "eps"),
])
def test_a_configuration_that_does_not_fit_is_refused_with_its_key(change, needle):
    from lmsf_b200.config import ConfigError
    cfg = copy.deepcopy(CFG)
    change(cfg)
    with pytest.raises(ConfigError) as e:
        build(cfg)
    assert needle in str(e.value)


def test_missing_and_misshapen_tensors_are_reported_together(tmp_path):
    from lmsf_b200.weights.loader import WeightError, check_tensors
    from lmsf_b200.weights.safetensors_io import open_model_tensors, write_safetensors
    _, model = build(CFG)
    w = P.random_weights(CFG, 0)
    del w["l0.mix.sink"]
    w["l1.mix.r1"] = torch.ones(3, dtype=torch.bfloat16)
    w["l9.extra"] = torch.ones(2, dtype=torch.bfloat16)
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    write_safetensors(str(tmp_path / "model.safetensors"), [(n, t.dtype, tuple(t.shape)) for n, t in w.items()], lambda n: w[n])
    with pytest.raises(WeightError) as e:
        check_tensors(model, open_model_tensors(str(tmp_path)), str(tmp_path))
    assert e.value.missing == ["l0.mix.sink"] and e.value.unexpected == ["l9.extra"] and e.value.wrong_shape[0][0] == "l1.mix.r1"


def test_attention_on_the_cached_row_equals_attention_on_expanded_keys_and_values():
    """q_plain . (Wuk c) + q_rot . k_rot = [Wuk^T q_plain | q_rot] . [c | k_rot], and sum p (Wuv c) = Wuv (sum p c): the
    identity behind caching one row [c | k_rot] per token; the sink only joins the denominator."""
    g = torch.Generator().manual_seed(0)
    m = CFG["layers"][0]["mixer"]
    H, dk, dr, dv, r, D, T = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], 24, 15
    W = {"q": torch.randn(H * (dk + dr), D, generator=g), "dkv": torch.randn(r + dr, D, generator=g),
         "dkv.norm": torch.rand(r, generator=g) + 0.5, "uk": torch.randn(H * dk, r, generator=g),
         "uv": torch.randn(H * dv, r, generator=g), "sink": torch.randn(H, generator=g), "o": torch.randn(D, H * dv, generator=g)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(T, D, generator=g).double()
    want = P.latent_attention_mixer(h, W, m, 1e-5)
    pos = torch.arange(T)
    d = h @ W["dkv"].T
    row = torch.cat([P.rms_norm(d[:, :r], W["dkv.norm"], 1e-5), P.rotate_halves(d[:, r:], pos, m["rot"]["base"])], -1)
    q = (h @ W["q"].T).view(T, H, dk + dr)
    out = torch.zeros(T, H, dv, dtype=torch.float64)
    for i in range(T):
        for hd in range(H):
            qa = torch.cat([W["uk"][hd * dk:(hd + 1) * dk].T @ q[i, hd, :dk],
                            P.rotate_halves(q[i:i + 1, hd, dk:], pos[i:i + 1], m["rot"]["base"])[0]])
            s = (row[:i + 1] @ qa) * m["scale"]
            e = torch.exp(s)
            p = e / (e.sum() + torch.exp(W["sink"][hd]))
            out[i, hd] = W["uv"][hd * dv:(hd + 1) * dv] @ (p @ row[:i + 1, :r])
    assert torch.allclose(out.view(T, H * dv) @ W["o"].T, want, rtol=1e-9, atol=1e-9)


def test_a_sink_takes_weight_away_and_a_far_sink_changes_nothing():
    s = torch.tensor([[0.3, -1.0, 2.0]], dtype=torch.float64)
    seen = torch.ones(1, 3, dtype=torch.bool)
    p = P.softmax_with_sink(s, seen, 1.5)
    assert abs(float(p.sum()) - float(torch.exp(s).sum() / (torch.exp(s).sum() + math.exp(1.5)))) < 1e-12
    assert torch.allclose(P.softmax_with_sink(s, seen, -80.0), torch.softmax(s, -1), atol=1e-12)
    assert float(P.softmax_with_sink(s, seen, 80.0).sum()) < 1e-30         # a sink far above every score takes all


def test_chunks_count_from_position_zero_and_the_bias_grows_with_the_distance():
    """One key is made to stand out: a query of the same chunk finds it, the first query of the next chunk does not;
    with equal content the nearer of two keys gets the larger weight, by exactly (1 + r2 d)^-r1."""
    m = {"heads": 1, "kv_heads": 1, "dim": 4, "vdim": 4, "scale": 1.0, "mask": {"size": 5}}
    D, T = 4, 11
    eye = torch.eye(4, dtype=torch.float64)
    W = {"q": eye, "k": eye, "v": eye, "g": torch.zeros(1, 4, dtype=torch.float64), "o": eye,
         "r1": torch.tensor([0.7], dtype=torch.float64), "r2": torch.tensor([0.5], dtype=torch.float64)}
    h = torch.zeros(T, D, dtype=torch.float64)
    h[:, 0] = 1.0                                                          # every token alike: only the distance tells keys apart
    out = P.chunk_attention_mixer(h, W, m, 1e-6)
    assert torch.allclose(out[5], out[0])                                  # position 5 starts a chunk: it sees itself alone
    # weights of position 9 over keys 5..9
    dist = torch.arange(4, -1, -1, dtype=torch.float64)
    w = (1 + 0.5 * dist) ** -0.7
    v = P.rms_norm(h[:1], None, 1e-6)[0]
    assert torch.allclose(out[9], 0.5 * v * (w / w.sum()).sum())           # the gate is sigmoid(0)
    hot = h.clone()
    hot[4] = torch.tensor([0.0, 3.0, 0.0, 0.0])
    hot[9] = torch.tensor([0.0, 1.0, 0.0, 0.0])
    o2 = P.chunk_attention_mixer(hot, W, m, 1e-6)
    hot[5] = hot[4]
    o3 = P.chunk_attention_mixer(hot, W, m, 1e-6)
    assert float(o3[9, 1]) > float(o2[9, 1])                               # key 5 is inside position 9's chunk, key 4 is not


def test_the_expert_reads_its_input_times_the_score():
    """expert(w h) is not w expert(h): silu is not homogeneous, so the place of the weight shows."""
    g = torch.Generator().manual_seed(3)
    D, F, E = 8, 6, 3
    f = {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": 2}}
    W = {"router": torch.randn(E, D, generator=g).double()}
    for e in range(E):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = (torch.randn(*s, generator=g).double() for s in ((F, D), (F, D), (D, F)))
    h = torch.randn(4, D, generator=g).double()
    got = P.moe_feed_forward(h, W, f)
    s = P.sigmoid(h @ W["router"].T)
    val, idx = torch.topk(s, 2, dim=-1)
    inside, outside = torch.zeros_like(h), torch.zeros_like(h)
    for t in range(4):
        for j in range(2):
            e = int(idx[t, j])
            ex = lambda x: (P.silu(x @ W[f"e{e}.gate"].T) * (x @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
            inside[t] += ex(val[t, j] * h[t])
            outside[t] += val[t, j] * ex(h[t])
    assert torch.allclose(got, inside, rtol=1e-12, atol=1e-12) and not torch.allclose(got, outside, atol=1e-3)


def test_the_plain_model_is_causal_and_its_span_has_one_cache_per_pass():
    w = P.random_weights(CFG, 1, dtype=torch.float32)
    toks = [3, 9, 1, 44, 20, 7, 7, 30, 12, 5, 100, 2, 2, 61, 17]
    a = P.forward(CFG, w, toks)
    b = P.forward(CFG, w, toks[:9] + [1, 2, 3, 4, 5, 6])
    assert torch.allclose(a[:9], b[:9], rtol=1e-9, atol=1e-9) and not torch.allclose(a[9:], b[9:], atol=1e-3)
    more = copy.deepcopy(CFG)
    more["loop"]["times"] = 3
    w3 = dict(w, **{"loop.step": torch.cat([w["loop.step"], w["loop.step"][:1]])})
    assert not torch.allclose(P.forward(more, w3, toks), a, atol=1e-3)
    streams = []
    P.forward(CFG, w, toks, streams=streams)
    assert len(streams) == len(P.run_order(CFG)) == 6
