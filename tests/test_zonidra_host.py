"""Host side of the Zonidra design: its configuration, its description as data, its tensor names, what its cache keeps, and
the properties of the plain implementation that the GPU tests rest on."""
import copy
import json

import pytest
import torch

import plain_zonidra as P
from zonidra_configs import CONFIGS, attention, dense, embedding, with_mlp

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
    assert [c.cache_of for c in model.calls] == [None, 0, None, None]
    m0, m1 = model.blocks[0]._mixer, model.blocks[1]._mixer
    assert m0.own_kv and not m1.own_kv and m1.sigmoid_weights and m1.value_gate and m1.has_head_bias
    assert (m0.window, m0.keep_first, m1.window, m1.keep_first) == (21, 3, 50, 5)
    # the cache of layer 0 keeps what its reader sees: the wider window and the longer kept start
    groups, where = plan_groups(model)
    by_calls = {tuple(g.calls): (g.spec.num_kv_heads, g.spec.head_dim, g.spec.window, g.spec.keep_first) for g in groups}
    assert by_calls == {(0,): (2, 32, 50, 5), (2,): (2, 48, 9, 0), (3,): (1, 16, 33, 1)}
    assert where[1] == where[0]
    # every layer shifts its mixer's input and keeps a row per request for it; the embedding keeps the token before
    assert all(set(model.call_extra_state_specs(j)) == {"mixer_shift"} for j in range(4))
    assert model.call_extra_state_specs(0)["mixer_shift"].shape == (72,)
    assert model.embedding_state_spec().dtype == torch.int32
    assert model.blocks[2].feed_forward is None
    ff = model.blocks[0].feed_forward
    assert (ff.routing, ff.identity_experts, ff.route_scale, ff.shared_size, ff.gated) == ("softmax_all", 2, 1.7, 20, True)
    assert all(getattr(p, "graph_safe", False) for p, _ in model.parts_with_specs())


def test_a_reader_of_a_layer_that_sees_everything_leaves_its_cache_whole():
    from lmsf_b200.cache.storage import plan_groups
    _, model = build(CONFIGS["Y"])
    groups, _ = plan_groups(model)
    assert [(g.spec.window, g.spec.keep_first) for g in groups] == [(None, 0), (None, 0)]
    assert model.blocks[1]._mixer.window == 17 and model.blocks[1]._mixer.keep_first == 2


def test_tensor_names_and_shapes_are_those_of_the_design():
    from lmsf_b200.weights.loader import collect_requirements
    for name, cfg in CONFIGS.items():
        _, model = build(cfg)
        asked = {}
        for _, _, wspec, names in collect_requirements(model):
            asked.update(dict(zip(names, [tuple(s) for s in wspec.shapes])))
        want = {k: tuple(v) for k, v in P.tensor_shapes(cfg).items()}
        assert asked == want, (name, set(asked) ^ set(want))


@pytest.mark.parametrize("change,needle", [
    (lambda c: c["layers"][0].update(type="convolution"), "type"),
    (lambda c: c["layers"][0]["mixer"].pop("heads"), "heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("low"), "low"),
    (lambda c: c["layers"][0]["mixer"].update(kv_heads=3), "kv heads"),
    (lambda c: c["layers"][1]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=0), "kv_from"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=8), "top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="conv"), "kind"),
    (lambda c: c["embedding"]["bigram"].pop("mul_cur"), "mul_cur"),
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
    del w["l0.mix.pb"]
    w["l1.shift"] = torch.ones(3, dtype=torch.bfloat16)
    w["l1.mix.k"] = torch.ones(2, dtype=torch.bfloat16)            # a reader of another layer's cache stores no keys
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    write_safetensors(str(tmp_path / "model.safetensors"), [(n, t.dtype, tuple(t.shape)) for n, t in w.items()], lambda n: w[n])
    with pytest.raises(WeightError) as e:
        check_tensors(model, open_model_tensors(str(tmp_path)), str(tmp_path))
    assert e.value.missing == ["l0.mix.pb"] and e.value.unexpected == ["l1.mix.k"] and e.value.wrong_shape[0][0] == "l1.shift"


def test_a_window_group_keeps_the_pages_of_the_first_positions():
    from lmsf_b200.cache.manager import CacheManager, GroupSpec
    bs, w, keep = 4, 6, 5
    m = CacheManager([GroupSpec(window=w, keep_first=keep), GroupSpec(window=w)], [64, 64], block_size=bs, num_state_slots=1)
    m.add("a")
    total = 0
    for n in [3, 2, 9, 1, 1, 1, 17, 1, 30]:
        m.reserve("a", n)
        m.commit("a", n)
        total += n
        first_needed = max(0, total - w + 1) // bs
        kept = (keep + bs - 1) // bs
        t0, t1 = m.block_table("a", 0), m.block_table("a", 1)
        for i in range(len(t0)):
            assert (t0[i] >= 0) == (i < kept or i >= first_needed), (total, i, t0)
            assert (t1[i] >= 0) == (i >= first_needed), (total, i, t1)
        m.check_invariants()
    m.free("a")
    assert m.num_free_pages(0) == 64 and m.num_free_pages(1) == 64


def test_the_shift_reads_the_row_before_as_it_was_before_the_shift():
    g = torch.Generator().manual_seed(0)
    h, mix = torch.randn(6, 5, generator=g, dtype=torch.float64), torch.rand(5, generator=g, dtype=torch.float64)
    out = P.token_shift(h, mix)
    assert torch.allclose(out[0], h[0] * (1 - mix))                       # nothing before the first token: zeros
    for t in range(1, 6):
        assert torch.allclose(out[t], h[t] + (h[t - 1] - h[t]) * mix)
    chained = h.clone()                                                # the other reading, which the design does not mean
    for t in range(1, 6):
        chained[t] = h[t] + (chained[t - 1] - h[t]) * mix
    assert not torch.allclose(chained[2:], out[2:])


def test_the_window_keeps_the_first_tokens_at_their_places():
    seen = P.visible(12, {"size": 4, "keep_first": 2})
    assert seen[9].nonzero().flatten().tolist() == [0, 1, 6, 7, 8, 9]
    assert seen[3].nonzero().flatten().tolist() == [0, 1, 2, 3] and seen[1].nonzero().flatten().tolist() == [0, 1]
    assert P.visible(5, None).sum() == 15 and P.visible(5, {"size": 2}).sum() == 9


def test_weights_are_not_normalised_and_a_bias_of_a_head_moves_them_all():
    g = torch.Generator().manual_seed(1)
    D, T = 16, 9
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 4, "scale": 0.3}
    W = {"q": torch.randn(16, D, generator=g), "k": torch.randn(8, D, generator=g), "v": torch.randn(4, D, generator=g),
         "g": torch.zeros(8, D), "o": torch.eye(8), "pb": torch.tensor([0.0, 0.0])}
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(T, D, generator=g).double()
    a, _ = P.sigmoid_attention_mixer(h, W, m, None)
    # a key's weight is its own sigmoid whatever the other keys are: no denominator couples the weights
    k, v = P.keys_and_values(h, W, m)
    alone = 0.5 * P.sigmoid((h[T - 1] @ W["q"][:8].T) @ k[T - 1, 0] * 0.3) * v[T - 1, 0]
    assert torch.allclose(P.sigmoid_attention_mixer(h[T - 1:], W, m, None)[0][0, :4], alone)
    up, _ = P.sigmoid_attention_mixer(h, dict(W, pb=torch.tensor([300.0, -300.0]).double()), m, None)
    assert torch.allclose(up[:, 4:], torch.zeros(T, 4).double(), atol=1e-9)                  # a bias far below every score: the head is silent
    assert torch.allclose(up[T - 1, :4], 0.5 * v[:, 0].sum(0), atol=1e-9)                    # far above: every key counts fully
    wts = P.sigmoid((h[T - 1] @ W["q"][:8].T) @ k[:, 0].T * 0.3)
    assert torch.allclose(a[T - 1, :4], 0.5 * wts @ v[:, 0])


def test_outputs_behind_the_experts_return_the_input_and_the_correction_only_chooses():
    g = torch.Generator().manual_seed(2)
    D = 12
    f = {"kind": "moe", "expert": {"ff": 6}, "router": {"experts": 2, "top": 1, "identity": 2, "scale": 1.5}}
    W = {"router": torch.randn(4, D, generator=g), "correction": torch.zeros(4)}
    for e in range(2):
        W.update({f"e{e}.gate": torch.randn(6, D, generator=g), f"e{e}.up": torch.randn(6, D, generator=g), f"e{e}.down": torch.randn(D, 6, generator=g)})
    W = {k: v.double() for k, v in W.items()}
    h = torch.randn(5, D, generator=g).double()
    s = torch.softmax(h @ W["router"].T, -1)
    forced = dict(W, correction=torch.tensor([0.0, 0.0, 0.0, 9.0]).double())       # the last output always wins the choice ...
    out = P.routed_feed_forward(h, forced, f)
    assert torch.allclose(out, 1.5 * s[:, 3:4] * h)                                # ... and weighs by its plain score
    forced = dict(W, correction=torch.tensor([9.0, 0.0, 0.0, 0.0]).double())
    assert torch.allclose(P.routed_feed_forward(h, forced, f), 1.5 * s[:, 0:1] * P.gated_expert(h, W, "e0."))


def test_the_plain_model_is_causal_and_a_reader_sees_its_owner_keys():
    for name in ("X", "Y"):
        cfg = CONFIGS[name]
        w = P.random_weights(cfg, 3)
        toks = [(7 * i + 3) % cfg["vocab"] for i in range(40)]
        a = P.forward(cfg, w, toks)
        b = P.forward(cfg, w, toks[:25])
        assert torch.allclose(a[:25], b, atol=1e-9)
        other = dict(w)
        other["l0.mix.k"] = -w["l0.mix.k"]                                         # the reader (layer 1) follows its owner's keys
        layers_a, layers_b = [], []
        P.forward(cfg, w, toks, layers_out=layers_a)
        P.forward(cfg, dict(other, **{"l0.mix.q": -w["l0.mix.q"]}), toks, layers_out=layers_b)
        assert torch.allclose(layers_a[0], layers_b[0], atol=1e-9)                 # layer 0 itself: q and k both negated
        assert not torch.allclose(layers_a[1], layers_b[1], atol=1e-3)             # its reader: the keys alone changed


def test_a_design_without_a_pair_table_takes_the_plain_embedding():
    cfg = {"architecture": "Zonidra", "vocab": 50, "width": 16, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
           "layers": [with_mlp(attention(2, 1, 8, 8, 0.3), dense(12))]}
    typed, model = build(cfg)
    assert typed.pair_buckets == 0 and model.embedding_state_spec() is None and model.embedding.scale == 2.0
    cfg["embedding"] = embedding(1.0, 7, 3, 2)
    typed, model = build(cfg)
    assert (model.embedding.buckets, model.embedding.mul_prev, model.embedding.mul_cur) == (7, 3, 2)
