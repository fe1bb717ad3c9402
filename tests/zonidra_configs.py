"""Tiny Zonidra configurations for the tests: sizes that share nothing with each other, every branch of the design."""


def attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=0, rot=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window, "keep_first": keep_first}
    if rot:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def rotation(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, identity=0, scale=1.0, shared=0):
    f = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "identity": identity, "scale": scale}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


def embedding(scale, buckets, mul_prev, mul_cur):
    return {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


CONFIGS = {
    # experts first; a reader of layer 0 with a WIDER window and more kept tokens than its owner; a layer without feed-forward;
    # windows that no page or tile size divides; rotation of a part of the head with stretched frequencies
    "X": {"architecture": "Zonidra", "vocab": 211, "width": 72, "norm": {"eps": 1e-5}, "embedding": embedding(3.0, 37, 5, 3),
          "layers": [with_mlp(attention(4, 2, 24, 16, 0.2, 21, 3, rotation(8, 300.0, (3.0, 1.0, 5.0, 40))), moe(5, 2, 24, 2, 1.7, 20)),
                     with_mlp(attention(4, 2, 24, 16, 0.3, 50, 5, rotation(8, 300.0, (3.0, 1.0, 5.0, 40)), kv_from=0), dense(100)),
                     with_mlp(attention(2, 2, 32, 40, 0.25, 9, 0, rotation(32, 50.0)), None),
                     with_mlp(attention(6, 1, 16, 16, 0.35, 33, 1), dense(60))]},
    # one kv head for six query heads; every router output chosen; no identity output, no shared expert; a layer that sees
    # every earlier token read by a layer with a window; no rotation in one layer
    "Y": {"architecture": "Zonidra", "vocab": 130, "width": 64, "norm": {"eps": 1e-6}, "embedding": embedding(1.0, 1, 0, 1),
          "layers": [with_mlp(attention(6, 1, 16, 16, 0.4, None, 0, rotation(16, 10000.0)), moe(3, 3, 16)),
                     with_mlp(attention(6, 1, 16, 16, 0.2, 17, 2, rotation(16, 10000.0), kv_from=0), None),
                     with_mlp(attention(3, 3, 40, 24, 0.15), moe(1, 1, 32, 1, 3.0, 8))]},
    # head sizes of the tensor-core kernels with windows longer than a tile; more identity outputs than experts; two
    # readers of one layer
    "Z": {"architecture": "Zonidra", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "embedding": embedding(8.0, 101, 29, 11),
          "layers": [with_mlp(attention(4, 2, 64, 64, 0.125, 150, 6, rotation(32, 5.0e5, (6.0, 1.0, 3.0, 64))), dense(40)),
                     with_mlp(attention(4, 2, 64, 64, 0.2, 70, 130, rotation(32, 5.0e5, (6.0, 1.0, 3.0, 64)), kv_from=0), moe(2, 2, 32, 3, 0.7)),
                     with_mlp(attention(4, 2, 64, 64, 0.1, 300, 0, rotation(32, 5.0e5, (6.0, 1.0, 3.0, 64)), kv_from=0), moe(7, 1, 8, 0, 1.0, 24)),
                     with_mlp(attention(2, 1, 128, 48, 0.09, 129, 1, rotation(2, 100.0)), dense(72))]},
}
BLOCK = {"X": 8, "Y": 16, "Z": 16}
