"""Tiny Bedenex configurations for the tests: sizes that share nothing with each other, every branch of the design."""


def attention(heads, kv_heads, dim, vdim, scale, chunk=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    return {"type": "attention", "mixer": m}


def latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"dims": rot_dim, "base": base}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def with_mlp(layer, mlp):
    return dict(layer, mlp=mlp)


CONFIGS = {
    # a span of two layers in the middle that runs twice; a layer without feed-forward; chunks of 12 and of 7 positions
    "X": {"architecture": "Bedenex", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
          "layers": [with_mlp(latent(3, 24, 8, 20, 40, 0.2, 7000.0), moe(5, 2, 24)),
                     with_mlp(attention(4, 2, 16, 24, 0.3, 12), dense(100)),
                     with_mlp(attention(2, 2, 32, 16, 0.25, 7), None),
                     with_mlp(latent(2, 16, 12, 32, 20, 0.35, 100.0), dense(60))],
          "loop": {"start": 1, "stop": 3, "times": 2}},
    # no span; one kv head for six query heads; every expert chosen; one latent head with two rotated pairs
    "Y": {"architecture": "Bedenex", "vocab": 130, "width": 64, "norm": {"eps": 1e-6},
          "layers": [with_mlp(attention(6, 1, 16, 16, 0.4, 32), moe(3, 3, 16)),
                     with_mlp(latent(1, 32, 4, 8, 16, 0.18, 50000.0), None)]},
    # the whole model is the span, three times; an attention layer that sees every earlier token; one expert; head sizes
    # that 16 does not divide; a latent vector wider than the tensor-core kernels take
    "Z": {"architecture": "Bedenex", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
          "layers": [with_mlp(latent(5, 8, 6, 12, 130, 0.3, 300.0), dense(40)),
                     with_mlp(attention(3, 3, 40, 24, 0.15), moe(1, 1, 32)),
                     with_mlp(attention(2, 1, 64, 64, 0.125, 16), moe(7, 1, 8))],
          "loop": {"start": 0, "stop": 3, "times": 3}},
}
BLOCK = {"X": 8, "Y": 16, "Z": 16}
