"""A plain, slow implementation of the Bedenex design on whole sequences: one function per mechanism, float64 or
float32 on the CPU, no cache, no batching, nothing shared with the package.  The tests compare the engine with it.

A model is (config dict, {tensor name: tensor}).  Notation: T tokens, D width, x the residual stream [T, D].
"""
import math

import torch


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension; w None: no weight."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def sigmoid(z):
    return 1 / (1 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_halves(x, positions, base):
    """x [T, ..., n]: value i and value i + n/2 turn by the angle position * base^(-2i/n)."""
    n = x.shape[-1]
    half = n // 2
    freq = torch.tensor([base ** (-2.0 * i / n) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype).reshape(-1, *([1] * (x.dim() - 1))) * freq
    u, v = x[..., :half], x[..., half:]
    return torch.cat([u * torch.cos(ang) - v * torch.sin(ang), v * torch.cos(ang) + u * torch.sin(ang)], -1)


def softmax_with_sink(s, seen, sink):
    """Rows of s over the keys that `seen` allows; `sink` (a number, or None) joins the denominator as exp(sink)
    without a key or a value."""
    s = s.masked_fill(~seen, float("-inf"))
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, torch.full_like(m, float(sink)))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - m)
    return e / den


def latent_attention_mixer(h, W, m, eps):
    """Keys and values expanded from one normed low-rank vector per token; one rotated key part that all heads share;
    every earlier token is seen; a sink in the softmax."""
    T = h.shape[0]
    H, dk, dr, dv, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ W["q"].T).reshape(T, H, dk + dr)
    q_plain, q_rot = q[..., :dk], rotate_halves(q[..., dk:], pos, m["rot"]["base"])
    d = h @ W["dkv"].T
    c = rms_norm(d[:, :r], W["dkv.norm"], eps)
    k_rot = rotate_halves(d[:, r:], pos, m["rot"]["base"])               # [T, dr], the same for every head
    k_plain = (c @ W["uk"].T).reshape(T, H, dk)
    v = (c @ W["uv"].T).reshape(T, H, dv)
    seen = pos[None, :] <= pos[:, None]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        s = (q_plain[:, hd] @ k_plain[:, hd].T + q_rot[:, hd] @ k_rot.T) * m["scale"]
        out[:, hd] = softmax_with_sink(s, seen, W["sink"][hd]) @ v[:, hd]
    return out.reshape(T, H * dv) @ W["o"].T


def chunk_attention_mixer(h, W, m, eps):
    """Grouped heads, unit-RMS queries, keys and values, a bias that grows with the logarithm of the distance, keys of
    the query's own chunk of positions only, a sigmoid gate per head on the output."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rms_norm((h @ W["q"].T).reshape(T, H, dk), None, eps)
    k = rms_norm((h @ W["k"].T).reshape(T, G, dk), None, eps)
    v = rms_norm((h @ W["v"].T).reshape(T, G, dv), None, eps)
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).clamp(min=0).to(h.dtype)
    seen = pos[None, :] <= pos[:, None]
    size = (m.get("mask") or {}).get("size")
    if size:
        seen = seen & (pos[None, :] // size == pos[:, None] // size)
    gate = sigmoid(h @ W["g"].T)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] - W["r1"][hd] * torch.log(1 + W["r2"][hd] * dist)
        out[:, hd] = (softmax_with_sink(s, seen, None) @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv) @ W["o"].T


def dense_feed_forward(h, W):
    return (gelu_tanh(h @ W["gate"].T) * (h @ W["up"].T)) @ W["down"].T


def moe_feed_forward(h, W, f):
    """Every token goes to the `top` experts of largest sigmoid score; the score multiplies what the expert reads."""
    top = f["router"]["top"]
    s = sigmoid(h @ W["router"].T)
    val, idx = torch.topk(s, top, dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(top):
            e = int(idx[t, j])
            x = val[t, j] * h[t]
            out[t] += (silu(x @ W[f"e{e}.gate"].T) * (x @ W[f"e{e}.up"].T)) @ W[f"e{e}.down"].T
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x, cfg, weights, i):
    """x + gate1 * mixer(h) + gate2 * ff(h), h = norm(x): both branches read the same normed stream."""
    L = cfg["layers"][i]
    eps = cfg["norm"]["eps"]
    p = f"l{i}."
    h = rms_norm(x, weights[p + "norm1"], eps)
    mix = latent_attention_mixer if L["type"] == "latent_attention" else chunk_attention_mixer
    y = sigmoid(h @ weights[p + "rg1"].T + weights[p + "rg1.b"]) * mix(h, sub(weights, p + "mix."), L["mixer"], eps)
    if L.get("mlp"):
        W = sub(weights, p + "mlp.")
        f = dense_feed_forward(h, W) if L["mlp"]["kind"] == "dense" else moe_feed_forward(h, W, L["mlp"])
        y = y + sigmoid(h @ weights[p + "rg2"].T + weights[p + "rg2.b"]) * f
    return x + y


def run_order(cfg):
    """[(layer, number of the pass that starts here or None)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop["stop"] <= loop["start"]:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, weights, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one whole sequence.  `streams`: a list that receives x after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    x0 = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x = x0
    for i, start_of_pass in run_order(cfg):
        if start_of_pass is not None:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][start_of_pass]
        x = layer(x, cfg, W, i)
        if streams is not None:
            streams.append(x)
    return rms_norm(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T


def tensor_shapes(cfg):
    """{tensor name: shape} of a model of this configuration."""
    D, V = cfg["width"], cfg["vocab"]
    s = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    loop = cfg.get("loop")
    if loop and loop["stop"] > loop["start"]:
        s["loop.in"] = (D, 2 * D)
        s["loop.step"] = (loop["times"], D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        s[p + "norm1"] = (D,)
        s[p + "rg1"], s[p + "rg1.b"] = (D, D), (D,)
        H, dk, dv = m["heads"], m["dim"], m["vdim"]
        if L["type"] == "latent_attention":
            r, dr = m["kv_rank"], m["rot_dim"]
            s.update({p + "mix.q": (H * (dk + dr), D), p + "mix.dkv": (r + dr, D), p + "mix.dkv.norm": (r,),
                      p + "mix.uk": (H * dk, r), p + "mix.uv": (H * dv, r), p + "mix.sink": (H,), p + "mix.o": (D, H * dv)})
        else:
            G = m["kv_heads"]
            s.update({p + "mix.q": (H * dk, D), p + "mix.k": (G * dk, D), p + "mix.v": (G * dv, D), p + "mix.r1": (H,),
                      p + "mix.r2": (H,), p + "mix.g": (H, D), p + "mix.o": (D, H * dv)})
        f = L.get("mlp")
        if f:
            s[p + "rg2"], s[p + "rg2.b"] = (D, D), (D,)
            if f["kind"] == "dense":
                s.update({p + "mlp.gate": (f["ff"], D), p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"])})
            else:
                F = f["expert"]["ff"]
                s[p + "mlp.router"] = (f["router"]["experts"], D)
                for e in range(f["router"]["experts"]):
                    s.update({p + f"mlp.e{e}.gate": (F, D), p + f"mlp.e{e}.up": (F, D), p + f"mlp.e{e}.down": (D, F)})
    return s


def random_weights(cfg, seed=0, std=None, dtype=torch.bfloat16):
    """Weights whose branches all matter: matrices of standard deviation 1 / sqrt(columns) (or `std`), norm weights
    around 1, positive distance constants, sinks of a size that changes the softmax."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name.endswith(".norm"):
            t = 1 + 0.2 * torch.randn(shape, generator=g)
        elif name.endswith(".r1"):
            t = 0.3 + torch.rand(shape, generator=g)
        elif name.endswith(".r2"):
            t = 0.2 + torch.rand(shape, generator=g)
        elif name.endswith(".sink"):
            t = torch.randn(shape, generator=g)
        elif name.endswith(".b") or name == "loop.step":
            t = 0.3 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        elif name.endswith(".router"):
            t = torch.randn(shape, generator=g) * 2.0 / math.sqrt(shape[-1])
        else:
            t = torch.randn(shape, generator=g) * (std if std is not None else 1.0 / math.sqrt(shape[-1]))
        W[name] = t.to(dtype)
    return W
