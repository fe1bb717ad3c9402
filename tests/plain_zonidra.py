"""A plain, slow implementation of the Zonidra design on whole sequences: one function per mechanism, float64 or
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


def embed(tokens, W, cfg, dtype):
    """Row of the token times a scale, plus a row of a second table chosen by the pair (token before, token); the
    sequence's first token takes that table's last row."""
    e = cfg["embedding"]
    b = e.get("bigram")
    x = W["embed"][tokens].to(dtype) * e.get("scale", 1.0)
    if b:
        rows = [b["buckets"] if i == 0 else (tokens[i - 1] * b["mul_prev"] + t * b["mul_cur"]) % b["buckets"]
                for i, t in enumerate(tokens)]
        x = x + W["bigram"][rows].to(dtype)
    return x


def token_shift(h, mix):
    """h_t + (h_{t-1} - h_t) * mix, h_{-1} = 0; the earlier token's h is the one before this replacement."""
    before = torch.cat([torch.zeros_like(h[:1]), h[:-1]], 0)
    return h + (before - h) * mix


def scaled_frequencies(rot, dtype):
    """base^(-2i/n), then stretched by wavelength: short waves stay, long ones are divided by `factor`, those between are
    interpolated."""
    n = rot["dims"]
    f = [rot["base"] ** (-2.0 * i / n) for i in range(n // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for v in f:
            wave = 2 * math.pi / v
            if wave < sc["original"] / sc["high"]:
                out.append(v)
            elif wave > sc["original"] / sc["low"]:
                out.append(v / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1 - s) * v / sc["factor"] + s * v)
        f = out
    return torch.tensor(f, dtype=dtype)


def rotate_front(x, positions, rot):
    """x [T, heads, d]: of the first `dims` values of every head, value i and value i + dims/2 turn by the angle
    position * f_i; the rest stays."""
    if not rot or not rot.get("dims"):
        return x
    n = rot["dims"]
    half = n // 2
    ang = positions.to(x.dtype)[:, None, None] * scaled_frequencies(rot, x.dtype)
    u, v = x[..., :half], x[..., half:n]
    return torch.cat([u * torch.cos(ang) - v * torch.sin(ang), v * torch.cos(ang) + u * torch.sin(ang), x[..., n:]], -1)


def visible(T, mask):
    """[query, key]: the key is not later than the query and either among the last `size` or among the first
    `keep_first` of the sequence."""
    p = torch.arange(T)
    d = p[:, None] - p[None, :]
    seen = d >= 0
    if mask and mask.get("size"):
        near = d < mask["size"]
        if mask.get("keep_first"):
            near = near | (p[None, :] < mask["keep_first"])
        seen = seen & near
    return seen


def keys_and_values(h, W, m):
    """What a layer with projections of its own puts into its cache: rotated keys [T, G, dk] and values [T, G, dv]."""
    T = h.shape[0]
    G, dk, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rotate_front((h @ W["k"].T).reshape(T, G, dk), torch.arange(T), m.get("rot"))
    v = (h @ W["v"].T).reshape(T, G, dv)
    return k, v


def sigmoid_attention_mixer(h, W, m, kv):
    """Grouped heads, the front of every head rotated, weights sigmoid(score * scale + bias of the head) that are not
    normalised over the keys, an element-wise sigmoid gate on the concatenated heads.  kv: (keys, values) of the layer
    whose cache this one reads, or None (then its own)."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = rotate_front((h @ W["q"].T).reshape(T, H, dk), torch.arange(T), m.get("rot"))
    k, v = kv if kv is not None else keys_and_values(h, W, m)
    seen = visible(T, m.get("mask"))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"] + W["pb"][hd]
        out[:, hd] = (sigmoid(s) * seen) @ v[:, g]
    out = out.reshape(T, H * dv) * sigmoid(h @ W["g"].T)
    return out @ W["o"].T, (k, v)


def poly_norm(z, coef, eps):
    """a N(z) + b N(z^2) + c N(z^3) + e, N: division by the root mean square over the row."""
    a, b, c, e = [coef[i] for i in range(4)]
    return a * rms_norm(z, None, eps) + b * rms_norm(z * z, None, eps) + c * rms_norm(z * z * z, None, eps) + e


def dense_feed_forward(h, W, eps):
    return poly_norm(h @ W["up"].T, W["act"], eps) @ W["down"].T


def gated_expert(h, W, prefix):
    return (silu(h @ W[prefix + "gate"].T) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def routed_feed_forward(h, W, f):
    """Scores: a softmax over all router outputs; the choice is made with a correction added, the weights are the plain
    scores times a constant; the last `identity` outputs stand for experts that return their input."""
    r = f["router"]
    E, I, top = r["experts"], r.get("identity", 0), r["top"]
    s = torch.softmax((h @ W["router"].T), -1)
    choice = s + W["correction"] if "correction" in W else s
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in torch.topk(choice[t], top).indices.tolist():
            w = s[t, e] * r.get("scale", 1.0)
            out[t] += w * (h[t] if e >= E else gated_expert(h[t:t + 1], W, f"e{e}.")[0])
    assert W["router"].shape[0] == E + I
    if f.get("shared"):
        out = out + sigmoid(h @ W["shared.sg"].T) * gated_expert(h, W, "shared.")
    return out


def sub(W, prefix):
    return {k[len(prefix):]: v for k, v in W.items() if k.startswith(prefix)}


def forward(cfg, W, tokens, dtype=torch.float64, layers_out=None):
    """logits [T, vocab] of one whole sequence; layers_out (a list) receives the stream after every layer."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in W.items()}
    eps = cfg["norm"]["eps"]
    x = embed(list(tokens), W, cfg, dtype)
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = L["mixer"]
        h = rms_norm(x, W[p + "norm1"], eps)
        if p + "shift" in W:
            h = token_shift(h, W[p + "shift"])
        a, kept[i] = sigmoid_attention_mixer(h, sub(W, p + "mix."), m, kept[m["kv_from"]] if m.get("kv_from") is not None else None)
        x = x + rms_norm(a, W[p + "norm1b"], eps) * W[p + "ls1"]
        f = L.get("mlp")
        if f is not None:
            h = rms_norm(x, W[p + "norm2"], eps)
            y = dense_feed_forward(h, sub(W, p + "mlp."), eps) if f["kind"] == "dense" else routed_feed_forward(h, sub(W, p + "mlp."), f)
            x = x + rms_norm(y, W[p + "norm2b"], eps) * W[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T


# ----------------------------------------------------------------------------- tensors of a configuration

def tensor_shapes(cfg):
    """{name: shape} of every tensor that a model of this configuration stores, from the configuration alone."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    b = cfg["embedding"].get("bigram")
    if b:
        out["bigram"] = (b["buckets"] + 1, D)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        out.update({p + "norm1": (D,), p + "norm1b": (D,), p + "ls1": (D,), p + "shift": (D,), p + "mix.q": (H * dk, D),
                    p + "mix.pb": (H,), p + "mix.g": (H * dv, D), p + "mix.o": (D, H * dv)})
        if m.get("kv_from") is None:
            out.update({p + "mix.k": (G * dk, D), p + "mix.v": (G * dv, D)})
        f = L.get("mlp")
        if f is None:
            continue
        out.update({p + "norm2": (D,), p + "norm2b": (D,), p + "ls2": (D,)})
        if f["kind"] == "dense":
            out.update({p + "mlp.up": (f["ff"], D), p + "mlp.down": (D, f["ff"]), p + "mlp.act": (4,)})
        else:
            r, F = f["router"], f["expert"]["ff"]
            R = r["experts"] + r.get("identity", 0)
            out.update({p + "mlp.router": (R, D), p + "mlp.correction": (R,)})
            for e in range(r["experts"]):
                out.update({p + f"mlp.e{e}.gate": (F, D), p + f"mlp.e{e}.up": (F, D), p + f"mlp.e{e}.down": (D, F)})
            if f.get("shared"):
                S = f["shared"]["ff"]
                out.update({p + "mlp.shared.gate": (S, D), p + "mlp.shared.up": (S, D), p + "mlp.shared.down": (D, S),
                            p + "mlp.shared.sg": (1, D)})
    return out


def random_weights(cfg, seed=0, std=None, dtype=torch.bfloat16):
    """Weights under which every mechanism moves the result: norm weights and layer scales around 1, shift vectors between 0
    and 1, biases per head of either sign, polynomial coefficients of order 1, corrections that change some choices."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.split(".")[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b", "norm", "ls1", "ls2"):
            t = 0.6 + 0.8 * torch.rand(shape, generator=g)
        elif last == "shift":
            t = torch.rand(shape, generator=g)
        elif last == "pb":
            t = torch.randn(shape, generator=g) - 1.0
        elif last == "act":
            t = torch.randn(shape, generator=g)
        elif last == "correction":
            t = 0.1 * torch.randn(shape, generator=g)
        elif name in ("embed", "bigram"):
            t = torch.randn(shape, generator=g) * (std or 0.5)
        else:
            t = torch.randn(shape, generator=g) * (std or 1.0 / math.sqrt(shape[-1]))
        W[name] = t.to(dtype)
    return W
