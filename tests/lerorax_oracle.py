"""A plain, slow evaluation of the Lerorax design, written from its equations: one function per mechanism, loops over
tokens where the design is sequential, float64 by default.  It shares no code with the framework.

Weights are a dict of checkpoint-named tensors (``embed``, ``bigram``, ``l<i>.mix...``, ``head`` ...), linear weights
``[out, in]``.
"""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    return rms(x, eps) * (1 + w)


def bigram_rows(tokens, bg):
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(bg["buckets"] if t == 0 else (tokens[t - 1] * bg["mul_prev"] + tok * bg["mul_cur"]) % bg["buckets"])
    return rows


def short_conv(u, w):
    """y_t = sum_j w[:, j] * u_(t - taps + 1 + j), zeros before the start."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                y[t] += w[:, j] * u[s]
    return y


def rotary_frequencies(rot):
    dims = rot["dims"]
    out = []
    sc = rot.get("scaling")
    for i in range(dims // 2):
        f = rot["base"] ** (-2.0 * i / dims)
        if sc:
            lam = 2 * math.pi / f
            if lam > sc["original"] / sc["low"]:
                f = f / sc["factor"]
            elif lam >= sc["original"] / sc["high"]:
                s = (sc["original"] / lam - sc["low"]) / (sc["high"] - sc["low"])
                f = (1 - s) * f / sc["factor"] + s * f
        out.append(f)
    return out


def rotate(x, pos, freqs):
    """x [heads, dim]: pairs (2i, 2i + 1) of the first 2 * len(freqs) dimensions of every head."""
    y = x.clone()
    for i, f in enumerate(freqs):
        a = pos * f
        c, s = math.cos(a), math.sin(a)
        y[:, 2 * i] = x[:, 2 * i] * c - x[:, 2 * i + 1] * s
        y[:, 2 * i + 1] = x[:, 2 * i + 1] * c + x[:, 2 * i] * s
    return y


def head_mixing_attention(q, k, v, scale, talk):
    """q [T, H, d], k [T, G, d], v [T, G, dv]: causal softmax per head, weights mixed over heads, values of the own kv head."""
    T, H, _ = q.shape
    G, dv = k.shape[1], v.shape[2]
    rep = H // G
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for i in range(T):
        P = torch.zeros(H, i + 1, dtype=q.dtype)
        for g in range(H):
            s = (k[:i + 1, g // rep] @ q[i, g]) * scale
            P[g] = torch.softmax(s, 0)
        M = talk @ P
        for h in range(H):
            out[i, h] = M[h] @ v[:i + 1, h // rep]
    return out


def attention_branch(h, W, p, mx, eps, pos0=0):
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx.get("kv_heads", mx["heads"]), mx["dim"], mx.get("vdim", mx["dim"])
    q = short_conv(h @ W[p + "q"].T + W[p + "q.b"], W[p + "q.conv"])
    k = short_conv(h @ W[p + "k"].T + W[p + "k.b"], W[p + "k.conv"])
    v = short_conv(h @ W[p + "v"].T + W[p + "v.b"], W[p + "v.conv"])
    q = (rms(q, eps) * W[p + "q.norm"]).view(T, H, d)
    k = (rms(k, eps) * W[p + "k.norm"]).view(T, G, d)
    rot = mx.get("rot")
    if rot and rot.get("dims"):
        fr = rotary_frequencies(rot)
        q = torch.stack([rotate(q[t], pos0 + t, fr) for t in range(T)])
        k = torch.stack([rotate(k[t], pos0 + t, fr) for t in range(T)])
    o = head_mixing_attention(q, k, v.view(T, G, dv), mx["scale"], W[p + "talk"]).reshape(T, H * dv)
    return (o * torch.sigmoid(h @ W[p + "g"].T)) @ W[p + "o"].T


def delta_memory_loop(r, k, v, w, a, S=None):
    """r, k, w, a [T, H, d], v [T, H, dv] -> o [T, H, dv]; S_t = diag(w) S - (a u)(u^T S) + k v^T, o = S^T r."""
    T, H, d = k.shape
    dv = v.shape[2]
    S = torch.zeros(H, d, dv, dtype=k.dtype) if S is None else S.clone()
    o = torch.zeros(T, H, dv, dtype=k.dtype)
    for t in range(T):
        for h in range(H):
            u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + 1e-6)
            old = S[h]
            S[h] = w[t, h].unsqueeze(1) * old - torch.outer(a[t, h] * u, u @ old) + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ r[t, h]
    return o, S


def delta_branch(h, W, p, mx, eps):
    T, H, d = h.shape[0], mx["heads"], mx["dim"]
    r, k, v = ((h @ W[p + n].T).view(T, H, d) for n in "rkv")
    w = torch.exp(-math.exp(-0.5) * torch.sigmoid(torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(T, H, d)
    a = torch.sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).view(T, H, d)
    o, _ = delta_memory_loop(r, k, v, w, a)
    o = rms(o, eps).reshape(T, H * d) * W[p + "norm"] * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def parallel_mixer(h, W, p, mx, eps):
    a = attention_branch(h, W, p + "left.", mx["left"], eps)
    b = delta_branch(h, W, p + "right.", mx["right"], eps)
    return 0.5 * (rms(a, eps) * W[p + "left.out"] + rms(b, eps) * W[p + "right.out"])


def mingru_loop(z, u, S=None):
    S = torch.zeros(z.shape[1], dtype=z.dtype) if S is None else S.clone()
    out = torch.zeros_like(z)
    for t in range(z.shape[0]):
        cand = torch.where(u[t] >= 0, u[t] + 0.5, torch.sigmoid(u[t]))
        S = (1 - z[t]) * S + z[t] * cand
        out[t] = S
    return out, S


def mingru_mixer(h, W, p):
    z = torch.sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    S, _ = mingru_loop(z, u)
    g = h @ W[p + "g"].T
    return (S * g * torch.sigmoid(g)) @ W[p + "o"].T


def clamped_ffn(h, W, p, mlp):
    lim = mlp["limit"]
    g = torch.clamp(h @ W[p + "gate"].T, max=lim)
    u = torch.clamp(h @ W[p + "up"].T, -lim, lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T


def owner(config, i):
    while config["layers"][i].get("weights_of") is not None:
        i = config["layers"][i]["weights_of"]
    return i


def forward(config, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits ``[T, vocab]`` of one sequence (and the residual stream after every layer run)."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)]
    bg = (config.get("embedding") or {}).get("bigram")
    if bg:
        x = x + W["bigram"][torch.tensor(bigram_rows(tokens, bg))]
    layers = []
    for i, l in enumerate(config["layers"]):
        p = f"l{owner(config, i)}."
        m = parallel_mixer(x, W, p + "mix.", l["mixer"], eps) if l["type"] == "parallel" else mingru_mixer(x, W, p + "mix.")
        x = x + one_plus_norm(m, W[p + "norm1"], eps)
        if l.get("mlp"):
            x = x + one_plus_norm(clamped_ffn(x, W, p + "mlp.", l["mlp"]), W[p + "norm2"], eps)
        layers.append(x.clone())
    logits = one_plus_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, layers) if return_layers else logits


def random_weights(config, seed=0, dtype=torch.float32, decay_rank=5):
    """Random tensors for every name the design defines, at scales that keep all gates and norms away from saturation."""
    g = torch.Generator().manual_seed(seed)
    W = {}
    width = config["width"]

    def lin(name, out, inp, std=None):
        W[name] = torch.randn(out, inp, generator=g) * (std if std is not None else inp ** -0.5)

    def vec(name, n, std=0.3, mean=0.0):
        W[name] = mean + torch.randn(n, generator=g) * std

    W["embed"] = torch.randn(config["vocab"], width, generator=g)
    bg = (config.get("embedding") or {}).get("bigram")
    if bg:
        W["bigram"] = torch.randn(bg["buckets"] + 1, width, generator=g) * 0.7
    for i, l in enumerate(config["layers"]):
        if l.get("weights_of") is not None:
            continue
        p = f"l{i}."
        vec(p + "norm1", width, 0.2)
        if l["type"] == "mingru":
            n = l["mixer"]["width"]
            for nm in "zxg":
                lin(p + "mix." + nm, n, width, 1.5 * width ** -0.5)
            vec(p + "mix.z.b", n, 0.5)
            vec(p + "mix.x.b", n, 0.5)
            lin(p + "mix.o", width, n)
        else:
            a, r = l["mixer"]["left"], l["mixer"]["right"]
            H, G, d, dv = a["heads"], a.get("kv_heads", a["heads"]), a["dim"], a.get("vdim", a["dim"])
            q = p + "mix.left."
            for nm, n in (("q", H * d), ("k", G * d), ("v", G * dv)):
                lin(q + nm, n, width)
                vec(q + nm + ".b", n, 0.3)
                W[q + nm + ".conv"] = torch.randn(n, a.get("conv", 1), generator=g) * 0.6
            vec(q + "q.norm", H * d, 0.3, 1.5)
            vec(q + "k.norm", G * d, 0.3, 1.5)
            W[q + "talk"] = torch.eye(H) * 0.7 + torch.randn(H, H, generator=g) * 0.3
            lin(q + "g", H * dv, width)
            lin(q + "o", width, H * dv)
            q = p + "mix.right."
            n = r["heads"] * r["dim"]
            for nm in ("r", "k", "v", "g", "a"):
                lin(q + nm, n, width)
            vec(q + "a.b", n, 0.5)
            lin(q + "w1", decay_rank, width)
            lin(q + "w2", n, decay_rank, 1.0)
            vec(q + "w0", n, 1.0)
            vec(q + "norm", n, 0.3, 1.0)
            lin(q + "o", width, n)
            vec(p + "mix.left.out", width, 0.3, 1.0)
            vec(p + "mix.right.out", width, 0.3, 1.0)
        if l.get("mlp"):
            vec(p + "norm2", width, 0.2)
            ff = l["mlp"]["ff"]
            lin(p + "mlp.gate", ff, width, 2.0 * width ** -0.5)
            lin(p + "mlp.up", ff, width, 2.0 * width ** -0.5)
            lin(p + "mlp.down", width, ff)
    vec("final.norm", width, 0.2)
    lin("head", config["vocab"], width)
    return {k: v.to(dtype) for k, v in W.items()}
