"""Slow, loop-by-loop evaluation of a Zikunex model, written from the design's equations: the oracle of the tests.

One function per mechanism, whole sequences only (no cache, no state hand-over, no batching), token by token where the
design is recurrent.  Nothing here is imported by the package and nothing of the package is imported here.

``weights`` maps the checkpoint's tensor names (``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``,
``head``) to tensors; ``config`` is the parsed ``config.json``.
"""
import math

import torch


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def relu2_ffn(h, up, down):
    return (torch.relu(h @ up.T) ** 2) @ down.T


def route(z, top, n_groups, keep):
    """z [E] router logits of one token -> (expert ids, weights)."""
    s = torch.softmax(z, -1)
    E = s.numel()
    per = E // n_groups
    group_best = s.view(n_groups, per).max(-1).values
    kept = torch.topk(group_best, keep).indices.tolist()
    allowed = torch.full_like(s, -1.0)
    for g in kept:
        allowed[g * per:(g + 1) * per] = s[g * per:(g + 1) * per]
    idx = torch.topk(allowed, top).indices
    w = s[idx]
    return idx.tolist(), w / (w.sum() + 1e-20)


def moe_ffn(h, W, pre, mlp):
    r = mlp["router"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    out = torch.zeros(h.shape[0], W[pre + "e0.down"].shape[0], dtype=h.dtype)
    z = h @ W[pre + "router"].T
    for t in range(h.shape[0]):
        ids, ws = route(z[t], r["top"], groups["count"], groups["keep"])
        for e, w in zip(ids, ws):
            out[t] += w * relu2_ffn(h[t], W[f"{pre}e{e}.up"], W[f"{pre}e{e}.down"])
    if mlp.get("shared"):
        out = out + relu2_ffn(h, W[pre + "shared.up"], W[pre + "shared.down"])
    return out


def latent_of(h, W, pre, eps):
    return rms_norm(h @ W[pre + "dkv"].T, W[pre + "dkv.norm"], eps)


def latent_attention(h, c, W, pre, mx, eps):
    """h [T, width]; c [T, kv_rank] the latents this layer attends over (its own or another layer's)."""
    T, H, d, dv = h.shape[0], mx["heads"], mx["dim"], mx["vdim"]
    q = (rms_norm(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps) @ W[pre + "uq"].T).view(T, H, d)
    k = (c @ W[pre + "uk"].T).view(T, H, d)
    v = (c @ W[pre + "uv"].T).view(T, H, dv)
    out = causal_attention_loop(q, k, v, mx["scale"])
    return out.reshape(T, H * dv) @ W[pre + "o"].T


def causal_attention_loop(q, k, v, scale):
    """q, k [T, H, d], v [T, H, dv] -> [T, H, dv]; position i sees every j <= i."""
    T, H = q.shape[0], q.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for i in range(T):
        for a in range(H):
            s = (k[:i + 1, a] @ q[i, a]) * scale
            out[i, a] = torch.softmax(s, 0) @ v[:i + 1, a]
    return out


def short_conv_silu(x, w):
    """x [T, C], w [C, taps] (last column = current token), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    y = torch.zeros_like(x)
    for t in range(T):
        for j in range(taps):
            src = t - (taps - 1 - j)
            if src >= 0:
                y[t] += w[:, j] * x[src]
    return y * torch.sigmoid(y)


def channel_delta(h, W, pre, mx, eps):
    T, H, KH, d, dv = h.shape[0], mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = short_conv_silu(h @ W[pre + "q"].T, W[pre + "q.conv"]).view(T, KH, d)
    k = short_conv_silu(h @ W[pre + "k"].T, W[pre + "k.conv"]).view(T, KH, d)
    v = short_conv_silu(h @ W[pre + "v"].T, W[pre + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[pre + "b"].T)                                             # [T, H]
    dt = torch.nn.functional.softplus((h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "dt_bias"]).view(T, H, d)
    g = torch.exp(-torch.exp(W[pre + "A_log"]).view(1, H, 1) * dt)                       # [T, H, d]
    gate = torch.sigmoid((h @ W[pre + "g1"].T) @ W[pre + "g2"].T).view(T, H, dv)
    out = delta_rule_loop(q, k, v, g, beta)
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * W[pre + "norm"] * gate
    return out.reshape(T, H * dv) @ W[pre + "o"].T


def delta_rule_loop(q, k, v, g, beta):
    """q, k [T, KH, d] (already unit length / scaled), v [T, H, dv], decay g [T, H, d], beta [T, H] -> o [T, H, dv]."""
    T, H, dv = v.shape
    KH, d = q.shape[1], q.shape[2]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for a in range(H):
        kh = a // (H // KH)
        S = torch.zeros(d, dv, dtype=q.dtype)
        for t in range(T):
            S = g[t, a].unsqueeze(1) * S
            u = beta[t, a] * (v[t, a] - S.T @ k[t, kh])
            S = S + torch.outer(k[t, kh], u)
            out[t, a] = S.T @ q[t, kh]
    return out


def mlstm(h, W, pre, mx, eps):
    T, H, d, dv, cap = h.shape[0], mx["heads"], mx["dim"], mx["vdim"], mx["gate_cap"]
    q = (h @ W[pre + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ W[pre + "k"].T).view(T, H, d)
    v = (h @ W[pre + "v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ W[pre + "i"].T + W[pre + "i.b"]) / cap)                   # [T, H]
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ W[pre + "f"].T + W[pre + "f.b"]) / cap))
    out = mlstm_loop(q, k, v, ig, fg)
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps)
    out = out.reshape(T, H * dv) * W[pre + "norm"] * torch.sigmoid(h @ W[pre + "g"].T)
    return out @ W[pre + "o"].T


def mlstm_loop(q, k, v, ig, fg):
    """q (scaled), k [T, H, d], v [T, H, dv], log gates ig, fg [T, H] -> o [T, H, dv]."""
    T, H, dv = v.shape
    d = q.shape[2]
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for a in range(H):
        S = torch.zeros(d, dv, dtype=q.dtype)
        n = torch.zeros(d, dtype=q.dtype)
        m = torch.zeros((), dtype=q.dtype)
        for t in range(T):
            m_new = torch.maximum(fg[t, a] + m, ig[t, a])
            keep, put = torch.exp(fg[t, a] + m - m_new), torch.exp(ig[t, a] - m_new)
            S = keep * S + put * torch.outer(k[t, a], v[t, a])
            n = keep * n + put * k[t, a]
            m = m_new
            out[t, a] = S.T @ q[t, a] / (torch.maximum((n @ q[t, a]).abs(), torch.exp(-m)) + 1e-6)
    return out


def forward(config, weights, tokens, dtype=torch.float64, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the residual stream after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens)] * config["embedding"]["scale"]
    latents, layers = {}, []
    for i, layer in enumerate(config["layers"]):
        mx, pre = layer["mixer"], f"l{i}.mix."
        h = rms_norm(x, W[f"l{i}.norm1"], eps)
        if layer["type"] == "latent_attention":
            if mx.get("kv_from") is None:
                latents[i] = latent_of(h, W, pre, eps)
            y = latent_attention(h, latents[mx["kv_from"] if mx.get("kv_from") is not None else i], W, pre, mx, eps)
        elif layer["type"] == "channel_delta":
            y = channel_delta(h, W, pre, mx, eps)
        elif layer["type"] == "mlstm":
            y = mlstm(h, W, pre, mx, eps)
        else:
            raise ValueError(layer["type"])
        x = x + y
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm(x, W[f"l{i}.norm2"], eps)
            if mlp["kind"] == "dense":
                x = x + relu2_ffn(h, W[f"l{i}.mlp.up"], W[f"l{i}.mlp.down"])
            else:
                x = x + moe_ffn(h, W, f"l{i}.mlp.", mlp)
        layers.append(x)
    logits = rms_norm(x, W["final.norm"], eps) @ W["head"].T
    return (logits, torch.stack(layers)) if return_layers else logits


def random_weights(config, seed=0, dtype=torch.float32, low_rank=8):
    """Random tensors with the checkpoint's names and shapes for ``config`` (gains near 1, small projections);
    ``low_rank`` is the inner width of the decay and gate projections of channel_delta layers."""
    g = torch.Generator().manual_seed(seed)
    width, W = config["width"], {}

    def lin(name, out, inp, std=None):
        W[name] = (torch.randn(out, inp, generator=g) * (std or inp ** -0.5)).to(dtype)

    def gain(name, n):
        W[name] = (1.0 + 0.1 * torch.randn(n, generator=g)).to(dtype)

    lin("embed", config["vocab"], width, 1.0)
    for i, layer in enumerate(config["layers"]):
        mx, p = layer["mixer"], f"l{i}.mix."
        gain(f"l{i}.norm1", width)
        if layer["type"] == "latent_attention":
            H, d, dv, r, rq = mx["heads"], mx["dim"], mx["vdim"], mx["kv_rank"], mx["q_rank"]
            lin(p + "dq", rq, width), gain(p + "dq.norm", rq), lin(p + "uq", H * d, rq)
            if mx.get("kv_from") is None:
                lin(p + "dkv", r, width), gain(p + "dkv.norm", r)
            lin(p + "uk", H * d, r), lin(p + "uv", H * dv, r), lin(p + "o", width, H * dv)
        elif layer["type"] == "channel_delta":
            H, KH, d, dv, taps = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"], mx["conv"]
            lo = low_rank
            for nm, n in (("q", KH * d), ("k", KH * d), ("v", H * dv)):
                lin(p + nm, n, width)
                W[p + nm + ".conv"] = (torch.randn(n, taps, generator=g) * 0.5).to(dtype)
            lin(p + "b", H, width)
            W[p + "A_log"] = (torch.rand(H, generator=g) * 2 - 1).to(dtype)
            gain(p + "norm", dv)
            lin(p + "a1", lo, width), lin(p + "a2", H * d, lo)
            W[p + "dt_bias"] = (torch.randn(H * d, generator=g) - 2.0).to(dtype)
            lin(p + "g1", lo, width), lin(p + "g2", H * dv, lo), lin(p + "o", width, H * dv)
        else:
            H, d, dv = mx["heads"], mx["dim"], mx["vdim"]
            lin(p + "q", H * d, width), lin(p + "k", H * d, width), lin(p + "v", H * dv, width)
            lin(p + "g", H * dv, width), lin(p + "o", width, H * dv), gain(p + "norm", H * dv)
            lin(p + "i", H, width), lin(p + "f", H, width)
            W[p + "i.b"] = torch.randn(H, generator=g).to(dtype)
            W[p + "f.b"] = (torch.randn(H, generator=g) + 3.0).to(dtype)
        mlp = layer.get("mlp")
        if mlp:
            gain(f"l{i}.norm2", width)
            m = f"l{i}.mlp."
            if mlp["kind"] == "dense":
                lin(m + "up", mlp["ff"], width), lin(m + "down", width, mlp["ff"])
            else:
                for e in range(mlp["router"]["experts"]):
                    lin(f"{m}e{e}.up", mlp["expert"]["ff"], width), lin(f"{m}e{e}.down", width, mlp["expert"]["ff"])
                lin(m + "router", mlp["router"]["experts"], width, 1.0 * width ** -0.5 * 3)
                if mlp.get("shared"):
                    lin(m + "shared.up", mlp["shared"]["ff"], width), lin(m + "shared.down", width, mlp["shared"]["ff"])
    gain("final.norm", width)
    lin("head", config["vocab"], width)
    return W
