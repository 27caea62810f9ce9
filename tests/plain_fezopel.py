"""A plain, slow implementation of the Fezopel decoder: whole sequences, no cache, no batching, one function for
each mechanism, float64. It shares no code with the engine (its own reader of model folders is the one in
`plain_model`) and is what the engine's Fezopel results are compared with.

The design in this file's notation (x: residual stream [T, d]; h: the normed rows a sublayer reads):

    layer:      m = mixer(h1) * sigmoid(h1 Rg1^T + b1),  h1 = LN1(x);   x <- x + LN1b(m)
                f = ff(h2)    * sigmoid(h2 Rg2^T + b2),  h2 = LN2(x);   x <- x + LN2b(f)       (only with a feed-forward)
    depth mix:  X_0 = embedding rows, X_(i+1) = x after layer i;  the next layer (or the final norm) reads
                sum_(j <= i+1) a_i[j] X_j
    mixers:     windowed attention with a sink, a gated linear recurrence, a gated delta rule with decays per channel
"""
import math

import torch


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_interleaved(x, positions, base, n_rot):
    """x [T, heads, dh]: dimensions (2i, 2i + 1), i < n_rot / 2, turn by angle position * base^(-2i / n_rot); the
    dimensions from n_rot on pass unchanged."""
    out = x.clone()
    i = torch.arange(n_rot // 2, dtype=torch.float64)
    freq = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / n_rot)
    ang = torch.as_tensor(positions, dtype=torch.float64)[:, None] * freq[None, :]          # [T, n_rot / 2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:n_rot:2], x[..., 1:n_rot:2]
    out[..., 0:n_rot:2] = u * c - v * s
    out[..., 1:n_rot:2] = v * c + u * s
    return out


def sink_window_attention(q, k, v, scale, window, sinks):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv] of one sequence from its start; query head h reads key/value head
    h // (H / G); position i sees j with 0 <= i - j < window (window 0: every j <= i); the softmax's denominator also
    holds exp(sinks[h]), which has no value. Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window > 0 else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), float(sinks[h]))
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(0) / (e.sum() + math.exp(float(sinks[h]) - m))
    return out


def attention_mixer(h, W, p, mc, eps, positions=None):
    """The attention mixer on normed rows h [T, d]; W: tensors by name, p: the layer's prefix ('l0.mix.')."""
    T = h.shape[0]
    H, G, dk, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    positions = list(range(T)) if positions is None else positions
    q = rms_unit(h @ W[p + "q"].T, eps) * W[p + "q.norm"]              # over the whole projection, before the heads are split
    k = rms_unit(h @ W[p + "k"].T, eps) * W[p + "k.norm"]
    v = (h @ W[p + "v"].T).reshape(T, G, dv)
    q = rotate_interleaved(q.reshape(T, H, dk), positions, mc["rot"]["base"], mc["rot"]["dims"])
    k = rotate_interleaved(k.reshape(T, G, dk), positions, mc["rot"]["base"], mc["rot"]["dims"])
    o = sink_window_attention(q, k, v, mc["scale"], mc["mask"]["size"], W[p + "sink"])
    gate = torch.sigmoid(h @ W[p + "g"].T)                              # [T, H]
    return (o * gate[:, :, None]).reshape(T, H * dv) @ W[p + "o"].T


def gated_linear_recurrence(q, k, v, alpha):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T; o_t = S_t^T q_t. q, k, alpha [T, H, dk], v [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def gla_mixer(h, W, p, mc, eps):
    T = h.shape[0]
    H, dk, dv = mc["heads"], mc["dim"], mc["vdim"]
    q = (h @ W[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ W[p + "k"].T).reshape(T, H, dk)
    v = (h @ W[p + "v"].T).reshape(T, H, dv)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "a2.b"]
    alpha = torch.sigmoid(z).reshape(T, H, dk) ** (1.0 / mc["tau"])
    o = gated_linear_recurrence(q, k, v, alpha)
    o = rms_unit(o, eps) * W[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def short_conv(x, taps):
    """y[t, c] = sum_j taps[c, j] x[t - (n - 1) + j, c] with zeros before the start (the last tap is the current token's)."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([torch.zeros(n - 1, C, dtype=x.dtype), x], 0)
    y = torch.zeros_like(x)
    for j in range(n):
        y = y + padded[j:j + T] * taps[:, j]
    return y


def delta_recurrence(q, k, v, g, beta):
    """Per head: S <- g * S (rows); u = beta (v - S^T k); S <- S + k u^T; o = S^T q. q, k, g [T, H, dk]; v [T, H, dv];
    beta [T, H]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def channel_delta_mixer(h, W, p, mc, eps):
    T = h.shape[0]
    H, G, dk, dv = mc["heads"], mc["kv_heads"], mc["dim"], mc["vdim"]
    q = silu(short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).reshape(T, G, dk)
    k = silu(short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).reshape(T, G, dk)
    v = silu(short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).reshape(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q, k = q.repeat_interleave(rep, 1), k.repeat_interleave(rep, 1)      # head h reads q/k head h // rep
    beta = torch.sigmoid(h @ W[p + "b"].T)
    z = ((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).reshape(T, H, dk)
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * softplus(z))
    o = delta_recurrence(q, k, v, g, beta)
    o = rms_unit(o, eps) * W[p + "norm"]
    gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).reshape(T, H, dv)
    return (o * gate).reshape(T, H * dv) @ W[p + "o"].T


def dense_ff(h, W, p):
    return gelu_erf(h @ W[p + "up"].T) @ W[p + "down"].T


MIXERS = {"attention": attention_mixer, "gla": gla_mixer, "channel_delta": channel_delta_mixer}


def forward(cfg, W, tokens, return_layers=False):
    """float64 logits [T, vocab] of one sequence from its start (and the stream after every layer, depth mix included)."""
    W = {n: t.double() for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    history, after = [x], []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = layer_norm(x, W[p + "norm1"], W[p + "norm1.b"], eps)
        m = MIXERS[layer["type"]](h, W, p + "mix.", layer["mixer"], eps)
        m = m * torch.sigmoid(h @ W[p + "rg1"].T + W[p + "rg1.b"])
        x = x + layer_norm(m, W[p + "norm1b"], W[p + "norm1b.b"], eps)
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"plain Fezopel: feed-forward kind {layer['mlp']['kind']!r}")
            h = layer_norm(x, W[p + "norm2"], W[p + "norm2.b"], eps)
            f = dense_ff(h, W, p + "mlp.") * torch.sigmoid(h @ W[p + "rg2"].T + W[p + "rg2.b"])
            x = x + layer_norm(f, W[p + "norm2b"], W[p + "norm2b.b"], eps)
        history.append(x)
        x = sum(W[p + "dwa"][j] * history[j] for j in range(i + 2))
        after.append(x)
    logits = layer_norm(x, W["final.norm"], W["final.norm.b"], eps) @ W["head"].T
    return (logits, torch.stack(after)) if return_layers else logits
