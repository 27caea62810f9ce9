"""A plain, slow implementation of the Kavotar decoder: whole sequences, no cache, no batching, one function for each
mechanism, float64. It shares no code with the engine and is what the engine's Kavotar results are compared with.

The design in this file's notation (x: residual stream [T, d]; the sublayers read x itself, the norms stand BEHIND them):

    layer:      x <- x + LN1(mixer(x));   x <- x + LN2(ff(x))             (LN: layer norm with a weight, no bias)
    mixers:     'mlstm'     a matrix memory per head with exponential gates held against a running maximum
                'parallel'  the mean of two mixers that read the same rows, each RMS-normed over the width first:
                            chunk-masked attention whose heads' weights are mixed after the softmax, and a linear
                            recurrence with token-shifted inputs, a decay per key channel and a bonus for the current token
    ff:         routed experts (sigmoid scores, a correction for the choice only, groups of neighbours)
    output:     final layer norm, head, soft cap c * tanh(logits / c)
"""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def log_sigmoid(z):
    return -torch.where(z < -30, -z, torch.log1p(torch.exp(-torch.clamp(z, min=-30.0))))


def soft_cap(z, cap):
    return cap * torch.tanh(z / cap)


# ------------------------------------------------------------------------------------------------ matrix memory
def matrix_memory(q, k, v, i_log, f_log):
    """One sequence from its start. q, k [T, H, dk] (q already scaled), v [T, H, dv], log gates i_log, f_log [T, H].
    Per head, with S, n, m starting at zero:  m' = max(f + m, i);  S' = e^(f + m - m') S + e^(i - m') k v^T;
    n' likewise with k alone;  o = S'^T q / (max(|n' . q|, e^(-m')) + 1e-6). Returns [T, H, dv]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=F64)
    n = torch.zeros(H, dk, dtype=F64)
    m = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(f_log[t] + m, i_log[t])
        a = torch.exp(f_log[t] + m - m_new)
        b = torch.exp(i_log[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hkv,hk->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out


def mlstm_mixer(h, w, H, dk, dv, cap, eps):
    """w: this mixer's tensors by their local names ('q', 'k', 'v', 'g', 'o', 'norm', 'i', 'i.b', 'f', 'f.b')."""
    T = h.shape[0]
    q = (h @ w["q"].T).view(T, H, dk) * dk ** -0.5
    k = (h @ w["k"].T).view(T, H, dk)
    v = (h @ w["v"].T).view(T, H, dv)
    i_log = soft_cap(h @ w["i"].T + w["i.b"], cap)
    f_log = log_sigmoid(soft_cap(h @ w["f"].T + w["f.b"], cap))
    o = rms_unit(matrix_memory(q, k, v, i_log, f_log), eps).reshape(T, H * dv)
    return (o * w["norm"] * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


# ------------------------------------------------------------------------------------------ chunk-masked attention
def rotate_halves(x, positions, base, n_rot):
    """x [T, heads, dh]: dimension i turns with dimension i + n_rot / 2 (i < n_rot / 2) by position * base^(-2i / n_rot);
    the dimensions from n_rot on pass unchanged."""
    out = x.clone()
    half = n_rot // 2
    if half == 0:
        return out
    i = torch.arange(half, dtype=F64)
    freq = torch.tensor(float(base), dtype=F64) ** (-2.0 * i / n_rot)
    ang = torch.as_tensor(positions, dtype=F64)[:, None] * freq[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:n_rot]
    out[..., :half] = u * c - v * s
    out[..., half:n_rot] = v * c + u * s
    return out


def chunk_mask(T, size):
    """[T, T] bool: i sees j when j <= i and both lie in the same chunk of `size` positions counted from 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def talking_attention(q, k, v, scale, temp, talk, size):
    """q [T, H, dk], k [T, G, dk], v [T, G, dv]. Head h's scores q_h . k_(h // (H/G)) * scale * temp[h] go through a
    softmax over the keys `chunk_mask` lets it see; the heads' weights are then mixed, W'_h = sum_g talk[h, g] W_g, and
    head h applies W'_h to the values of its own key/value head. Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)
    vv = v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale * temp[:, None, None]
    s = s.masked_fill(~chunk_mask(T, size)[None], float("-inf"))
    wts = torch.softmax(s, dim=-1)
    mixed = torch.einsum("hg,gij->hij", talk, wts)
    return torch.einsum("hij,jhd->ihd", mixed, vv)


def attention_mixer(h, w, c, eps):
    """c: heads, kv_heads, dim, vdim, size, rot_base, rot_dims, scale."""
    T = h.shape[0]
    H, G, dk, dv = c["heads"], c["kv_heads"], c["dim"], c["vdim"]
    pos = torch.arange(T)
    q = rms_unit((h @ w["q"].T).view(T, H, dk), eps) * w["q.norm"]
    k = rms_unit((h @ w["k"].T).view(T, G, dk), eps) * w["k.norm"]
    v = (h @ w["v"].T).view(T, G, dv)
    q = rotate_halves(q, pos, c["rot_base"], c["rot_dims"])
    k = rotate_halves(k, pos, c["rot_base"], c["rot_dims"])
    o = talking_attention(q, k, v, c["scale"], w["temp"], w["talk"], c["size"])
    return o.reshape(T, H * dv) @ w["o"].T


# ------------------------------------------------------------------------------------------- shifted recurrence
def bonus_recurrence(r, k, v, w, u):
    """r, k, w [T, H, dk], v [T, H, dv], u [H, dk]. Per head, S starting at zero:
    o_t = (S + diag(u) k_t v_t^T)^T r_t, then S <- diag(w_t) S + k_t v_t^T. Returns [T, H, dv]."""
    T, H, dk = r.shape
    dv = v.shape[2]
    S = torch.zeros(H, dk, dv, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    return out


def shifted_mixer(h, w, H, dk, eps):
    """The inputs of r, k, v, g and the decay are each h + (h' - h) * mu, h' the row before (zeros before the first)."""
    T = h.shape[0]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    mix = lambda s: h + (prev - h) * w["mu." + s]
    r = (mix("r") @ w["r"].T).view(T, H, dk)
    k = (mix("k") @ w["k"].T).view(T, H, dk)
    v = (mix("v") @ w["v"].T).view(T, H, dk)
    gate = silu(mix("g") @ w["g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(mix("w") @ w["w1"].T) @ w["w2"].T + w["w0"])).view(T, H, dk)
    o = rms_unit(bonus_recurrence(r, k, v, decay, w["u"]), eps).reshape(T, H * dk)
    return (o * w["norm"] * gate) @ w["o"].T


def parallel_mixer(h, w, c, eps):
    """c: {'left': attention sizes, 'right': {'heads', 'dim'}}; w: tensors under 'left.*', 'right.*'."""
    sub = lambda p: {n[len(p):]: t for n, t in w.items() if n.startswith(p)}
    a = attention_mixer(h, sub("left."), c["left"], eps)
    b = shifted_mixer(h, sub("right."), c["right"]["heads"], c["right"]["dim"], eps)
    return 0.5 * (rms_unit(a, eps) * w["left.out"] + rms_unit(b, eps) * w["right.out"])


# ------------------------------------------------------------------------------------------------ routed experts
def route(h, router, correction, top, groups, keep):
    """Returns (experts [T, top], weights [T, top]): scores sigmoid(h router^T); the choice runs on score + correction,
    among the experts of the `keep` groups (of `groups` equal runs of neighbours) whose two largest choice scores add up
    highest; the weights are the scores themselves, as they are."""
    return route_from_logits(h @ router.T, correction, top, groups, keep)


def route_from_logits(z, correction, top, groups, keep, margins=False):
    """With `margins` also returns, per token, how far the choice is from another one: the smaller of the gap between the
    last chosen and the best unchosen open expert and the gap between the last kept and the best closed group."""
    s = torch.sigmoid(z)
    choice = s + correction
    T, E = s.shape
    per = E // groups
    g = choice.view(T, groups, per)
    gscore = g.topk(min(2, per), dim=-1).values.sum(-1)
    kept = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = choice.masked_fill(~allowed[:, :, None].expand(T, groups, per).reshape(T, E), float("-inf"))
    idx = masked.topk(top, dim=-1).indices
    if not margins:
        return idx, s.gather(1, idx)
    margin = torch.full((T,), float("inf"), dtype=F64)
    if top < keep * per:
        best = masked.topk(top + 1, dim=-1).values
        margin = torch.minimum(margin, best[:, top - 1] - best[:, top])
    if keep < groups:
        best = gscore.topk(keep + 1, dim=-1).values
        margin = torch.minimum(margin, best[:, keep - 1] - best[:, keep])
    return idx, s.gather(1, idx), margin


def routed_experts(h, w, c, forced=None, info=None):
    """c: experts, top, groups, keep; w: 'router', 'correction', 'e<j>.gate' / '.up' / '.down'. `forced` [T, top]: experts
    to use instead of the own choice (their weights are still the own scores); `info`: a list that receives (own choice,
    margin of the own choice)."""
    z = h @ w["router"].T
    idx, wt, margin = route_from_logits(z, w["correction"], c["top"], c["groups"], c["keep"], margins=True)
    if info is not None:
        info.append((idx, margin))
    if forced is not None:
        idx = torch.as_tensor(forced, dtype=torch.long)
        wt = torch.sigmoid(z).gather(1, idx)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for j in range(c["top"]):
            e = int(idx[t, j])
            a = silu(h[t] @ w[f"e{e}.gate"].T) * (h[t] @ w[f"e{e}.up"].T)
            out[t] += wt[t, j] * (a @ w[f"e{e}.down"].T)
    return out


# ------------------------------------------------------------------------------------------------------- model
def _mixer_sizes(layer):
    m = layer["mixer"]
    if layer["type"] == "mlstm":
        return m
    l = m["left"]
    return {"left": dict(heads=l["heads"], kv_heads=l.get("kv_heads", l["heads"]), dim=l["dim"], vdim=l.get("vdim", l["dim"]),
                         size=l["mask"]["size"], rot_base=l["rot"]["base"], rot_dims=l["rot"]["dims"], scale=l["scale"]),
            "right": m["right"]}


def forward(config: dict, tensors: dict, tokens, streams: bool = False, forced=None, info=None):
    """Logits [T, vocab] of one sequence from its start (and, with `streams`, the residual stream after every layer
    [layers, T, width]). `forced` {layer: experts [T, top]}: the experts to use in that layer's feed-forward; `info` {}:
    receives {layer: (own choice, margin)}."""
    W = {n: t.to(F64) for n, t in tensors.items()}
    eps = float(config["norm"]["eps"])
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kept = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        w = {n[len(p) + 4:]: t for n, t in W.items() if n.startswith(p + "mix.")}
        sizes = _mixer_sizes(layer)
        if layer["type"] == "mlstm":
            y = mlstm_mixer(x, w, sizes["heads"], sizes["dim"], sizes.get("vdim", sizes["dim"]), float(sizes["gate_cap"]), eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(x, w, sizes, eps)
        else:
            raise ValueError(layer["type"])
        x = x + layer_norm(y, W[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            r = layer["mlp"]["router"]
            w = {n[len(p) + 4:]: t for n, t in W.items() if n.startswith(p + "mlp.")}
            got = []
            y = routed_experts(x, w, dict(experts=r["experts"], top=r["top"], groups=r["groups"]["count"], keep=r["groups"]["keep"]),
                               forced=None if forced is None else forced.get(i), info=got)
            if info is not None:
                info[i] = got[0]
            x = x + layer_norm(y, W[p + "norm2"], eps)
        kept.append(x)
    logits = layer_norm(x, W["final.norm"], eps) @ W["head"].T
    logits = soft_cap(logits, float(config["logit_softcap"]))
    return (logits, torch.stack(kept)) if streams else logits
