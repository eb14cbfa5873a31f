"""The Lomusun decoder stated plainly: whole sequences, 64-bit, no cache, one function per mechanism.

It shares no code with the package; tests compare the package's results with it.  Weights come as a dict of
tensors under the checkpoint's own names, the configuration as the config.json dict.

    embedding        x_t = embed[tok_t] + pos[t]
    layer            h = rms(x) * w;  x <- x + mixer(h) + ff(h)        (one norm, both sublayers read it)
    'attention'      q, k, v = projections, each through a causal convolution over time (no activation);
                     score(i, j) = scale q_i.k_j + rel[bucket(i - j), head], window, softmax, a sigmoid gate per head;
                     a layer with 'kv_from' has only queries and reads another layer's keys and values
    'parallel'       left_scale * windowed attention (q and k normed over the whole projection, score minus
                     slope_head * (i - j), a sink in the softmax denominator, an element-wise sigmoid gate)
                     + right_scale * gated delta rule with one decay per head
    feed-forward     mixture of experts, sigmoid router with a correction on the choice only, clamped experts
    output           embed rms(x)
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def causal_conv(x, w):
    """x [T, C], w [C, taps] whose last column meets the current token; zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    out = torch.zeros_like(x)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += x[:T - back] * w[:, j]
    return out


def bucket(n, rows, far):
    """The row of the distance table for distance n >= 0: one row per distance below rows // 2, then rows that grow
    logarithmically up to distance `far`, the last row for everything beyond."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def window_mask(T, size):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def group_of(h, heads, kv_heads):
    return h // (heads // kv_heads)


def table_attention_scores(q, k, m, rel):
    """q [T, H, d], k [T, G, d] -> softmax weights [H, T, T] of the 'attention' mixer."""
    T, H = q.shape[0], m["heads"]
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0)
    rows = torch.tensor([[bucket(int(n), rel.shape[0], m["bias_max"]) for n in r] for r in dist.tolist()])
    mask = window_mask(T, m["mask"]["size"])
    out = []
    for h in range(H):
        g = group_of(h, H, m["kv_heads"])
        s = q[:, h] @ k[:, g].T * m["scale"] + rel[rows, h]
        out.append(torch.softmax(s.masked_fill(~mask, -math.inf), -1))
    return torch.stack(out)


def conv_attention(h, W, p, m, shared=None):
    """The 'attention' mixer.  shared: (k, v) of the layer this one reads from; returns (y, (k, v))."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = causal_conv(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, H, d)
    if shared is None:
        k = causal_conv(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, d)
        v = causal_conv(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, G, dv)
    else:
        k, v = shared
    w = table_attention_scores(q, k, m, W[p + "rel"])
    gate = torch.sigmoid(h @ W[p + "g"].T)                      # [T, H]
    o = torch.stack([w[hh] @ v[:, group_of(hh, H, G)] * gate[:, hh:hh + 1] for hh in range(H)], 1)
    return o.reshape(T, H * dv) @ W[p + "o"].T, (k, v)


def sink_attention(h, W, p, m, eps):
    """The left half of the 'parallel' mixer."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (rms(h @ W[p + "q"].T, eps) * W[p + "q.norm"]).view(T, H, d)
    k = (rms(h @ W[p + "k"].T, eps) * W[p + "k.norm"]).view(T, G, d)
    v = (h @ W[p + "v"].T).view(T, G, dv)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).to(F64)
    mask = window_mask(T, m["mask"]["size"])
    heads = []
    for hh in range(H):
        g = group_of(hh, H, G)
        slope = 2.0 ** (-8.0 * (hh + 1) / H)
        s = (q[:, hh] @ k[:, g].T * m["scale"] - slope * dist).masked_fill(~mask, -math.inf)
        s = torch.cat([s, W[p + "sink"][hh].expand(T, 1)], 1)   # the sink: one more term of the softmax, without a value
        heads.append(torch.softmax(s, -1)[:, :T] @ v[:, g])
    o = torch.cat(heads, 1) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def head_delta_rule(h, W, p, m, eps):
    """The right half of the 'parallel' mixer: gated delta rule, one decay per head and token."""
    T = h.shape[0]
    H, J, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, J, d)
    k = silu(causal_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, J, d)
    v = silu(causal_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * softplus(h @ W[p + "a"].T + W[p + "dt_bias"]))      # [T, H]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hh in range(H):
        j = group_of(hh, H, J)
        S = torch.zeros(d, dv, dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, j])
            S = S + torch.outer(k[t, j], u)
            out[t, hh] = S.T @ q[t, j]
    y = rms(out, eps) * W[p + "norm"] * silu(h @ W[p + "g"].T).view(T, H, dv)
    return y.reshape(T, H * dv) @ W[p + "o"].T


def expert(h, W, p, limit):
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1)) @ W[p + "down"].T


def mixture(h, W, p, mlp):
    r = mlp["router"]
    s = torch.sigmoid(h @ W[p + "router"].T)                    # [T, E]
    chosen = torch.topk(s + W[p + "correction"], r["top"], dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        picked = s[t, chosen[t]]
        weights = picked / (picked.sum() + 1e-20) * r["scale"]
        for e, w in zip(chosen[t].tolist(), weights):
            out[t] += w * expert(h[t], W, f"{p}e{e}.", mlp["expert"]["limit"])
    return out


def forward(cfg, weights, tokens, dtype=F64, keep_layers=False):
    """Logits [T, vocab] of one whole sequence (and, with keep_layers, the stream after every layer)."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    T = len(tokens)
    x = W["embed"][torch.tensor(tokens)] + W["pos"][:T]
    kept, kv = [], {}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        h = rms(x, eps) * W[p + "norm1"]
        if L["type"] == "attention":
            src = m.get("kv_from")
            y, kv[i] = conv_attention(h, W, p + "mix.", m, None if src is None else kv[src])
        elif L["type"] == "parallel":
            y = (m["left_scale"] * sink_attention(h, W, p + "mix.left.", m["left"], eps)
                 + m["right_scale"] * head_delta_rule(h, W, p + "mix.right.", m["right"], eps))
        else:
            raise ValueError(f"layer type {L['type']!r}")
        if L.get("mlp") is not None:
            y = y + mixture(h, W, p + "mlp.", L["mlp"])
        x = x + y
        if keep_layers:
            kept.append(x.clone())
    logits = (rms(x, eps) * W["final.norm"]) @ W["embed"].T
    return (logits, torch.stack(kept)) if keep_layers else logits
