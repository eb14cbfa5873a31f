"""The Tapupel decoder stated plainly: whole sequences, 64-bit, no cache, one function per mechanism.

It shares no code with the package; tests compare the package's results with it.  Weights come as a dict of
tensors under the checkpoint's own names, the configuration as the config.json dict.

    embedding        x_t = embed[tok_t] * s
    layer            x <- x + n1(mixer(x));  x <- x + n2(ff(x));   n(v) = v / sqrt(mean(v^2) + eps) * (1 + w)
    'attention'      q = Wq x, k = Wk x, values = the keys as projected; q, k rotated (half-split pairs, the leading
                     `rot.dims`, frequencies rescaled by wavelength), then divided by their root mean square per head;
                     score = cap tanh(scale q.k / cap); key j visible to i if j <= i and (i - j < W or j < F); softmax
    'rglru'          y = gelu(Wy x + by);  u = conv(Wx x + bx) + bc;  per block b of the channels:
                     r = sigmoid(Ra_b u_b + ra_b), g = sigmoid(Ri_b u_b + ri_b);  a = exp(-8 r softplus(lam));
                     S <- a S + sqrt(1 - a^2) g u;  out = Wo (S y)
    'attention_2'    two softmax maps per head over the same values: q, k normed per head and map (weight shared), rotated
                     (interleaved pairs), causal;  o = a1 - L a2,  L = exp(lq1.lk1) - exp(lq2.lk2) + c;
                     o / rms(o) (1 - c);  a layer with 'kv_from' reads another layer's normed, rotated keys and its values
    feed-forward     Wd (silu(Wg x) Wu x), or `top` of E such experts chosen by the largest router logits, weighted by the
                     softmax over the chosen logits, plus a shared expert times sigmoid(w_s . x)
    output           head n(x)
"""
import math

import torch

F64 = torch.float64
DECAY_FACTOR = 8.0


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(x):
    return x * torch.sigmoid(x)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (x + 0.044715 * x ** 3)))


def softplus(x):
    return torch.where(x > 30, x, torch.log1p(torch.exp(torch.clamp(x, max=30))))


def one_plus_norm(v, w, eps):
    return rms(v, eps) * (1.0 + w)


def frequencies(rot):
    """One frequency per rotated pair; with `scaling` the slow ones are divided by `factor`, the fast ones kept and
    those between blended linearly in original / wavelength."""
    dims = rot["dims"]
    f = [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if sc:
        out = []
        for x in f:
            wave = 2 * math.pi / x
            if wave < sc["original"] / sc["high"]:
                out.append(x)
            elif wave > sc["original"] / sc["low"]:
                out.append(x / sc["factor"])
            else:
                s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
                out.append((1 - s) * x / sc["factor"] + s * x)
        f = out
    return torch.tensor(f, dtype=F64)


def rotate(x, rot, pairing, start=0):
    """x [T, heads, d]: the leading rot.dims dimensions of every head turned by the token's position."""
    T, dims = x.shape[0], rot["dims"]
    ang = (torch.arange(start, start + T, dtype=F64)[:, None] * frequencies(rot)[None, :])[:, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    if pairing == "half":
        a, b = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2], out[..., dims // 2:dims] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2], out[..., 1:dims:2] = a * c - b * s, b * c + a * s
    return out


def visible(T, window=None, keep_first=0):
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & ((i - j < window) | (j < keep_first))
    return seen


def softmax_rows(s, mask):
    return torch.softmax(s.masked_fill(~mask, -math.inf), -1)


def window_attention(x, m, w, eps):
    """The 'attention' mixer on x [T, D]; w: the layer's tensors by their short names (q, k, o)."""
    T = x.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (x @ w["q"].T).view(T, H, d)
    k = (x @ w["k"].T).view(T, G, d)
    v = k.clone()
    q, k = rms(rotate(q, m["rot"], "half"), eps), rms(rotate(k, m["rot"], "half"), eps)
    mask = visible(T, m["mask"]["size"], m["mask"]["keep_first"]) if m.get("mask") else visible(T)
    cap = m.get("softcap")
    heads = []
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        heads.append(softmax_rows(s, mask) @ v[:, g])
    return torch.cat(heads, -1) @ w["o"].T


def causal_conv(x, w, bias):
    """x [T, C], w [C, taps] whose last column meets the current token; zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x) + bias
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            out[back:] += x[:T - back] * w[:, j]
    return out


def rglru_gates(u, w, blocks):
    """(a, b) of the recurrence S <- a S + b for every token: u [T, C]."""
    T, C = u.shape
    ub = u.view(T, blocks, C // blocks)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ra"]) + w["ra.b"]).reshape(T, C)
    g = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w["ri"]) + w["ri.b"]).reshape(T, C)
    a = torch.exp(-DECAY_FACTOR * r * softplus(w["lam"]))
    return a, torch.sqrt(1 - a * a) * g * u


def linear_scan(a, b):
    S = torch.zeros_like(a[0])
    out = []
    for t in range(a.shape[0]):
        S = a[t] * S + b[t]
        out.append(S)
    return torch.stack(out)


def rglru(x, m, w):
    y = gelu_tanh(x @ w["y"].T + w["y.b"])
    u = causal_conv(x @ w["x"].T + w["x.b"], w["conv"], w["conv.b"])
    a, b = rglru_gates(u, w, m["blocks"])
    return (linear_scan(a, b) * y) @ w["o"].T


def diff_keys_values(x, m, w, eps):
    """Keys (normed, rotated) [T, G, 2, d] and values [T, G, dv] of an 'attention_2' layer that has its own."""
    T, G, d, dv = x.shape[0], m["kv_heads"], m["dim"], m["vdim"]
    k = (x @ w["k"].T).view(T, G * 2, d)
    k = rotate(rms(k, eps) * w["k.norm"], m["rot"], "interleaved")
    return k.view(T, G, 2, d), (x @ w["v"].T).view(T, G, dv)


def diff_lambda(m, w):
    return float(torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + m["diff"])


def diff_attention(x, m, w, eps, keys_values):
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = keys_values
    q = (x @ w["q"].T).view(T, H * 2, d)
    q = rotate(rms(q, eps) * w["q.norm"], m["rot"], "interleaved").view(T, H, 2, d)
    mask, lam = visible(T), diff_lambda(m, w)
    heads = []
    for h in range(H):
        g = h // (H // G)
        a = [softmax_rows(q[:, h, i] @ k[:, g, i].T * m["scale"], mask) @ v[:, g] for i in range(2)]
        heads.append(rms(a[0] - lam * a[1], eps) * (1.0 - m["diff"]))
    return torch.cat(heads, -1) @ w["o"].T


def gated_ff(x, w):
    return (silu(x @ w["gate"].T) * (x @ w["up"].T)) @ w["down"].T


def router_choice(z, top):
    """The `top` largest logits of every row (lowest index first on ties) and the softmax over just those."""
    idx = torch.sort(z, dim=-1, descending=True, stable=True).indices[:, :top]
    return idx, torch.softmax(z.gather(1, idx), -1)


def experts(x, mlp, w, margins=None):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = x @ w["router"].T
    idx, wt = router_choice(z, top)
    if margins is not None:
        # how far the last chosen logit lies above the first one left out, per token, in units of the spread of the token's
        # logits (infinite where all are chosen)
        zs = z.sort(-1, descending=True).values
        margins.append((zs[:, top - 1] - zs[:, top]) / (z.std(-1) + 1e-30) if top < E else torch.full((x.shape[0],), math.inf, dtype=F64))
    out = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for r in range(top):
            e = int(idx[t, r])
            out[t] += wt[t, r] * gated_ff(x[t:t + 1], {n: w[f"e{e}.{n}"] for n in ("gate", "up", "down")})[0]
    if mlp.get("shared"):
        sh = {n: w[f"shared.{n}"] for n in ("gate", "up", "down")}
        out = out + gated_ff(x, sh) * torch.sigmoid(x @ w["shared.sg"].T)
    return out


def sub(tensors, prefix):
    return {k[len(prefix):]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, streams=None, margins=None):
    """Logits [T, vocab] (64-bit) of one whole sequence; `streams` (a list) receives x behind every layer, `margins` (a
    list) the router's margin per token of every layer with experts."""
    eps = cfg["norm"]["eps"]
    x = tensors["embed"].to(F64)[torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        m, w = L["mixer"], sub(tensors, f"l{i}.mix.")
        if L["type"] == "attention":
            y = window_attention(x, m, w, eps)
        elif L["type"] == "rglru":
            y = rglru(x, m, w)
        elif L["type"] == "attention_2":
            if m.get("kv_from") is None:
                kept[i] = diff_keys_values(x, m, w, eps)
            y = diff_attention(x, m, w, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        else:
            raise ValueError(L["type"])
        x = x + one_plus_norm(y, tensors[f"l{i}.norm1"].to(F64), eps)
        if L.get("mlp"):
            w = sub(tensors, f"l{i}.mlp.")
            y = gated_ff(x, w) if L["mlp"]["kind"] == "dense" else experts(x, L["mlp"], w, margins)
            x = x + one_plus_norm(y, tensors[f"l{i}.norm2"].to(F64), eps)
        if streams is not None:
            streams.append(x.clone())
    return one_plus_norm(x, tensors["final.norm"].to(F64), eps) @ tensors["head"].to(F64).T
