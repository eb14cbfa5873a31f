"""The tensor-core kernels that Lomusun's layers use at the head sizes of real models, each against a plain 64-bit
statement of the same operation written here: attention with a bias by head and distance (a table, or slopes beside a sink)
in the tcgen05 prompt kernels and in the decode kernel, and the experts' products on the tensor cores."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import PagedKV
from test_kernels_gpu import DEV, make_batch

pytestmark = pytest.mark.gpu


def plain_biased_attention(q, k, v, scale, window, sink, table, slopes):
    """q [L, H, d], k and v [L, G, d] in float64; the output [L, H, d].  Position i sees j with 0 <= i - j < window (all
    earlier ones without a window); the scaled score takes table[min(i - j, rows - 1), h] and loses slopes[h] * (i - j); the
    softmax denominator also holds exp(sink[h])."""
    L, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(L, H, d, dtype=torch.float64)
    i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
    n = i - j
    seen = (n >= 0) & ((n < window) if window else True)
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].t() * scale
        if table is not None:
            s = s + table[n.clamp(0, table.shape[0] - 1), h]
        if slopes is not None:
            s = s - slopes[h] * n
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(dim=1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=1, keepdim=True) + (torch.exp(sink[h] - m) if sink is not None else 0.0)
        out[:, h] = (e / den) @ v[:, g]
    return out


def run(q_lens, starts, H, G, d, scale, window, sink, table, slopes, k_all, v_all, q_all, force):
    dtype = torch.bfloat16
    batch, pt, n_pages = make_batch(q_lens, starts, len(q_lens) + 2, 64, max(-(-(s + q) // 64) for s, q in zip(starts, q_lens)), seed=4)
    kp = torch.zeros(n_pages, G, 64, d, dtype=dtype, device=DEV)
    vp = torch.zeros(n_pages, G, 64, d, dtype=dtype, device=DEV)
    qs = []
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        slot = int(batch.slots[s])
        L = p0 + n
        for page_i in range(-(-L // 64)):
            page = int(pt[slot, page_i])
            rows = slice(page_i * 64, min(L, page_i * 64 + 64))
            kp[page, :, :rows.stop - rows.start] = k_all[s][rows].to(dtype).transpose(0, 1).to(DEV)
            vp[page, :, :rows.stop - rows.start] = v_all[s][rows].to(dtype).transpose(0, 1).to(DEV)
        qs.append(q_all[s][p0:p0 + n])
    q = torch.cat(qs).to(dtype).to(DEV).contiguous()
    out = torch.empty(batch.n_tokens, H * d, dtype=dtype, device=DEV)
    kv = PagedKV(kp, vp, pt, 64)
    kw = dict(bias=None if table is None else table.float().to(DEV).contiguous(), slopes=None if slopes is None else slopes.float().to(DEV))
    sk = None if sink is None else sink.float().to(DEV)
    if force is None:
        ops.attention(q, kv, batch, out, H, G, d, scale, window, None, sk, d, **kw)
    else:
        ops.kernels()._attention_bf16(q, kv, batch, out, H, G, d, scale, window, sink=sk, **kw, **force)
    ops.check_status(batch.status)
    return out.double().cpu()


FORCES = [pytest.param(None, id="dispatch"), pytest.param(dict(prefill=True, tiles=1), id="prompt-one-tile"),
          pytest.param(dict(prefill=True, tiles=2), id="prompt-two-tiles"), pytest.param(dict(splits=1), id="decode"),
          pytest.param(dict(splits=3), id="decode-three-slices")]


@pytest.mark.parametrize("force", FORCES)
@pytest.mark.parametrize("H,G,d,window,rows,kind", [
    (4, 2, 128, 150, 150, "table"),        # a table as long as the window
    (8, 1, 64, None, 40, "table"),         # no window: far keys all take the last row
    (6, 2, 128, 333, 97, "table"),         # the table ends inside the window
    (2, 2, 64, 70, 70, "table"),
    (4, 1, 128, 200, 0, "slopes"),         # slopes beside a sink
    (3, 3, 64, None, 0, "slopes"),
    (4, 2, 128, 65, 30, "both"),
])
def test_attention_with_a_distance_bias(force, H, G, d, window, rows, kind):
    """Prompts from position 0, portions that go on behind cached tokens, and single decoded tokens around page and window
    edges, through each tensor-core kernel by name and through the dispatch."""
    if force and force.get("tiles") == 2 and d != 128:
        pytest.skip("the two-tile kernel is built for heads of 128")
    decode = force is not None and "splits" in force
    q_lens, starts = ([1, 1, 1, 1, 1], [0, 63, 64, 300, 511]) if decode else ([300, 1, 70, 3, 129], [0, 63, 130, 126, 383])
    g = torch.Generator().manual_seed(21)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).double()   # the oracle sees what the cache stores
    L = [s + n for s, n in zip(starts, q_lens)]
    k_all, v_all, q_all = [bf(n, G, d) for n in L], [bf(n, G, d) for n in L], [bf(n, H, d) for n in L]
    table = torch.randn(rows, H, generator=g).double() * 2 if kind in ("table", "both") else None
    slopes = torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=torch.float64) if kind in ("slopes", "both") else None
    sink = torch.randn(H, generator=g).double() * 2 if kind in ("slopes", "both") else None
    scale = 0.11
    out = run(q_lens, starts, H, G, d, scale, window, sink, table, slopes, k_all, v_all, q_all, force)
    at = 0
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        f32 = lambda t: None if t is None else t.float().double()
        want = plain_biased_attention(q_all[s], k_all[s], v_all[s], scale, window, f32(sink), f32(table), f32(slopes))[p0:].reshape(n, H * d)
        torch.testing.assert_close(out[at:at + n], want, rtol=3e-2, atol=3e-2)
        at += n
    # the bias matters at these sizes: without it the last sequence's result is another
    bare = plain_biased_attention(q_all[-1], k_all[-1], v_all[-1], scale, window, sink, None, None)[starts[-1]:].reshape(q_lens[-1], H * d)
    assert (bare - out[at - q_lens[-1]:at]).abs().max() > 0.05


@pytest.mark.parametrize("force", FORCES)
@pytest.mark.parametrize("gap", ["inside", "outside"])
def test_one_strong_key_at_the_edge_of_table_and_window(force, gap):
    """The query meets one key far stronger than the rest on the last position the window keeps (found, through the table's
    last row of +4) or one beyond it (not seen, whatever the table says)."""
    H, G, d, window, rows = 2, 1, 128, 201, 50
    decode = force is not None and "splits" in force
    p = 64 * 5 + 17
    key_at = p - (window - 1 if gap == "inside" else window)
    g = torch.Generator().manual_seed(22)
    k = torch.randn(p + 1, G, d, generator=g) * 0.1
    v = torch.randn(p + 1, G, d, generator=g)
    q = torch.randn(p + 1, H, d, generator=g) * 0.1
    q[p, :, 0], k[key_at, :, 0] = 30.0, 30.0
    table = torch.zeros(rows, H, dtype=torch.float64)
    table[-1] = 4.0
    q_lens, starts = ([1], [p]) if decode else ([p + 1], [0])
    out = run(q_lens, starts, H, G, d, 0.05, window, None, table, None, [k.double()], [v.double()], [q.double()], force)[-1].view(H, d)
    target = v[key_at, 0].to(torch.bfloat16).double()
    if gap == "inside":
        torch.testing.assert_close(out, target.expand(H, d), rtol=2e-2, atol=2e-2)
    else:
        assert (out - target).abs().max() > 0.3


# ---- the experts' products on the tensor cores ------------------------------------------------------------------------------

@pytest.mark.parametrize("T,E,top,F,D,limit", [(300, 6, 2, 136, 320, 1.5), (5, 3, 3, 8, 8, 0.0), (130, 2, 1, 264, 72, 0.7), (64, 16, 4, 72, 192, 1.2),
                                                   (1, 4, 2, 200, 328, 1.0), (900, 2, 1, 136, 320, 1.5), (1300, 3, 1, 40, 264, 0.0),
                                                   (700, 4, 3, 264, 72, 0.9), (20, 5, 2, 24, 40, 0.8)],
                         ids=["several-tiles-each-way", "smallest", "one-expert-two-row-tiles", "a-decode-batch", "one-token",
                              "tiles-of-256-rows", "tiles-of-256-rows-all-of-one-expert", "tiles-of-256-rows-three-each", "tiles-of-32-tokens"])
def test_experts_on_the_tensor_cores(T, E, top, F, D, limit):
    """Rows sorted by expert in tiles (16 to 64 tokens as the columns of the swapped MMA in a decode step, 128 rows, 256 rows for
    pairs of SMs from about two full tiles per expert on), the gate/up product with the clamped activation in its epilogue, the down
    product and the weighted sum, against the same sums in 64-bit; some experts get no token at all."""
    g = torch.Generator().manual_seed(T + E)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16)
    h, gate, up, down = bf(T, D), bf(E, F, D, s=D ** -0.5), bf(E, F, D, s=D ** -0.5), bf(E, D, F, s=F ** -0.5)
    busy = max(top, E - 2)                                    # the last experts stay idle
    idx = torch.stack([torch.randperm(busy, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    w = torch.rand(T, top, generator=g) + 0.1
    alpha, shift = 1.702, 1.0
    want = torch.zeros(T, D, dtype=torch.float64)
    for t in range(T):
        for r in range(top):
            e = int(idx[t, r])
            a, b = gate[e].double() @ h[t].double(), up[e].double() @ h[t].double()
            if limit > 0:
                a, b = a.clamp(max=limit), b.clamp(-limit, limit)
            act = (a * torch.sigmoid(alpha * a) * (b + shift)).to(torch.bfloat16).double()
            want[t] += float(w[t, r]) * (down[e].double() @ act)
    w13 = torch.stack([gate, up], dim=2).reshape(E, 2 * F, D).contiguous().cuda()
    x = torch.full((T, D), 0.25, dtype=torch.float32, device="cuda")
    assert T > ops.kernels().MOE_TC_FEW_TOKENS
    ops.moe_experts(h.cuda(), idx.cuda(), w.cuda(), w13, down.cuda(), x, limit, alpha, shift)
    ops.check_status(ops.kernels().status)
    err = (x.cpu().double() - 0.25 - want).abs().max() / want.abs().max()
    assert float(err) < 6e-3, float(err)                      # one bfloat16 rounding of the activation, 32-bit sums


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,E,top,D", [(1, 5, 2, 40), (7, 40, 3, 200), (64, 130, 32, 72)])
def test_router_in_one_launch(dtype, T, E, top, D):
    """A decode step's router (logits and choice by one kernel) against sigmoid, correction, top and weights in 64-bit; the
    correction decides a choice here and there, and the weights leave it out."""
    g = torch.Generator().manual_seed(E)
    h = torch.randn(T, D, generator=g).to(dtype)
    router = (torch.randn(E, D, generator=g) * D ** -0.5).to(dtype)
    corr = (torch.randn(E, generator=g) * 0.2).float()
    pad = torch.cat([router, torch.zeros(-E % 8, D, dtype=dtype)])
    idx = torch.empty(T, top, dtype=torch.int32, device="cuda")
    w = torch.empty(T, top, dtype=torch.float32, device="cuda")
    assert ops.kernels().moe_router(h.cuda(), pad.cuda(), corr.cuda(), top, 1.7, idx, w)
    s = torch.sigmoid(h.double() @ router.double().T)
    choice = s + corr.double()
    for t in range(T):
        order = sorted(range(E), key=lambda e: (-float(choice[t, e]), e))[:top]
        gap = float(choice[t].sort(descending=True).values[top - 1] - choice[t].sort(descending=True).values[top]) if top < E else 1.0
        if gap < 1e-3:
            continue                                           # a close call may fall either way in bfloat16
        assert sorted(idx[t].tolist()) == sorted(order), (t, idx[t].tolist(), order)
        picked = s[t, idx[t].long().cpu()]
        torch.testing.assert_close(w[t].cpu().double(), picked / picked.sum() * 1.7, rtol=2e-3, atol=1e-5)
