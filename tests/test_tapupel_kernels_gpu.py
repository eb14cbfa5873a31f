"""The tensor-core kernels that Tapupel's layers use at the head sizes of real models, each against a plain 64-bit statement
of the same operation written here: attention with a capped score and a window that keeps the sequence's first positions,
in the tcgen05 prompt kernel and in the decode kernel, where one strong key sits just inside or outside what a query sees;
differential attention as ordinary heads over spread queries; and the recurrence at a real width."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.ops.types import PagedKV
from test_kernels_gpu import DEV, make_batch

pytestmark = pytest.mark.gpu


def plain_attention(q, k, v, scale, window, keep_first, cap):
    """q [L, H, d], k [L, G, d], v [L, G, dv] in float64 -> [L, H, dv].  Position i sees j <= i with i - j < window or
    j < keep_first (all earlier ones without a window); the scaled score s becomes cap tanh(s / cap)."""
    L, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(L)[:, None], torch.arange(L)[None, :]
    seen = j <= i
    if window:
        seen = seen & ((i - j < window) | (j < keep_first))
    out = []
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].t() * scale
        if cap:
            s = cap * torch.tanh(s / cap)
        out.append(torch.softmax(s.masked_fill(~seen, -math.inf), -1) @ v[:, g])
    return torch.stack(out, 1)


def fill_cache(batch, pt, n_pages, q_lens, starts, G, dk, dv, k_all, v_all):
    kp = torch.zeros(n_pages, G, 64, dk, dtype=torch.bfloat16, device=DEV)
    vp = torch.zeros(n_pages, G, 64, dv, dtype=torch.bfloat16, device=DEV)
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        slot = int(batch.slots[s])
        L = p0 + n
        for page_i in range(-(-L // 64)):
            page = int(pt[slot, page_i])
            rows = slice(page_i * 64, min(L, page_i * 64 + 64))
            kp[page, :, :rows.stop - rows.start] = k_all[s][rows].to(torch.bfloat16).transpose(0, 1).to(DEV)
            vp[page, :, :rows.stop - rows.start] = v_all[s][rows].to(torch.bfloat16).transpose(0, 1).to(DEV)
    return PagedKV(kp, vp, pt, 64)


FORCES = [pytest.param(None, id="dispatch"), pytest.param(dict(prefill=True, tiles=1), id="prompt"),
          pytest.param(dict(splits=1), id="decode"), pytest.param(dict(splits=3), id="decode-three-slices")]


@pytest.mark.parametrize("force", FORCES)
@pytest.mark.parametrize("H,G,d,window,keep,cap", [
    (4, 2, 128, 150, 4, 30.0),
    (8, 1, 64, 70, 70, 8.0),             # as many kept positions as the window is long: more than a page of them
    (6, 2, 128, 333, 1, None),           # kept positions without a cap
    (2, 2, 64, None, 0, 5.0),            # a cap without a window
    (4, 1, 128, 64, 130, 50.0),          # the kept positions span three pages
    (3, 3, 64, 1, 2, 12.0),              # a window of the token itself
])
def test_capped_window_attention(force, H, G, d, window, keep, cap):
    """Prompts from position 0, portions that go on behind cached tokens, and single decoded tokens around page and window
    edges, through each tensor-core kernel by name and through the dispatch.  In every sequence one early key is made strong for
    all queries: it is among the kept positions in some sequences and just behind them in others."""
    decode = force is not None and "splits" in force
    q_lens, starts = ([1, 1, 1, 1, 1, 1], [0, 63, 64, 300, 511, 212]) if decode else ([300, 1, 70, 3, 129], [0, 63, 130, 126, 383])
    g = torch.Generator().manual_seed(23)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).double()   # the oracle sees what the cache stores
    L = [s + n for s, n in zip(starts, q_lens)]
    k_all, v_all, q_all = [bf(n, G, d) for n in L], [bf(n, G, d) for n in L], [bf(n, H, d) for n in L]
    scale = 0.11
    u = torch.where(torch.rand(d, generator=g) < 0.5, -1.0, 1.0).double()       # a direction all queries share
    for s in range(len(L)):
        at = max(0, keep - 1 + (s % 2))                         # the last kept position, or the first one that is not kept
        if at < L[s]:
            q_all[s] = q_all[s] + u
            k_all[s][at] = (u * (12.0 / (scale * d))).to(torch.bfloat16).double()   # its scaled score is about 12 for every query: it takes nearly all the weight
    batch, pt, n_pages = make_batch(q_lens, starts, len(q_lens) + 2, 64, max(-(-n // 64) for n in L), seed=4)
    kv = fill_cache(batch, pt, n_pages, q_lens, starts, G, d, d, k_all, v_all)
    q_all = [x.to(torch.bfloat16).double() for x in q_all]
    q = torch.cat([q_all[s][p0:p0 + n] for s, (n, p0) in enumerate(zip(q_lens, starts))]).to(torch.bfloat16).to(DEV).contiguous()
    out = torch.empty(batch.n_tokens, H * d, dtype=torch.bfloat16, device=DEV)
    if force is None:
        ops.attention(q, kv, batch, out, H, G, d, scale, window, softcap=cap, keep_first=keep)
    else:
        if "splits" in force and keep and window:
            force = dict(splits=force["splits"] + 1)             # the kept positions' slice
        ops.kernels()._attention_bf16(q, kv, batch, out, H, G, d, scale, window, softcap=cap, keep_first=keep if window else 0, **force)
    ops.check_status(batch.status)
    out = out.double().cpu()
    at = 0
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        want = plain_attention(q_all[s], k_all[s], v_all[s], scale, window, keep, cap)[p0:].reshape(n, H * d)
        torch.testing.assert_close(out[at:at + n], want, rtol=3e-2, atol=3e-2)
        at += n
    if window and keep:
        # the kept positions matter at these sizes: without them the longest sequence's results are others
        s = max(range(len(L)), key=lambda i: L[i])
        bare = plain_attention(q_all[s], k_all[s], v_all[s], scale, window, 0, cap)[starts[s]:].reshape(q_lens[s], H * d)
        first = sum(q_lens[:s])
        assert (bare - out[first:first + q_lens[s]]).abs().max() > 0.05


@pytest.mark.parametrize("decode", [False, True], ids=["prompt", "decode"])
@pytest.mark.parametrize("H,G,d,dv", [(4, 2, 64, 128), (8, 2, 32, 64), (2, 2, 64, 128)])
def test_two_maps_as_ordinary_heads(decode, H, G, d, dv):
    """Differential attention with spread queries on the tensor-core kernels against the two softmax maps stated plainly."""
    assert ops.spread_queries(torch.bfloat16, H, G, d, dv, 2, 64)
    q_lens, starts = ([1, 1, 1, 1], [0, 63, 300, 511]) if decode else ([300, 1, 70, 129], [0, 63, 130, 383])
    g = torch.Generator().manual_seed(29)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).double()
    L = [s + n for s, n in zip(starts, q_lens)]
    k_all, v_all, q_all = [bf(n, G, 2 * d) for n in L], [bf(n, G, dv) for n in L], [bf(n, H, 2, d) for n in L]
    scale, lam, eps, out_scale = 0.2, 0.7, 1e-5, 0.6
    batch, pt, n_pages = make_batch(q_lens, starts, len(q_lens) + 2, 64, max(-(-n // 64) for n in L), seed=5)
    kv = fill_cache(batch, pt, n_pages, q_lens, starts, G, 2 * d, dv, k_all, v_all)
    T = sum(q_lens)
    q = torch.zeros(T, H * 2, 2, d, dtype=torch.bfloat16, device=DEV)
    packed = torch.cat([q_all[s][p0:p0 + n] for s, (n, p0) in enumerate(zip(q_lens, starts))]).to(torch.bfloat16).to(DEV)   # [T, H, 2, d]
    for m in range(2):
        q[:, m::2, m] = packed[:, :, m]
    out = torch.empty(T, H * dv, dtype=torch.bfloat16, device=DEV)
    ops.attention(q.view(T, H * 2, 2 * d), kv, batch, out, H, G, d, scale, v_head_dim=dv, maps=2, diff=(lam, eps, out_scale))
    ops.check_status(batch.status)
    out = out.double().cpu()
    at = 0
    for s, (n, p0) in enumerate(zip(q_lens, starts)):
        maps = [plain_attention(q_all[s][:, :, m], k_all[s].view(L[s], G, 2, d)[:, :, m], v_all[s], scale, None, 0, None) for m in range(2)]
        o = maps[0] - lam * maps[1]
        want = (o / torch.sqrt((o * o).mean(-1, keepdim=True) + eps) * out_scale)[p0:].reshape(n, H * dv)
        torch.testing.assert_close(out[at:at + n], want, rtol=4e-2, atol=4e-2)
        at += n


@pytest.mark.parametrize("T,C,B", [(1, 1024, 4), (8, 1024, 4), (300, 512, 2), (77, 640, 1)])
def test_recurrence_at_real_widths(T, C, B):
    """The gate and scan kernels at widths of real layers, several sequences, against the recurrence written out in 64-bit."""
    g = torch.Generator().manual_seed(31)
    bw = C // B
    n_seqs = 1 if T == 1 else 3
    lens = [T] if n_seqs == 1 else [T - 2 * (T // 3), T // 3, T // 3]
    batch, _, _ = make_batch(lens, [0] * n_seqs, n_seqs + 2, 64, -(-max(lens) // 64), seed=6)
    u = torch.randn(T, C, generator=g)
    wa, wi = (torch.randn(B, bw, bw, generator=g) * bw ** -0.5).to(torch.bfloat16), (torch.randn(B, bw, bw, generator=g) * bw ** -0.5).to(torch.bfloat16)
    ba, bi, lam, yb = (torch.randn(C, generator=g) * 0.3 for _ in range(4))
    y = torch.randn(T, C + 8, generator=g).to(torch.bfloat16)
    state = torch.randn(n_seqs + 2, C + 5, generator=g)
    dev = lambda t: t.to(DEV).contiguous()
    st = dev(state)
    out = torch.empty(T, C, dtype=torch.bfloat16, device=DEV)
    ops.rglru(dev(u), dev(wa), dev(wi), dev(ba), dev(bi), dev(lam), 8.0, dev(y), 8, dev(yb), st, 5, out, batch)
    r = torch.sigmoid(torch.einsum("tbi,bio->tbo", u.double().view(T, B, bw), wa.double()).reshape(T, C) + ba.double())
    i = torch.sigmoid(torch.einsum("tbi,bio->tbo", u.double().view(T, B, bw), wi.double()).reshape(T, C) + bi.double())
    a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
    b = torch.sqrt(1 - a * a) * i * u.double()
    z = y[:, 8:].double() + yb.double()
    gate = 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))
    at = 0
    for s, n in enumerate(lens):
        slot = int(batch.slots[s])
        S = state[slot, 5:].double()
        for t in range(at, at + n):
            S = a[t] * S + b[t]
            torch.testing.assert_close(out[t].double().cpu(), S * gate[t], rtol=2e-2, atol=2e-2)
        torch.testing.assert_close(st[slot, 5:].double().cpu(), S, rtol=1e-4, atol=1e-4)
        at += n
