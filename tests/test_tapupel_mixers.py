"""Each mechanism of the Tapupel design alone, as a part with a cache entry of its own, against the plain statement of the
mechanism in `plain_tapupel.py`: the input goes in whole, in portions and as a batch of two sequences, and what the part adds
to an empty stream is compared.  Where random inputs would hide a fault (a key at a window's edge, among the kept first
positions or hundreds of positions back, the second score map) the inputs are made so that one score stands out.  Three back
ends as in `test_tapupel.py`."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.cache import Cache
from gpt_fast_b200.cache.paged import EntryView
from gpt_fast_b200.config.spec import PartSpec
from gpt_fast_b200.ops.types import BatchMeta
from gpt_fast_b200.parts import FEED_FORWARDS, MIXERS, POSITIONS, build_part
from gpt_fast_b200.parts.residual import Branch
from gpt_fast_b200.parts.rope import rope_frequencies
import plain_tapupel as pt
import plain_ops

BACKENDS = [
    pytest.param(("cpu", torch.float32), id="cpu-standin-f32"),
    pytest.param(("cuda", torch.float32), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", torch.bfloat16), id="cuda-bf16", marks=pytest.mark.gpu),
]
D, EPS = 40, 1e-5


@pytest.fixture(params=BACKENDS)
def backend(request):
    device, dtype = request.param
    prev = ops.use_kernels(plain_ops.PlainOps()) if device == "cpu" else None
    yield device, dtype
    if device == "cpu":
        ops.use_kernels(prev)


def rand(shape, seed, scale=1.0, shift=0.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale + shift).to(torch.bfloat16)


def batch_of(cache, live, q_lens, device):
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    return BatchMeta(torch.tensor(cu, dtype=torch.int32).to(device),
                     torch.tensor([i for i, q in enumerate(q_lens) for _ in range(q)], dtype=torch.int32).to(device),
                     torch.tensor(live, dtype=torch.int32).to(device), cache.lengths, len(live), cu[-1], max(q_lens),
                     max(cache.lengths_host[s] + q for s, q in zip(live, q_lens)), ops.new_status(device))


def run(mixers, h, seqs, cuts, device, dtype, width=D):
    """Feed the sequences (lists of row ranges of h) through the mixers (entry 0 owns keys and values; a second mixer reads
    them) as one batch, each cut at `cuts`; returns what each mixer added, in h's row order."""
    cache = Cache({i: m.cache_needs() for i, m in enumerate(mixers)}, dtype, device, max_tokens=2048, max_seqs=4)
    for m in mixers:
        if getattr(m, "position", None) is not None:
            m.position.prepare(cache.max_pages * cache.page_size, device)
    slots = cache.begin(len(seqs))
    outs = [torch.zeros(h.shape[0], width) for _ in mixers]
    bounds = [0] + list(cuts) + [max(len(s) for s in seqs)]
    for lo, hi in zip(bounds[:-1], bounds[1:]):
        live = [(slot, s[lo:hi]) for slot, s in zip(slots, seqs) if len(s[lo:hi])]
        if not live:
            continue
        rows = [r for _, part in live for r in part]
        q_lens = [len(part) for _, part in live]
        for slot, part in live:
            cache.reserve(slot, cache.lengths_host[slot] + len(part))
        cache.sync_tables()
        batch = batch_of(cache, [s for s, _ in live], q_lens, device)
        x = h[rows].to(dtype).to(device).contiguous()
        for i, m in enumerate(mixers):
            y = Branch(len(rows), width, device)
            if i == 0:
                m.forward(x, batch, cache.view(0), residual=y, append=True)
            else:
                m.forward(x, batch, EntryView(kv=cache.view(0).kv, state=cache.view(i).state), residual=y, append=False)
            outs[i][rows] = y.tensor().float().cpu()
        ops.advance_lengths(batch)
        cache.note_advance([s for s, _ in live], q_lens)
        ops.check_status(batch.status)
    cache.end(slots)
    return outs


def judge(got, want, dtype, where, rows=None, bf16=0.03):
    if rows is not None:
        got, want = got[rows], want[rows]
    if dtype == torch.float32:
        torch.testing.assert_close(got, want.float(), rtol=3e-4, atol=3e-4, msg=lambda m: f"{where}\n{m}")
    else:
        scale = float(want.pow(2).mean().sqrt())
        assert float((got - want.float()).pow(2).mean().sqrt()) <= bf16 * scale, where


def load(part, weights, names, backend):
    """Matrices in the compute type, vectors in 32-bit, under the part's own parameter names."""
    device, dtype = backend
    specs = part.param_specs()
    part.load({k: weights[v].to(dtype if specs[k].role == "matrix" else torch.float32).to(device) for k, v in names.items()})


def f64(w):
    return {k: v.double() for k, v in w.items()}


CUTS = (([], "whole"), ([1, 3, 64, 66], "portions"), (list(range(60, 75)), "a prompt, then token by token"))

# ---- the rotary frequencies with their rescaling ---------------------------------------------------------------------

def test_frequencies_hit_all_three_branches():
    rot = {"dims": 16, "base": 10000.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    want = pt.frequencies(rot)
    plain_f = torch.tensor([10000.0 ** (-2.0 * i / 16) for i in range(8)], dtype=torch.float64)
    kept, divided = (want == plain_f), torch.isclose(want, plain_f / 4.0, rtol=1e-12)
    assert kept.any() and divided.any() and (~kept & ~divided).any()              # fast, slow and blended pairs
    sc = rot["scaling"]
    got = rope_frequencies(16, 10000.0, dict(factor=sc["factor"], low_freq_factor=sc["low"], high_freq_factor=sc["high"],
                                            original_max_position_embeddings=sc["original"]), "float64")
    torch.testing.assert_close(got.double(), want, rtol=1e-6, atol=0)


# ---- the 'attention' mixer: values that are the keys, rotation then a bare norm, a capped score, a window with kept first positions ----

ATT = dict(heads=4, kv_heads=2, dim=12, vdim=12, scale=0.3, softcap=5.0, mask=dict(size=19, keep_first=3),
           rot=dict(dims=8, base=10000.0, scaling=dict(factor=4.0, low=1.0, high=4.0, original=16)))
ATT_NAMES = dict(wq="q", wk="k", wo="o")


def att_weights(m, seed, s=0.3):
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    return {"q": rand((H * d, D), seed, s), "k": rand((G * d, D), seed + 1, s), "o": rand((D, H * d), seed + 2, s)}


def att_part(m, dtype):
    rot, sc = m["rot"], m["rot"].get("scaling")
    scaling = None if sc is None else dict(factor=sc["factor"], low_freq_factor=sc["low"], high_freq_factor=sc["high"],
                                           original_max_position_embeddings=sc["original"])
    pos = build_part(POSITIONS, PartSpec("rope", dict(head_dim=rot["dims"], base=rot["base"], scaling=scaling, pairing="half", freq_dtype="float64")))
    mask = m.get("mask") or {}
    return build_part(MIXERS, PartSpec("attention", dict(dim=D, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], scale=m["scale"],
                                                         window=mask.get("size"), keep_first=mask.get("keep_first", 0), softcap=m.get("softcap"),
                                                         qk_norm_eps=EPS, qk_norm_weight=False, qk_norm_last=True, values_are_keys=True)),
                      dtype=dtype, position=pos)


@pytest.mark.parametrize("m", [
    pytest.param(ATT, id="window-19-keep-3"),
    pytest.param(dict(ATT, heads=2, kv_heads=2, dim=20, vdim=20, mask=dict(size=1, keep_first=5), softcap=None, rot=dict(dims=20, base=300.0)), id="window-1-keep-5"),
    pytest.param(dict(ATT, heads=1, kv_heads=1, mask=None, rot=dict(dims=2, base=20.0)), id="no-window"),
    pytest.param(dict(ATT, mask=dict(size=70, keep_first=0)), id="window-70-keep-0"),
])
def test_window_attention(backend, m):
    device, dtype = backend
    w = att_weights(m, 1)
    a = att_part(m, dtype)
    load(a, w, ATT_NAMES, backend)
    h = rand((80, D), 5).float()
    s0, s1 = list(range(0, 75)), list(range(75, 80))
    want = torch.cat([pt.window_attention(h[s].double(), m, f64(w), EPS) for s in (s0, s1)])
    for cuts, where in CUTS + (([2, 4], "a batch of two, cut"),):
        seqs = [s0, s1] if "batch" in where else [s0]
        (got,) = run([a], h, seqs, cuts, device, dtype)
        judge(got, want, dtype, f"attention: {where}", [r for s in seqs for r in s])


@pytest.mark.parametrize("where_key", ["window edge", "kept first", "far back"])
def test_one_key_that_stands_out(backend, where_key):
    """One key whose direction every query shares on the unrotated dimensions and whose value is unlike all others: whether it
    is seen decides the output.  It sits just inside / outside the window, among / behind the kept first positions, or hundreds
    of positions back where only the kept first positions reach; in a whole prompt and in decode steps."""
    device, dtype = backend
    W, F = 70, 4
    m = dict(heads=2, kv_heads=1, dim=16, vdim=16, scale=3.0, softcap=40.0, mask=dict(size=W, keep_first=F), rot=dict(dims=4, base=100.0))
    n = 330
    key_at = {"window edge": 200, "kept first": F - 1, "far back": F}[where_key]
    h = rand((n, D), 11, 0.2).float()
    h[:, 0] = 0.0
    h[key_at, 0] = 6.0                                      # column 0 marks the key ...
    h[:, 1] = 1.0                                           # ... and column 1 makes every query look for it
    w = att_weights(m, 3, 0.05)
    wq, wk = w["q"].float(), w["k"].float()
    wq[:, 1], wk[:, 0] = 0.0, 0.0
    for head in range(2):
        wq[head * 16 + 8:head * 16 + 16, 1] = 1.0           # unrotated dimensions of every query head
    wk[8:16, 0] = 1.0
    w["q"], w["k"] = wq.to(torch.bfloat16), wk.to(torch.bfloat16)
    a = att_part(m, dtype)
    load(a, w, ATT_NAMES, backend)
    want = pt.window_attention(h.double(), m, f64(w), EPS)
    # the test is sharp: the rows that just lose sight of the key differ from their neighbours by about the output's scale
    if where_key == "window edge":
        last_in, first_out = key_at + W - 1, key_at + W
    else:
        last_in, first_out = (n - 1, None) if where_key == "kept first" else (key_at + W - 1, key_at + W)
    if first_out is not None:
        assert float((want[first_out] - want[last_in]).norm()) > 0.5 * float(want[last_in].norm())
    seq = list(range(n))
    for cuts, where in (([], "whole"), ([key_at + 1, key_at + W - 2] + list(range(key_at + W - 1, key_at + W + 3)), "decoded over the edge"),
                        (list(range(300, n)), "long prompt, then decoded")):
        (got,) = run([a], h, [seq], sorted(set(c for c in cuts if 0 < c < n)), device, dtype)
        judge(got, want, dtype, f"{where_key}: {where}", bf16=0.05)


# ---- the gated linear recurrence -----------------------------------------------------------------------------------------

RG_NAMES = dict(wy="y", y_bias="y.b", wx="x", x_bias="x.b", conv="conv", conv_bias="conv.b", gate_a="ra", gate_a_bias="ra.b",
                gate_i="ri", gate_i_bias="ri.b", lam="lam", wo="o")


def rg_weights(C, B, taps, seed, lam_shift=0.0):
    bw = C // B
    return {"y": rand((C, D), seed, 0.3), "y.b": rand((C,), seed + 1, 0.2), "x": rand((C, D), seed + 2, 0.3), "x.b": rand((C,), seed + 3, 0.2),
            "conv": rand((C, taps), seed + 4, 0.5), "conv.b": rand((C,), seed + 5, 0.2), "ra": rand((B, bw, bw), seed + 6, 0.3),
            "ra.b": rand((B, bw), seed + 7, 0.3), "ri": rand((B, bw, bw), seed + 8, 0.3), "ri.b": rand((B, bw), seed + 9, 0.3),
            "lam": rand((C,), seed + 10, 1.0, lam_shift), "o": rand((D, C), seed + 11, 0.3)}


@pytest.mark.parametrize("C,B,taps", [(48, 3, 4), (32, 1, 1), (40, 2, 2), (136, 1, 3)])
def test_gated_linear_recurrence(backend, C, B, taps):
    device, dtype = backend
    w = rg_weights(C, B, taps, 7)
    part = build_part(MIXERS, PartSpec("rglru", dict(dim=D, width=C, blocks=B, taps=taps)), dtype=dtype, position=None)
    load(part, w, RG_NAMES, backend)
    h = rand((80, D), 9).float()
    s0, s1 = list(range(0, 75)), list(range(75, 80))
    m = dict(width=C, blocks=B, conv=taps)
    want = torch.cat([pt.rglru(h[s].double(), m, f64(w)) for s in (s0, s1)])
    for cuts, where in CUTS + (([2, 4], "a batch of two, cut"),):
        seqs = [s0, s1] if "batch" in where else [s0]
        (got,) = run([part], h, seqs, cuts, device, dtype)
        judge(got, want, dtype, f"recurrence of {C} channels in {B} blocks, {taps} taps: {where}", [r for s in seqs for r in s])


def test_a_state_that_remembers(backend):
    """Decays close to one: what the first tokens wrote still decides the output hundreds of steps later, in a prompt cut
    anywhere and decoded token by token; a state that is lost or zeroed on the way shows."""
    device, dtype = backend
    C, B, taps = 24, 2, 3
    w = rg_weights(C, B, taps, 21, lam_shift=-7.0)         # softplus(lam) ~ 1e-3: a ~ 0.996 per step
    part = build_part(MIXERS, PartSpec("rglru", dict(dim=D, width=C, blocks=B, taps=taps)), dtype=dtype, position=None)
    load(part, w, RG_NAMES, backend)
    h = rand((300, D), 4, 0.1).float()
    h[:6] *= 400.0                                          # a loud start, then near silence
    m = dict(width=C, blocks=B, conv=taps)
    want = pt.rglru(h.double(), m, f64(w))
    quiet = pt.rglru(h[6:].double(), m, f64(w))
    assert float((want[200:] - quiet[194:]).norm()) > 0.5 * float(want[200:].norm())     # the start is still heard at the end
    for cuts in ([], [3, 64, 128, 130, 192], [100] + list(range(250, 300))):
        (got,) = run([part], h, [list(range(300))], cuts, device, dtype)
        judge(got, want, dtype, f"a long memory, cut at {cuts[:4]}", bf16=0.05)


# ---- differential attention and a reader of its keys and values -------------------------------------------------------------

DIFF = dict(heads=4, kv_heads=2, dim=10, vdim=14, scale=0.4, diff=0.3, rot=dict(dims=6, base=100.0))
DIFF_NAMES = dict(wq="q", wk="k", wv="v", wo="o", q_norm="q.norm", k_norm="k.norm", lq1="lq1", lk1="lk1", lq2="lq2", lk2="lk2")


def diff_weights(m, seed, reader=False, s=0.3):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"q": rand((H * 2 * d, D), seed, s), "q.norm": rand((d,), seed + 1, 0.2, 1.0), "o": rand((D, H * dv), seed + 2, s)}
    for i, n in enumerate(("lq1", "lk1", "lq2", "lk2")):
        w[n] = rand((d,), seed + 3 + i, 0.4)
    if not reader:
        w.update({"k": rand((G * 2 * d, D), seed + 8, s), "k.norm": rand((d,), seed + 9, 0.2, 1.0), "v": rand((G * dv, D), seed + 10, s)})
    return w


def diff_part(m, dtype, reader=False):
    pos = build_part(POSITIONS, PartSpec("rope", dict(head_dim=m["rot"]["dims"], base=m["rot"]["base"], pairing="interleaved", freq_dtype="float64")))
    return build_part(MIXERS, PartSpec("diff_attention", dict(dim=D, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                              scale=m["scale"], diff=m["diff"], eps=EPS, shared_kv=reader)),
                      dtype=dtype, position=pos)


@pytest.mark.parametrize("m", [pytest.param(DIFF, id="grouped"),
                               pytest.param(dict(DIFF, heads=1, kv_heads=1, dim=8, vdim=6, rot=dict(dims=8, base=50.0), diff=0.8), id="one-head")])
def test_differential_attention_and_its_reader(backend, m):
    device, dtype = backend
    reader_m = dict(m, scale=0.25, diff=0.55)
    w0, w1 = diff_weights(m, 1), diff_weights(reader_m, 30, reader=True)
    assert abs(pt.diff_lambda(m, f64(w0)) - m["diff"]) > 0.05            # the learned part of lambda counts
    a, b = diff_part(m, dtype), diff_part(reader_m, dtype, reader=True)
    load(a, w0, DIFF_NAMES, backend)
    load(b, w1, {k: v for k, v in DIFF_NAMES.items() if k in b.param_specs()}, backend)
    h = rand((80, D), 5).float()
    s0, s1 = list(range(0, 75)), list(range(75, 80))
    want0, want1 = [], []
    for s in (s0, s1):
        kv = pt.diff_keys_values(h[s].double(), m, f64(w0), EPS)
        want0.append(pt.diff_attention(h[s].double(), m, f64(w0), EPS, kv))
        want1.append(pt.diff_attention(h[s].double(), reader_m, f64(w1), EPS, kv))
    want0, want1 = torch.cat(want0), torch.cat(want1)
    for cuts, where in CUTS + (([2, 4], "a batch of two, cut"),):
        seqs = [s0, s1] if "batch" in where else [s0]
        got0, got1 = run([a, b], h, seqs, cuts, device, dtype)
        rows = [r for s in seqs for r in s]
        judge(got0, want0, dtype, f"differential attention: {where}", rows)
        judge(got1, want1, dtype, f"a reader of its keys and values: {where}", rows)


def test_a_far_key_in_the_second_map_only(backend):
    """A key 300 positions back that only the second map's queries look for: a map that reads the other map's keys, or a
    lambda with the wrong sign, shows at once."""
    device, dtype = backend
    m = dict(heads=2, kv_heads=1, dim=8, vdim=12, scale=3.0, diff=0.4, rot=dict(dims=2, base=10.0))
    n = 320
    h = rand((n, D), 13, 0.2).float()
    h[:, 0] = 0.0
    h[7, 0] = 6.0
    h[:, 1] = 1.0
    w = diff_weights(m, 17, s=0.05)
    wq, wk = w["q"].float(), w["k"].float()
    wq[:, 1], wk[:, 0] = 0.0, 0.0
    for head in range(2):
        wq[head * 16 + 8 + 2:head * 16 + 16, 1] = 1.0       # the second map's unrotated dimensions
    wk[8 + 2:16, 0] = 1.0
    w["q"], w["k"] = wq.to(torch.bfloat16), wk.to(torch.bfloat16)
    a = diff_part(m, dtype)
    load(a, w, DIFF_NAMES, backend)
    want = pt.diff_attention(h.double(), m, f64(w), EPS, pt.diff_keys_values(h.double(), m, f64(w), EPS))
    for cuts in ([], [8, 64, 128, 256] + list(range(300, n))):
        (got,) = run([a], h, [list(range(n))], cuts, device, dtype)
        judge(got, want, dtype, f"a far key of the second map, cut at {cuts[:4]}", bf16=0.05)


# ---- the experts: the largest logits, a softmax over the chosen ones, a shared expert behind a gate per token ----------------

@pytest.mark.parametrize("E,top,F,Fs", [(5, 2, 24, 16), (40, 1, 8, 0), (3, 3, 8, 24), (12, 3, 16, 16), (1, 1, 8, 8)])
def test_experts(backend, E, top, F, Fs):
    device, dtype = backend
    part = build_part(FEED_FORWARDS, PartSpec("moe", dict(dim=D, hidden=F, n_experts=E, top=top, score="softmax_top", correction=False,
                                                          alpha=1.0, shift=0.0, limit=0.0, shared_hidden=Fs, shared_gate=Fs > 0)), dtype=dtype)
    w = {"router": rand((E, D), 1, 0.5)}
    for e in range(E):
        w.update({f"e{e}.gate": rand((F, D), 10 + 3 * e, 0.3), f"e{e}.up": rand((F, D), 11 + 3 * e, 0.3), f"e{e}.down": rand((D, F), 12 + 3 * e, 0.3)})
    names = {}
    if Fs:
        w.update({"shared.gate": rand((Fs, D), 200, 0.3), "shared.up": rand((Fs, D), 201, 0.3), "shared.down": rand((D, Fs), 202, 0.3),
                  "shared.sg": rand((1, D), 203, 0.5)})
        names = dict(shared_gate="shared.gate", shared_up="shared.up", shared_down="shared.down", shared_sg="shared.sg")
    tensors = {"router": w["router"], "gate": torch.stack([w[f"e{e}.gate"] for e in range(E)]), "up": torch.stack([w[f"e{e}.up"] for e in range(E)]),
               "down": torch.stack([w[f"e{e}.down"] for e in range(E)])}
    tensors.update({k: w[v] for k, v in names.items()})
    part.load({k: v.to(dtype).to(device) for k, v in tensors.items()})
    mlp = {"router": {"experts": E, "top": top}, "shared": {"ff": Fs} if Fs else None}
    for T in (1, 7, 40, 150):                              # decode steps and prompts take other kernels
        h = rand((T, D), 50 + T).float()
        if dtype == torch.bfloat16:
            # no close calls: rows whose top-th and next logits are nearer than bfloat16 can tell apart are left out
            z = (h.double() @ w["router"].double().T).sort(-1, descending=True).values
            keep = torch.ones(T, dtype=torch.bool) if top == E else (z[:, top - 1] - z[:, top]) > 0.15
        else:
            keep = torch.ones(T, dtype=torch.bool)
        want = pt.experts(h.double(), mlp, f64(w))
        y = Branch(T, D, device)
        part.forward(h.to(dtype).to(device), residual=y)
        got = y.tensor().float().cpu()
        judge(got[keep], want[keep], dtype, f"{top} of {E} experts of {F}, shared {Fs}, {T} tokens", bf16=0.04)


def test_the_chosen_experts_and_their_weights(backend):
    device, dtype = backend
    z = torch.tensor([[0.1, 2.0, -1.0, 1.5, 0.3], [3.0, 3.0, 3.0, -9.0, 2.0]])
    idx = torch.empty(2, 3, dtype=torch.int32, device=device)
    wts = torch.empty(2, 3, dtype=torch.float32, device=device)
    ops.moe_route(z.to(device), torch.zeros(5, device=device), 3, 1.0, idx, wts, score="softmax_top")
    want_idx, want_w = pt.router_choice(z.double(), 3)
    assert idx.cpu().tolist() == want_idx.tolist() == [[1, 3, 4], [0, 1, 2]]
    torch.testing.assert_close(wts.cpu().double(), want_w, rtol=1e-6, atol=1e-7)
