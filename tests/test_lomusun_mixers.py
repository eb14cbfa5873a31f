"""Each mechanism of the Lomusun design alone, as a part with a cache entry of its own, against the plain statement of the
mechanism in `plain_lomusun.py`: the normed input goes in whole, in portions and as a batch of two sequences, and what the
part adds to an empty stream is compared.  Where random inputs would hide a fault (a key at a window's edge or hundreds of
positions back, the sink) the inputs are made so that one score stands out.  Three back ends as in `test_lomusun.py`."""
import math

import pytest
import torch

from gpt_fast_b200 import ops
from gpt_fast_b200.cache import Cache
from gpt_fast_b200.cache.paged import EntryView
from gpt_fast_b200.config.spec import PartSpec
from gpt_fast_b200.ops.types import BatchMeta
from gpt_fast_b200.parts import EMBEDDINGS, FEED_FORWARDS, MIXERS, build_part
from gpt_fast_b200.parts.attention import distance_bucket
from gpt_fast_b200.parts.residual import Branch
import plain_lomusun as pl
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
    them with a state entry of its own) as one batch, each cut at `cuts`; returns what each mixer added, in h's row order."""
    cache = Cache({i: m.cache_needs() for i, m in enumerate(mixers)}, dtype, device, max_tokens=2048, max_seqs=4)
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


def judge(got, want, dtype, where, rows=None):
    if rows is not None:
        got, want = got[rows], want[rows]
    if dtype == torch.float32:
        torch.testing.assert_close(got, want.float(), rtol=3e-4, atol=3e-4, msg=lambda m: f"{where}\n{m}")
    else:
        scale = float(want.pow(2).mean().sqrt())
        assert float((got - want.float()).pow(2).mean().sqrt()) <= 0.03 * scale, where


def load(mixer, weights, names, backend):
    device, dtype = backend
    mixer.load({k: weights[v].to(dtype if weights[v].dim() > 1 and "conv" not in v and v != "rel" else torch.float32).to(device)
                for k, v in names.items()})


CUTS = (([], "whole"), ([1, 3, 64, 66], "portions"), (list(range(60, 75)), "a prompt, then token by token"))

# ---- the 'attention' mixer: convolved q/k/v, a learned distance table, a window, a gate per head; and a reader ------

ATT = dict(heads=4, kv_heads=2, dim=12, vdim=10, conv=3, scale=0.3, bias_max=30, mask=dict(size=19))
ATT_NAMES = dict(wq="q", wk="k", wv="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", rel="rel", wg="g", wo="o")


def att_weights(m, rows, seed, reader=False):
    H, G, d, dv, t = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    w = {"q": rand((H * d, D), seed, 0.3), "q.conv": rand((H * d, t), seed + 1, 0.5), "rel": rand((rows, H), seed + 2),
         "g": rand((H, D), seed + 3, 0.3), "o": rand((D, H * dv), seed + 4, 0.3)}
    if not reader:
        w.update({"k": rand((G * d, D), seed + 5, 0.3), "k.conv": rand((G * d, t), seed + 6, 0.5),
                  "v": rand((G * dv, D), seed + 7, 0.3), "v.conv": rand((G * dv, t), seed + 8, 0.5)})
    return w


def att_part(m, rows, dtype, reader=False):
    return build_part(MIXERS, PartSpec("attention", dict(dim=D, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                         window=m["mask"]["size"], scale=m["scale"], conv_taps=m["conv"], gate="head",
                                                         distance_bias=dict(kind="table", rows=rows, far=m["bias_max"]), shared_kv=reader)),
                      dtype=dtype, position=None)


def test_table_attention_and_its_reader(backend):
    device, dtype = backend
    owner, reader_m = ATT, dict(ATT, heads=2, conv=2, scale=0.4, bias_max=12, mask=dict(size=33))
    w0, w1 = att_weights(owner, 10, 1), att_weights(reader_m, 7, 20, reader=True)
    a, b = att_part(owner, 10, dtype), att_part(reader_m, 7, dtype, reader=True)
    load(a, w0, ATT_NAMES, backend)
    load(b, w1, {k: v for k, v in ATT_NAMES.items() if k in b.param_specs()}, backend)
    h = rand((80, D), 5).float()
    s0, s1 = list(range(0, 75)), list(range(75, 80))
    want0, want1 = [], []
    for s in (s0, s1):
        y, kv = pl.conv_attention(h[s].double(), {"p." + k: v.double() for k, v in w0.items()}, "p.", owner)
        want0.append(y)
        want1.append(pl.conv_attention(h[s].double(), {"p." + k: v.double() for k, v in w1.items()}, "p.", reader_m, shared=kv)[0])
    want0, want1 = torch.cat(want0), torch.cat(want1)
    for cuts, where in CUTS + (([2, 4], "a batch of two, cut"),):
        seqs = [s0, s1] if "batch" in where else [s0]
        got0, got1 = run([a, b], h, seqs, cuts, device, dtype)
        rows = [r for s in seqs for r in s]
        judge(got0, want0, dtype, f"attention: {where}", rows)
        judge(got1, want1, dtype, f"a reader of its keys and values: {where}", rows)


def test_buckets_of_the_distance_table():
    assert [distance_bucket(n, 8, 16.0) for n in (0, 3, 4, 5, 7, 8, 15, 16, 400)] == [0, 3, 4, 4, 5, 6, 7, 7, 7]
    assert [distance_bucket(n, 7, 12.5) for n in (0, 2, 3, 4, 12, 13)] == [0, 2, 3, 3, 6, 6]
    for rows, far in ((8, 16.0), (7, 12.5), (20, 300.0)):
        assert all(distance_bucket(n, rows, far) == pl.bucket(n, rows, far) for n in range(400))


def spike(h, at, axis, size):
    h[at] = 0
    h[at, axis] = size


@pytest.mark.parametrize("gap", ["inside", "outside"])
def test_a_key_at_the_window_edge_of_table_attention(backend, gap):
    """One taps, identity-like projections: the query at i meets one key far stronger than the rest, which sits on the last
    position the window keeps or one beyond it; with a far table row of -3 or +3 nothing else could make up for it."""
    device, dtype = backend
    m = dict(heads=1, kv_heads=1, dim=D, vdim=D, conv=1, scale=1.0, bias_max=9, mask=dict(size=70))
    eye = torch.eye(D).to(torch.bfloat16)
    w = {"q": eye, "k": eye, "v": eye, "q.conv": torch.ones(D, 1).to(torch.bfloat16), "k.conv": torch.ones(D, 1).to(torch.bfloat16),
         "v.conv": torch.ones(D, 1).to(torch.bfloat16), "rel": torch.linspace(-3, 3, 6)[:, None].to(torch.bfloat16),
         "g": torch.zeros(1, D).to(torch.bfloat16), "o": eye}
    part = att_part(m, 6, dtype)
    load(part, w, ATT_NAMES, backend)
    T, i = 150, 140
    j = i - (69 if gap == "inside" else 70)
    h = rand((T, D), 3, 0.2).float()
    spike(h, j, 0, 6.0)                                      # the key (and a value that points along axis 0)
    spike(h, i, 0, 4.0)                                      # the query: score 24 against everything else's 1 or so
    want, _ = pl.conv_attention(h.double(), {"p." + k: v.double() for k, v in w.items()}, "p.", m)
    assert (want[i, 0] > 2.0) == (gap == "inside")           # the plain statement itself tells the two cases apart
    for cuts, where in (([], "whole"), ([64, 128, 139], "portions"), (list(range(100, T)), "decoded")):
        (got,) = run([part], h, [list(range(T))], cuts, device, dtype)
        judge(got, want, dtype, f"key just {gap} the window, {where}", rows=list(range(i - 3, i + 3)))


# ---- the left half of 'parallel': whole-projection q/k norm, slopes, a sink, an element-wise gate --------------------

LEFT = dict(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.4, mask=dict(size=23))
LEFT_NAMES = dict(wq="q", wk="k", wv="v", q_norm="q.norm", k_norm="k.norm", sink="sink", wg="g", wo="o")


def left_part(m, dtype):
    return build_part(MIXERS, PartSpec("attention", dict(dim=D, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                         window=m["mask"]["size"], scale=m["scale"], qk_norm_eps=EPS, qk_norm_whole=True,
                                                         sink=True, distance_bias=dict(kind="slopes", exponent=-8.0), gate="element")),
                      dtype=dtype, position=None)


def left_weights(m, seed):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {"q": rand((H * d, D), seed, 0.3), "k": rand((G * d, D), seed + 1, 0.3), "v": rand((G * dv, D), seed + 2, 0.3),
            "q.norm": rand((H * d,), seed + 3, 0.3, 1.0), "k.norm": rand((G * d,), seed + 4, 0.3, 1.0), "sink": rand((H,), seed + 5, 1.5),
            "g": rand((H * dv, D), seed + 6, 0.3), "o": rand((D, H * dv), seed + 7, 0.3)}


@pytest.mark.parametrize("m", [LEFT, dict(LEFT, heads=1, kv_heads=1, dim=16, vdim=24, mask=dict(size=1)),
                               dict(LEFT, heads=3, kv_heads=3, mask=dict(size=500))], ids=["grouped", "one-head-window-1", "window-beyond"])
def test_sink_attention(backend, m):
    device, dtype = backend
    w = left_weights(m, 40)
    part = left_part(m, dtype)
    load(part, w, LEFT_NAMES, backend)
    h = rand((80, D), 6).float()
    s0, s1 = list(range(0, 75)), list(range(75, 80))
    W = {"p." + k: v.double() for k, v in w.items()}
    want = torch.cat([pl.sink_attention(h[s].double(), W, "p.", m, EPS) for s in (s0, s1)])
    for cuts, where in CUTS + (([2, 4], "a batch of two, cut"),):
        seqs = [s0, s1] if "batch" in where else [s0]
        (got,) = run([part], h, seqs, cuts, device, dtype)
        judge(got, want, dtype, f"sink attention: {where}", [r for s in seqs for r in s])


def test_the_sink_and_the_slopes_show(backend):
    """A large sink takes most of the softmax (leaving it out would multiply the output), and with equal keys the slopes
    alone decide the weights: head 0's slope 2^(-8/H) weighs the near keys, the last head's 2^-8 hardly any."""
    device, dtype = backend
    m = dict(heads=2, kv_heads=1, dim=8, vdim=D, scale=1.0, mask=dict(size=300))
    w = left_weights(m, 50)
    w["k"] = torch.zeros_like(w["k"])                        # every score is 0: only slope * distance and the sink remain
    w["sink"] = torch.tensor([2.0, 4.0]).to(torch.bfloat16)
    w["g"] = torch.zeros_like(w["g"])
    part = left_part(m, dtype)
    load(part, w, LEFT_NAMES, backend)
    h = rand((260, D), 7).float()
    want = pl.sink_attention(h.double(), {"p." + k: v.double() for k, v in w.items()}, "p.", m, EPS)
    for cuts, where in (([], "whole"), ([64, 200], "portions"), (list(range(230, 260)), "decoded")):
        (got,) = run([part], h, [list(range(260))], cuts, device, dtype)
        judge(got, want, dtype, f"sink and slopes: {where}")


@pytest.mark.parametrize("gap", ["inside", "outside"])
def test_a_far_key_at_the_window_edge_of_sink_attention(backend, gap):
    """A key hundreds of positions back, across several pages, on the last position the window keeps or one beyond."""
    device, dtype = backend
    m = dict(heads=1, kv_heads=1, dim=D, vdim=D, scale=1.0, mask=dict(size=260))
    eye = torch.eye(D).to(torch.bfloat16)
    ones = torch.ones(D).to(torch.bfloat16)
    w = {"q": eye, "k": eye, "v": eye, "q.norm": ones, "k.norm": ones, "sink": torch.zeros(1).to(torch.bfloat16),
         "g": torch.zeros(D, D).to(torch.bfloat16), "o": eye}
    part = left_part(m, dtype)
    load(part, w, LEFT_NAMES, backend)
    T, i = 330, 321
    j = i - (259 if gap == "inside" else 260)
    h = rand((T, D), 8, 0.05).float()
    spike(h, j, 1, 20.0)                                     # normed, key j equals the query's own key: q . k = 40 for both,
    spike(h, i, 1, 2.0)                                      # less a slope of 2^-8 * 260; j's value is ten times the query's
    want = pl.sink_attention(h.double(), {"p." + k: v.double() for k, v in w.items()}, "p.", m, EPS)
    assert (want[i, 1] > 2.0) == (gap == "inside")
    for cuts, where in (([], "whole"), ([64, 320], "portions"), (list(range(300, T)), "decoded")):
        (got,) = run([part], h, [list(range(T))], cuts, device, dtype)
        judge(got, want, dtype, f"far key just {gap} the window, {where}", rows=list(range(i - 2, i + 3)))


# ---- the right half of 'parallel': the gated delta rule with one decay per head ---------------------------------------

RIGHT = dict(heads=4, kv_heads=2, dim=8, vdim=12, conv=3)
RIGHT_NAMES = dict(wq="q", wk="k", wv="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", wb="b", a_log="A_log", norm="norm", wa="a",
                   dt_bias="dt_bias", wg="g", wo="o")


@pytest.mark.parametrize("m", [RIGHT, dict(heads=1, kv_heads=1, dim=16, vdim=16, conv=1), dict(heads=2, kv_heads=2, dim=24, vdim=5, conv=5)],
                         ids=["grouped", "one-head-one-tap", "five-taps"])
def test_head_decay_delta_rule(backend, m):
    device, dtype = backend
    H, J, d, dv, t = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
    w = {"q": rand((J * d, D), 1, 0.3), "q.conv": rand((J * d, t), 2, 0.5), "k": rand((J * d, D), 3, 0.3), "k.conv": rand((J * d, t), 4, 0.5),
         "v": rand((H * dv, D), 5, 0.3), "v.conv": rand((H * dv, t), 6, 0.5), "b": rand((H, D), 7, 0.3), "A_log": rand((H,), 8, 0.5, -1.0),
         "norm": rand((dv,), 9, 0.2, 1.0), "a": rand((H, D), 10, 0.3), "dt_bias": rand((H,), 11, 0.5), "g": rand((H * dv, D), 12, 0.3),
         "o": rand((D, H * dv), 13, 0.3)}
    part = build_part(MIXERS, PartSpec("delta_rule", dict(dim=D, n_head=H, n_qk=J, head_dim=d, v_head_dim=dv, taps=t, decay_rank=0, gate_rank=0,
                                                          eps=EPS, head_decay=True, gate_act="silu")), dtype=dtype, position=None)
    load(part, w, RIGHT_NAMES, backend)
    h = rand((80, D), 9).float()
    s0, s1 = list(range(0, 75)), list(range(75, 80))
    W = {"p." + k: v.double() for k, v in w.items()}
    want = torch.cat([pl.head_delta_rule(h[s].double(), W, "p.", m, EPS) for s in (s0, s1)])
    for cuts, where in CUTS + (([2, 4], "a batch of two, cut"),):
        seqs = [s0, s1] if "batch" in where else [s0]
        (got,) = run([part], h, seqs, cuts, device, dtype)
        judge(got, want, dtype, f"delta rule: {where}", [r for s in seqs for r in s])


# ---- the two halves added with their factors ----------------------------------------------------------------------------

def test_sum_of_two_mixers(backend):
    device, dtype = backend
    le, ri = LEFT, RIGHT
    wl = left_weights(le, 70)
    H, J, d, dv, t = ri["heads"], ri["kv_heads"], ri["dim"], ri["vdim"], ri["conv"]
    wr = {"q": rand((J * d, D), 1, 0.3), "q.conv": rand((J * d, t), 2, 0.5), "k": rand((J * d, D), 3, 0.3), "k.conv": rand((J * d, t), 4, 0.5),
          "v": rand((H * dv, D), 5, 0.3), "v.conv": rand((H * dv, t), 6, 0.5), "b": rand((H, D), 7, 0.3), "A_log": rand((H,), 8, 0.5, -1.0),
          "norm": rand((dv,), 9, 0.2, 1.0), "a": rand((H, D), 10, 0.3), "dt_bias": rand((H,), 11, 0.5), "g": rand((H * dv, D), 12, 0.3),
          "o": rand((D, H * dv), 13, 0.3)}
    left = left_part(le, dtype)
    spec = PartSpec("sum", dict(dim=D, factors=dict(left=0.7, right=1.4), mixers=dict(
        left=PartSpec("attention", dict(dim=D, n_head=le["heads"], n_kv=le["kv_heads"], head_dim=le["dim"], v_head_dim=le["vdim"],
                                        window=le["mask"]["size"], scale=le["scale"], qk_norm_eps=EPS, qk_norm_whole=True, sink=True,
                                        distance_bias=dict(kind="slopes", exponent=-8.0), gate="element")),
        right=PartSpec("delta_rule", dict(dim=D, n_head=H, n_qk=J, head_dim=d, v_head_dim=dv, taps=t, decay_rank=0, gate_rank=0, eps=EPS,
                                          head_decay=True, gate_act="silu")))))
    part = build_part(MIXERS, spec, dtype=dtype, position=None)
    assert left.cache_needs().kv == part.cache_needs().kv and part.cache_needs().state is not None
    tensors = {"left." + k: wl[v] for k, v in LEFT_NAMES.items()}
    tensors.update({"right." + k: wr[v] for k, v in RIGHT_NAMES.items()})
    part.load({k: v.to(dtype if v.dim() > 1 and "conv" not in k else torch.float32).to(device) for k, v in tensors.items()})
    h = rand((75, D), 10).float()
    want = (0.7 * pl.sink_attention(h.double(), {"p." + k: v.double() for k, v in wl.items()}, "p.", le, EPS)
            + 1.4 * pl.head_delta_rule(h.double(), {"p." + k: v.double() for k, v in wr.items()}, "p.", ri, EPS))
    for cuts, where in CUTS:
        (got,) = run([part], h, [list(range(75))], cuts, device, dtype)
        judge(got, want, dtype, f"the sum of two mixers: {where}")


# ---- the mixture of experts ------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("E,top,F,T", [(5, 2, 24, 9), (40, 1, 8, 3), (3, 3, 16, 150), (9, 4, 12, 700)],
                         ids=["2-of-5", "1-of-40", "3-of-3-many-tokens", "4-of-9-tiles"])
def test_mixture_of_experts(backend, E, top, F, T):
    device, dtype = backend
    mlp = dict(expert=dict(ff=F, limit=0.8), router=dict(experts=E, top=top, scale=1.7))
    g = torch.Generator().manual_seed(E)
    w = {"router": rand((E, D), 1, 0.4), "correction": (torch.randperm(E, generator=g).float() * 0.3 - 0.3).to(torch.bfloat16)}
    for e in range(E):
        w.update({f"e{e}.gate": rand((F, D), 10 + 3 * e, 0.3), f"e{e}.up": rand((F, D), 11 + 3 * e, 0.3), f"e{e}.down": rand((D, F), 12 + 3 * e, 0.3)})
    part = build_part(FEED_FORWARDS, PartSpec("moe", dict(dim=D, hidden=F, n_experts=E, top=top, router_scale=1.7, limit=0.8, alpha=1.702,
                                                          shift=1.0, correction=True)), dtype=dtype)
    stack = lambda name: torch.stack([w[f"e{e}.{name}"] for e in range(E)]).to(dtype).to(device)
    part.load({"router": w["router"].to(dtype).to(device), "correction": w["correction"].float().to(device),
               "gate": stack("gate"), "up": stack("up"), "down": stack("down")})
    h = rand((T, D), 2).float()                               # bfloat16 values: the router sees the same input in every back end
    want = pl.mixture(h.double(), {"p." + k: v.double() for k, v in w.items()}, "p.", mlp)
    x = torch.zeros(T, D, dtype=torch.float32, device=device)
    part.forward(h.to(dtype).to(device), residual=x)
    judge(x.cpu(), want, dtype, f"{top} of {E} experts, {T} tokens")
    assert float(want.abs().max()) > 0.1                      # the clamps bite: the limit is below the products' spread


def test_router_weights_leave_the_correction_out(plain_kernels):
    z = torch.tensor([[0.0, 2.0, -1.0, 0.5]])
    corr = torch.tensor([3.0, 0.0, 0.0, -5.0])
    idx, wt = torch.empty(1, 2, dtype=torch.int32), torch.empty(1, 2)
    ops.moe_route(z, corr, 2, 2.0, idx, wt)
    s = torch.sigmoid(z[0])
    assert idx.tolist() == [[0, 1]]                           # the correction lifts expert 0 above expert 1 and drops expert 3
    torch.testing.assert_close(wt[0], torch.stack([s[0], s[1]]) / (s[0] + s[1]) * 2.0)


# ---- the learned position embedding -----------------------------------------------------------------------------------------

def test_learned_positions(backend):
    device, dtype = backend
    table, pos = rand((30, D), 1).to(dtype).to(device), rand((50, D), 2).to(dtype).to(device)
    part = build_part(EMBEDDINGS, PartSpec("learned_position", dict(dim=D, max_positions=50)), dtype=dtype)
    part.load({"table": pos})
    cache = Cache({0: part.cache_needs()}, dtype, device, max_tokens=128, max_seqs=2)
    slots = cache.begin(2)
    got = {s: [] for s in slots}
    toks = {slots[0]: [3, 3, 7, 29, 0, 3], slots[1]: [3, 5]}
    for lo, hi in ((0, 1), (1, 4), (4, 6)):
        live = [s for s in slots if toks[s][lo:hi]]
        q = [len(toks[s][lo:hi]) for s in live]
        batch = batch_of(cache, live, q, device)
        out = torch.empty(sum(q), D, dtype=torch.float32, device=device)
        part.forward(torch.tensor([t for s in live for t in toks[s][lo:hi]], dtype=torch.int32).to(device), table, out, batch, cache.view(0), 1.0)
        ops.advance_lengths(batch)
        cache.note_advance(live, q)
        at = 0
        for s, n in zip(live, q):
            got[s].append(out[at:at + n].cpu())
            at += n
    for s in slots:
        want = table.float().cpu()[toks[s]] + pos.float().cpu()[:len(toks[s])]
        torch.testing.assert_close(torch.cat(got[s]), want, rtol=1e-6, atol=1e-6)
