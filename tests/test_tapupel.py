"""The Tapupel decoder through the whole engine, against the plain statement in `plain_tapupel.py`: two small
configurations that differ in every size and option (grouped and ungrouped heads, one head, rotation of a part of the head
and of all of it, with and without rescaled frequencies, windows of one position and longer than any prompt, no window at
all, 0 to 5 kept first positions, with and without a score cap, recurrences of 1 to 3 blocks behind convolutions of 1 to 4
taps and of another width than the model, value heads larger and smaller than two keys, readers of another layer's keys,
1 of 40 and 3 of 3 experts, with and without a shared expert, dense and absent feed-forwards, every order of the kinds),
random weights.

Every test runs three ways: the host logic on the CPU against the plain statement of the kernels, and the kernels
themselves in 32-bit and in bfloat16 on a GPU."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch
from safetensors.torch import load_file

import gpt_fast_b200 as gf
from gpt_fast_b200 import ops
from gpt_fast_b200.engine.step import Stepper
import plain_tapupel as pt
import plain_ops
import traces

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
NAMES = ["tapupel-tiny-a", "tapupel-tiny-b"]
BACKENDS = [
    pytest.param(("cpu", "float32"), id="cpu-standin-f32"),
    pytest.param(("cuda", "float32"), id="cuda-f32", marks=pytest.mark.gpu),
    pytest.param(("cuda", "bfloat16"), id="cuda-bf16", marks=pytest.mark.gpu),
]


@pytest.fixture(params=BACKENDS)
def backend(request):
    device, dtype = request.param
    prev = ops.use_kernels(plain_ops.PlainOps()) if device == "cpu" else None
    yield device, dtype
    if device == "cpu":
        ops.use_kernels(prev)


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, name in enumerate(NAMES):
        d = str(tmp_path_factory.mktemp(name.replace("-", "_")))
        gf.write_model_folder(d, name, seed=83 + i, std=0.11, jitter=0.2, vector_dtype="float32" if i else "bfloat16")
        out[name] = d
    return out


_plain_cache = {}
CLOSE_CALL = 0.08          # a router margin, in units of the spread of a token's logits, that bfloat16 inputs may tip (their
                           # noise on these models' router logits was seen at 0.01 to 0.03 of the spread)


def plain(folder, tokens, with_first_close_call=False):
    key = (folder, tuple(tokens))
    if key not in _plain_cache:
        with open(os.path.join(folder, "config.json")) as f:
            cfg = json.load(f)
        margins = []
        logits = pt.forward(cfg, load_file(os.path.join(folder, "model.safetensors")), tokens, margins=margins).float()
        close = torch.stack(margins).min(0).values < CLOSE_CALL if margins else torch.zeros(len(tokens), dtype=torch.bool)
        _plain_cache[key] = (logits, int(close.nonzero()[0]) if close.any() else len(tokens))
    return _plain_cache[key] if with_first_close_call else _plain_cache[key][0]


def judge(got, folder, tokens, rows, dtype, where):
    """32-bit: equal to rounding.  bfloat16: up to the sequence's first token at which a router's choice is a close call, every
    row within a tenth of the logits' own scale and all together within a few per cent of it.  A bfloat16 input may tip a
    close call, which moves that token's logits by a fraction of their scale, and the recurrent and attention layers carry
    it on to later tokens (every sublayer's output is normed to unit size, so another expert is a change of the stream's own
    order); from there on half of the rows must still be within 0.3 of the scale (a wrong key, page or state moves the rows by
    about the scale).  The 32-bit runs are the sharp ones."""
    want, first_close = plain(folder, tokens, True)
    positions = torch.arange(len(tokens))[rows]
    want = want[rows]
    got = got.float().cpu()
    if dtype == "float32":
        torch.testing.assert_close(got, want, rtol=3e-4, atol=3e-4, msg=lambda m: f"{where}\n{m}")
    else:
        scale = float(want.pow(2).mean().sqrt())
        per_row = (got - want).pow(2).mean(-1).sqrt() / scale
        sure = per_row[positions < first_close]
        if sure.numel():
            assert float(sure.pow(2).mean().sqrt()) <= 0.06, f"{where}: rms error {float(sure.pow(2).mean().sqrt()):.4f} of the scale"
            assert float(sure.max()) <= 0.15, f"{where}: a row is off by {float(sure.max()):.3f} of the scale ahead of any close call"
        assert float(per_row.median()) <= 0.3, f"{where}: half of the rows are off by {float(per_row.median()):.3f} of the scale or more"


def tokens_of(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def stepped(stepper, slot, toks, cuts):
    outs, at = [], 0
    for c in list(cuts) + [len(toks)]:
        if c > at:
            outs.append(stepper.step([slot], [toks[at:c]], "all"))
            at = c
    stepper.check()
    return torch.cat(outs)


def make(folder, backend, max_tokens=2048, max_seqs=8):
    device, dtype = backend
    model = gf.load(folder, dtype=dtype, device=device)
    cache = model.new_cache(max_tokens=max_tokens, max_seqs=max_seqs)
    return model, cache, Stepper(model, cache)


# ---- whole prompts, and the first tokens of a sequence ------------------------------------------------

@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(folders, backend, name):
    model, cache, st = make(folders[name], backend)
    for n in (1, 2, 3, 6, 64, 71, 150):
        toks = tokens_of(model.vocab_size, n, seed=n)
        (slot,) = cache.begin(1)
        got = st.step([slot], [toks], "all")
        st.check()
        cache.end([slot])
        judge(got, folders[name], toks, slice(None), backend[1], f"{name}: prompt of {n}")


@pytest.mark.parametrize("name", NAMES)
def test_the_stream_after_every_layer(folders, backend, name):
    """The residual stream behind each layer, not only the logits: a layer that is wrong by little does not hide
    behind the layers after it."""
    model, cache, st = make(folders[name], backend)
    toks = tokens_of(model.vocab_size, 75, seed=8)
    kept = []
    model.after_layer = lambda x: kept.append(x.tensor().float().cpu().clone())
    (slot,) = cache.begin(1)
    st.step([slot], [toks], "all")
    cache.end([slot])
    model.after_layer = None
    with open(os.path.join(folders[name], "config.json")) as f:
        cfg = json.load(f)
    want = []
    pt.forward(cfg, load_file(os.path.join(folders[name], "model.safetensors")), toks, want)
    assert len(kept) == len(want)
    sure = len(toks) if backend[1] == "float32" else max(1, plain(folders[name], toks, True)[1])    # bfloat16: up to the first close call
    for i, got in enumerate(kept):
        tol = 3e-4 if backend[1] == "float32" else 0.05 * float(want[i].float().pow(2).mean().sqrt())
        assert float((got[:sure] - want[i][:sure].float()).pow(2).mean().sqrt()) <= tol, f"the stream behind layer {i}"


def test_one_token_repeated(folders, backend):
    """Positions count from 0 in every sequence and go on across steps: one token repeated."""
    name = NAMES[0]
    model, cache, st = make(folders[name], backend)
    for toks in ([7, 7, 7, 7, 7], [9], [9, 9]):
        (slot,) = cache.begin(1)
        got = stepped(st, slot, toks, range(1, len(toks)))
        cache.end([slot])
        judge(got, folders[name], toks, slice(None), backend[1], f"{name}: {toks}")


# ---- prefill against token-by-token decoding, portions down to two tokens, long decoding ----------------

@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("cuts", [
    pytest.param(lambda n: range(1, n), id="token-by-token"),
    pytest.param(lambda n: [20] + list(range(21, n)), id="prefill-then-long-decode"),
    pytest.param(lambda n: [2, 4, 5, 9, 10, 36, 38, 64, 66, 69, 70, 72, 128, 130, 139, 141], id="portions"),
    pytest.param(lambda n: [63, 65, 140], id="page-edges"),
])
def test_cuts_agree_with_the_whole(folders, backend, name, cuts):
    model, cache, st = make(folders[name], backend)
    toks = tokens_of(model.vocab_size, 143, seed=5)
    (slot,) = cache.begin(1)
    got = stepped(st, slot, toks, cuts(len(toks)))
    cache.end([slot])
    judge(got, folders[name], toks, slice(None), backend[1], f"{name}: cut prompt")
    if backend[1] == "float32":
        (slot,) = cache.begin(1)
        whole = st.step([slot], [toks], "all")
        cache.end([slot])
        torch.testing.assert_close(got, whole, rtol=1e-4, atol=1e-4)


def test_long_decoding(folders, backend):
    """Windows pass over decoded tokens several times and the recurrent state carries over hundreds of steps."""
    name = NAMES[0]
    model, cache, st = make(folders[name], backend)
    toks = tokens_of(model.vocab_size, 310, seed=9)
    (slot,) = cache.begin(1)
    got = stepped(st, slot, toks, [5] + list(range(6, len(toks))))
    cache.end([slot])
    judge(got[-40:], folders[name], toks, slice(len(toks) - 40, len(toks)), backend[1], f"{name}: the last of 305 decode steps")


# ---- batches of unequal requests against each alone; slots, pages and state used again ------------------

@pytest.mark.parametrize("name", NAMES)
def test_batches_and_reuse(folders, backend, name):
    model, cache, st = make(folders[name], backend, max_tokens=1024, max_seqs=4)
    V = model.vocab_size
    for turn in range(3):                                  # the later rounds get slots, pages and state that were used before
        lens = [[70, 3, 131], [1, 66, 9, 20], [129, 2]][turn]
        reqs = [tokens_of(V, n + 6, seed=100 * turn + n) for n in lens]
        slots = cache.begin(len(reqs))
        rows = {i: [] for i in range(len(reqs))}
        out = st.step(slots, [r[:n] for r, n in zip(reqs, lens)], "all")       # packed prefill
        at = 0
        for i, n in enumerate(lens):
            rows[i].append(out[at:at + n])
            at += n
        live = list(range(len(reqs)))
        for k in range(6):                                   # decode together; the shorter ones (by index) leave early
            live = [i for i in live if not (k >= 2 + 2 * i and i < len(reqs) - 1)]
            out = st.step([slots[i] for i in live], [[reqs[i][lens[i] + k]] for i in live], "all")
            for j, i in enumerate(live):
                rows[i].append(out[j:j + 1])
        st.check()
        cache.end(slots)
        for i, r in enumerate(reqs):
            got = torch.cat(rows[i])
            judge(got, folders[name], r, slice(0, got.shape[0]), backend[1], f"{name}: pass {turn}, request {i}")
    assert cache.slots.n_free == cache.n_slots and all(g.pages.n_free == cache.n_pages for g in cache.kv_groups)


# ---- greedy generation through the library's entry point and scheduler -----------------------------------

@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation(folders, backend, name):
    device, dtype = backend
    model = gf.load(folders[name], dtype=dtype, device=device)
    prompts = [tokens_of(model.vocab_size, n, seed=7 * n) for n in (5, 1, 68, 12)]
    seqs, stats = gf.generate(model, prompts, 9, temperature=0.0, batch_size=3)
    assert stats.batches == 2 and [len(s) for s in seqs] == [len(p) + 9 for p in prompts]
    for p, s in zip(prompts, seqs):
        assert s[:len(p)] == p
        logits = plain(folders[name], s[:-1])
        for j in range(len(p) - 1, len(s) - 1):
            margin = 1e-3 if dtype == "float32" else 0.1 * float(logits[j].pow(2).mean().sqrt()) + 0.05
            assert logits[j, s[j + 1]] >= logits[j].max() - margin, f"{name}: token {j + 1} is not the plain argmax"


# ---- what the model asks of the cache -----------------------------------------------------------------------

def test_cache_entries(folders, backend):
    model, cache, st = make(folders[NAMES[0]], backend)
    needs = model.cache_needs()
    # layer 0: keys, and the keys as projected in the place of values, both of the key size; a window
    assert needs[0].kv.n_kv == 2 and needs[0].kv.head_dim == 12 and needs[0].kv.v_head_dim is None and needs[0].kv.window == 37
    assert needs[1].kv is None and needs[1].state.shape == (48 * 4,)                  # S and three carried rows of inputs
    assert needs[2].kv.n_kv == 1 and needs[2].kv.head_dim == 20 and needs[2].kv.v_head_dim == 14     # two keys side by side
    assert needs[3].kv is None and needs[3].state is None                             # a reader keeps nothing
    assert needs[4].kv is None and needs[4].state.shape == (32,)                      # one tap: only S
    sched = model.spec.schedule
    assert [e.kv_from for e in sched] == [None, None, None, 2, None, None] and all(e.owns_cache for e in sched)


# ---- configuration and weights ------------------------------------------------------------------------------

def test_config_errors_name_the_key():
    cfg = gf.config_from_name("tapupel-tiny-a")
    for path, value, word in [(("layers", 0, "type"), "mamba2", "type"), (("layers", 0, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 3, "mixer", "kv_from"), 1, "kv_from"), (("layers", 3, "mixer", "kv_from"), 3, "kv_from"),
                              (("layers", 3, "mixer", "dim"), 16, "dim"), (("layers", 0, "mlp", "kind"), "sparse", "mlp"),
                              (("layers", 0, "mlp", "router", "top"), 6, "experts"), (("layers", 0, "mixer", "mask"), 5, "mask"),
                              (("layers", 1, "mixer", "conv"), 0, "conv"), (("layers", 1, "mixer", "blocks"), 5, "blocks"),
                              (("norm",), 1e-5, "norm"), (("layers", 0, "mixer", "rot", "dims"), 14, "dims"),
                              (("layers", 0, "mixer", "vdim"), 10, "vdim"), (("layers", 0, "mixer", "softcap"), 0.0, "softcap"),
                              (("embedding",), 3, "embedding")]:
        bad = json.loads(json.dumps(cfg))
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(gf.ConfigError, match=word):
            gf.load(bad, device="cpu", random_weights=True)


def test_weights_roundtrip_and_one_error(folders, tmp_path):
    from safetensors.torch import save_file
    name = NAMES[0]
    model = gf.load(folders[name], dtype="bfloat16", device="cpu")
    gf.save_folder(model, str(tmp_path / "again"))
    a, b = load_file(os.path.join(folders[name], "model.safetensors")), load_file(str(tmp_path / "again" / "model.safetensors"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert "l3.mix.k" not in a and "l3.mix.k.norm" not in a and "l3.mix.q.norm" in a and "l0.mix.v" not in a
    broken = dict(a)
    del broken["l1.mix.lam"]
    broken["l1.mix.ra"] = torch.zeros(3, 16, 15)
    broken["l3.mix.k"] = torch.zeros(1)
    os.makedirs(tmp_path / "broken")
    save_file(broken, str(tmp_path / "broken" / "model.safetensors"))
    with open(tmp_path / "broken" / "config.json", "w") as f:
        json.dump(gf.config_from_name(name), f)
    with pytest.raises(gf.WeightError) as e:
        gf.load(str(tmp_path / "broken"), device="cpu")
    assert e.value.missing == ["l1.mix.lam"] and e.value.unexpected == ["l3.mix.k"] and e.value.wrong_shape[0][0] == "l1.mix.ra"


# ---- the trace program and the command line as a user runs them ----------------------------------------------

@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_run(folders, tmp_path, dtype):
    name = NAMES[1]
    folder = folders[name]
    V = gf.config_from_name(name)["vocab"]
    reqs = traces.make_requests(V, [40, 3, 77, 65], seed=3)
    for cut, steps in (("whole", traces.whole(reqs)), ("stepped", traces.stepped(reqs)), ("batched", traces.batched(reqs, 3))):
        out_dir = str(tmp_path / cut)
        cmd = [sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out_dir,
               "--max-tokens", str(traces.peak_tokens(steps))]
        proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
        try:
            for s in steps:
                proc.stdin.write(json.dumps(s) + "\n")
                proc.stdin.flush()
                assert proc.stdout.readline().strip() == f"done {s['step']}"
            proc.stdin.close()
            assert proc.wait(timeout=120) == 0
        finally:
            if proc.poll() is None:
                proc.kill()
        outputs = {}
        for s in steps:
            wanted = sum(len(e["want"]) for e in s["entries"])
            if wanted:
                outputs[s["step"]] = np.fromfile(os.path.join(out_dir, f"{s['step']}.f32"), dtype="<f4").reshape(wanted, V)
        by_request = {}
        for (rid, j), row in traces.collect(steps, outputs, V).items():
            by_request.setdefault(rid, []).append((j, row))
        for rid, rows in by_request.items():
            rows.sort(key=lambda x: x[0])
            got = torch.from_numpy(np.stack([r for _, r in rows]))
            judge(got, folder, reqs[rid], [j for j, _ in rows], dtype, f"{cut}: {rid}")


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_cli_greedy(folders, tmp_path, dtype):
    from test_cli_gpu import read_lines, run_cli
    name = NAMES[1]
    out = tmp_path / "tokens.jsonl"
    r = run_cli("--checkpoint_path", folders[name], "--prompt", "4,13", "--max_new_tokens", "7", "--temperature", "0",
                "--dtype", dtype, "--output", str(out))
    assert r.returncode == 0, r.stderr[-2000:]
    rows = read_lines(out)
    assert [len(x["prompt"]) for x in rows] == [4, 13]
    for x in rows:
        assert len(x["tokens"]) == 7


# ---- head sizes and widths of whole 16-byte rows, at which the tensor-core products run, through the whole engine ---------

def _moe(E, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": E, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


WIDE = {
    "architecture": "Tapupel", "vocab": 211, "width": 192, "embedding": {"scale": 1.3}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mlp": _moe(6, 2, 48, 64),
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.2, "softcap": 8.0, "mask": {"size": 150, "keep_first": 9},
                   "rot": {"dims": 32, "base": 10000.0, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}}},
        {"type": "rglru", "mlp": {"kind": "dense", "ff": 256}, "mixer": {"width": 256, "blocks": 4, "conv": 4}},
        {"type": "attention_2", "mlp": _moe(12, 5, 40),
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 128, "scale": 0.15, "diff": 0.5, "rot": {"dims": 64, "base": 5000.0}}},
        {"type": "attention", "mlp": None,
         "mixer": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.1, "softcap": 20.0, "mask": {"size": 70, "keep_first": 70},
                   "rot": {"dims": 128, "base": 100000.0}}},
        {"type": "attention_2", "mlp": _moe(3, 1, 64, 32),
         "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 128, "scale": 0.2, "diff": 0.2, "rot": {"dims": 64, "base": 5000.0}, "kv_from": 2}},
    ]}


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_wide_sizes_through_the_engine(tmp_path, dtype):
    """Heads of 64 and 128 and a width of whole 16-byte rows: in bfloat16 the tensor-core products (the grouped expert products
    among them) and the fast attention kernels run, in prompts longer than every window, in portions, in a batch of unequal
    requests and in decode steps; 32-bit runs the same model on CUDA cores."""
    folder = str(tmp_path / "wide")
    gf.write_model_folder(folder, WIDE, seed=77, std=0.08, jitter=0.2)
    model, cache, st = make(folder, ("cuda", dtype))
    toks = tokens_of(WIDE["vocab"], 520, seed=8)
    (slot,) = cache.begin(1)
    whole = st.step([slot], [toks], "all")
    st.check()
    cache.end([slot])
    judge(whole, folder, toks, slice(None), dtype, "a prompt longer than every window")
    (slot,) = cache.begin(1)
    cut = stepped(st, slot, toks, (130, 132, 389, 390, 391, 392, 393, 394, 395, 396, 397, 398, 399, 400))
    cache.end([slot])
    judge(cut, folder, toks, slice(None), dtype, "portions and decode steps")
    others = [tokens_of(WIDE["vocab"], n, seed=n) for n in (77, 9)]
    slots = cache.begin(3)
    got = st.step(slots, [toks[:300], others[0][:71], others[1][:3]], "all")
    steps = [st.step(slots, [[toks[300 + i]], [others[0][71 + i]], [others[1][3 + i]]], "all") for i in range(6)]   # decoded together
    st.check()
    cache.end(slots)
    judge(got[:300], folder, toks, slice(0, 300), dtype, "the long request of a batch")
    judge(got[300:371], folder, others[0], slice(0, 71), dtype, "the second request of a batch")
    decoded = torch.stack(steps)                                 # [step, request, vocab]
    judge(decoded[:, 0], folder, toks, slice(300, 306), dtype, "the long request decoded in a batch")
    judge(decoded[:, 1], folder, others[0], slice(71, 77), dtype, "the second request decoded in a batch")
    judge(decoded[:, 2], folder, others[1], slice(3, 9), dtype, "the short request decoded in a batch")
