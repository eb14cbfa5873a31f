"""Random Lomusun configurations (widths with and without whole 16-byte rows, head sizes on and off the tensor-core kernels,
1 to 64 experts, windows of 1 to 1,000 positions, tables of 2 to 64 rows, readers of other layers' keys, layers without a
feed-forward) through the engine against the plain statement: a prompt beyond most windows, decode steps, another portion.
32-bit must agree to rounding at every position; bfloat16 in the median row and in all but a few rows (random weights leave
the router close calls, and a bfloat16 input may tip one, which moves that token and the few that attend to it)."""
import json
import os
import random

import pytest
import torch
from safetensors.torch import load_file

import gpt_fast_b200 as gf
from gpt_fast_b200.engine.step import Stepper
import plain_lomusun as pl

pytestmark = pytest.mark.gpu


def moe(r):
    E = r.choice([1, 2, 3, 8, 17, 64]); top = r.randint(1, min(E, 6))
    return {"kind": "moe", "expert": {"ff": r.choice([8, 20, 24, 33, 64, 136]), "limit": r.choice([0.5, 2.0, 7.0])},
            "router": {"experts": E, "top": top, "scale": r.choice([1.0, 2.5])}}

def heads(r):
    G = r.choice([1, 2, 3]); rep = r.choice([1, 2, 4]) if G < 3 else r.choice([1, 2])
    return G * rep, G

def config(seed):
    r = random.Random(seed)
    W = r.choice([36, 100, 64, 192, 256, 72])
    layers, owners = [], []
    for i in range(r.randint(2, 6)):
        mlp = None if r.random() < 0.15 else moe(r)
        if r.random() < 0.6:
            H, G = heads(r)
            m = {"heads": H, "kv_heads": G, "dim": r.choice([8, 24, 64, 80, 128]), "vdim": r.choice([8, 40, 64, 128]), "conv": r.randint(1, 5),
                 "mask": {"size": r.choice([1, 2, 7, 64, 65, 130, 300, 1000])}, "scale": r.choice([0.1, 0.2]), "bias_rows": r.choice([2, 3, 8, 31, 64])}
            m["bias_max"] = m["bias_rows"] // 2 + r.choice([1, 2.5, 40, 200])
            if owners and r.random() < 0.4:
                j = r.choice(owners)
                src = layers[j]["mixer"]
                m.update(kv_from=j, kv_heads=src["kv_heads"], dim=src["dim"], vdim=src["vdim"], heads=src["kv_heads"] * r.choice([1, 2, 4]))
            else:
                owners.append(i)
            layers.append({"type": "attention", "mixer": m, "mlp": mlp})
        else:
            H, G = heads(r); H2, G2 = heads(r)
            layers.append({"type": "parallel", "mlp": mlp, "mixer": {
                "left": {"heads": H, "kv_heads": G, "dim": r.choice([8, 16, 64, 128]), "vdim": r.choice([8, 24, 64, 128]),
                         "mask": {"size": r.choice([1, 5, 64, 96, 129, 400])}, "scale": r.choice([0.125, 0.3])},
                "right": {"heads": H2, "kv_heads": G2, "dim": r.choice([8, 16, 32, 64]), "vdim": r.choice([6, 16, 64, 128]), "conv": r.randint(1, 4)},
                "left_scale": r.choice([1.0, 1.2, 0.5]), "right_scale": r.choice([1.0, 1.1])}})
    return {"architecture": "Lomusun", "vocab": r.choice([97, 512, 1000]), "width": W, "max_positions": 600, "norm": {"eps": r.choice([1e-5, 1e-6])},
            "layers": layers}


@pytest.mark.parametrize("seed", [0, 3, 4, 9, 11, 25, 31, 44])
def test_random_configurations(tmp_path, seed):
    cfg = config(seed)
    folder = str(tmp_path / "m")
    gf.write_model_folder(folder, cfg, seed=seed, std=0.1, jitter=0.2)
    weights = load_file(os.path.join(folder, "model.safetensors"))
    with open(os.path.join(folder, "config.json")) as f:
        stored = json.load(f)
    toks = torch.randint(0, cfg["vocab"], (470,), generator=torch.Generator().manual_seed(seed)).tolist()
    want = pl.forward(stored, weights, toks).float()
    scale = float(want.pow(2).mean().sqrt())
    for dtype in ("float32", "bfloat16"):
        model = gf.load(folder, dtype=dtype, device="cuda:0")
        cache = model.new_cache(max_tokens=1024, max_seqs=2)
        st = Stepper(model, cache)
        (slot,) = cache.begin(1)
        outs = [st.step([slot], [toks[:401]], "all")] + [st.step([slot], [[t]], "all") for t in toks[401:440]] + [st.step([slot], [toks[440:]], "all")]
        st.check()
        err = (torch.cat(outs).float().cpu() - want).pow(2).mean(-1).sqrt() / scale
        if dtype == "float32":
            assert float(err.max()) < 2e-3, f"seed {seed}: 32-bit differs by {float(err.max()):.5f} of the logits' scale at row {int(err.argmax())}"
        else:
            assert float(err.median()) < 0.02, f"seed {seed}: bfloat16 median row error {float(err.median()):.4f}"
            assert int((err > 0.1).sum()) <= 30, f"seed {seed}: {int((err > 0.1).sum())} of {err.numel()} rows off by a tenth of the scale"
