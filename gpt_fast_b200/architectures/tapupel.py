"""The Tapupel decoder as data: which parts each layer has and which checkpoint tensors fill which parameter.

The design: a scaled token embedding; layers in an order that config.json lists, each a block whose sublayers READ THE
STREAM ITSELF and whose outputs are normed before they are added, x += n1(mixer(x)), x += n2(ff(x)), with root-mean-square
norms whose stored weight lies around zero (the factor is 1 + w); a final norm of the same kind and an output matrix of
its own.  Three kinds of mixer:

    'attention'    grouped-query softmax attention whose values are its keys as projected; q and k are rotated on their
                   leading dimensions (half-split pairs, frequencies rescaled by wavelength) and then divided by their root
                   mean square per head; the scaled score is squashed by a soft cap; a sliding window that also keeps the
                   sequence's first positions visible
    'rglru'        a gated linear recurrence per channel behind a short convolution, times a GELU gate branch
    'attention_2'  differential attention: two softmax maps per head over one set of values, subtracted, normed per head;
                   a layer with 'kv_from' has queries only and reads the keys and values that another such layer cached

The feed-forward is a SwiGLU ('dense'), a mixture of SwiGLU experts chosen by the largest router logits and weighted by
the softmax over the chosen ones, with an optional shared expert behind a sigmoid gate per token ('moe'), or absent.

config.json keys: architecture, vocab, width, embedding.scale, norm.eps, layers [{type, mixer {...}, mlp {kind, ...} | null}].
Tensor names: embed, head, final.norm, l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.{gate, up, down} or
l<i>.mlp.{router, e<j>.{gate, up, down}, shared.{gate, up, down, sg}}.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch

from ..config.args import ConfigError
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..weights.plan import Recipe, Source, WeightPlan
from .lasezen import _int, _num

KINDS = ("attention", "rglru", "attention_2")
DECAY_SCALE = 8.0                    # a = exp(-8 r softplus(lam)) in the recurrence


@dataclass(frozen=True)
class MlpArgs:
    kind: str                        # 'dense' or 'moe'
    ff: int                          # hidden size (of one expert)
    experts: int = 0
    top: int = 0
    shared_ff: int = 0               # 0: no shared expert


@dataclass(frozen=True)
class LayerArgs:
    kind: str
    mixer: Dict[str, Any]            # the layer's sizes and constants, checked
    mlp: Optional[MlpArgs] = None    # None: the layer has no feed-forward


@dataclass(frozen=True)
class TapupelArgs:
    vocab: int
    width: int
    embed_scale: float
    norm_eps: float
    layers: Tuple[LayerArgs, ...]
    source: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def to_json(self) -> Dict[str, Any]:
        return dict(self.source)


def _obj(d: Any, key: str, where: str) -> Dict[str, Any]:
    v = d.get(key) if isinstance(d, dict) else None
    if not isinstance(v, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object")
    return v


def _rot(m: Dict[str, Any], where: str, dim: int) -> Dict[str, Any]:
    rot = _obj(m, "rot", where)
    w = where + "rot."
    out = dict(dims=_int(rot, "dims", w), base=_num(rot, "base", w), scaling=None)
    if out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"config.json: {w}dims = {out['dims']} must be even and at most the head size {dim}")
    if rot.get("scaling") is not None:
        sc = _obj(rot, "scaling", w)
        out["scaling"] = {k: _num(sc, k, w + "scaling.") for k in ("factor", "low", "high", "original")}
        if out["scaling"]["high"] == out["scaling"]["low"]:
            raise ConfigError(f"config.json: {w}scaling.high must differ from scaling.low")
    return out


def _heads(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    out = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim")}
    out["vdim"] = out["dim"] if m.get("vdim") is None else _int(m, "vdim", where)      # not given: as wide as the keys
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}{out['heads']} heads do not divide into {out['kv_heads']} kv_heads")
    out["scale"] = _num(m, "scale", where)
    return out


def _mixer(kind: Any, m: Any, where: str) -> Dict[str, Any]:
    if kind not in KINDS:
        raise ConfigError(f"config.json: {where}'type' is {kind!r}; this design has {', '.join(KINDS)}")
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where}'mixer' must be an object")
    w = where + "mixer."
    if kind == "rglru":
        out = dict(width=_int(m, "width", w), blocks=_int(m, "blocks", w), conv=_int(m, "conv", w))
        if out["width"] % out["blocks"]:
            raise ConfigError(f"config.json: {w}width = {out['width']} does not divide into {out['blocks']} blocks")
        return out
    out = _heads(m, w)
    out["rot"] = _rot(m, w, out["dim"])
    if kind == "attention":
        if out["vdim"] != out["dim"]:
            raise ConfigError(f"config.json: {w}vdim = {out['vdim']}: the values of this mixer are its keys, of size dim = {out['dim']}")
        out.update(window=None, keep_first=0, softcap=None)
        if m.get("mask") is not None:
            mask = _obj(m, "mask", w)
            out["window"] = _int(mask, "size", w + "mask.")
            if mask.get("keep_first") is not None:
                out["keep_first"] = _int(mask, "keep_first", w + "mask.", 0)
        if m.get("softcap") is not None:
            out["softcap"] = _num(m, "softcap", w)
            if not out["softcap"] > 0:
                raise ConfigError(f"config.json: {w}softcap must be positive")
        return out
    out["diff"] = _num(m, "diff", w)
    out["kv_from"] = None if m.get("kv_from") is None else _int(m, "kv_from", w, 0)
    return out


def _mlp(mlp: Any, where: str) -> Optional[MlpArgs]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
        raise ConfigError(f"config.json: {where}'mlp' must be null or an object of kind 'dense' or 'moe'")
    w = where + "mlp."
    if mlp["kind"] == "dense":
        return MlpArgs("dense", _int(mlp, "ff", w))
    expert, router = _obj(mlp, "expert", w), _obj(mlp, "router", w)
    out = MlpArgs("moe", _int(expert, "ff", w + "expert."), experts=_int(router, "experts", w + "router."),
                  top=_int(router, "top", w + "router."),
                  shared_ff=0 if mlp.get("shared") is None else _int(_obj(mlp, "shared", w), "ff", w + "shared."))
    if out.top > out.experts:
        raise ConfigError(f"config.json: {w}router: {out.top} of {out.experts} experts per token")
    return out


def parse(cfg: Dict[str, Any]) -> TapupelArgs:
    if not isinstance(cfg, dict):
        raise ConfigError("config.json must hold one JSON object")
    layers = cfg.get("layers")
    if not isinstance(layers, list) or not layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    parsed = []
    for i, L in enumerate(layers):
        where = f"layers[{i}]."
        if not isinstance(L, dict):
            raise ConfigError(f"config.json: layers[{i}] must be an object")
        parsed.append(LayerArgs(L.get("type"), _mixer(L.get("type"), L.get("mixer"), where), _mlp(L.get("mlp"), where)))
    for i, L in enumerate(parsed):
        j = L.mixer.get("kv_from") if L.kind == "attention_2" else None
        if j is None:
            continue
        where = f"layers[{i}].mixer."
        if j >= i or parsed[j].kind != "attention_2" or parsed[j].mixer["kv_from"] is not None:
            raise ConfigError(f"config.json: {where}kv_from = {j} must name an earlier 'attention_2' layer with keys and values of its own")
        for k in ("kv_heads", "dim", "vdim", "rot"):
            if parsed[j].mixer[k] != L.mixer[k]:
                raise ConfigError(f"config.json: {where}{k} differs from layer {j}'s, whose keys and values it reads")
    eps = _num(_obj(cfg, "norm", ""), "eps", "norm.")
    if eps < 0:
        raise ConfigError("config.json: norm.eps must not be negative")
    scale = 1.0 if cfg.get("embedding") is None else _num(_obj(cfg, "embedding", ""), "scale", "embedding.")
    return TapupelArgs(vocab=_int(cfg, "vocab", ""), width=_int(cfg, "width", ""), embed_scale=scale, norm_eps=eps,
                       layers=tuple(parsed), source=dict(cfg))


def _position(m: Dict[str, Any], pairing: str) -> PartSpec:
    rot, sc = m["rot"], m["rot"]["scaling"]
    scaling = None if sc is None else dict(factor=sc["factor"], low_freq_factor=sc["low"], high_freq_factor=sc["high"],
                                           original_max_position_embeddings=sc["original"])
    return PartSpec("rope", dict(head_dim=rot["dims"], base=rot["base"], scaling=scaling, pairing=pairing, freq_dtype="float64"))


def build_spec(a: TapupelArgs) -> ModelSpec:
    D = a.width
    out_norm = PartSpec("rmsnorm", dict(dim=D, eps=a.norm_eps, one_plus=True))
    reads_stream = PartSpec("none", dict(dim=D))
    layers, schedule = [], []
    for i, L in enumerate(a.layers):
        m, position, kv_from = L.mixer, None, None
        if L.kind == "attention":
            position = _position(m, "half")
            mixer = PartSpec("attention", dict(dim=D, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], scale=m["scale"],
                                               window=m["window"], keep_first=m["keep_first"], softcap=m["softcap"],
                                               qk_norm_eps=a.norm_eps, qk_norm_weight=False, qk_norm_last=True, values_are_keys=True))
        elif L.kind == "rglru":
            mixer = PartSpec("rglru", dict(dim=D, width=m["width"], blocks=m["blocks"], taps=m["conv"], decay_scale=DECAY_SCALE))
        else:
            position, kv_from = _position(m, "interleaved"), m["kv_from"]
            mixer = PartSpec("diff_attention", dict(dim=D, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                                    scale=m["scale"], diff=m["diff"], eps=a.norm_eps, shared_kv=kv_from is not None))
        parts = dict(mixer=mixer, mixer_norm=reads_stream, mixer_post_norm=out_norm)
        if L.mlp is not None:
            if L.mlp.kind == "dense":
                ff = PartSpec("swiglu", dict(dim=D, hidden=L.mlp.ff))
            else:
                ff = PartSpec("moe", dict(dim=D, hidden=L.mlp.ff, n_experts=L.mlp.experts, top=L.mlp.top, score="softmax_top",
                                          correction=False, alpha=1.0, shift=0.0, limit=0.0, shared_hidden=L.mlp.shared_ff,
                                          shared_gate=L.mlp.shared_ff > 0))
            parts.update(feed_forward=ff, ffn_norm=reads_stream, ffn_post_norm=out_norm)
        layers.append(LayerSpec(block="sandwich", parts=parts, position=position))
        schedule.append(ScheduleEntry(layer=i, cache=i, kv_from=kv_from))
    # launch_overlap off: with kernels allowed to start under their predecessor, prompt steps of 2,048 tokens of this design at
    # layer sizes of real models stopped making progress in some runs (never with the launches strictly in turn); until the
    # pair of kernels behind that is found the design runs its steps in turn
    spec = ModelSpec(architecture="tapupel", dim=D, vocab_size=a.vocab, layers=layers, schedule=schedule, final_norm=out_norm,
                     embed_scale=a.embed_scale, launch_overlap=False)
    spec.validate()
    return spec


def _stack(*tensors):
    return torch.stack(tensors)


def _unstack(t):
    return list(t.unbind(0))


def weight_plan(a: TapupelArgs) -> WeightPlan:
    D, V = a.width, a.vocab
    r = [Recipe("embed.weight", [Source("embed", (V, D), "embedding")]), Recipe("head.weight", [Source("head", (V, D))]),
         Recipe("final_norm.weight", [Source("final.norm", (D,), "bias")])]
    for i, L in enumerate(a.layers):
        s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
        x, y = s + "mix.", t + "mixer."
        r.append(Recipe(t + "mixer_post_norm.weight", [Source(s + "norm1", (D,), "bias")]))
        if L.kind == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            r += [Recipe(y + "wq", [Source(x + "q", (H * d, D))]), Recipe(y + "wk", [Source(x + "k", (G * d, D))]),
                  Recipe(y + "wo", [Source(x + "o", (D, H * d))])]
        elif L.kind == "rglru":
            C, B, taps = m["width"], m["blocks"], m["conv"]
            bw = C // B
            r += [Recipe(y + "wy", [Source(x + "y", (C, D))]), Recipe(y + "y_bias", [Source(x + "y.b", (C,), "bias")]),
                  Recipe(y + "wx", [Source(x + "x", (C, D))]), Recipe(y + "x_bias", [Source(x + "x.b", (C,), "bias")]),
                  Recipe(y + "conv", [Source(x + "conv", (C, taps), "conv")]), Recipe(y + "conv_bias", [Source(x + "conv.b", (C,), "bias")]),
                  Recipe(y + "gate_a", [Source(x + "ra", (B, bw, bw))]), Recipe(y + "gate_a_bias", [Source(x + "ra.b", (B, bw), "bias")]),
                  Recipe(y + "gate_i", [Source(x + "ri", (B, bw, bw))]), Recipe(y + "gate_i_bias", [Source(x + "ri.b", (B, bw), "bias")]),
                  Recipe(y + "lam", [Source(x + "lam", (C,), "unit")]), Recipe(y + "wo", [Source(x + "o", (D, C))])]
        else:
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            r += [Recipe(y + "wq", [Source(x + "q", (H * 2 * d, D))]), Recipe(y + "q_norm", [Source(x + "q.norm", (d,), "norm")])]
            if m["kv_from"] is None:
                r += [Recipe(y + "wk", [Source(x + "k", (G * 2 * d, D))]), Recipe(y + "k_norm", [Source(x + "k.norm", (d,), "norm")]),
                      Recipe(y + "wv", [Source(x + "v", (G * dv, D))])]
            r += [Recipe(y + n, [Source(x + n, (d,), "bias")]) for n in ("lq1", "lk1", "lq2", "lk2")]
            r.append(Recipe(y + "wo", [Source(x + "o", (D, H * dv))]))
        if L.mlp is None:
            continue
        x, y = s + "mlp.", t + "feed_forward."
        r.append(Recipe(t + "ffn_post_norm.weight", [Source(s + "norm2", (D,), "bias")]))
        if L.mlp.kind == "dense":
            F = L.mlp.ff
            r += [Recipe(y + "w1", [Source(x + "gate", (F, D))]), Recipe(y + "w3", [Source(x + "up", (F, D))]),
                  Recipe(y + "w2", [Source(x + "down", (D, F))])]
            continue
        E, F, Fs = L.mlp.experts, L.mlp.ff, L.mlp.shared_ff
        r.append(Recipe(y + "router", [Source(x + "router", (E, D))]))
        for name, shape in (("gate", (F, D)), ("up", (F, D)), ("down", (D, F))):
            r.append(Recipe(y + name, [Source(f"{x}e{e}.{name}", shape) for e in range(E)], _stack, _unstack))
        if Fs:
            r += [Recipe(y + "shared_gate", [Source(x + "shared.gate", (Fs, D))]), Recipe(y + "shared_up", [Source(x + "shared.up", (Fs, D))]),
                  Recipe(y + "shared_down", [Source(x + "shared.down", (D, Fs))]), Recipe(y + "shared_sg", [Source(x + "shared.sg", (1, D))])]
    return WeightPlan(recipes=r)


TAPUPEL = register_architecture(Architecture(
    name="tapupel", aliases=("Tapupel",), parse=parse, build_spec=build_spec, weight_plan=weight_plan,
))
