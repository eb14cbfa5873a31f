"""The Lomusun decoder as data: which parts each layer has and which checkpoint tensors fill which parameter.

The design: a token embedding plus a learned vector per position; layers in an order that config.json lists, each a
parallel block with ONE root-mean-square norm that mixer and feed-forward both read, x += mixer(h) + feed_forward(h);
a final norm of the same kind and the output product with the embedding table.  Two kinds of layer:

    'attention'  windowed softmax attention without rotation: q, k and v each pass a short causal convolution right
                 behind their projections, the scaled score takes a learned bias by head and (bucketed) distance, every
                 head's output a sigmoid gate of its own.  A layer with 'kv_from' has queries only and reads the keys and
                 values that another attention layer cached.
    'parallel'   two mixers on the same input, added with a constant factor each: on the left windowed attention whose
                 q and k are normed over the whole projection, whose score loses slope_head * distance and whose
                 softmax has a learned sink, gated element by element; on the right the gated delta rule with one decay
                 per head and token, a normed read-out and a SiLU gate.

The feed-forward is a mixture of experts (sigmoid router, a correction that counts for the choice only, clamped gated
experts); a layer may have none.

config.json keys: architecture, vocab, width, max_positions, norm.eps, layers [{type, mixer {...}, mlp {kind: 'moe',
expert {ff, limit}, router {experts, top, scale}} | null}].  Tensor names: embed, pos, final.norm, l<i>.norm1,
l<i>.mix.*, l<i>.mlp.{router, correction, e<j>.{gate, up, down}}.
"""
from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

import torch

from ..config.args import ConfigError
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from ..weights.plan import Recipe, Source, WeightPlan
from .lasezen import _int, _num

KINDS = ("attention", "parallel")
SLOPE_EXPONENT = -8.0                # slope of head h of H: 2^(-8 (h + 1) / H)
EXPERT_ALPHA = 1.702                 # an expert's activation: g * sigmoid(1.702 g) * (u + 1)
EXPERT_SHIFT = 1.0
DEFAULT_BIAS_ROWS = 16               # rows of a distance table when neither a checkpoint nor config.json gives them


@dataclass(frozen=True)
class MoeArgs:
    ff: int
    limit: float
    experts: int
    top: int
    scale: float


@dataclass(frozen=True)
class LayerArgs:
    kind: str
    mixer: Dict[str, Any]                  # the layer's sizes and constants, checked
    mlp: Optional[MoeArgs] = None          # None: the layer has no feed-forward


@dataclass(frozen=True)
class LomusunArgs:
    vocab: int
    width: int
    max_positions: int
    norm_eps: float
    layers: Tuple[LayerArgs, ...]
    source: Dict[str, Any] = field(default_factory=dict, compare=False, repr=False)

    def to_json(self) -> Dict[str, Any]:
        return dict(self.source)


def _window(m: Dict[str, Any], where: str) -> Optional[int]:
    mask = m.get("mask")
    if mask is None:
        return None
    if not isinstance(mask, dict):
        raise ConfigError(f"config.json: {where}'mask' must be an object with 'size'")
    return _int(mask, "size", where + "mask.")


def _heads(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where[:-1]} must be an object")
    out = {k: _int(m, k, where) for k in ("heads", "kv_heads", "dim", "vdim")}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}{out['heads']} heads do not divide into {out['kv_heads']} kv_heads")
    return out


def _mixer(kind: str, m: Any, where: str) -> Dict[str, Any]:
    if kind not in KINDS:
        raise ConfigError(f"config.json: {where}'type' is {kind!r}; this design has {', '.join(KINDS)}")
    if not isinstance(m, dict):
        raise ConfigError(f"config.json: {where}'mixer' must be an object")
    w = where + "mixer."
    if kind == "attention":
        out = _heads(m, w)
        out.update(conv=_int(m, "conv", w), scale=_num(m, "scale", w), bias_max=_num(m, "bias_max", w), window=_window(m, w),
                   kv_from=None, bias_rows=None)
        if m.get("kv_from") is not None:
            out["kv_from"] = _int(m, "kv_from", w, 0)
        if m.get("bias_rows") is not None:
            out["bias_rows"] = _int(m, "bias_rows", w, 2)
        return out
    left = _heads(m.get("left"), w + "left.")
    left.update(scale=_num(m["left"], "scale", w + "left."), window=_window(m["left"], w + "left."))
    right = _heads(m.get("right"), w + "right.")
    right["conv"] = _int(m["right"], "conv", w + "right.")
    return dict(left=left, right=right, left_scale=_num(m, "left_scale", w), right_scale=_num(m, "right_scale", w))


def _mlp(mlp: Any, where: str) -> Optional[MoeArgs]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}'mlp' must be null or an object of kind 'moe'")
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, dict) or not isinstance(router, dict):
        raise ConfigError(f"config.json: {where}mlp needs the objects 'expert' and 'router'")
    out = MoeArgs(ff=_int(expert, "ff", where + "mlp.expert."), limit=_num(expert, "limit", where + "mlp.expert."),
                  experts=_int(router, "experts", where + "mlp.router."), top=_int(router, "top", where + "mlp.router."),
                  scale=_num(router, "scale", where + "mlp.router."))
    if out.top > out.experts:
        raise ConfigError(f"config.json: {where}mlp.router: {out.top} of {out.experts} experts per token")
    if not out.limit > 0:
        raise ConfigError(f"config.json: {where}mlp.expert.limit must be positive")
    return out


def parse(cfg: Dict[str, Any]) -> LomusunArgs:
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
        j = L.mixer.get("kv_from") if L.kind == "attention" else None
        if j is None:
            continue
        where = f"layers[{i}].mixer."
        if j >= i or parsed[j].kind != "attention" or parsed[j].mixer["kv_from"] is not None:
            raise ConfigError(f"config.json: {where}kv_from = {j} must name an earlier 'attention' layer with keys and values of its own")
        for k in ("kv_heads", "dim", "vdim"):
            if parsed[j].mixer[k] != L.mixer[k]:
                raise ConfigError(f"config.json: {where}{k} differs from layer {j}'s, whose keys and values it reads")
    norm = cfg.get("norm")
    if not isinstance(norm, dict):
        raise ConfigError("config.json: 'norm' must be an object with 'eps'")
    eps = _num(norm, "eps", "norm.")
    if eps < 0:
        raise ConfigError("config.json: norm.eps must not be negative")
    return LomusunArgs(vocab=_int(cfg, "vocab", ""), width=_int(cfg, "width", ""), max_positions=_int(cfg, "max_positions", ""),
                       norm_eps=eps, layers=tuple(parsed), source=dict(cfg))


def bias_rows(a: LomusunArgs, layer: int, shapes: Optional[Dict[str, Tuple[int, ...]]]) -> int:
    """Rows of an 'attention' layer's distance table.  config.json does not have to name them: the checkpoint's tensor
    l<i>.mix.rel has them as its first dimension.  Without a checkpoint (random weights) `mixer.bias_rows`, else 16."""
    if shapes is not None and f"l{layer}.mix.rel" in shapes:
        return int(shapes[f"l{layer}.mix.rel"][0])
    return a.layers[layer].mixer["bias_rows"] or DEFAULT_BIAS_ROWS


def _attention(a: LomusunArgs, i: int, shapes) -> PartSpec:
    m = a.layers[i].mixer
    return PartSpec("attention", dict(dim=a.width, n_head=m["heads"], n_kv=m["kv_heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                      window=m["window"], scale=m["scale"], conv_taps=m["conv"], gate="head",
                                      distance_bias=dict(kind="table", rows=bias_rows(a, i, shapes), far=m["bias_max"]),
                                      shared_kv=m["kv_from"] is not None))


def _two_mixers(a: LomusunArgs, i: int) -> PartSpec:
    m = a.layers[i].mixer
    le, ri = m["left"], m["right"]
    left = PartSpec("attention", dict(dim=a.width, n_head=le["heads"], n_kv=le["kv_heads"], head_dim=le["dim"], v_head_dim=le["vdim"],
                                      window=le["window"], scale=le["scale"], qk_norm_eps=a.norm_eps, qk_norm_whole=True, sink=True,
                                      distance_bias=dict(kind="slopes", exponent=SLOPE_EXPONENT), gate="element"))
    right = PartSpec("delta_rule", dict(dim=a.width, n_head=ri["heads"], n_qk=ri["kv_heads"], head_dim=ri["dim"], v_head_dim=ri["vdim"],
                                        taps=ri["conv"], decay_rank=0, gate_rank=0, eps=a.norm_eps, head_decay=True, gate_act="silu"))
    return PartSpec("sum", dict(dim=a.width, mixers=dict(left=left, right=right),
                                factors=dict(left=m["left_scale"], right=m["right_scale"])))


def build_spec(a: LomusunArgs, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(dim=a.width, eps=a.norm_eps))
    layers, schedule = [], []
    for i, L in enumerate(a.layers):
        parts = dict(mixer=_attention(a, i, shapes) if L.kind == "attention" else _two_mixers(a, i), mixer_norm=norm)
        if L.mlp is not None:
            parts["feed_forward"] = PartSpec("moe", dict(dim=a.width, hidden=L.mlp.ff, n_experts=L.mlp.experts, top=L.mlp.top,
                                                         router_scale=L.mlp.scale, limit=L.mlp.limit, alpha=EXPERT_ALPHA,
                                                         shift=EXPERT_SHIFT, correction=True))
        layers.append(LayerSpec(block="parallel", parts=parts))
        schedule.append(ScheduleEntry(layer=i, cache=i, kv_from=L.mixer.get("kv_from") if L.kind == "attention" else None))
    spec = ModelSpec(architecture="lomusun", dim=a.width, vocab_size=a.vocab, layers=layers, schedule=schedule, final_norm=norm,
                     tie_embeddings=True, max_position=a.max_positions,
                     embedding=PartSpec("learned_position", dict(dim=a.width, max_positions=a.max_positions)))
    spec.validate()
    return spec


def _stack(*tensors):
    return torch.stack(tensors)


def _unstack(t):
    return list(t.unbind(0))


def weight_plan(a: LomusunArgs, shapes: Optional[Dict[str, Tuple[int, ...]]] = None) -> WeightPlan:
    D, V = a.width, a.vocab
    r = [Recipe("embed.weight", [Source("embed", (V, D), "embedding")]),
         Recipe("embedding.table", [Source("pos", (a.max_positions, D), "embedding")]),
         Recipe("final_norm.weight", [Source("final.norm", (D,), "norm")])]
    for i, L in enumerate(a.layers):
        s, t, m = f"l{i}.", f"layers.{i}.", L.mixer
        r.append(Recipe(t + "mixer_norm.weight", [Source(s + "norm1", (D,), "norm")]))
        if L.kind == "attention":
            x, y = s + "mix.", t + "mixer."
            H, G, d, dv, taps = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            r += [Recipe(y + "wq", [Source(x + "q", (H * d, D))]), Recipe(y + "q_conv", [Source(x + "q.conv", (H * d, taps), "conv")])]
            if m["kv_from"] is None:
                r += [Recipe(y + "wk", [Source(x + "k", (G * d, D))]), Recipe(y + "k_conv", [Source(x + "k.conv", (G * d, taps), "conv")]),
                      Recipe(y + "wv", [Source(x + "v", (G * dv, D))]), Recipe(y + "v_conv", [Source(x + "v.conv", (G * dv, taps), "conv")])]
            r += [Recipe(y + "rel", [Source(x + "rel", (bias_rows(a, i, shapes), H), "unit")]),
                  Recipe(y + "wg", [Source(x + "g", (H, D))]), Recipe(y + "wo", [Source(x + "o", (D, H * dv))])]
        else:
            x, y, le = s + "mix.left.", t + "mixer.left.", m["left"]
            H, G, d, dv = le["heads"], le["kv_heads"], le["dim"], le["vdim"]
            r += [Recipe(y + "wq", [Source(x + "q", (H * d, D))]), Recipe(y + "wk", [Source(x + "k", (G * d, D))]),
                  Recipe(y + "wv", [Source(x + "v", (G * dv, D))]),
                  Recipe(y + "q_norm", [Source(x + "q.norm", (H * d,), "norm")]), Recipe(y + "k_norm", [Source(x + "k.norm", (G * d,), "norm")]),
                  Recipe(y + "sink", [Source(x + "sink", (H,), "unit")]),
                  Recipe(y + "wg", [Source(x + "g", (H * dv, D))]), Recipe(y + "wo", [Source(x + "o", (D, H * dv))])]
            x, y, ri = s + "mix.right.", t + "mixer.right.", m["right"]
            H, J, d, dv, taps = ri["heads"], ri["kv_heads"], ri["dim"], ri["vdim"], ri["conv"]
            r += [Recipe(y + "wq", [Source(x + "q", (J * d, D))]), Recipe(y + "q_conv", [Source(x + "q.conv", (J * d, taps), "conv")]),
                  Recipe(y + "wk", [Source(x + "k", (J * d, D))]), Recipe(y + "k_conv", [Source(x + "k.conv", (J * d, taps), "conv")]),
                  Recipe(y + "wv", [Source(x + "v", (H * dv, D))]), Recipe(y + "v_conv", [Source(x + "v.conv", (H * dv, taps), "conv")]),
                  Recipe(y + "wb", [Source(x + "b", (H, D))]), Recipe(y + "a_log", [Source(x + "A_log", (H,), "bias")]),
                  Recipe(y + "norm", [Source(x + "norm", (dv,), "norm")]), Recipe(y + "wa", [Source(x + "a", (H, D))]),
                  Recipe(y + "dt_bias", [Source(x + "dt_bias", (H,), "bias")]),
                  Recipe(y + "wg", [Source(x + "g", (H * dv, D))]), Recipe(y + "wo", [Source(x + "o", (D, H * dv))])]
        if L.mlp is not None:
            x, y, E, F = s + "mlp.", t + "feed_forward.", L.mlp.experts, L.mlp.ff
            r += [Recipe(y + "router", [Source(x + "router", (E, D))]),
                  Recipe(y + "correction", [Source(x + "correction", (E,), "bias")])]
            for name, shape in (("gate", (F, D)), ("up", (F, D)), ("down", (D, F))):
                r.append(Recipe(y + name, [Source(f"{x}e{e}.{name}", shape) for e in range(E)], _stack, _unstack))
    return WeightPlan(recipes=r, aliases={"head.weight": "embed.weight"})


LOMUSUN = register_architecture(Architecture(
    name="lomusun", aliases=("Lomusun",), parse=parse, build_spec=build_spec, weight_plan=weight_plan, shapes_from_checkpoint=True,
))
