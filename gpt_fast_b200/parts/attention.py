"""Causal grouped-query attention with a fused q/k/v projection
(gpt-fast model.py:167-216).

Steps: qkv = h Wqkv^T; prepare q and k (rotate by each token's position, or
norm per head), append k, v to the sequence's place in the cache and attend
over the cache; residual += y Wo^T.  Query head h reads key/value head
h // (n_head / n_kv); the scale is 1/sqrt(head_dim) unless given.

Options beyond gpt-fast's attention, each off by default:
  position=None    no rotation: positions do not enter the scores
  qk_norm_eps      q and k are divided by their root mean square over the head (+ eps inside the root) and
                   multiplied by a weight [head_dim] shared by the heads (parameters q_norm, k_norm)
  chunk            a query sees only keys of its own block of `chunk` positions, blocks counted from the
                   sequence's first position
  sink             a learned number per query head (parameter sink) whose exponential joins the softmax
                   denominator; it has no key and no value and is not scaled
  v_head_dim       a head size of the values that differs from the keys'
  window           only the latest `window` positions are seen
  qk_norm_whole    the q/k norm runs over the whole projection (all heads of q, or of k, as one vector) with a weight
                   per column, instead of per head
  conv_taps        q, k and v each pass a causal convolution over time per channel (`conv_taps` wide, no bias, no
                   activation) right behind the projection; the last conv_taps - 1 projected rows of a sequence are
                   per-sequence state (parameters q_conv, k_conv, v_conv [channels, taps], the last column the current token's)
  distance_bias    a bias on the scaled score that depends on the head and on the distance n = i - j:
                   {"kind": "slopes", "exponent": e}: minus 2^(e (h + 1) / H) * n  (no parameters);
                   {"kind": "table", "rows": B, "far": D}: plus rel[bucket(n), h], a learned table (parameter rel [B, H])
                   with one row per distance below B // 2 and logarithmic rows from there to distance D
  gate             'head': head h's output times sigmoid(Wg h)_h, one gate per head; 'element': the concatenated heads times
                   sigmoid(Wg h), one gate per column (parameter wg)
  shared_kv        the layer has no key/value projections: it attends over the cache entry of another run with its own queries
  qk_norm_weight   False: the per-head q/k norm has no weights
  qk_norm_last     the per-head q/k norm follows the rotation instead of preceding it
  values_are_keys  no value projection: a position's values are its keys as projected, ahead of norm and rotation
  softcap          the scaled score s becomes softcap * tanh(s / softcap)
  keep_first       with a window: the sequence's first `keep_first` positions stay visible to every later query
With none of them the rotate-and-append kernel and the tensor-core attention kernels run; the others go through
`ops.qkv_prepare` and the options of `ops.attention`."""
import math
from typing import Optional

import torch

from .. import ops
from ..cache.needs import CacheNeeds, KVNeed, StateNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


def distance_bucket(n: int, rows: int, far: float) -> int:
    """The row of a distance table for distance n >= 0: one row per distance below rows // 2, then
    rows // 2 + floor(ln(n / half) / ln(far / half) * (rows - half)), at most the last row."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    extra = -w.shape[0] % multiple
    return w.contiguous() if extra == 0 else torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous()


@register_mixer("attention")
class Attention:
    def __init__(self, dim: int, n_head: int, n_kv: int, head_dim: int, dtype: torch.dtype, position,
                 window: Optional[int] = None, scale: Optional[float] = None, v_head_dim: Optional[int] = None,
                 qk_norm_eps: Optional[float] = None, chunk: Optional[int] = None, sink: bool = False,
                 qk_norm_whole: bool = False, conv_taps: Optional[int] = None, distance_bias: Optional[dict] = None,
                 gate: Optional[str] = None, shared_kv: bool = False, qk_norm_weight: bool = True, qk_norm_last: bool = False,
                 values_are_keys: bool = False, softcap: Optional[float] = None, keep_first: int = 0):
        if n_head % n_kv:
            raise ValueError(f"{n_head} query heads do not divide into {n_kv} key/value heads")
        if chunk is not None and chunk < 1:
            raise ValueError(f"a chunk of {chunk} positions")
        self.dim, self.n_head, self.n_kv, self.head_dim = dim, n_head, n_kv, head_dim
        self.v_head_dim = int(v_head_dim) if v_head_dim else head_dim
        self.window, self.dtype, self.position = window, dtype, position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.chunk, self.has_sink = chunk, bool(sink)
        self.qk_norm_whole = bool(qk_norm_whole) and self.qk_norm_eps is not None
        self.conv_taps = int(conv_taps) if conv_taps else None
        self.gate, self.shared_kv = gate, bool(shared_kv)
        self.qk_norm_weight, self.qk_norm_last = bool(qk_norm_weight), bool(qk_norm_last)
        self.values_are_keys = bool(values_are_keys)
        self.softcap = float(softcap) if softcap else None
        self.keep_first = int(keep_first or 0)
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError(f"a soft cap of {softcap} on the scores")
        if self.keep_first < 0:
            raise ValueError(f"{keep_first} kept first positions")
        if self.values_are_keys and (self.v_head_dim != head_dim or self.shared_kv or conv_taps):
            raise ValueError("values that are the projected keys have the keys' head size, a cache entry of their own and no convolution")
        if self.qk_norm_whole and (not self.qk_norm_weight or self.qk_norm_last):
            raise ValueError("a q/k norm over the whole projection has weights and precedes the rotation")
        if gate not in (None, "head", "element"):
            raise ValueError(f"an output gate is 'head' or 'element', not {gate!r}")
        self.distance_bias = dict(distance_bias) if distance_bias else None
        if self.distance_bias is not None:
            kind = self.distance_bias.get("kind")
            if kind == "table":
                if int(self.distance_bias["rows"]) < 2 or not float(self.distance_bias["far"]) > int(self.distance_bias["rows"]) // 2:
                    raise ValueError("a distance table needs at least two rows and a far distance beyond its linear half")
            elif kind != "slopes":
                raise ValueError(f"a distance bias is of kind 'slopes' or 'table', not {kind!r}")
        extras = (self.qk_norm_whole or self.conv_taps or self.distance_bias is not None or gate is not None or self.shared_kv
                  or self.values_are_keys or self.softcap is not None or self.keep_first)
        self.plain = (position is not None and self.v_head_dim == head_dim and self.qk_norm_eps is None
                      and chunk is None and not self.has_sink and getattr(position, "head_dim", head_dim) == head_dim
                      and not extras)
        self.wqkv = self.wo = self.q_norm = self.k_norm = self.sink = None
        self.conv = self.bias_table = self.slopes = None
        # columns of the fused projection: q, then k and v (unless shared), then the gates
        self.kv_cols = 0 if self.shared_kv else n_kv * head_dim if self.values_are_keys else n_kv * (head_dim + self.v_head_dim)
        self.conv_channels = n_head * head_dim + self.kv_cols
        self.gate_cols = {None: 0, "head": n_head, "element": n_head * self.v_head_dim}[gate]

    def param_specs(self):
        H, G, d, dv, D = self.n_head, self.n_kv, self.head_dim, self.v_head_dim, self.dim
        specs = {"wq": ParamSpec((H * d, D)), "wo": ParamSpec((D, H * dv))}
        if not self.shared_kv:
            specs["wk"] = ParamSpec((G * d, D))
            if not self.values_are_keys:
                specs["wv"] = ParamSpec((G * dv, D))
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            specs["q_norm"] = ParamSpec(((H if self.qk_norm_whole else 1) * d,), "vector")
            if not self.shared_kv:
                specs["k_norm"] = ParamSpec(((G if self.qk_norm_whole else 1) * d,), "vector")
        if self.has_sink:
            specs["sink"] = ParamSpec((H,), "vector")
        if self.conv_taps:
            specs["q_conv"] = ParamSpec((H * d, self.conv_taps), "vector")
            if not self.shared_kv:
                specs.update(k_conv=ParamSpec((G * d, self.conv_taps), "vector"), v_conv=ParamSpec((G * dv, self.conv_taps), "vector"))
        if self.gate is not None:
            specs["wg"] = ParamSpec((self.gate_cols, D))
        if self.distance_bias is not None and self.distance_bias["kind"] == "table":
            specs["rel"] = ParamSpec((int(self.distance_bias["rows"]), H), "vector")
        return specs

    def load(self, tensors):
        # rows: q heads, then k heads, then v heads (gpt-fast model.py:184-189)
        self._stored = {k: v for k, v in tensors.items() if k not in ("wq", "wk", "wv", "wg", "wo")}
        rows = [tensors["wq"]] + ([] if self.shared_kv else [tensors["wk"]] if self.values_are_keys else [tensors["wk"], tensors["wv"]])
        if self.gate is not None:
            rows.append(tensors["wg"])
        self.wqkv = torch.cat(rows).contiguous() if self.plain or len(rows) == 3 and self.gate is None else _pad_rows(torch.cat(rows))
        self.wo = tensors["wo"]
        if self.qk_norm_eps is not None and self.qk_norm_weight:
            self.q_norm = tensors["q_norm"]
            self.k_norm = None if self.shared_kv else tensors["k_norm"].to(tensors["q_norm"].dtype)
        if self.has_sink:
            self._sink_stored = tensors["sink"]
            self.sink = tensors["sink"].float().contiguous()        # softmax terms are 32-bit
        if self.conv_taps:
            taps = [tensors["q_conv"]] + ([] if self.shared_kv else [tensors["k_conv"], tensors["v_conv"]])
            self.conv = torch.cat([t.to(taps[0].dtype) for t in taps]).contiguous()
        if self.distance_bias is not None:
            dev = self.wo.device
            if self.distance_bias["kind"] == "slopes":
                e = float(self.distance_bias["exponent"])
                self.slopes = torch.tensor([2.0 ** (e * (h + 1) / self.n_head) for h in range(self.n_head)],
                                           dtype=torch.float32).to(dev)
            else:
                # the table by distance: row n = rel[bucket(n)], up to the distance from which the last row holds
                rows_, far = int(self.distance_bias["rows"]), float(self.distance_bias["far"])
                reach = int(math.ceil(far)) + 1
                if self.window:
                    reach = min(reach, int(self.window))
                pick = torch.tensor([distance_bucket(n, rows_, far) for n in range(max(reach, 1))], dtype=torch.long)
                self.bias_table = tensors["rel"].float().cpu()[pick].contiguous().to(dev)

    def export(self):
        """The parameters as `load` received them (the way back from the fused layout)."""
        H, G, d, dv = self.n_head, self.n_kv, self.head_dim, self.v_head_dim
        kv = [] if self.shared_kv else [("wk", G * d)] if self.values_are_keys else [("wk", G * d), ("wv", G * dv)]
        sizes = [H * d] + [n for _, n in kv] + ([self.gate_cols] if self.gate is not None else [])
        names = ["wq"] + [k for k, _ in kv] + (["wg"] if self.gate is not None else [])
        out = dict(zip(names, self.wqkv[:sum(sizes)].split(sizes)), wo=self.wo)
        out.update({k: self._stored[k] for k in self.param_specs() if k not in out})
        return out

    def cache_needs(self) -> CacheNeeds:
        dv = self.v_head_dim if self.v_head_dim != self.head_dim else None
        kv = None if self.shared_kv else KVNeed(self.n_kv, self.head_dim, self.window, dv)
        state = StateNeed(((self.conv_taps - 1) * self.conv_channels,), torch.float32) if self.conv_taps and self.conv_taps > 1 else None
        return CacheNeeds(kv=kv, state=state)

    def forward(self, h, batch, view, residual, append: bool = True):
        T = batch.n_tokens
        H, G, d, dv = self.n_head, self.n_kv, self.head_dim, self.v_head_dim
        if self.shared_kv and append:
            raise ValueError("an attention layer without key/value projections reads another run's cache entry")
        if not self.shared_kv and not append and self.conv_taps:
            raise ValueError("a run on another run's cache entry cannot advance a convolution over keys and values")
        qkv = torch.empty(T, self.wqkv.shape[0], dtype=self.dtype, device=h.device)
        # a split sum is finished by the kernel that reads it; a convolution or a gate reads the finished rows
        partials = ops.linear(h, self.wqkv, qkv, defer=not (self.conv_taps or self.gate))
        y = torch.empty(T, H * dv, dtype=self.dtype, device=h.device)
        if self.plain:
            ops.rope_append_attention(qkv, partials, view.kv, batch, self.position.table, y, H, G, d, self.position.pairing,
                                      append, self.scale, self.window)
        else:
            q = torch.empty(T, H, d, dtype=self.dtype, device=h.device)
            pos = self.position
            src = qkv
            if self.conv_taps:
                C = self.conv_channels
                conv = torch.empty(T, C, dtype=torch.float32, device=h.device)
                state = view.state if self.conv_taps > 1 else conv          # one tap keeps nothing
                ops.short_conv(qkv, 0, C, self.conv, None, state, 0, conv, batch, act=False)
                src, partials = None, conv.view(1, T, C)                    # the 32-bit rows, taken as a sum of one part
            kw = {"norm_whole": True} if self.qk_norm_whole else {}
            if self.qk_norm_eps is not None and not self.qk_norm_weight:
                kw["norm_bare"] = True
            if self.qk_norm_last:
                kw["norm_last"] = True
            # values that are the keys as projected: the value columns of the row are its key columns
            ops.qkv_prepare(src, partials, (0, H * d, H * d if self.values_are_keys else (H + G) * d), q, view.kv, batch, H, G, d, dv,
                            table=None if pos is None else pos.table, rot_dims=0 if pos is None else pos.head_dim,
                            pairing="half" if pos is None else pos.pairing, q_norm=self.q_norm, k_norm=self.k_norm,
                            norm_eps=self.qk_norm_eps or 0.0, append=append, **kw)
            kw = {}
            if self.bias_table is not None:
                kw["bias"] = self.bias_table
            if self.slopes is not None:
                kw["slopes"] = self.slopes
            if self.softcap is not None:
                kw["softcap"] = self.softcap
            if self.keep_first and self.window:
                kw["keep_first"] = self.keep_first
            ops.attention(q, view.kv, batch, y, H, G, d, self.scale, self.window, self.chunk, self.sink, dv, **kw)
            if self.gate is not None:
                ops.sigmoid_gate(y, qkv, H * d + self.kv_cols, dv if self.gate == "head" else 1)
        as_residual(residual).add_linear(y, self.wo)
