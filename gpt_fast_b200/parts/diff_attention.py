"""Differential attention: every head has two softmax score maps over one set of values, and what it hands on is their
difference.

    q = Wq h  [H heads x 2 maps x d],   k = Wk h  [G x 2 x d],   v = Wv h  [G x dv]       (laid out head by head, map by map)
    q, k <- root-mean-square norm over d per head and map, times a weight [d] that all heads and maps share, then
            rotated by the token's position (each map like a head of its own)
    a_m = softmax(scale q_m . k_m, causal) v                                  m = 1, 2;  query head h reads key/value head h // (H / G)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + c                              one number for the layer, from four learned vectors [d]
    o = a_1 - lambda a_2;   o <- o / sqrt(mean(o^2) + eps) * (1 - c)          per head, over dv
    y = Wo concat_h o_h

The cache holds, per position and key/value head, the two normed and rotated keys side by side and the value.  With
`shared_kv` the layer has no key/value projections and no key norm: it reads the cache entry of another run with its own
queries.  Scores, softmax, lambda and the head norm are 32-bit."""
import math
from typing import Optional

import torch

from .. import ops
from ..cache.needs import CacheNeeds, KVNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual

MAPS = 2


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    extra = -w.shape[0] % multiple
    return w.contiguous() if extra == 0 else torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous()


@register_mixer("diff_attention")
class DiffAttention:
    def __init__(self, dim: int, n_head: int, n_kv: int, head_dim: int, v_head_dim: int, diff: float, eps: float,
                 dtype: torch.dtype, position, scale: Optional[float] = None, shared_kv: bool = False):
        if n_head % n_kv:
            raise ValueError(f"{n_head} query heads do not divide into {n_kv} key/value heads")
        self.dim, self.n_head, self.n_kv, self.head_dim, self.v_head_dim = dim, n_head, n_kv, head_dim, int(v_head_dim)
        self.diff, self.eps, self.dtype, self.position = float(diff), float(eps), dtype, position
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.shared_kv = bool(shared_kv)
        self.kv_cols = 0 if self.shared_kv else n_kv * (MAPS * head_dim + self.v_head_dim)
        self.wqkv = self.wo = self.q_norm = self.k_norm = None
        self.lam = None                                    # lambda, made once when the weights arrive

    def param_specs(self):
        H, G, d, dv, D = self.n_head, self.n_kv, self.head_dim, self.v_head_dim, self.dim
        specs = {"wq": ParamSpec((H * MAPS * d, D)), "wo": ParamSpec((D, H * dv)), "q_norm": ParamSpec((d,), "vector")}
        if not self.shared_kv:
            specs.update(wk=ParamSpec((G * MAPS * d, D)), wv=ParamSpec((G * dv, D)), k_norm=ParamSpec((d,), "vector"))
        for name in ("lq1", "lk1", "lq2", "lk2"):
            specs[name] = ParamSpec((d,), "vector")
        return specs

    def load(self, tensors):
        self._stored = {k: v for k, v in tensors.items() if k not in ("wq", "wk", "wv", "wo")}
        rows = [tensors["wq"]] + ([] if self.shared_kv else [tensors["wk"], tensors["wv"]])
        self.wqkv = _pad_rows(torch.cat(rows))
        self.wo = tensors["wo"]
        self.q_norm = tensors["q_norm"]
        self.k_norm = None if self.shared_kv else tensors["k_norm"].to(self.q_norm.dtype)
        lq1, lk1, lq2, lk2 = (tensors[n].float() for n in ("lq1", "lk1", "lq2", "lk2"))
        self.lam = float(torch.exp((lq1 * lk1).sum()) - torch.exp((lq2 * lk2).sum())) + self.diff

    def export(self):
        H, G, d, dv = self.n_head, self.n_kv, self.head_dim, self.v_head_dim
        sizes = [H * MAPS * d] + ([] if self.shared_kv else [G * MAPS * d, G * dv])
        names = ["wq"] + ([] if self.shared_kv else ["wk", "wv"])
        out = dict(zip(names, self.wqkv[:sum(sizes)].split(sizes)), wo=self.wo)
        out.update(self._stored)
        return out

    def cache_needs(self) -> CacheNeeds:
        if self.shared_kv:
            return CacheNeeds()
        dk = MAPS * self.head_dim
        return CacheNeeds(kv=KVNeed(self.n_kv, dk, None, self.v_head_dim if self.v_head_dim != dk else None))

    def forward(self, h, batch, view, residual, append: bool = True):
        T = batch.n_tokens
        H, G, d, dv = self.n_head, self.n_kv, self.head_dim, self.v_head_dim
        if self.shared_kv and append:
            raise ValueError("a differential attention layer without key/value projections reads another run's cache entry")
        qkv = torch.empty(T, self.wqkv.shape[0], dtype=self.dtype, device=h.device)
        partials = ops.linear(h, self.wqkv, qkv, defer=True)
        # where the kernels' fast attention takes heads of 2 d, every map runs as an ordinary head: its query lies in the
        # columns of its own key and zeros face the other map's
        spread = ops.spread_queries(self.dtype, H, G, d, dv, MAPS, view.kv.page_size)
        q = (torch.zeros(T, H * MAPS, MAPS * d, dtype=self.dtype, device=h.device) if spread
             else torch.empty(T, H * MAPS, d, dtype=self.dtype, device=h.device))
        pos = self.position
        ops.qkv_prepare(qkv, partials, (0, H * MAPS * d, (H + G) * MAPS * d), q, view.kv, batch, H, G, d, dv,
                        table=None if pos is None else pos.table, rot_dims=0 if pos is None else pos.head_dim,
                        pairing="half" if pos is None else pos.pairing, q_norm=self.q_norm, k_norm=self.k_norm,
                        norm_eps=self.eps, append=append, maps=MAPS, **({"q_spread": True} if spread else {}))
        y = torch.empty(T, H * dv, dtype=self.dtype, device=h.device)
        ops.attention(q, view.kv, batch, y, H, G, d, self.scale, v_head_dim=dv, maps=MAPS, diff=(self.lam, self.eps, 1.0 - self.diff))
        as_residual(residual).add_linear(y, self.wo)
