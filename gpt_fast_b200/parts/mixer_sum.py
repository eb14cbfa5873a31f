"""Several mixers side by side on the same input, their results added with a constant factor each:

    y = sum_i factor_i * mixer_i(h)

Each sub-mixer is any registered mixer, given as a `PartSpec`; its parameters carry its name as a prefix
('left.wq', ...).  Every sub-mixer writes into a branch of its own (32-bit); the factors are applied when the branches
join the stream, which the stream's next norm does on its way.  Of the sub-mixers at most one may keep keys and values
and at most one per-sequence state: they share the layer's cache entry."""
from typing import Dict, Sequence

import torch

from ..cache.needs import CacheNeeds
from ..config.spec import PartSpec
from . import MIXERS, build_part, register_mixer
from .residual import Branch, as_residual


@register_mixer("sum")
class MixerSum:
    def __init__(self, dim: int, mixers: Dict[str, PartSpec], factors: Dict[str, float], dtype: torch.dtype, position=None):
        if not mixers or set(mixers) != set(factors):
            raise ValueError("a sum of mixers needs one factor per mixer")
        self.dim, self.dtype = dim, dtype
        self.names = list(mixers)
        self.mixers = {n: build_part(MIXERS, mixers[n], dtype=dtype, position=position) for n in self.names}
        self.factors = {n: float(factors[n]) for n in self.names}
        self._vectors = {}
        kv = [m.cache_needs().kv for m in self.mixers.values() if m.cache_needs().kv is not None]
        state = [m.cache_needs().state for m in self.mixers.values() if m.cache_needs().state is not None]
        if len(kv) > 1 or len(state) > 1:
            raise ValueError("of the mixers of a sum at most one keeps keys and values and at most one keeps state")
        self._needs = CacheNeeds(kv=kv[0] if kv else None, state=state[0] if state else None)

    def param_specs(self):
        return {f"{n}.{k}": s for n, m in self.mixers.items() for k, s in m.param_specs().items()}

    def load(self, tensors):
        for n, m in self.mixers.items():
            m.load({k[len(n) + 1:]: v for k, v in tensors.items() if k.startswith(n + ".")})
        dev = next(iter(tensors.values())).device
        self._vectors = {n: torch.full((self.dim,), f, dtype=torch.float32, device=dev) for n, f in self.factors.items()}

    def export(self):
        return {f"{n}.{k}": v for n, m in self.mixers.items() for k, v in m.export().items()}

    def cache_needs(self) -> CacheNeeds:
        return self._needs

    def forward(self, h, batch, view, residual, append: bool = True):
        r = as_residual(residual)
        for n in self.names:
            y = Branch(batch.n_tokens, self.dim, h.device)
            self.mixers[n].forward(h, batch, view, residual=y, append=append)
            r.add_scaled(y, self._vectors[n])
