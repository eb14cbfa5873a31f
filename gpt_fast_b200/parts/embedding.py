"""What a model may add to its token embedding.

'bigram_hash': a second table indexed by a hash of the previous and the current token,

    x_t = table[tok_t] + extra[(tok_(t-1) * mul_prev + tok_t * mul_cur) mod buckets]

with the table's last row (number `buckets`) for a sequence's first token.  The previous token is per-sequence
state (one int32 in the cache), so a sequence may arrive in portions of any size.

'learned_position': a learned vector per position, x_t = table[tok_t] + positions[p_t], p_t counted from 0 in each
sequence; it keeps no state (a token's position is its sequence's cached length plus its place in the step)."""
import torch

from .. import ops
from ..cache.needs import CacheNeeds, StateNeed
from ..weights.loader import ParamSpec
from . import register_embedding


@register_embedding("bigram_hash")
class BigramHash:
    def __init__(self, dim: int, buckets: int, mul_prev: int, mul_cur: int, dtype: torch.dtype):
        if buckets < 1:
            raise ValueError(f"a hashed embedding needs at least one bucket, got {buckets}")
        self.dim, self.buckets, self.mul_prev, self.mul_cur, self.dtype = dim, int(buckets), int(mul_prev), int(mul_cur), dtype
        self.table = None

    def param_specs(self):
        return {"table": ParamSpec((self.buckets + 1, self.dim))}

    def load(self, tensors):
        self.table = tensors["table"]

    def export(self):
        return {"table": self.table}

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateNeed((1,), torch.int32))

    def forward(self, tokens, table, out, batch, view, scale: float = 1.0):
        """out float32 [T, dim] = table[tokens] * scale + the hashed rows; view.state int32 [n_slots, 1]."""
        ops.embed_hashed(tokens, table, self.table, out, batch, view.state.view(-1), self.buckets, self.mul_prev, self.mul_cur, scale)


@register_embedding("learned_position")
class LearnedPosition:
    def __init__(self, dim: int, max_positions: int, dtype: torch.dtype):
        if max_positions < 1:
            raise ValueError(f"a position table needs at least one row, got {max_positions}")
        self.dim, self.max_positions, self.dtype = dim, int(max_positions), dtype
        self.table = None

    def param_specs(self):
        return {"table": ParamSpec((self.max_positions, self.dim))}

    def load(self, tensors):
        self.table = tensors["table"]

    def export(self):
        return {"table": self.table}

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds()

    def forward(self, tokens, table, out, batch, view, scale: float = 1.0):
        """out float32 [T, dim] = table[tokens] * scale + the rows of the tokens' positions."""
        ops.embed_positions(tokens, table, self.table, out, batch, scale)
