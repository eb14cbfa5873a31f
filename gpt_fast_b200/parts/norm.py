"""Norms over the 32-bit residual stream.  RMSNorm (gpt-fast model.py:230-241): x * rsqrt(mean(x^2) + eps) * weight;
LayerNorm: (x - mean) / sqrt(variance + eps) * weight + bias.  Statistics and products are 32-bit.  'none' is no norm at
all: the stream in the compute type, for sublayers that read it as it is."""
import torch

from .. import ops
from ..weights.loader import ParamSpec
from . import register_norm
from .residual import Residual


def _owed_rms_branch(x: Residual, rows):
    """The normed branch a stream still owes, as the norm kernel takes it, if one kernel can add it on its way (the
    branch's norm is a root-mean-square norm, no rows are gathered, nothing else is pending); else None."""
    owed = x.normed
    if owed is None or rows is not None or not isinstance(owed[1], RMSNorm) or x.pending is not None or x.scaled:
        return None
    branch, norm, mult = x.take_normed()
    return (branch.value(), norm.weight, None, norm.eps, mult)


@register_norm("rmsnorm")
class RMSNorm:
    """one_plus: the stored weight w lies around zero and the factor is 1 + w (the sum is made once, in 32-bit)."""

    def __init__(self, dim: int, eps: float, dtype: torch.dtype, one_plus: bool = False):
        self.dim, self.eps, self.dtype, self.one_plus = dim, float(eps), dtype, bool(one_plus)
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), "vector")}

    def load(self, tensors):
        self._stored = tensors["weight"]
        self.weight = (self._stored.float() + 1.0).contiguous() if self.one_plus else self._stored

    def export(self):
        return {"weight": self._stored}

    def forward(self, x, out, rows=None):
        """x: the residual stream (a `Residual`, or a complete float32 tensor
        [T, dim]) -> out [R, dim] in the compute dtype; `rows` (int32 [R]) picks
        input rows, else R = T.  Partial sums pending on the stream are added
        by the same kernel, and so is a branch with a root-mean-square norm of its own."""
        if isinstance(x, Residual):
            branch = _owed_rms_branch(x, rows)
            if branch is not None:
                ops.layernorm(x.x, self.weight, None, self.eps, out, None, branch=branch, rms=True)
            else:
                ops.rmsnorm(x.x, self.weight, self.eps, out, rows, x.take_pending())
        else:
            ops.rmsnorm(x, self.weight, self.eps, out, rows)
        return out

    def add_into(self, x32, branch, mult: float) -> None:
        """x32 (float32 [T, dim], complete) += mult * norm(branch)."""
        ops.layernorm(x32, None, None, 0.0, None, None, branch=(branch.value(), self.weight, None, self.eps, mult), rms=True)


@register_norm("none")
class NoNorm:
    """No norm: the stream itself in the compute type, for an arrangement whose sublayers read x and norm their own
    output.  It has no parameters.  A branch that the stream still owes is added by the same kernel."""

    def __init__(self, dim: int, dtype: torch.dtype):
        self.dim, self.dtype = dim, dtype

    def param_specs(self):
        return {}

    def load(self, tensors):
        pass

    def export(self):
        return {}

    def forward(self, x, out, rows=None):
        if isinstance(x, Residual):
            branch = _owed_rms_branch(x, rows)
            if branch is not None:
                ops.layernorm(x.x, None, None, 0.0, out, None, branch=branch, rms=True)
            else:
                ops.layernorm(x.tensor(), None, None, 0.0, out, rows, rms=True)
        else:
            ops.layernorm(x, None, None, 0.0, out, rows, rms=True)
        return out


@register_norm("layernorm")
class LayerNorm:
    """Layer norm with weight and bias: (x - mean) / sqrt(variance + eps) * weight + bias, the variance being the
    mean of the squared deviations, all in 32-bit.  Besides norming the stream it can add a normed branch to it
    (`add_into`: x += mult * norm(y)), which a sandwich block uses behind each sublayer; when the stream still owes
    such a sum as it is normed, one kernel does both."""

    def __init__(self, dim: int, eps: float, dtype: torch.dtype, bias: bool = True):
        self.dim, self.eps, self.dtype, self.has_bias = dim, float(eps), dtype, bool(bias)
        self.weight = self.bias = None

    def param_specs(self):
        specs = {"weight": ParamSpec((self.dim,), "vector")}
        if self.has_bias:
            specs["bias"] = ParamSpec((self.dim,), "vector")
        return specs

    def load(self, tensors):
        self.weight = tensors["weight"]
        if self.has_bias:
            self.bias = tensors["bias"]
            if self.bias.dtype != self.weight.dtype:
                self.bias = self.bias.to(self.weight.dtype)

    def export(self):
        return {"weight": self.weight, "bias": self.bias} if self.has_bias else {"weight": self.weight}

    def _branch_args(self, owed):
        branch, norm, mult = owed
        return (branch.value(), norm.weight, norm.bias, norm.eps, mult)

    def forward(self, x, out, rows=None):
        """x: the residual stream (a `Residual`, or a complete float32 tensor [T, dim]) -> out [R, dim] in the
        compute dtype; `rows` (int32 [R]) picks input rows."""
        if not isinstance(x, Residual):
            ops.layernorm(x, self.weight, self.bias, self.eps, out, rows)
            return out
        owed = x.normed
        if owed is not None and rows is None and isinstance(owed[1], LayerNorm) and x.pending is None:
            x.take_normed()
            ops.layernorm(x.x, self.weight, self.bias, self.eps, out, None, branch=self._branch_args(owed))
        else:
            ops.layernorm(x.tensor(), self.weight, self.bias, self.eps, out, rows)
        return out

    def add_into(self, x32, branch, mult: float) -> None:
        """x32 (float32 [T, dim], complete) += mult * norm(branch)."""
        ops.layernorm(x32, None, None, 0.0, None, None, branch=(branch.value(), self.weight, self.bias, self.eps, mult))

    def forward_with(self, other: "LayerNorm", x: Residual, out, other_out):
        """Two norms of the same rows in one pass: out = self(x), other_out = other(x), from one mean and variance.
        Scaled branches that the stream still owes (`Residual.add_scaled`) are added by the same kernel.  Both norms
        are without bias."""
        if self.has_bias or other.has_bias:
            raise ValueError("two norms of one row in one kernel: only for norms without bias")
        owed = x.take_scaled()
        pending = x.take_pending()
        if pending is not None:
            owed = owed + [(pending, None)]
        if len(owed) > 2:
            x.scaled = owed[2:]
            x.resolve()
            owed = owed[:2]
        ops.layernorm_multi(x.x, [(b if torch.is_tensor(b) else b.value(), s) for b, s in owed],
                            [(self.weight, self.eps, out), (other.weight, other.eps, other_out)])
