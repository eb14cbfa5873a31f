"""A recurrent mixer around a gated linear recurrence per channel (the recurrent block of the Griffin models with its
real-gated linear recurrent unit).

    y = gelu_tanh(Wy h + by)                          the gate branch
    u = conv(Wx h + bx) + bc                          a causal convolution over time per channel, `taps` wide, no activation
    per block b of the channels (C / blocks each, a square matrix per block and gate):
        r = sigmoid(Ra_b u_b + ra_b),   i = sigmoid(Ri_b u_b + ri_b)
    a = exp(-decay_scale r softplus(lam))
    S_t = a S_(t-1) + sqrt(1 - a^2) i u,   S = 0 ahead of a sequence's first token
    out = Wo (S y)

Per sequence the cache keeps S (one 32-bit number per channel) and the convolution's last taps - 1 inputs (bias
included); both start at zero.  Gates, decay and state are 32-bit."""
import torch

from .. import ops
from ..cache.needs import CacheNeeds, StateNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    extra = -w.shape[0] % multiple
    return w.contiguous() if extra == 0 else torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous()


@register_mixer("rglru")
class GatedLinearRecurrence:
    def __init__(self, dim: int, width: int, blocks: int, taps: int, dtype: torch.dtype, decay_scale: float = 8.0, position=None):
        if blocks < 1 or width % blocks:
            raise ValueError(f"{width} channels do not divide into {blocks} blocks")
        if taps < 1:
            raise ValueError(f"a convolution of {taps} taps")
        self.dim, self.width, self.blocks, self.taps, self.dtype = dim, int(width), int(blocks), int(taps), dtype
        self.decay_scale = float(decay_scale)
        self.w_in = self.wo = self.conv = self.conv_bias = self.x_bias = self.y_bias = None
        self.gate_a = self.gate_i = self.gate_a_bias = self.gate_i_bias = self.lam = None

    def param_specs(self):
        C, D, B = self.width, self.dim, self.blocks
        bw = C // B
        return {"wy": ParamSpec((C, D)), "wx": ParamSpec((C, D)), "y_bias": ParamSpec((C,), "vector"), "x_bias": ParamSpec((C,), "vector"),
                "conv": ParamSpec((C, self.taps), "vector"), "conv_bias": ParamSpec((C,), "vector"),
                "gate_a": ParamSpec((B, bw, bw)), "gate_i": ParamSpec((B, bw, bw)),
                "gate_a_bias": ParamSpec((B, bw), "vector"), "gate_i_bias": ParamSpec((B, bw), "vector"),
                "lam": ParamSpec((C,), "vector"), "wo": ParamSpec((D, C))}

    def load(self, tensors):
        C = self.width
        self.w_in = _pad_rows(torch.cat([tensors["wy"], tensors["wx"]]))          # columns of the product: y, then x
        self.wo = tensors["wo"]
        self.conv = tensors["conv"]
        vt = self.conv.dtype                                                       # the vectors in one type
        self.conv_bias, self.x_bias = tensors["conv_bias"].to(vt), tensors["x_bias"].to(vt)
        self.y_bias = tensors["y_bias"].to(vt)
        self.gate_a_bias = tensors["gate_a_bias"].to(vt).reshape(C).contiguous()
        self.gate_i_bias = tensors["gate_i_bias"].to(vt).reshape(C).contiguous()
        self.lam = tensors["lam"].to(vt)
        # [block][in][out]: a thread of the gate kernel owns an output and a warp reads consecutive outputs
        self.gate_a = tensors["gate_a"].transpose(1, 2).contiguous()
        self.gate_i = tensors["gate_i"].transpose(1, 2).contiguous()

    def export(self):
        C, B = self.width, self.blocks
        return {"wy": self.w_in[:C], "wx": self.w_in[C:2 * C], "y_bias": self.y_bias, "x_bias": self.x_bias, "conv": self.conv,
                "conv_bias": self.conv_bias, "gate_a": self.gate_a.transpose(1, 2), "gate_i": self.gate_i.transpose(1, 2),
                "gate_a_bias": self.gate_a_bias.view(B, C // B), "gate_i_bias": self.gate_i_bias.view(B, C // B),
                "lam": self.lam, "wo": self.wo}

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateNeed((self.width * self.taps,), torch.float32))   # S, then taps - 1 rows of inputs

    def forward(self, h, batch, view, residual, append: bool = True):
        if not append:
            raise ValueError("a recurrent layer owns its state: it cannot run on another run's cache entry")
        T, C = batch.n_tokens, self.width
        proj = torch.empty(T, self.w_in.shape[0], dtype=self.dtype, device=h.device)
        ops.linear(h, self.w_in, proj)
        u = torch.empty(T, C, dtype=torch.float32, device=h.device)
        ops.short_conv(proj, C, C, self.conv, self.conv_bias, view.state, C, u, batch, act=False, in_bias=self.x_bias)
        out = torch.empty(T, C, dtype=self.dtype, device=h.device)
        ops.rglru(u, self.gate_a, self.gate_i, self.gate_a_bias, self.gate_i_bias, self.lam, self.decay_scale, proj, 0, self.y_bias,
                  view.state, 0, out, batch)
        as_residual(residual).add_linear(out, self.wo)
