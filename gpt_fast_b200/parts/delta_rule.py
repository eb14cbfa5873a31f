"""The gated delta rule with a decay per head and key channel.

    q = Wq h, k = Wk h (qk_heads x head_dim), v = Wv h (heads x v_head_dim); each passes a causal convolution over time
    per channel (`taps` wide, no bias) and SiLU; q and k are then made unit vectors per head (x / sqrt(sum x^2 + 1e-6)),
    q also times head_dim^-1/2
    beta = sigmoid(Wb h)                                         one per head
    g = exp(-exp(A_log_h) softplus(Wa2 (Wa1 h) + dt_bias))       heads x head_dim: one decay per row of S
    S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q          per head, S [head_dim, v_head_dim]
    y = Wo concat_h (o / rms(o) * norm * sigmoid(Wg2 (Wg1 h)))                  rms over v_head_dim, eps inside the root

Head h reads query/key head h // (heads / qk_heads); the read-out sees the current token's write.  Per sequence the
cache keeps S (32-bit) and the convolutions' last taps - 1 inputs; both start at zero.

Variants: decay_rank = 0 with head_decay: one decay per head and token from one projection, g = exp(-exp(A_log_h)
softplus(Wa h + dt_bias_h)), Wa [heads, dim]; gate_rank = 0: the gate is one projection Wg [heads * v_head_dim, dim];
gate_act 'silu' or 'sigmoid' names the gate's function."""
import torch

from .. import ops
from ..cache.needs import CacheNeeds, StateNeed
from ..weights.loader import ParamSpec
from . import register_mixer
from .residual import as_residual
from .state_space import _pad_rows


@register_mixer("delta_rule")
class DeltaRule:
    def __init__(self, dim: int, n_head: int, n_qk: int, head_dim: int, v_head_dim: int, taps: int, decay_rank: int, gate_rank: int,
                 eps: float, dtype: torch.dtype, position=None, head_decay: bool = False, gate_act: str = "sigmoid"):
        if n_head % n_qk:
            raise ValueError(f"{n_head} heads do not divide into {n_qk} query/key heads")
        if bool(decay_rank) != bool(gate_rank):
            raise ValueError("decay and gate are both low-rank products or both single projections")
        if head_decay and decay_rank:
            raise ValueError("one decay per head comes from a single projection (decay_rank = 0)")
        if gate_act not in ("sigmoid", "silu"):
            raise ValueError(f"unknown gate function {gate_act!r}")
        self.head_decay, self.gate_act = bool(head_decay), gate_act
        self.decays = n_head if head_decay else n_head * head_dim           # decay inputs per token
        self.dim, self.n_head, self.n_qk, self.head_dim, self.v_head_dim = dim, n_head, n_qk, head_dim, v_head_dim
        self.taps, self.decay_rank, self.gate_rank, self.eps, self.dtype = int(taps), decay_rank, gate_rank, float(eps), dtype
        self.conv_channels = 2 * n_qk * head_dim + n_head * v_head_dim
        self.state_floats = n_head * head_dim * v_head_dim
        self.w_in = self.w_low = self.w_up = self.wo = self.conv = self.dt_bias = self.a_log = self.norm = None

    def param_specs(self):
        H, J, d, dv, D = self.n_head, self.n_qk, self.head_dim, self.v_head_dim, self.dim
        if self.decay_rank:
            low = {"wa1": ParamSpec((self.decay_rank, D)), "wa2": ParamSpec((self.decays, self.decay_rank)),
                   "wg1": ParamSpec((self.gate_rank, D)), "wg2": ParamSpec((H * dv, self.gate_rank))}
        else:
            low = {"wa": ParamSpec((self.decays, D)), "wg": ParamSpec((H * dv, D))}
        return {"wq": ParamSpec((J * d, D)), "wk": ParamSpec((J * d, D)), "wv": ParamSpec((H * dv, D)), "wb": ParamSpec((H, D)), **low,
                "q_conv": ParamSpec((J * d, self.taps), "vector"), "k_conv": ParamSpec((J * d, self.taps), "vector"),
                "v_conv": ParamSpec((H * dv, self.taps), "vector"), "dt_bias": ParamSpec((self.decays,), "vector"),
                "a_log": ParamSpec((H,), "vector"), "norm": ParamSpec((dv,), "vector"), "wo": ParamSpec((D, H * dv))}

    def load(self, tensors):
        t = tensors
        mats = ("wa1", "wa2", "wg1", "wg2") if self.decay_rank else ("wa", "wg")
        self._stored = {k: t[k] for k in ("wq", "wk", "wv", "wb", "q_conv", "k_conv", "v_conv") + mats}
        # one product for q, k, v and beta; one for the two low-rank inputs; one block-diagonal product for their outputs
        self.w_in = _pad_rows(torch.cat([t["wq"], t["wk"], t["wv"], t["wb"]]))
        if self.decay_rank:
            self.w_low = _pad_rows(torch.cat([t["wa1"], t["wg1"]]))
            ra, rg = self.decay_rank, self.gate_rank
            up = t["wa2"].new_zeros(t["wa2"].shape[0] + t["wg2"].shape[0], self.w_low.shape[0])
            up[:t["wa2"].shape[0], :ra] = t["wa2"]
            up[t["wa2"].shape[0]:, ra:ra + rg] = t["wg2"]
            self.w_up = _pad_rows(up)
        else:
            self.w_low, self.w_up = None, _pad_rows(torch.cat([t["wa"], t["wg"]]))      # decay inputs, then gate inputs, from h
        self.conv = torch.cat([t["q_conv"], t["k_conv"].to(t["q_conv"].dtype), t["v_conv"].to(t["q_conv"].dtype)]).contiguous()
        self.dt_bias, self.a_log, self.norm, self.wo = t["dt_bias"], t["a_log"].to(t["dt_bias"].dtype), t["norm"], t["wo"]

    def export(self):
        return dict(self._stored, dt_bias=self.dt_bias, a_log=self.a_log, norm=self.norm, wo=self.wo)

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateNeed((self.state_floats + (self.taps - 1) * self.conv_channels,), torch.float32))

    def forward(self, h, batch, view, residual, append: bool = True):
        if not append:
            raise ValueError("a delta-rule layer owns its state: it cannot run on another run's cache entry")
        T = batch.n_tokens
        H, J, d, dv = self.n_head, self.n_qk, self.head_dim, self.v_head_dim
        C = self.conv_channels
        proj = torch.empty(T, self.w_in.shape[0], dtype=self.dtype, device=h.device)
        ops.linear(h, self.w_in, proj)
        low = h
        if self.w_low is not None:
            low = torch.empty(T, self.w_low.shape[0], dtype=self.dtype, device=h.device)
            ops.linear(h, self.w_low, low)
        ag = torch.empty(T, self.w_up.shape[0], dtype=torch.float32, device=h.device)      # decay inputs, then gate inputs
        ops.linear(low, self.w_up, ag)
        qkv = torch.empty(T, C, dtype=torch.float32, device=h.device)
        ops.short_conv(proj, 0, C, self.conv, None, view.state, self.state_floats, qkv, batch)
        o = torch.empty(T, H, dv, dtype=torch.float32, device=h.device)
        kw = {"head_decay": True} if self.head_decay else {}
        ops.delta_rule(qkv, (0, J * d, 2 * J * d), proj, C, ag, 0, self.dt_bias, self.a_log, view.state, 0, o, batch, H, J, d, dv,
                       q_scale=float(d) ** -0.5, **kw)
        y = torch.empty(T, H * dv, dtype=self.dtype, device=h.device)
        ops.gated_norm(o.view(T, H * dv), ag, self.decays, self.norm, y, dv, self.eps, act=self.gate_act, gate_first=False)
        as_residual(residual).add_linear(y, self.wo)
