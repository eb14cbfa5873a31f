"""Mixture of experts as a feed-forward: every token runs `top` of `n_experts` small gated feed-forwards.

    z = W_router h                      router logits, 32-bit
    s = sigmoid(z);  chosen = the `top` experts with the largest s + correction  (the correction counts for the choice only)
    w_e = s_e / (sum of the chosen s + 1e-20) * scale
    expert e:  g = min(W_gate h, limit),  u = clamp(W_up h, -limit, limit),  y = W_down (g * sigmoid(alpha g) * (u + shift))
    result = sum over the chosen e of w_e * y_e

Options: score 'softmax_top' chooses the `top` largest logits themselves (plus the correction, if there is one) and weighs
the chosen experts by the softmax over just their logits (times scale).  `shared_hidden`: one more expert of that size, a
plain SwiGLU that every token runs; with `shared_gate` its output is multiplied by sigmoid(w_s . h), one number per token,
whose row rides behind the router's rows in one product.

The experts have no biases.  Their gate and up rows alternate in one matrix per expert, so one product yields both and
applies the activation before anything is written; the weighted sum of the chosen experts' outputs is added to the
residual stream in 32-bit by the kernel that does the down products (or by the one behind it)."""
import torch

from .. import ops
from ..weights.loader import ParamSpec
from . import register_feed_forward
from .residual import as_residual


def _pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    extra = -w.shape[0] % multiple
    return w.contiguous() if extra == 0 else torch.cat([w, w.new_zeros(extra, w.shape[1])]).contiguous()


@register_feed_forward("moe")
class MixtureOfExperts:
    def __init__(self, dim: int, hidden: int, n_experts: int, top: int, dtype: torch.dtype, router_scale: float = 1.0,
                 limit: float = 0.0, alpha: float = 1.0, shift: float = 0.0, correction: bool = True, score: str = "sigmoid",
                 shared_hidden: int = 0, shared_gate: bool = False):
        if not 1 <= top <= n_experts:
            raise ValueError(f"{top} of {n_experts} experts per token")
        if score not in ("sigmoid", "softmax_top"):
            raise ValueError(f"a router score is 'sigmoid' or 'softmax_top', not {score!r}")
        if shared_gate and not shared_hidden:
            raise ValueError("a gate for a shared expert that is not there")
        self.score, self.shared_hidden, self.shared_gate = score, int(shared_hidden or 0), bool(shared_gate)
        self.shared_w13 = self.shared_w2 = None
        self.dim, self.hidden, self.n_experts, self.top, self.dtype = dim, hidden, int(n_experts), int(top), dtype
        self.router_scale, self.limit, self.alpha, self.shift = float(router_scale), float(limit), float(alpha), float(shift)
        self.has_correction = bool(correction)
        self.router = self.correction = self.w13 = self.w2 = None

    def param_specs(self):
        E, F, D = self.n_experts, self.hidden, self.dim
        specs = {"router": ParamSpec((E, D)), "gate": ParamSpec((E, F, D)), "up": ParamSpec((E, F, D)), "down": ParamSpec((E, D, F))}
        if self.has_correction:
            specs["correction"] = ParamSpec((E,), "vector")
        if self.shared_hidden:
            Fs = self.shared_hidden
            specs.update(shared_gate=ParamSpec((Fs, D)), shared_up=ParamSpec((Fs, D)), shared_down=ParamSpec((D, Fs)))
            if self.shared_gate:
                specs["shared_sg"] = ParamSpec((1, D))
        return specs

    def load(self, tensors):
        E, F, D = self.n_experts, self.hidden, self.dim
        self._router_stored = tensors["router"]
        self.router = _pad_rows(torch.cat([tensors["router"], tensors["shared_sg"]]) if self.shared_gate else tensors["router"])
        if self.shared_hidden:
            self.shared_w13 = torch.stack([tensors["shared_gate"], tensors["shared_up"]], dim=1).reshape(2 * self.shared_hidden, D).contiguous()
            self.shared_w2 = tensors["shared_down"]
        self.correction = tensors["correction"] if self.has_correction else torch.zeros(E, dtype=torch.float32, device=tensors["router"].device)
        # rows alternate gate, up within every expert
        self.w13 = torch.stack([tensors["gate"], tensors["up"]], dim=2).reshape(E, 2 * F, D).contiguous()
        self.w2 = tensors["down"]

    def export(self):
        w = self.w13.view(self.n_experts, self.hidden, 2, self.dim)
        out = {"router": self._router_stored, "gate": w[:, :, 0], "up": w[:, :, 1], "down": self.w2}
        if self.has_correction:
            out["correction"] = self.correction
        if self.shared_hidden:
            sw = self.shared_w13.view(self.shared_hidden, 2, self.dim)
            out.update(shared_gate=sw[:, 0], shared_up=sw[:, 1], shared_down=self.shared_w2)
            if self.shared_gate:
                out["shared_sg"] = self.router[self.n_experts:self.n_experts + 1]
        return out

    def forward(self, h, residual):
        T = h.shape[0]
        idx = torch.empty(T, self.top, dtype=torch.int32, device=h.device)
        w = torch.empty(T, self.top, dtype=torch.float32, device=h.device)
        if self.score == "sigmoid" and not self.shared_gate:
            gate = ops.moe_router(h, self.router, self.correction, self.top, self.router_scale, idx, w)
        else:
            gate = ops.moe_router(h, self.router, self.correction, self.top, self.router_scale, idx, w, score=self.score,
                                  n_extra=1 if self.shared_gate else 0)
        residual = as_residual(residual)
        x = residual.tensor()                                  # complete: the experts' kernel adds into it
        ops.moe_experts(h, idx, w, self.w13, self.w2, x, self.limit, self.alpha, self.shift)
        if self.shared_hidden:
            act = torch.empty(T, self.shared_hidden, dtype=self.dtype, device=h.device)
            ops.linear(h, self.shared_w13, act, mode="swiglu")
            if self.shared_gate:
                # a factor per token commutes with the down product: it goes onto the activations
                ops.sigmoid_gate(act, gate[0], gate[1], self.shared_hidden)
            residual.add_linear(act, self.shared_w2)
