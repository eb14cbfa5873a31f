"""Arrangements of a layer's parts.  'prenorm' is gpt-fast's TransformerBlock
(model.py:153-164): x += mixer(norm(x)); x += feed_forward(norm(x)), with the
residual stream x kept in 32-bit.  'sandwich' norms a sublayer's output as well
and scales it before the sum; its feed-forward is optional.  'parallel' runs mixer and
feed-forward side by side on two norms of the same x.

An arrangement declares `roles`: the names of the parts it is made of, each with
the kind of part that fills it ('mixer', 'feed_forward', 'norm': the registries of
`parts`).  The model builds one part per role from the layer's `LayerSpec.parts`
and hands them over as a dict; mixers also receive the layer's position encoding."""
import torch

from ..weights.loader import ParamSpec
from . import register_block
from .residual import Branch, as_residual


@register_block("prenorm")
class PreNormBlock:
    roles = {"mixer": "mixer", "feed_forward": "feed_forward", "mixer_norm": "norm", "ffn_norm": "norm"}

    def __init__(self, parts: dict, dim: int, dtype: torch.dtype):
        self.mixer, self.feed_forward = parts["mixer"], parts["feed_forward"]
        self.mixer_norm, self.ffn_norm = parts["mixer_norm"], parts["ffn_norm"]
        self.dim, self.dtype = dim, dtype

    def parts(self):
        return {"mixer": self.mixer, "feed_forward": self.feed_forward,
                "mixer_norm": self.mixer_norm, "ffn_norm": self.ffn_norm}

    def cache_needs(self):
        """What one run of this layer keeps per sequence (its mixer's keys/values or state)."""
        return self.mixer.cache_needs()

    def forward(self, x, batch, view, append: bool = True):
        """x: the residual stream (`parts.residual.Residual`), updated in place."""
        x = as_residual(x)
        h = torch.empty(x.x.shape[0], self.dim, dtype=self.dtype, device=x.x.device)
        self.mixer_norm.forward(x, h)
        self.mixer.forward(h, batch, view, residual=x, append=append)
        self.ffn_norm.forward(x, h)
        self.feed_forward.forward(h, residual=x)


@register_block("sandwich")
class SandwichBlock:
    """Norms on both sides of every sublayer and a constant factor on the branch:

        x += mult * post_norm(mixer(pre_norm(x)));   x += mult * post_norm(feed_forward(pre_norm(x)))

    The feed-forward (with its two norms) is optional: a layer without one has only the first sublayer.  A
    sublayer writes into a `Branch` (32-bit); the normed sum is left to the stream, whose next norm does it on
    the way (`Residual.add_normed`)."""
    roles = {"mixer": "mixer", "mixer_norm": "norm", "mixer_post_norm": "norm",
             "feed_forward": "feed_forward", "ffn_norm": "norm", "ffn_post_norm": "norm"}
    optional_roles = ("feed_forward", "ffn_norm", "ffn_post_norm")

    def __init__(self, parts: dict, dim: int, dtype: torch.dtype, residual_mult: float = 1.0):
        self._parts = dict(parts)
        ffn = [r for r in self.optional_roles if r in parts]
        if ffn and len(ffn) != len(self.optional_roles):
            raise ValueError(f"a sandwich block has a feed-forward with both of its norms or none of the three; got {ffn}")
        self.mixer, self.mixer_norm, self.mixer_post_norm = parts["mixer"], parts["mixer_norm"], parts["mixer_post_norm"]
        self.feed_forward = parts.get("feed_forward")
        self.ffn_norm, self.ffn_post_norm = parts.get("ffn_norm"), parts.get("ffn_post_norm")
        self.dim, self.dtype, self.mult = dim, dtype, float(residual_mult)

    def parts(self):
        return dict(self._parts)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def forward(self, x, batch, view, append: bool = True):
        x = as_residual(x)
        T, dev = x.x.shape[0], x.x.device
        h = torch.empty(T, self.dim, dtype=self.dtype, device=dev)
        self.mixer_norm.forward(x, h)
        y = Branch(T, self.dim, dev)
        self.mixer.forward(h, batch, view, residual=y, append=append)
        x.add_normed(y, self.mixer_post_norm, self.mult)
        if self.feed_forward is not None:
            self.ffn_norm.forward(x, h)
            y = Branch(T, self.dim, dev)
            self.feed_forward.forward(h, residual=y)
            x.add_normed(y, self.ffn_post_norm, self.mult)


class LayerScale:
    """A learned factor per column on a sublayer's output."""

    def __init__(self, dim: int):
        self.dim = dim
        self.weight = None

    def param_specs(self):
        return {"weight": ParamSpec((self.dim,), "vector")}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def export(self):
        return {"weight": self.weight}


@register_block("parallel")
class ParallelBlock:
    """Mixer and feed-forward read two norms of the SAME x and their results are added together:

        x += s1 * mixer(norm1(x)) + s2 * feed_forward(norm2(x))

    s1, s2: learned per-column factors (`layer_scale`; without it they are 1).  The feed-forward with its norm is
    optional.  The two norms share mean and variance and differ in their weights, so one kernel writes both normed
    rows; the two scaled sums are left to the stream and done by the next layer's norm kernel on its way
    (`Residual.add_scaled`).  The norms are layer norms without bias.

    A feed-forward WITHOUT a norm of its own reads the mixer's norm: x += mixer(h) + feed_forward(h), h = norm1(x); the
    norm may then be of any kind.  Without layer scale both sublayers add straight into the stream."""
    roles = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "ffn_norm": "norm"}
    optional_roles = ("feed_forward", "ffn_norm")

    def __init__(self, parts: dict, dim: int, dtype: torch.dtype, layer_scale: bool = False):
        if "ffn_norm" in parts and "feed_forward" not in parts:
            raise ValueError("a parallel block has no norm for a feed-forward it lacks")
        self._parts = dict(parts)
        self.mixer, self.mixer_norm = parts["mixer"], parts["mixer_norm"]
        self.feed_forward, self.ffn_norm = parts.get("feed_forward"), parts.get("ffn_norm")
        self.dim, self.dtype = dim, dtype
        self.mixer_scale = self.ffn_scale = None
        if layer_scale:
            self.mixer_scale = self._parts["mixer_scale"] = LayerScale(dim)
            if self.feed_forward is not None:
                self.ffn_scale = self._parts["ffn_scale"] = LayerScale(dim)

    def parts(self):
        return dict(self._parts)

    def cache_needs(self):
        return self.mixer.cache_needs()

    def forward(self, x, batch, view, append: bool = True):
        x = as_residual(x)
        T, dev = x.x.shape[0], x.x.device
        h1 = torch.empty(T, self.dim, dtype=self.dtype, device=dev)
        if self.ffn_norm is None:                              # one norm, read by both sublayers
            self.mixer_norm.forward(x, h1)
            if self.mixer_scale is None:
                self.mixer.forward(h1, batch, view, residual=x, append=append)
                if self.feed_forward is not None:
                    self.feed_forward.forward(h1, residual=x)
                return
            h2 = h1
        elif self.feed_forward is not None:
            h2 = torch.empty(T, self.dim, dtype=self.dtype, device=dev)
            self.mixer_norm.forward_with(self.ffn_norm, x, h1, h2)
        else:
            self.mixer_norm.forward(x, h1)
        y1 = Branch(T, self.dim, dev)
        self.mixer.forward(h1, batch, view, residual=y1, append=append)
        x.add_scaled(y1, None if self.mixer_scale is None else self.mixer_scale.weight)
        if self.feed_forward is not None:
            y2 = Branch(T, self.dim, dev)
            self.feed_forward.forward(h2, residual=y2)
            x.add_scaled(y2, None if self.ffn_scale is None else self.ffn_scale.weight)
