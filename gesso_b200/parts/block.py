"""Block arrangements: how a layer's parts and residuals are ordered.

``prenorm`` (src/Inference/Inference.jl:278-363, 3322-3378)::

    h = h + Mixer(Norm_m(h))
    h = h + FeedForward(Norm_f(h))

The residual stream ``h`` is float32 and is updated in place.  A sublayer's output is not
added at once: it travels as ``pending = (delta, bias)`` to the next norm, which adds it into
``h`` and norms the sum in one kernel (the reference fuses the same add+norm on its decode
path, src/Inference/Inference.jl:3239-3247).

``sandwich``: each sublayer's output is normed once more before it is added (see :class:`SandwichBlock`).

``parallel``: a single norm feeds the mixer and the feed-forward alike (see :class:`ParallelBlock`).
"""
from __future__ import annotations

from typing import Dict

from .. import ops
from ..errors import invalid
from .base import ParamDecl
from .registry import (build_feed_forward, build_mixer, build_norm, register_block)


class PreNormBlock:
    def __init__(self, block_spec):
        self.spec = block_spec
        self.mixer = build_mixer(block_spec.mixer)
        self.feed_forward = build_feed_forward(block_spec.feed_forward)
        self.mixer_norm = build_norm(block_spec.mixer_norm)
        self.ff_norm = build_norm(block_spec.ff_norm)

    def parts(self):
        return (("mixer_norm.", self.mixer_norm), ("mixer.", self.mixer),
                ("ff_norm.", self.ff_norm), ("feed_forward.", self.feed_forward))

    def param_decls(self) -> Dict[str, ParamDecl]:
        out = {}
        for prefix, part in self.parts():
            for name, decl in part.param_decls().items():
                out[prefix + name] = decl
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def bind(self, tensors, rt) -> None:
        for prefix, part in self.parts():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, rt)
        # a norm's weight may move into the first matrix of the part it feeds (bfloat16 runs): the
        # norm then only divides by the root mean square, which the consumer's skinny matrix product
        # gathers on the fly
        for norm, consumer in ((self.mixer_norm, self.mixer), (self.ff_norm, self.feed_forward)):
            fold = getattr(norm, "fold_into", None)
            if fold is not None:
                fold(consumer)

    def forward(self, h, pending, ctx, cache):
        """``pending`` is the previous sublayer's (delta, bias) not yet added to ``h`` (or Nones).

        Parts that set ``accepts_lazy_norm`` may be handed a norm that has not run yet; parts that
        set ``fuses_residual`` are given ``residual=h`` and may add their output into it themselves
        (they then return ``(None, None)``)."""
        x = self._norm(self.mixer_norm, self.mixer, h, pending)
        if getattr(self.mixer, "fuses_residual", False):
            m = self.mixer.forward(x, ctx, cache, residual=h)
        else:
            m = self.mixer.forward(x, ctx, cache)
        x = self._norm(self.ff_norm, self.feed_forward, h, m)
        if getattr(self.feed_forward, "fuses_residual", False):
            return self.feed_forward.forward(x, ctx, residual=h)
        return self.feed_forward.forward(x, ctx)

    @staticmethod
    def _norm(norm, consumer, h, pending):
        if getattr(consumer, "accepts_lazy_norm", False) and getattr(norm, "supports_lazy", False):
            return norm.add_norm(h, pending[0], pending[1], lazy=True)
        return norm.add_norm(h, pending[0], pending[1])


class SandwichBlock:
    """Norm before AND after each sublayer::

        h = h + PostNorm_m( Mixer(Norm_m(h)) )
        h = h + PostNorm_f( FeedForward(Norm_f(h)) )        (left out when the layer has no feed-forward)

    A sublayer's output travels on as ``pending = (PostNormed(delta, post norm), None)``: the next pre norm
    norms it, adds it into the float32 stream and norms the sum in one kernel.  The post norms must be of a kind
    that offers ``params()`` (Dynamic Tanh, RMS norm in groups: the fused kernels' forms); the pre norms may be any
    registered norm."""

    def __init__(self, block_spec):
        self.spec = block_spec
        if block_spec.mixer_post_norm is None:
            raise invalid("sandwich block: needs a mixer_post_norm")
        self.mixer = build_mixer(block_spec.mixer)
        self.mixer_norm = build_norm(block_spec.mixer_norm)
        self.mixer_post_norm = build_norm(block_spec.mixer_post_norm)
        self.feed_forward = self.ff_norm = self.ff_post_norm = None
        if block_spec.feed_forward is not None:
            if block_spec.ff_norm is None or block_spec.ff_post_norm is None:
                raise invalid("sandwich block: a feed-forward needs ff_norm and ff_post_norm")
            self.feed_forward = build_feed_forward(block_spec.feed_forward)
            self.ff_norm = build_norm(block_spec.ff_norm)
            self.ff_post_norm = build_norm(block_spec.ff_post_norm)
        for n in (self.mixer_post_norm, self.ff_post_norm):
            if n is not None and not hasattr(n, "params"):
                raise invalid("sandwich block: post norms must be of a kind that fuses with the residual add "
                              "(dyt, group_rmsnorm)")

    def parts(self):
        out = [("mixer_norm.", self.mixer_norm), ("mixer.", self.mixer), ("mixer_post_norm.", self.mixer_post_norm)]
        if self.feed_forward is not None:
            out += [("ff_norm.", self.ff_norm), ("feed_forward.", self.feed_forward),
                    ("ff_post_norm.", self.ff_post_norm)]
        return tuple(out)

    def param_decls(self) -> Dict[str, ParamDecl]:
        out = {}
        for prefix, part in self.parts():
            for name, decl in part.param_decls().items():
                out[prefix + name] = decl
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def bind(self, tensors, rt) -> None:
        for prefix, part in self.parts():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, rt)

    def forward(self, h, pending, ctx, cache):
        x = self.mixer_norm.add_norm(h, pending[0], pending[1])
        d, b = self.mixer.forward(x, ctx, cache)
        pending = (ops.PostNormed(d, self.mixer_post_norm.params(), b), None)
        if self.feed_forward is None:
            return pending
        x = self.ff_norm.add_norm(h, pending[0], None)
        d, b = self.feed_forward.forward(x, ctx)
        return ops.PostNormed(d, self.ff_post_norm.params(), b), None


class ParallelBlock:
    """A single norm per layer feeds the mixer and the feed-forward alike::

        n = Norm(h);   h = h + (Mixer(n) + FeedForward(n))        (the feed-forward may be left out)

    The two outputs travel on together (``ops.SummedDeltas``): the next layer's norm adds both into the float32
    stream in the pass of its own norm.  The feed-forward's output is float32; the mixer's may be of the run type."""

    def __init__(self, block_spec):
        self.spec = block_spec
        self.mixer = build_mixer(block_spec.mixer)
        self.mixer_norm = build_norm(block_spec.mixer_norm)
        self.feed_forward = None if block_spec.feed_forward is None else build_feed_forward(block_spec.feed_forward)

    def parts(self):
        out = [("mixer_norm.", self.mixer_norm), ("mixer.", self.mixer)]
        if self.feed_forward is not None:
            out.append(("feed_forward.", self.feed_forward))
        return tuple(out)

    def param_decls(self) -> Dict[str, ParamDecl]:
        out = {}
        for prefix, part in self.parts():
            for name, decl in part.param_decls().items():
                out[prefix + name] = decl
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def bind(self, tensors, rt) -> None:
        for prefix, part in self.parts():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}, rt)

    def forward(self, h, pending, ctx, cache):
        x = self.mixer_norm.add_norm(h, pending[0], pending[1])
        d, b = self.mixer.forward(x, ctx, cache)
        if self.feed_forward is None:
            return d, b
        f, fb = self.feed_forward.forward(x, ctx)
        if fb is not None:
            raise invalid("parallel block: a feed-forward with an output bias is not supported")
        return ops.SummedDeltas(d, f), b


register_block("parallel", ParallelBlock, replace=True)
register_block("prenorm", PreNormBlock, replace=True)
register_block("sandwich", SandwichBlock, replace=True)
