"""Parts that act on the residual stream between two layers.

``reentry_mix``: the entry of a pass through a looped stack of layers.  With the stream ``x`` as the layers before
left it and ``x0`` the embedding's output of the same token::

    x <- W_in [x ; x0] + step[t]          (t: the number of the pass, the schedule entry's argument)

``W_in`` is ``[hidden, 2 hidden]`` (the columns of ``x`` first), ``step`` is ``[passes, hidden]``.  What the last
sublayer left pending is added into the stream first.  The two streams are float32; they are rounded to the run type
only as the operand of the matrix product, whose result is float32, and the step vector is added in float32.

Parameters: hidden_size, passes.  Tensors: ``in.weight`` [hidden, 2 hidden], ``step`` [passes, hidden].
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import ParamDecl, StreamPart
from .registry import register_stream


class ReentryMix(StreamPart):
    needs_embedding_output = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.passes = int(spec["passes"])
        if self.hidden < 1 or self.passes < 1:
            raise invalid("reentry_mix: hidden_size and passes must be positive")

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"in.weight": ParamDecl((self.hidden, 2 * self.hidden), fan_in=2 * self.hidden),
                "step": ParamDecl((self.passes, self.hidden), role="vector", init="zeros")}

    def bind(self, tensors, rt) -> None:
        self.w_in = tensors["in.weight"]
        self.step = tensors["step"]
        self.dtype = rt.dtype

    def forward(self, h, pending, ctx, arg):
        t = int(arg)
        if not (0 <= t < self.passes):
            raise invalid(f"reentry_mix: pass {t} of {self.passes}")
        ops.flush_pending(h, pending)
        both = ops.concat_cast(h, ctx.shared["embedding_output"], self.dtype)
        y = ops.linear(both, self.w_in, out_dtype=torch.float32)
        return ops.rows_add_vector(y, self.step[t]), (None, None)


register_stream("reentry_mix", ReentryMix, replace=True)
