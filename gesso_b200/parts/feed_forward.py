"""Dense feed-forwards.

``swiglu``: ``down( silu(gate(x)) * up(x) )``, no biases.

``g = x Wg^T``, ``u = x Wu^T``, ``a = (g / (1 + exp(-g))) * u``, ``d = a Wd^T``
(src/Inference/Inference.jl:869-882, src/Operators/cpu.jl:482-488).  Gate and up are fused
into one matrix at bind time.

``mlp``: ``down( act(up(x)) )`` with one activation between two matrices, no biases; ``activation`` is a parameter
(``gelu_erf``: the exact gelu, ``0.5 z (1 + erf(z / sqrt 2))``; ``xielu``: ``softplus(p) z^2 + z/2`` for ``z > 0`` and
``(1/2 + softplus(q)) (exp(z) - 1 - z) + z/2`` otherwise, with the two learned numbers of the tensor ``act`` [2]).  Its
output is float32.

``glu_clamped``: a gated unit with clamped inputs, ``down( g * sigmoid(1.702 g) * (u + 1) )`` with ``g = min(gate(x),
limit)`` and ``u = clamp(up(x), -limit, limit)``; ``limit`` is a parameter.  Its output is float32.  (The routed
feed-forward uses the same unit for its experts and runs one of these as its shared expert.)
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import FeedForward, ParamDecl
from .registry import register_feed_forward


class SwiGLU(FeedForward):
    accepts_lazy_norm = True
    fuses_residual = True

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["ff_dim"])

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {
            "gate_proj.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
            "up_proj.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
            "down_proj.weight": ParamDecl((self.hidden, self.ff), fan_in=self.ff),
        }

    def bind(self, tensors, rt) -> None:
        g, u = tensors["gate_proj.weight"], tensors["up_proj.weight"]
        common = torch.float32 if (g.dtype == torch.float32 or u.dtype == torch.float32) else g.dtype
        # groups of 8 gate rows followed by their 8 up rows when the width allows it (the layout
        # whose activation the skinny matrix product applies in its epilogue), else gate rows first
        self.packed = self.ff % 8 == 0
        if self.packed:
            self.w_gate_up = ops.pack_gate_up(g.to(common), u.to(common))
        else:
            self.w_gate_up = torch.cat([g.to(common), u.to(common)], dim=0).contiguous()
        self.w_down = tensors["down_proj.weight"]

    def fold_input_scale(self, scale) -> bool:
        self.w_gate_up = ops.fold_norm_weight(self.w_gate_up, scale)
        return True

    def forward(self, x, ctx, residual=None):
        a = ops.linear_swiglu(x, self.w_gate_up, self.packed)
        if residual is not None:
            return ops.linear_residual(a, self.w_down, residual, None), None
        return ops.linear(a, self.w_down, out_dtype=a.dtype), None


class MLP(FeedForward):
    ACTIVATIONS = {"gelu_erf": ops.gelu_erf, "xielu": ops.xielu}
    LEARNED = {"xielu": 2}          # activations with learned numbers: how many the tensor ``act`` holds

    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["ff_dim"])
        self.act = str(spec.get("activation", "gelu_erf"))
        if self.act not in self.ACTIVATIONS:
            raise invalid(f"mlp: unknown activation {self.act!r}; known: {sorted(self.ACTIVATIONS)}")

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {"up.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
             "down.weight": ParamDecl((self.hidden, self.ff), fan_in=self.ff)}
        if self.act in self.LEARNED:
            d["act"] = ParamDecl((self.LEARNED[self.act],), role="vector", init="zeros")
        return d

    def bind(self, tensors, rt) -> None:
        self.w_up, self.w_down = tensors["up.weight"], tensors["down.weight"]
        self.act_params = tensors.get("act")

    def forward(self, x, ctx):
        u = ops.linear(x, self.w_up, out_dtype=x.dtype)
        a = self.ACTIVATIONS[self.act](u, self.act_params) if self.act in self.LEARNED else self.ACTIVATIONS[self.act](u)
        return ops.linear(a, self.w_down, out_dtype=torch.float32), None


class ClampedGLU(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["ff_dim"])
        self.limit = float(spec["limit"])

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"gate.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
                "up.weight": ParamDecl((self.ff, self.hidden), fan_in=self.hidden),
                "down.weight": ParamDecl((self.hidden, self.ff), fan_in=self.ff)}

    def bind(self, tensors, rt) -> None:
        g, u = tensors["gate.weight"], tensors["up.weight"]
        common = torch.float32 if (g.dtype == torch.float32 or u.dtype == torch.float32) else g.dtype
        self.w_gate_up = torch.cat([g.to(common), u.to(common)], dim=0).contiguous()
        self.w_down = tensors["down.weight"]

    def forward(self, x, ctx):
        a = ops.glu_clamped(ops.linear(x, self.w_gate_up, out_dtype=x.dtype), self.limit)
        return ops.linear(a, self.w_down, out_dtype=torch.float32), None


register_feed_forward("swiglu", SwiGLU, replace=True)
register_feed_forward("mlp", MLP, replace=True)
register_feed_forward("glu_clamped", ClampedGLU, replace=True)
