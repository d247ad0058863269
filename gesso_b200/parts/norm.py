"""Norms with the residual add folded in: RMSNorm, Dynamic Tanh, RMS norm in groups.

``y = (x / sqrt(mean(x^2) + eps)) * w`` over the last axis, divide first, scale
second (src/Operators/cpu.jl:293-311).  The residual stream is float32; the sum
and the statistics are float32, the output is rounded to the run dtype.

With the parameter ``unit_offset`` the weight tensor holds the scale's offset from one, ``scale = 1 + w`` (formed once, in
float32, when the weights are bound).  A pending :class:`~gesso_b200.ops.SummedDeltas` (two sublayers' outputs
that are added together) is added in the same pass.

With ``lazy=True`` and nothing to add, the norm is not run: a
:class:`~gesso_b200.ops.LazyNorm` is returned, which the consumer's first matrix
product applies in its prologue for steps of few tokens (or materialises).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Norm, ParamDecl
from .registry import register_norm


class RMSNorm(Norm):
    supports_lazy = True

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.unit_offset = bool(spec.get("unit_offset", False))
        self.weight = None
        self.out_dtype = None
        self.folded = False      # True once the consumer's matrix carries this norm's weight

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.size,), role="vector", init="zeros" if self.unit_offset else "ones")}

    def bind(self, tensors, rt) -> None:
        self.weight = tensors["weight"]
        if self.unit_offset:
            self.weight = (self.weight.float() + 1.0).contiguous()
        self.out_dtype = rt.dtype

    def fold_into(self, consumer) -> bool:
        """Let ``consumer`` (a part with ``fold_input_scale``) absorb the weight into its first matrix.
        Only in bfloat16 runs: the 32-bit path keeps the reference's order of operations."""
        if self.folded or self.out_dtype != torch.bfloat16:
            return self.folded
        fold = getattr(consumer, "fold_input_scale", None)
        if fold is not None and fold(self.weight):
            self.folded = True
        return self.folded

    def add_norm(self, h, delta, delta_bias, rows=None, lazy=False):
        if isinstance(delta, ops.PostNormed):      # a sublayer's output that is normed before the add
            if rows is not None:
                raise NotImplementedError("rmsnorm: a post-normed delta cannot be added for a row list")
            delta.add_into(h)
            delta = None
        delta2 = None
        if isinstance(delta, ops.SummedDeltas):    # two sublayers' outputs, added in this pass
            delta, delta2 = delta.first, delta.second
        weight = None if self.folded else self.weight
        if lazy and delta is None and rows is None:
            return ops.LazyNorm(h, weight, self.eps, self.out_dtype)
        return ops.add_rmsnorm(h, delta, delta_bias, weight, self.eps, self.out_dtype, rows, delta2=delta2)


class DynamicTanh(Norm):
    """Dynamic Tanh: ``y = tanh(alpha * x) * weight + bias`` with a learned scalar ``alpha``; no mean, no
    variance, no eps.  Parameters: ``size``, ``bias`` (default true).  Tensors: ``weight`` [size], ``bias``
    [size], ``alpha`` [] (read once at bind time).

    ``add_norm`` adds the pending delta into the float32 stream and norms the sum in one kernel; a pending
    :class:`~gesso_b200.ops.PostNormed` (a sublayer's output that is itself normed before the add) is handled
    in the same pass.  ``params()`` hands the norm to such a caller."""

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec["size"])
        self.has_bias = bool(spec.get("bias", True))
        self.p = None
        self.out_dtype = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {"weight": ParamDecl((self.size,), role="vector", init="ones"),
             "alpha": ParamDecl((), role="vector", init="ones", alt_shapes=((1,),))}
        if self.has_bias:
            d["bias"] = ParamDecl((self.size,), role="vector", init="zeros")
        return d

    def bind(self, tensors, rt) -> None:
        self.p = ops.DytParams(float(tensors["alpha"].reshape(-1)[0].item()), tensors["weight"], tensors.get("bias"))
        self.out_dtype = rt.dtype

    def params(self) -> "ops.DytParams":
        return self.p

    def add_norm(self, h, delta, delta_bias, rows=None):
        post = None
        if isinstance(delta, ops.PostNormed):
            delta, post, delta_bias = delta.delta, delta.post, delta.bias
        return ops.add_dyt(h, delta, delta_bias, post, self.p, self.out_dtype, rows)


class GroupRMSNorm(Norm):
    """RMS norm in groups: a row is cut into ``groups`` equal consecutive parts; each part is divided by its own
    ``sqrt(mean(part^2) + eps)``, then the whole row is multiplied by ``weight``.  Parameters: ``size``, ``eps``,
    ``groups`` (default 1: the ordinary RMS norm).  Tensor: ``weight`` [size].

    ``add_norm`` adds the pending delta into the float32 stream and norms the sum in one kernel; a pending
    :class:`~gesso_b200.ops.PostNormed` whose own norm is of this kind (with the same eps and groups) is normed and
    added in the same pass.  ``params()`` hands the norm to such a caller.  Statistics, sums and the scaling are
    float32; only the result is rounded to the run type."""

    def __init__(self, spec):
        super().__init__(spec)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.groups = int(spec.get("groups") or 1)
        if self.groups < 1 or self.size % self.groups != 0:
            raise invalid(f"group_rmsnorm: {self.size} features do not form {self.groups} equal groups")
        self.p = None
        self.out_dtype = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        return {"weight": ParamDecl((self.size,), role="vector", init="ones")}

    def bind(self, tensors, rt) -> None:
        self.p = ops.GroupRmsParams(tensors["weight"], self.eps, self.groups)
        self.out_dtype = rt.dtype

    def params(self) -> "ops.GroupRmsParams":
        return self.p

    def add_norm(self, h, delta, delta_bias, rows=None):
        post = None
        if isinstance(delta, ops.PostNormed):
            fits = isinstance(delta.post, ops.GroupRmsParams) and \
                (delta.post.eps, delta.post.groups) == (self.eps, self.groups)
            if fits:
                delta, post, delta_bias = delta.delta, delta.post, delta.bias
            elif rows is None:
                delta.add_into(h)
                delta = None
            else:
                raise NotImplementedError("group_rmsnorm: a delta with another kind of post norm cannot be added for a row list")
        elif isinstance(delta, ops.SummedDeltas):
            if rows is not None:
                raise NotImplementedError("group_rmsnorm: two summed deltas cannot be added for a row list")
            ops.flush_pending(h, (delta, delta_bias))
            delta = delta_bias = None
        return ops.add_group_rmsnorm(h, delta, delta_bias, post, self.p, self.out_dtype, rows)


register_norm("group_rmsnorm", GroupRMSNorm, replace=True)
register_norm("rmsnorm", RMSNorm, replace=True)
register_norm("dyt", DynamicTanh, replace=True)
