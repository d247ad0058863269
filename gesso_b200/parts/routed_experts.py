"""Routed feed-forward: a mixture of small expert feed-forwards, of which each token uses a few.

Expert e computes ``W_down[e] act(W_up[e] x)`` (no biases; ``act`` is ``relu2`` = the square of relu,
``silu`` or ``gelu_tanh``).  The router scores every expert for every token in float32::

    z = W_router x (+ b_router),   s = sigmoid(z)   (or softmax over the experts, or ``softmax_chosen``: experts are
                                                     chosen by z itself and weighted by the softmax over the chosen
                                                     logits only)
    c = s + correction                 (the score an expert is CHOSEN by; ``correction`` is optional)

Experts form ``n_groups`` equal groups of neighbours; a group's score is the sum of its ``group_top``
largest ``c``; only experts of the ``keep_groups`` best groups can be chosen (the others' ``c`` count as
minus infinity, since choice scores can be negative).  The ``top_k`` largest ``c`` among those are chosen
and the token's output is ``sum_k weight_k * expert_k(x)`` with ``weight_k = s`` of the chosen expert
(divided by their sum with ``renormalize``, times ``weight_scale``).

A gated activation (``glu_clamped``: ``g = min(W_gate x, limit)``, ``u = clamp(W_up x, -limit, limit)``, ``act = g *
sigmoid(1.702 g) * (u + 1)``; ``limit`` is a parameter) takes two matrices per expert, ``experts.<e>.gate.weight``
and ``experts.<e>.up.weight``; they are stacked as one [2 ff, hidden] matrix per expert, in groups of 8 gate rows
and their 8 up rows where ``ff`` is a multiple of 8 (the layout the tensor-core epilogue pairs up), else all gate
rows first.  ``shared`` (a feed-forward part spec, e.g. kind ``glu_clamped``): a shared expert that runs for every
token; the routed sum is added to its output.

Parameters (all from the part spec): hidden_size, ff_dim, n_experts, top_k, n_groups (1), keep_groups
(= n_groups), group_top (2), score ("sigmoid"), correction (false), renormalize (false), weight_scale
(1.0), activation ("relu2"), router_bias (false; tensor ``router.bias`` [E]).  Tensors: ``router.weight`` [E, hidden] (the logits are a product with float32
accumulation and a float32 result, everything after them is float32 whatever the run type), ``correction``
[E], ``experts.<e>.up.weight`` [ff, hidden],
``experts.<e>.down.weight`` [hidden, ff]; the experts' matrices are stacked at bind time.

Which kernels run: bfloat16 steps with more (token, expert) pairs than ``ops.MOE_PAIR_MAX_ROWS`` group the rows by
expert and take the grouped tcgen05 product; fewer pairs, float32 runs and sizes that product does not take
go pair by pair (``ops.moe_experts_pairs``).  The output is float32 (it is normed or added in 32 bit).
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import FeedForward, ParamDecl
from .registry import build_feed_forward, register_feed_forward


class RoutedExperts(FeedForward):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.ff = int(spec["ff_dim"])
        self.E = int(spec["n_experts"])
        self.top = int(spec["top_k"])
        self.n_groups = int(spec.get("n_groups") or 1)
        self.keep_groups = int(spec.get("keep_groups") or self.n_groups)
        self.group_top = int(spec.get("group_top") or 2)
        self.score = str(spec.get("score", "sigmoid"))
        self.has_correction = bool(spec.get("correction", False))
        self.has_router_bias = bool(spec.get("router_bias", False))
        self.renorm = bool(spec.get("renormalize", False))
        self.weight_scale = float(spec.get("weight_scale", 1.0))
        self.act = str(spec.get("activation", "relu2"))
        self.gated = self.act in ops.MOE_GATED_ACTS
        self.limit = float(spec.get("limit") or 0.0)
        self.packed = self.gated and self.ff % 8 == 0
        self.shared = build_feed_forward(spec["shared"]) if spec.get("shared") is not None else None
        if self.gated and self.limit <= 0.0:
            raise invalid("routed experts: the gated activation needs a positive limit")
        if self.E < 1 or not (1 <= self.top <= min(self.E, 32)):
            raise invalid(f"routed experts: top_k {self.top} must be between 1 and min(n_experts, 32)")
        if self.n_groups < 1 or self.E % self.n_groups != 0:
            raise invalid(f"routed experts: {self.E} experts do not form {self.n_groups} equal groups")
        if not (1 <= self.keep_groups <= self.n_groups):
            raise invalid(f"routed experts: keep_groups {self.keep_groups} must be between 1 and n_groups")
        if (self.E // self.n_groups) * self.keep_groups < self.top:
            raise invalid("routed experts: the kept groups hold fewer experts than top_k")
        if self.group_top not in (1, 2):
            raise invalid("routed experts: group_top must be 1 or 2")
        if self.score not in ops.MOE_SCORES:
            raise invalid(f"routed experts: unknown score {self.score!r}; known: {sorted(ops.MOE_SCORES)}")
        if self.act not in ops.MOE_ACTS:
            raise invalid(f"routed experts: unknown activation {self.act!r}; known: {sorted(ops.MOE_ACTS)}")

    def param_decls(self) -> Dict[str, ParamDecl]:
        d = {"router.weight": ParamDecl((self.E, self.hidden), fan_in=self.hidden)}
        if self.has_correction:
            d["correction"] = ParamDecl((self.E,), role="vector", init="zeros")
        if self.has_router_bias:
            d["router.bias"] = ParamDecl((self.E,), role="vector", init="zeros")
        for e in range(self.E):
            if self.gated:
                d[f"experts.{e}.gate.weight"] = ParamDecl((self.ff, self.hidden), fan_in=self.hidden)
            d[f"experts.{e}.up.weight"] = ParamDecl((self.ff, self.hidden), fan_in=self.hidden)
            d[f"experts.{e}.down.weight"] = ParamDecl((self.hidden, self.ff), fan_in=self.ff)
        if self.shared is not None:
            for name, decl in self.shared.param_decls().items():
                d["shared." + name] = decl
        return d

    def bind(self, tensors, rt) -> None:
        self.w_router = tensors["router.weight"]
        self.correction = tensors.get("correction")
        self.router_bias = tensors.get("router.bias")
        ups = [tensors[f"experts.{e}.up.weight"] for e in range(self.E)]
        downs = [tensors[f"experts.{e}.down.weight"] for e in range(self.E)]
        gates = [tensors[f"experts.{e}.gate.weight"] for e in range(self.E)] if self.gated else []
        common = torch.float32 if any(w.dtype == torch.float32 for w in ups + downs + gates) else ups[0].dtype
        if self.gated:       # [E, 2 ff, hidden]: an expert's gate and up rows together
            both = [ops.pack_gate_up(g.to(common), u.to(common)) if self.packed else torch.cat([g.to(common), u.to(common)])
                    for g, u in zip(gates, ups)]
            self.w_up = torch.stack(both).contiguous()
        else:
            self.w_up = torch.stack([w.to(common) for w in ups]).contiguous()    # [E, ff, hidden]
        self.w_down = torch.stack([w.to(common) for w in downs]).contiguous()    # [E, hidden, ff]
        self.rt = rt
        if self.shared is not None:
            self.shared.bind({k[len("shared."):]: v for k, v in tensors.items() if k.startswith("shared.")}, rt)

    def forward(self, x, ctx):
        base = None
        if self.shared is not None:        # runs for every token; the routed sum is added to its float32 output
            base, bias = self.shared.forward(x, ctx)
            if bias is not None or base.dtype != torch.float32:
                raise invalid("routed experts: the shared expert must give a float32 output without a bias")
        idx, w = ops.moe_route(x, self.w_router, self.correction, self.top, self.n_groups, self.keep_groups,
                               self.group_top, self.score, self.renorm, self.weight_scale, self.router_bias)
        if ops.moe_grouped_takes(x, self.w_up, self.w_down, self.top, self.act, self.packed):
            return ops.moe_experts_grouped(x, self.w_up, self.w_down, idx, w, self.act, self.limit, add_to=base), None
        return ops.moe_experts_pairs(x, self.w_up, self.w_down, idx, w, self.act, self.limit, self.packed,
                                     add_to=base), None


register_feed_forward("routed_experts", RoutedExperts, replace=True)
