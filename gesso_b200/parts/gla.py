"""Gated linear attention: linear attention whose decay is computed from the input, one number per key channel and
token, as a recurrence over a per-request state.

With the mixer's input ``x``, per head h (``head_dim`` key features, ``v_head_dim`` value features)::

    q_t = W_q x_t * head_dim^(-1/2),   k_t = W_k x_t,   v_t = W_v x_t
    a_t = sigmoid(W_a2 (W_a1 x_t) + b_a2) ** (1 / tau)          (a low-rank projection; 0 < a_t < 1 per key channel)
    S_t = diag(a_t) S_{t-1} + k_t v_t^T                         (S_0 = 0; the decay scales the rows of the key channels)
    o_t = S_t^T q_t

Each head's ``o_t`` is normed by itself over its value features with one weight vector that all heads share, the heads
are put side by side, multiplied by ``silu(W_g x_t)`` and projected::

    y_t[h] = o_t[h] / sqrt(mean(o_t[h]^2) + eps) * w,      out_t = W_o (y_t * silu(W_g x_t))

The state S (``n_heads x v_head_dim x head_dim`` float32 numbers per request and layer, a value column's key
features contiguous) is all a request keeps.  The decay's logits from the second low-rank product on, the decay,
the state, the outer product, the read-out and the norm are float32 whatever the run type; q, k, v and the gate are one
fused matrix product.

Parameters: hidden_size, n_heads, head_dim, v_head_dim, decay_rank (the size random weights are drawn with; a
checkpoint's matrices decide), tau, norm_eps.  Tensors: ``q_proj.weight``,
``k_proj.weight`` [H * head_dim, hidden], ``v_proj.weight``, ``g_proj.weight`` [H * v_head_dim, hidden],
``a1.weight`` [decay_rank, hidden], ``a2.weight`` [H * head_dim, decay_rank], ``a2.bias`` [H * head_dim],
``norm.weight`` [v_head_dim], ``o_proj.weight`` [hidden, H * v_head_dim].
"""
from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, ParamDecl, StateNeed
from .registry import register_mixer


class GatedLinearAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["n_heads"])
        self.hd = int(spec["head_dim"])
        self.vd = int(spec.get("v_head_dim") or self.hd)
        self.rank = int(spec["decay_rank"])
        self.tau = float(spec["tau"])
        self.eps = float(spec["norm_eps"])
        if min(self.nh, self.hd, self.vd, self.rank) < 1:
            raise invalid("gated linear attention: sizes must be positive")
        if not self.tau > 0.0:
            raise invalid(f"gated linear attention: tau {self.tau} must be positive")
        if self.hd > 512:
            raise invalid(f"gated linear attention: head_dim {self.hd} is above 512, the most the recurrence kernel takes")
        self.q_scale = float(self.hd) ** -0.5

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, D, Dv, W, R = self.nh, self.hd, self.vd, self.hidden, self.rank
        return {
            "q_proj.weight": ParamDecl((H * D, W), fan_in=W),
            "k_proj.weight": ParamDecl((H * D, W), fan_in=W),
            "v_proj.weight": ParamDecl((H * Dv, W), fan_in=W),
            "g_proj.weight": ParamDecl((H * Dv, W), fan_in=W),
            # the rank of the decay's projection is the checkpoint's own
            "a1.weight": ParamDecl((R, W), fan_in=W, free_axes=(0,)),
            "a2.weight": ParamDecl((H * D, R), fan_in=R, free_axes=(1,)),
            "a2.bias": ParamDecl((H * D,), role="vector", init="zeros"),
            "norm.weight": ParamDecl((Dv,), role="vector", init="ones"),
            "o_proj.weight": ParamDecl((W, H * Dv), fan_in=H * Dv),
        }

    def cache_need(self):
        return StateNeed((self.nh, self.vd, self.hd), "float32")       # a value column's key features are contiguous

    def bind(self, tensors, rt) -> None:
        ws = [tensors[n + "_proj.weight"] for n in ("q", "k", "v", "g")] + [tensors["a1.weight"]]
        self.rank = int(tensors["a1.weight"].shape[0])
        if tensors["a2.weight"].shape[1] != self.rank:
            raise invalid("gated linear attention: the two matrices of the decay's projection have different ranks")
        common = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        # one product for q, k, v, the gate and the decay's inner projection (its columns come last)
        self.w_in = torch.cat([w.to(common) for w in ws], dim=0).contiguous()
        self.w_a2 = tensors["a2.weight"]
        self.b_a2 = tensors["a2.bias"]
        self.w_norm = tensors["norm.weight"]
        self.w_o = tensors["o_proj.weight"]

    def forward(self, x, ctx, cache):
        H, D, Dv = self.nh, self.hd, self.vd
        proj = ops.linear(x, self.w_in, out_dtype=x.dtype)
        g0 = 2 * H * D + H * Dv
        a0 = g0 + H * Dv
        inner = proj[:, a0:a0 + self.rank].contiguous()
        z = ops.linear(inner, self.w_a2, out_dtype=torch.float32)          # the decay's logits, float32 from here on
        # long prompt portions: the step's 64-token tiles side by side instead of token after token
        tiles = (ctx.tile_seg, ctx.tile_q0) if not ctx.decode_only and ops.gla_chunked_takes(ctx.max_seg_len) else (None, None)
        o = ops.gated_linear_attention(proj, z, self.b_a2, self.tau, self.q_scale, cache.state, ctx.seg_start,
                                       cache.slots, ctx.n_segs, H, D, Dv, *tiles)
        y = ops.head_gated_rmsnorm(o, self.w_norm, self.eps, proj[:, g0:g0 + H * Dv], H, x.dtype, gate_act="silu")
        return ops.linear(y, self.w_o, out_dtype=torch.float32), None


register_mixer("gated_linear_attention", GatedLinearAttention, replace=True)
