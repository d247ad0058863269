"""Grouped-query attention whose weights are sigmoids of the scores: no softmax, nothing is normalized over the keys.

With the mixer's input ``x``, ``n_heads`` query heads and ``n_kv_heads`` key/value heads (query head h reads kv head
``h // (n_heads / n_kv_heads)``), keys and queries of ``head_dim`` features and values of ``v_head_dim``::

    q = W_q x (+ b_q),  k = W_k x (+ b_k),  v = W_v x (+ b_v)
    q, k <- per head: divided by the root mean square over the head's features, times a weight [head_dim] that all
            heads share (``qk_norm_eps``; ``None``: no norm)
    score(i, j) = (q_i . k_j) * scale * temp(i) + bias[h, i - j]        for every j <= i (causal; no rotation)
    weight(i, j) = sigmoid(score(i, j))
    o_i[h] = ( sum_j weight(i, j) v_j ) * sigmoid(W_g x_i)[h]           (``head_gate``: one number per head)
    out_i = W_o concat_h(o_i[h]) (+ b_o)

``temp(i) = 1 + coef * ln(floor((i + 1) / every) + 1)`` is a temperature on the queries that grows with the position
(``q_temperature``: ``{"coef", "every"}``; ``None``: 1).  ``bias[h, n]`` (``distance_bias``) is a learned number per
head and distance: a table ``rel_bias`` [rows, n_heads] whose first ``rows // 2`` rows are the distances 0, 1, 2, ...
themselves, while further distances share rows that widen like a logarithm up to ``max_distance``::

    row(n) = n                                                                          for n < rows // 2
    row(n) = min(rows - 1, rows//2 + floor( ln(n / (rows//2)) / ln(max_distance / (rows//2)) * (rows - rows//2) ))

plus one number per head, ``head_bias`` [n_heads].  ``scale`` does not multiply the bias.  The number of rows is the
checkpoint table's own (``distance_bias["rows"]`` is the size random weights are drawn with).  At bind time the table
and the per-head number are laid out by distance, ``[n_heads, ceil(max_distance) + 1]`` float32 (every further
distance reads the last column), which is what the kernels take.

The cache holds the normed keys and the raw values in pages.  Scores, weights and the sums over the keys are float32
in every run type (the tensor-core kernels feed each weight to the product as two bfloat16 pieces); the projections,
and the cached keys and values, have the run type.  The output projection's result is float32.

Parameters: hidden_size, n_heads, n_kv_heads, head_dim, v_head_dim, scale, qk_norm_eps, qkv_bias, o_bias, head_gate,
q_temperature, distance_bias (``{"rows", "max_distance"}`` or ``None``), window (``None``: every earlier key).
Tensors: ``q_proj.weight`` ..., ``q_proj.bias`` ..., ``q_norm.weight``, ``k_norm.weight`` [head_dim], ``rel_bias`` [rows,
n_heads], ``head_bias`` [n_heads], ``g_proj.weight`` [n_heads, hidden], ``o_proj.weight``, ``o_proj.bias``.
"""
from __future__ import annotations

import math
from typing import Dict

import torch

from .. import ops
from ..errors import invalid
from .base import Mixer, PagedNeed, ParamDecl
from .registry import register_mixer


def distance_rows(n_max: int, rows: int, max_distance: float) -> torch.Tensor:
    """Row of the bias table for every distance 0 .. n_max (int64), by the rule in the module docstring."""
    half = rows // 2
    n = torch.arange(n_max + 1, dtype=torch.float64)
    far = half + torch.floor(torch.log(n.clamp(min=max(half, 1)) / half) / math.log(max_distance / half) * (rows - half))
    return torch.where(n < half, n, far.clamp(max=rows - 1)).to(torch.int64)


class SigmoidAttention(Mixer):
    def __init__(self, spec):
        super().__init__(spec)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["n_heads"])
        self.nkv = int(spec["n_kv_heads"])
        self.hd = int(spec["head_dim"])
        self.vd = int(spec.get("v_head_dim") or self.hd)
        self.eps = spec.get("qk_norm_eps")
        self.qkv_bias = bool(spec.get("qkv_bias", False))
        self.o_bias = bool(spec.get("o_bias", False))
        self.head_gate = bool(spec.get("head_gate", False))
        self.window = spec.get("window")
        self.scale = 1.0 / math.sqrt(self.hd) if spec.get("scale") is None else float(spec["scale"])
        if self.nh < 1 or self.nkv < 1 or self.nh % self.nkv != 0:
            raise invalid(f"sigmoid attention: {self.nh} heads are not a multiple of {self.nkv} kv heads")
        if not (1 <= self.hd <= 256 and 1 <= self.vd <= 256) or (self.eps is not None and self.hd % 2 != 0):
            raise invalid(f"sigmoid attention: head sizes {self.hd} / {self.vd} must be at most 256, and even where "
                          "heads are normed")
        if self.window is not None and int(self.window) < 1:
            raise invalid("sigmoid attention: window must be >= 1")
        self.temp_coef, self.temp_every = 0.0, 0
        qt = spec.get("q_temperature")
        if qt is not None:
            self.temp_coef, self.temp_every = float(qt["coef"]), int(qt["every"])
            if self.temp_every < 1:
                raise invalid("sigmoid attention: q_temperature.every must be >= 1")
        self.bias_rows, self.max_distance = 0, 0.0
        db = spec.get("distance_bias")
        if db is not None:
            self.bias_rows, self.max_distance = int(db.get("rows") or 32), float(db["max_distance"])
            if self.bias_rows < 2:
                raise invalid("sigmoid attention: the distance bias table has at least 2 rows")

    def param_decls(self) -> Dict[str, ParamDecl]:
        q, kv, v, o = self.nh * self.hd, self.nkv * self.hd, self.nkv * self.vd, self.nh * self.vd
        d = {
            "q_proj.weight": ParamDecl((q, self.hidden), fan_in=self.hidden),
            "k_proj.weight": ParamDecl((kv, self.hidden), fan_in=self.hidden),
            "v_proj.weight": ParamDecl((v, self.hidden), fan_in=self.hidden),
            "o_proj.weight": ParamDecl((self.hidden, o), fan_in=o),
        }
        if self.qkv_bias:
            d["q_proj.bias"] = ParamDecl((q,), role="vector", init="zeros")
            d["k_proj.bias"] = ParamDecl((kv,), role="vector", init="zeros")
            d["v_proj.bias"] = ParamDecl((v,), role="vector", init="zeros")
        if self.o_bias:
            d["o_proj.bias"] = ParamDecl((self.hidden,), role="vector", init="zeros")
        if self.head_gate:
            d["g_proj.weight"] = ParamDecl((self.nh, self.hidden), fan_in=self.hidden)
        if self.eps is not None:
            d["q_norm.weight"] = ParamDecl((self.hd,), role="vector", init="ones")
            d["k_norm.weight"] = ParamDecl((self.hd,), role="vector", init="ones")
        if self.bias_rows:
            # the checkpoint's table decides how many rows there are
            d["rel_bias"] = ParamDecl((self.bias_rows, self.nh), role="vector", free_axes=(0,))
            d["head_bias"] = ParamDecl((self.nh,), role="vector", init="zeros")
        return d

    def cache_need(self):
        return PagedNeed(self.nkv, self.hd, int(self.window) if self.window is not None else None, 0,
                         None if self.vd == self.hd else self.vd)

    def bind(self, tensors, rt) -> None:
        ws = [tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]]
        if self.head_gate:
            ws.append(tensors["g_proj.weight"])
        common = torch.float32 if any(w.dtype == torch.float32 for w in ws) else ws[0].dtype
        rows = sum(w.shape[0] for w in ws)
        pad = (-rows) % 16          # zero rows up to a multiple of 16: the widths the few-token product takes
        if pad:
            ws.append(torch.zeros((pad, self.hidden), dtype=common, device=ws[0].device))
        # the fused rows: q heads, k heads, v heads, then one gate row per head
        self.w_in = torch.cat([w.to(common) for w in ws], dim=0).contiguous()
        self.b_in = None
        if self.qkv_bias:
            self.b_in = torch.cat([tensors[n + "_proj.bias"].float() for n in ("q", "k", "v")]).contiguous()
        self.q_norm = tensors.get("q_norm.weight")
        self.k_norm = tensors.get("k_norm.weight")
        self.w_o = tensors["o_proj.weight"]
        self.b_o = tensors["o_proj.bias"].float().contiguous() if self.o_bias else None
        self.dist_bias = None
        if self.bias_rows:
            rel, pb = tensors["rel_bias"].float(), tensors["head_bias"].float()
            rows = rel.shape[0]
            if rows < 2 or not self.max_distance > rows // 2:
                raise invalid(f"sigmoid attention: a bias table of {rows} rows needs max_distance above {rows // 2}")
            which = distance_rows(int(math.ceil(self.max_distance)), rows, self.max_distance).to(rel.device)
            self.dist_bias = (rel[which] + pb[None, :]).t().contiguous()          # [heads, distances]
        self.rt = rt

    def forward(self, x, ctx, cache):
        if not cache.writes:
            raise invalid("sigmoid attention: a layer owns its cache")
        proj = ops.linear(x, self.w_in, out_dtype=x.dtype)
        q = ops.qk_norm_rope_store(proj, self.q_norm, self.k_norm, self.eps if self.eps is not None else 0.0,
                                   None, None, ctx.positions, ctx.seg_of_token, cache.block_table,
                                   cache.k_pages, cache.v_pages, self.nh, self.nkv, self.hd, True, ctx.status,
                                   tiles=None if ctx.decode_only else (ctx.seg_start, ctx.seg_pos0, ctx.tile_seg,
                                                                       ctx.tile_q0),
                                   bias=self.b_in, v_head_dim=self.vd)
        gate = None
        if self.head_gate:            # one gate column per head, behind q, k and v
            g0 = (self.nh + self.nkv) * self.hd + self.nkv * self.vd
            gate = proj[:, g0:g0 + self.nh]
        o = self.rt.sigmoid_attention(q, cache, ctx, self.scale, self.dist_bias, self.temp_coef, self.temp_every,
                                      gate, self.window)
        return ops.linear(o, self.w_o, out_dtype=torch.float32), self.b_o


register_mixer("sigmoid_attention", SigmoidAttention, replace=True)
