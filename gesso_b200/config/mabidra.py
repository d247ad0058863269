"""Typed Mabidra configuration, read from the architecture's own config.json keys.

Mabidra is a decoder-only stack whose every layer norms before AND after each sublayer with RMS norms in groups
(``x += norm1b(mixer(norm1(x)))``, ``x += norm2b(ff(norm2(x)))``), whose mixer is chosen per layer (gated linear
attention with a decay per key channel, or grouped-query attention with sigmoid weights, a bucketed distance bias and a
query temperature), whose feed-forward is dense (xIELU) or a mixture of squared-relu experts (router with a bias,
weights = softmax over the chosen logits), and in which a run of consecutive layers may be passed through several
times with the same tensors: before every pass the stream is mixed with the embedding's output by a matrix and a step
vector of the pass is added; every pass keeps caches and states of its own.  The embedding's output is scaled; the
output head is a matrix of its own.

config.json::

    {"architecture": "Mabidra", "vocab": V, "width": H, "embedding": {"scale": s}, "norm": {"eps": e, "groups": g},
     "loop": {"start": a, "stop": b, "times": n} | null,
     "layers": [{"type": "gla", "mixer": {"heads", "dim", "vdim", "tau"}, "mlp": ...},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "bias_max", "q_temp": {"coef", "every"}},
                 "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}} | null},
                ...]}

Every size and constant comes from there, nothing is assumed equal between layers; two sizes are the checkpoint's own:
the rank of the decay's low-rank projection (``mixer.decay_rank``, default 16, is what random weights are drawn with)
and the rows of the distance-bias table (``mixer.bias_rows``, default 32, likewise).  Checkpoint names: ``embed``,
``head``, ``final.norm``, ``loop.in``, ``loop.step``; ``l<i>.norm1|norm1b|norm2|norm2b``; gla: ``l<i>.mix.q|k|v|g|o``,
``l<i>.mix.a1``, ``l<i>.mix.a2`` (+ ``.b``), ``l<i>.mix.norm``; attention: ``l<i>.mix.q|k|v|o`` (+ ``.b``),
``l<i>.mix.q.norm``, ``l<i>.mix.k.norm``, ``l<i>.mix.rel``, ``l<i>.mix.pb``, ``l<i>.mix.g``; dense: ``l<i>.mlp.up|down|act``;
experts: ``l<i>.mlp.router`` (+ ``.b``), ``l<i>.mlp.e<k>.up|down``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional, Tuple, Union

from ..errors import invalid
from .registry import register_architecture
from .spec import BlockSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Mabidra"
MODEL_TYPE = "mabidra"


def _obj(v, what: str) -> Mapping[str, Any]:
    if not isinstance(v, Mapping):
        raise invalid(f"Mabidra config: {what} must be an object, got {v!r}")
    return v


def _int(d: Mapping[str, Any], key: str, what: str, minimum: int = 1, default: Optional[int] = None) -> int:
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise invalid(f"Mabidra config: {what} misses {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, int):
        raise invalid(f"Mabidra config: {what}.{key} must be an integer, got {v!r}")
    if v < minimum:
        raise invalid(f"Mabidra config: {what}.{key} must be >= {minimum}, got {v}")
    return v


def _num(d: Mapping[str, Any], key: str, what: str, default: Optional[float] = None) -> float:
    if key not in d or d[key] is None:
        if default is not None:
            return default
        raise invalid(f"Mabidra config: {what} misses {key!r}")
    v = d[key]
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise invalid(f"Mabidra config: {what}.{key} must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class MabidraGLA:
    heads: int
    dim: int
    vdim: int
    tau: float
    decay_rank: int

    @staticmethod
    def from_json(m: Mapping[str, Any], what: str) -> "MabidraGLA":
        dim = _int(m, "dim", what)
        tau = _num(m, "tau", what)
        if not tau > 0:
            raise invalid(f"Mabidra config: {what}.tau must be positive")
        return MabidraGLA(_int(m, "heads", what), dim, _int(m, "vdim", what, default=dim), tau,
                          _int(m, "decay_rank", what, default=16))


@dataclass(frozen=True)
class MabidraAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: float
    bias_rows: int
    temp_coef: float
    temp_every: int

    @staticmethod
    def from_json(m: Mapping[str, Any], what: str) -> "MabidraAttention":
        heads, kv = _int(m, "heads", what), _int(m, "kv_heads", what)
        if heads % kv != 0:
            raise invalid(f"Mabidra config: {what}: {heads} heads are not a multiple of {kv} kv_heads")
        dim = _int(m, "dim", what, 2)
        if dim % 2 != 0:
            raise invalid(f"Mabidra config: {what}.dim {dim} must be even")
        qt = _obj(m.get("q_temp"), what + ".q_temp")
        return MabidraAttention(heads, kv, dim, _int(m, "vdim", what, default=dim),
                                _num(m, "scale", what, default=float(dim) ** -0.5), _num(m, "bias_max", what),
                                _int(m, "bias_rows", what, 2, default=32), _num(qt, "coef", what + ".q_temp"),
                                _int(qt, "every", what + ".q_temp"))


@dataclass(frozen=True)
class MabidraDense:
    ff: int


@dataclass(frozen=True)
class MabidraMoE:
    ff: int
    experts: int
    top: int


def _mlp_from_json(m, what: str) -> Union[None, MabidraDense, MabidraMoE]:
    if m is None:
        return None
    m = _obj(m, what)
    kind = m.get("kind")
    if kind == "dense":
        return MabidraDense(_int(m, "ff", what))
    if kind == "moe":
        r = _obj(m.get("router"), what + ".router")
        experts, top = _int(r, "experts", what + ".router"), _int(r, "top", what + ".router")
        if top > experts:
            raise invalid(f"Mabidra config: {what}: {top} of {experts} experts cannot be chosen")
        return MabidraMoE(_int(_obj(m.get("expert"), what + ".expert"), "ff", what + ".expert"), experts, top)
    raise invalid(f"Mabidra config: {what}.kind {kind!r}; known kinds: ['dense', 'moe']")


MIXERS = {"gla": MabidraGLA, "attention": MabidraAttention}


@dataclass(frozen=True)
class MabidraLayer:
    kind: str
    mixer: Union[MabidraGLA, MabidraAttention]
    mlp: Union[None, MabidraDense, MabidraMoE]


@dataclass(frozen=True)
class MabidraLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class MabidraConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    norm_groups: int
    layers: Tuple[MabidraLayer, ...]
    loop: Optional[MabidraLoop]
    raw: Any = None

    @staticmethod
    def from_json(cfg: Mapping[str, Any]) -> "MabidraConfig":
        vocab, width = _int(cfg, "vocab", "config"), _int(cfg, "width", "config")
        norm = _obj(cfg.get("norm"), "norm")
        eps, groups = _num(norm, "eps", "norm"), _int(norm, "groups", "norm", default=1)
        if width % groups != 0:
            raise invalid(f"Mabidra config: width {width} does not form {groups} equal norm groups")
        scale = 1.0 if cfg.get("embedding") is None else _num(_obj(cfg["embedding"], "embedding"), "scale", "embedding",
                                                               default=1.0)
        raw_layers = cfg.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise invalid("Mabidra config: 'layers' must be a non-empty list")
        layers: List[MabidraLayer] = []
        for i, L in enumerate(raw_layers):
            L = _obj(L, f"layers[{i}]")
            kind = L.get("type")
            if kind not in MIXERS:
                raise invalid(f"Mabidra config: layers[{i}].type {kind!r}; known mixers: {sorted(MIXERS)}")
            mixer = MIXERS[kind].from_json(_obj(L.get("mixer"), f"layers[{i}].mixer"), f"layers[{i}].mixer")
            layers.append(MabidraLayer(kind, mixer, _mlp_from_json(L.get("mlp"), f"layers[{i}].mlp")))
        loop = None
        if cfg.get("loop") is not None:
            lp = _obj(cfg["loop"], "loop")
            loop = MabidraLoop(_int(lp, "start", "loop", 0), _int(lp, "stop", "loop"), _int(lp, "times", "loop"))
            if not (loop.start < loop.stop <= len(layers)):
                raise invalid(f"Mabidra config: loop {loop.start}..{loop.stop} does not lie inside {len(layers)} layers")
        return MabidraConfig(vocab, width, scale, eps, groups, tuple(layers), loop, raw=dict(cfg))

    def to_json(self) -> dict:
        if self.raw is not None:
            return dict(self.raw)
        raise invalid("Mabidra config: no source object to write")

    # ---- the model this configuration describes ---------------------------------------------------
    def layer_runs(self) -> List[Tuple[int, Optional[int]]]:
        """(layer, pass) per layer run in order; ``pass`` is the number of the loop's pass on its first layer."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        lp = self.loop
        runs: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(lp.start)]
        for t in range(lp.times):
            runs += [(i, t if i == lp.start else None) for i in range(lp.start, lp.stop)]
        return runs + [(i, None) for i in range(lp.stop, n)]

    def _mixer_spec(self, L: MabidraLayer) -> PartSpec:
        m = L.mixer
        if L.kind == "gla":
            return PartSpec("gated_linear_attention", {
                "hidden_size": self.width, "n_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "decay_rank": m.decay_rank, "tau": m.tau, "norm_eps": self.norm_eps})
        return PartSpec("sigmoid_attention", {
            "hidden_size": self.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim,
            "v_head_dim": m.vdim, "scale": m.scale, "qk_norm_eps": self.norm_eps, "qkv_bias": True, "o_bias": True,
            "head_gate": True, "q_temperature": {"coef": m.temp_coef, "every": m.temp_every},
            "distance_bias": {"rows": m.bias_rows, "max_distance": m.bias_max}, "window": None})

    def _mlp_spec(self, mlp) -> Optional[PartSpec]:
        if mlp is None:
            return None
        if isinstance(mlp, MabidraDense):
            return PartSpec("mlp", {"hidden_size": self.width, "ff_dim": mlp.ff, "activation": "xielu"})
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "ff_dim": mlp.ff, "n_experts": mlp.experts, "top_k": mlp.top,
            "score": "softmax_chosen", "router_bias": True, "correction": False, "renormalize": False,
            "activation": "relu2"})

    def to_spec(self) -> ModelSpec:
        norm = PartSpec("group_rmsnorm", {"size": self.width, "eps": self.norm_eps, "groups": self.norm_groups})
        names: Dict[str, Tuple[str, ...]] = {"embedding.weight": ("embed",), "lm_head.weight": ("head",),
                                             "final_norm.weight": ("final.norm",)}
        blocks: List[BlockSpec] = []
        for i, L in enumerate(self.layers):
            p, ck = f"layers.{i}.", f"l{i}."
            has_ff = L.mlp is not None
            blocks.append(BlockSpec("sandwich", self._mixer_spec(L), self._mlp_spec(L.mlp), norm,
                                    norm if has_ff else None, p, mixer_post_norm=norm,
                                    ff_post_norm=norm if has_ff else None))
            names[p + "mixer_norm.weight"] = (ck + "norm1",)
            names[p + "mixer_post_norm.weight"] = (ck + "norm1b",)
            if has_ff:
                names[p + "ff_norm.weight"] = (ck + "norm2",)
                names[p + "ff_post_norm.weight"] = (ck + "norm2b",)
            mx = p + "mixer."
            if L.kind == "gla":
                for t in ("q", "k", "v", "g", "o"):
                    names[mx + f"{t}_proj.weight"] = (ck + f"mix.{t}",)
                names[mx + "a1.weight"] = (ck + "mix.a1",)
                names[mx + "a2.weight"] = (ck + "mix.a2",)
                names[mx + "a2.bias"] = (ck + "mix.a2.b",)
                names[mx + "norm.weight"] = (ck + "mix.norm",)
            else:
                for t in ("q", "k", "v", "o"):
                    names[mx + f"{t}_proj.weight"] = (ck + f"mix.{t}",)
                    names[mx + f"{t}_proj.bias"] = (ck + f"mix.{t}.b",)
                names[mx + "q_norm.weight"] = (ck + "mix.q.norm",)
                names[mx + "k_norm.weight"] = (ck + "mix.k.norm",)
                names[mx + "rel_bias"] = (ck + "mix.rel",)
                names[mx + "head_bias"] = (ck + "mix.pb",)
                names[mx + "g_proj.weight"] = (ck + "mix.g",)
            ff = p + "feed_forward."
            if isinstance(L.mlp, MabidraDense):
                names[ff + "up.weight"] = (ck + "mlp.up",)
                names[ff + "down.weight"] = (ck + "mlp.down",)
                names[ff + "act"] = (ck + "mlp.act",)
            elif isinstance(L.mlp, MabidraMoE):
                names[ff + "router.weight"] = (ck + "mlp.router",)
                names[ff + "router.bias"] = (ck + "mlp.router.b",)
                for e in range(L.mlp.experts):
                    names[ff + f"experts.{e}.up.weight"] = (ck + f"mlp.e{e}.up",)
                    names[ff + f"experts.{e}.down.weight"] = (ck + f"mlp.e{e}.down",)
        stream_parts: Tuple[Tuple[str, PartSpec], ...] = ()
        if self.loop is not None:
            stream_parts = (("loop.", PartSpec("reentry_mix", {"hidden_size": self.width, "passes": self.loop.times})),)
            names["loop.in.weight"] = ("loop.in",)
            names["loop.step"] = ("loop.step",)
        # one schedule entry per layer run: a layer inside the loop runs with the same bound parts every pass,
        # each time on a cache or state of the entry's own
        schedule = tuple(ScheduleEntry(i, before=None if t is None else (0, t)) for i, t in self.layer_runs())
        ignorable = tuple(rf"^l{i}\.norm2b?$" for i, L in enumerate(self.layers) if L.mlp is None)
        return ModelSpec(
            architecture=ARCHITECTURE, vocab_size=self.vocab, hidden_size=self.width, blocks=tuple(blocks),
            schedule=schedule, final_norm=norm, tie_embedding=False, stream_parts=stream_parts,
            embedding_scale=self.embedding_scale, tensor_names=names, ignorable_tensors=ignorable, source=self)


def mabidra_adapter(cfg: Mapping[str, Any]) -> ModelSpec:
    return MabidraConfig.from_json(cfg).to_spec()


mabidra_adapter.model_type = MODEL_TYPE
register_architecture(ARCHITECTURE, mabidra_adapter, replace=True)
