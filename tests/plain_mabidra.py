"""A plain, slow Mabidra in float64 on the CPU: one function per mechanism, loops over positions where that is the
clearest way to say it.  It shares no code with the engine and is what the engine's tests compare with.

Notation: ``x`` [T, W] the residual stream of ONE sequence, ``n`` the normed rows, ``P`` a dict of the layer's
tensors by their checkpoint names without the ``l<i>.`` prefix, ``m`` the mixer's object of config.json.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ---- norms and activations -----------------------------------------------------------------------------
def group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """Every row is cut into ``groups`` equal consecutive parts; a part is divided by sqrt(mean(part^2) + eps);
    the whole row is then scaled by w."""
    T, W = x.shape
    parts = x.reshape(T, groups, W // groups)
    parts = parts / torch.sqrt((parts * parts).mean(dim=-1, keepdim=True) + eps)
    return parts.reshape(T, W) * w


def head_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """x [..., D]: divided by its root mean square over the last axis, times w [D]."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def softplus(a: float) -> float:
    return math.log1p(math.exp(-abs(a))) + max(a, 0.0)


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    pos = softplus(p) * z * z + 0.5 * z
    neg = (0.5 + softplus(q)) * (torch.expm1(z) - z) + 0.5 * z
    return torch.where(z > 0, pos, neg)


def relu2(z):
    return torch.clamp(z, min=0.0) ** 2


def silu(z):
    return z * torch.sigmoid(z)


# ---- gated linear attention ----------------------------------------------------------------------------------
def gla_decay(n, P, m):
    """alpha [T, H, D] = sigmoid(z) ** (1 / tau), z = W_a2 (W_a1 n) + b."""
    z = (n @ P["mix.a1"].T) @ P["mix.a2"].T + P["mix.a2.b"]
    return torch.sigmoid(z) ** (1.0 / float(m["tau"]))


def gla_recurrence(q, k, v, alpha, state=None):
    """q, k, alpha [T, H, D], v [T, H, Dv].  Per head S <- diag(alpha_t) S + k_t v_t^T (S is [D, Dv]: the decay
    scales the rows that belong to key channels), o_t = S^T q_t.  Returns o [T, H, Dv] and the last state."""
    T, H, D = q.shape
    Dv = v.shape[2]
    S = torch.zeros((H, D, Dv), dtype=F64) if state is None else state.clone()
    o = torch.zeros((T, H, Dv), dtype=F64)
    for t in range(T):
        for h in range(H):
            S[h] = alpha[t, h][:, None] * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


def mixer_gla(n, P, m, eps):
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = (n @ P["mix.q"].T).reshape(T, H, D) * float(D) ** -0.5
    k = (n @ P["mix.k"].T).reshape(T, H, D)
    v = (n @ P["mix.v"].T).reshape(T, H, Dv)
    alpha = gla_decay(n, P, m).reshape(T, H, D)
    o, _ = gla_recurrence(q, k, v, alpha)
    o = head_norm(o, P["mix.norm"], eps).reshape(T, H * Dv)
    return (o * silu(n @ P["mix.g"].T)) @ P["mix.o"].T


# ---- attention with sigmoid weights ------------------------------------------------------------------------------
def distance_bucket(n: int, B: int, D: float) -> int:
    """Distances below B/2 have a row each; further ones share rows that widen like a logarithm up to D."""
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def query_temperature(p: int, coef: float, every: int) -> float:
    return 1.0 + coef * math.log((p + 1) // every + 1)


def sigmoid_attend(q, k, v, scale: float, rel, pb, bias_max: float, group: int, pos0: int = 0):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; position i sees every j <= i with the weight
    sigmoid(scale * q_i.k_j + rel[bucket(i - j), h] + pb[h]); nothing is normalized over the keys."""
    T, H, D = q.shape
    Dv = v.shape[2]
    B = rel.shape[0]
    out = torch.zeros((T, H, Dv), dtype=F64)
    for h in range(H):
        g = h // group
        for i in range(T):
            for j in range(i + 1):
                s = float(q[i, h] @ k[j, g]) * scale + float(rel[distance_bucket(i - j, B, bias_max), h]) + float(pb[h])
                out[i, h] += (1.0 / (1.0 + math.exp(-s))) * v[j, g]
    return out


def sigmoid_attend_fast(q, k, v, scale, rel, pb, bias_max, group):
    """The same numbers as :func:`sigmoid_attend` by whole matrices (for long sequences in tests)."""
    T, H, D = q.shape
    B = rel.shape[0]
    kk = k.repeat_interleave(group, dim=1)
    vv = v.repeat_interleave(group, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    buckets = torch.tensor([distance_bucket(n, B, bias_max) for n in range(T)], dtype=torch.long)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    dist = (i - j).clamp(min=0)
    bias = rel.to(F64)[buckets[dist]]                        # [T, T, H]
    s = s + bias.permute(2, 0, 1) + pb.to(F64)[:, None, None]
    w = torch.sigmoid(s) * (i >= j)[None].to(F64)
    return torch.einsum("hij,jhd->ihd", w, vv)


def mixer_attention(n, P, m, eps, fast=True):
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = n.shape[0]
    q = (n @ P["mix.q"].T + P["mix.q.b"]).reshape(T, H, D)
    k = (n @ P["mix.k"].T + P["mix.k.b"]).reshape(T, G, D)
    v = (n @ P["mix.v"].T + P["mix.v.b"]).reshape(T, G, Dv)
    q = head_norm(q, P["mix.q.norm"], eps)
    k = head_norm(k, P["mix.k.norm"], eps)
    temp = torch.tensor([query_temperature(p, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"])) for p in range(T)],
                        dtype=F64)
    q = q * temp[:, None, None]
    f = sigmoid_attend_fast if fast else sigmoid_attend
    o = f(q, k, v, float(m["scale"]), P["mix.rel"], P["mix.pb"], float(m["bias_max"]), H // G)
    gate = torch.sigmoid(n @ P["mix.g"].T)                   # [T, H]: one number per head
    o = (o * gate[:, :, None]).reshape(T, H * Dv)
    return o @ P["mix.o"].T + P["mix.o.b"]


# ---- feed-forwards ---------------------------------------------------------------------------------------------
def ff_dense(n, P):
    p, q = float(P["mlp.act"][0]), float(P["mlp.act"][1])
    return xielu(n @ P["mlp.up"].T, p, q) @ P["mlp.down"].T


def route(n, P, top: int):
    """Router logits with their bias; the ``top`` largest are chosen, weights = softmax over the chosen logits."""
    z = n @ P["mlp.router"].T + P["mlp.router.b"]
    vals, idx = torch.topk(z, top, dim=-1)
    return idx, torch.softmax(vals, dim=-1)


def ff_moe(n, P, mlp):
    idx, w = route(n, P, int(mlp["router"]["top"]))
    out = torch.zeros((n.shape[0], P["mlp.e0.down"].shape[0]), dtype=F64)
    for t in range(n.shape[0]):
        for e, g in zip(idx[t].tolist(), w[t].tolist()):
            out[t] += g * (relu2(n[t] @ P[f"mlp.e{e}.up"].T) @ P[f"mlp.e{e}.down"].T)
    return out


# ---- the whole model ---------------------------------------------------------------------------------------------
def layer_order(cfg) -> List[dict]:
    """One dict per layer RUN: {"layer": i, "pass": t or None}; "pass" is set on the first layer of loop pass t."""
    L = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [{"layer": i, "pass": None} for i in range(L)]
    start, stop, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [{"layer": i, "pass": None} for i in range(start)]
    for t in range(times):
        for i in range(start, stop):
            runs.append({"layer": i, "pass": t if i == start else None})
    runs += [{"layer": i, "pass": None} for i in range(stop, L)]
    return runs


class PlainMabidra:
    def __init__(self, cfg: dict, tensors: Dict[str, torch.Tensor]):
        self.cfg = cfg
        self.T = {k: v.to(F64) for k, v in tensors.items()}
        self.eps = float(cfg["norm"]["eps"])
        self.groups = int(cfg["norm"]["groups"])

    def layer_tensors(self, i: int) -> Dict[str, torch.Tensor]:
        p = f"l{i}."
        return {k[len(p):]: v for k, v in self.T.items() if k.startswith(p)}

    def norm(self, x, w):
        return group_norm(x, w, self.groups, self.eps)

    def layer(self, x, i: int, fast=True):
        L, P = self.cfg["layers"][i], self.layer_tensors(i)
        n = self.norm(x, P["norm1"])
        if L["type"] == "gla":
            d = mixer_gla(n, P, L["mixer"], self.eps)
        elif L["type"] == "attention":
            d = mixer_attention(n, P, L["mixer"], self.eps, fast=fast)
        else:
            raise ValueError(L["type"])
        x = x + self.norm(d, P["norm1b"])
        if L.get("mlp") is None:
            return x
        n = self.norm(x, P["norm2"])
        d = ff_dense(n, P) if L["mlp"]["kind"] == "dense" else ff_moe(n, P, L["mlp"])
        return x + self.norm(d, P["norm2b"])

    def forward(self, tokens: List[int], taps: Optional[list] = None, fast=True) -> torch.Tensor:
        """Logits [T, vocab] of one sequence from position 0; ``taps`` collects the stream after every layer run."""
        x = self.T["embed"][torch.tensor(tokens, dtype=torch.long)] * float(self.cfg["embedding"]["scale"])
        x0 = x
        for run in layer_order(self.cfg):
            if run["pass"] is not None:
                x = torch.cat([x, x0], dim=1) @ self.T["loop.in"].T + self.T["loop.step"][run["pass"]]
            x = self.layer(x, run["layer"], fast=fast)
            if taps is not None:
                taps.append(x.clone())
        return self.norm(x, self.T["final.norm"]) @ self.T["head"].T

    # ---- what the tests ask of a model ------------------------------------------------------------------------
    @staticmethod
    def from_dir(model_dir: str) -> "PlainMabidra":
        import json
        import os
        from gesso_b200.weights.safetensors_io import read_safetensors_file
        with open(os.path.join(model_dir, "config.json")) as f:
            cfg = json.load(f)
        return PlainMabidra(cfg, read_safetensors_file(os.path.join(model_dir, "model.safetensors")))

    def logits(self, tokens) -> torch.Tensor:
        return self.forward(list(tokens))

    def stream(self, tokens) -> torch.Tensor:
        taps: list = []
        self.forward(list(tokens), taps=taps)
        return torch.stack(taps)

    def margins(self, tokens) -> torch.Tensor:
        """Per position: the smallest gap, over the routed layer runs, between the last chosen logit and the best one
        left out (infinite where every expert is chosen or no layer routes).  A bfloat16 run may choose otherwise
        where this is small."""
        tokens = list(tokens)
        out = torch.full((len(tokens),), math.inf, dtype=F64)
        x = self.T["embed"][torch.tensor(tokens, dtype=torch.long)] * float(self.cfg["embedding"]["scale"])
        x0 = x
        for run in layer_order(self.cfg):
            if run["pass"] is not None:
                x = torch.cat([x, x0], dim=1) @ self.T["loop.in"].T + self.T["loop.step"][run["pass"]]
            i = run["layer"]
            L, P = self.cfg["layers"][i], self.layer_tensors(i)
            mlp = L.get("mlp")
            if mlp is not None and mlp["kind"] == "moe" and mlp["router"]["top"] < mlp["router"]["experts"]:
                n1 = self.norm(x, P["norm1"])
                d = mixer_gla(n1, P, L["mixer"], self.eps) if L["type"] == "gla" else mixer_attention(n1, P, L["mixer"], self.eps)
                mid = x + self.norm(d, P["norm1b"])
                z = self.norm(mid, P["norm2"]) @ P["mlp.router"].T + P["mlp.router.b"]
                top = torch.sort(z, dim=-1, descending=True).values
                k = int(mlp["router"]["top"])
                out = torch.minimum(out, top[:, k - 1] - top[:, k])
            x = self.layer(x, i)
        return out

    def greedy(self, prompt, n_new: int):
        ids = list(prompt)
        for _ in range(n_new):
            ids.append(int(self.logits(ids)[-1].argmax()))
        return ids


# ---- random models for the tests -----------------------------------------------------------------------
def random_tensors(cfg: dict, seed: int, decay_rank: int = 5, bias_rows: int = 12) -> Dict[str, torch.Tensor]:
    """Tensors under their checkpoint names, rounded to bfloat16 (every run type sees the same numbers), drawn so that
    nothing is flat: projections N(0, gain^2 / fan_in), norm weights around one, biases and tables of order 0.3 to
    1.5, the decay's bias so that decays spread between slow and fast, the re-entry matrix near [I, I] / 2."""
    g = torch.Generator().manual_seed(seed)
    W: Dict[str, torch.Tensor] = {}

    def rnd(*shape, std=1.0, mean=0.0):
        return (mean + torch.randn(*shape, generator=g) * std).to(torch.bfloat16)

    def mat(rows, cols, gain=1.5):
        return rnd(rows, cols, std=gain / math.sqrt(cols))

    Wd, V = cfg["width"], cfg["vocab"]
    W["embed"] = rnd(V, Wd)
    W["head"] = mat(V, Wd, 1.0)
    W["final.norm"] = rnd(Wd, std=0.2, mean=1.0)
    if cfg.get("loop"):
        eye = torch.cat([torch.eye(Wd), torch.eye(Wd)], dim=1) * 0.5
        W["loop.in"] = (eye + torch.randn(Wd, 2 * Wd, generator=g) * 0.3 / math.sqrt(2 * Wd)).to(torch.bfloat16)
        W["loop.step"] = rnd(int(cfg["loop"]["times"]), Wd, std=0.3)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if L.get("mlp") is not None else ()):
            W[p + n] = rnd(Wd, std=0.2, mean=1.0)
        H, D = m["heads"], m["dim"]
        Dv = m.get("vdim", D)
        if L["type"] == "gla":
            W[p + "mix.q"], W[p + "mix.k"] = mat(H * D, Wd), mat(H * D, Wd)
            W[p + "mix.v"], W[p + "mix.g"] = mat(H * Dv, Wd), mat(H * Dv, Wd)
            W[p + "mix.a1"], W[p + "mix.a2"] = mat(decay_rank, Wd), mat(H * D, decay_rank, 2.0)
            W[p + "mix.a2.b"] = rnd(H * D, std=2.0, mean=2.0)
            W[p + "mix.norm"] = rnd(Dv, std=0.2, mean=1.0)
            W[p + "mix.o"] = mat(Wd, H * Dv)
        else:
            G = m["kv_heads"]
            for n, rows in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                W[p + "mix." + n] = mat(rows, Wd)
                W[p + "mix." + n + ".b"] = rnd(rows, std=0.3)
            W[p + "mix.q.norm"] = rnd(D, std=0.2, mean=1.0)
            W[p + "mix.k.norm"] = rnd(D, std=0.2, mean=1.0)
            W[p + "mix.rel"] = rnd(bias_rows, H, std=1.5)
            W[p + "mix.pb"] = rnd(H, std=1.0, mean=-1.0)
            W[p + "mix.g"] = mat(H, Wd, 2.0)
            W[p + "mix.o"] = mat(Wd, H * Dv)
            W[p + "mix.o.b"] = rnd(Wd, std=0.3)
        mlp = L.get("mlp")
        if mlp is None:
            continue
        if mlp["kind"] == "dense":
            W[p + "mlp.up"], W[p + "mlp.down"] = mat(mlp["ff"], Wd), mat(Wd, mlp["ff"])
            W[p + "mlp.act"] = rnd(2, std=1.0)
        else:
            F = mlp["expert"]["ff"]
            W[p + "mlp.router"] = mat(mlp["router"]["experts"], Wd, 3.0)
            W[p + "mlp.router.b"] = rnd(mlp["router"]["experts"], std=0.5)
            for e in range(mlp["router"]["experts"]):
                W[f"{p}mlp.e{e}.up"], W[f"{p}mlp.e{e}.down"] = mat(F, Wd), mat(Wd, F)
    return W


def write_model(model_dir: str, cfg: dict, seed: int, **sizes) -> None:
    import json
    import os
    from gesso_b200.weights.safetensors_io import write_safetensors_file
    os.makedirs(model_dir, exist_ok=True)
    with open(os.path.join(model_dir, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors_file(os.path.join(model_dir, "model.safetensors"), random_tensors(cfg, seed, **sizes))
