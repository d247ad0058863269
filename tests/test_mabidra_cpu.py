"""Mabidra without a device: the configuration reader, the model spec it makes, the checkpoint binding, the cache
plan of a looped stack, and the plain implementation's own mechanisms against closed forms."""
import copy
import math

import pytest
import torch

import configs_mabidra as cb
import plain_mabidra as pb
from gesso_b200.config import spec_from_config
from gesso_b200.config.mabidra import MabidraConfig
from gesso_b200.engine.model import CachePlan
from gesso_b200.errors import GessoError
from gesso_b200.parts.base import PagedNeed, StateNeed
from gesso_b200.parts.registry import build_block
from gesso_b200.parts.sigmoid_attention import distance_rows
from gesso_b200.weights.loader import bind_tensors


@pytest.mark.parametrize("name", list(cb.MBD))
def test_spec_parts_names_and_schedule(name):
    cfg, seed, sizes = cb.MBD[name]
    spec = spec_from_config(cfg)
    assert spec.architecture == "Mabidra" and not spec.tie_embedding and len(spec.blocks) == len(cfg["layers"])
    assert spec.embedding_scale == cfg["embedding"]["scale"]
    kinds = {"gla": "gated_linear_attention", "attention": "sigmoid_attention"}
    for L, b in zip(cfg["layers"], spec.blocks):
        assert b.arrangement == "sandwich" and b.mixer.kind == kinds[L["type"]]
        assert (b.feed_forward is None) == (L["mlp"] is None)
        assert b.mixer_norm.kind == "group_rmsnorm" and b.mixer_norm["groups"] == cfg["norm"]["groups"]
        assert b.mixer_post_norm["eps"] == cfg["norm"]["eps"]
        if L["type"] == "attention":
            assert b.mixer["scale"] == L["mixer"]["scale"] and b.mixer["window"] is None
            assert b.mixer["distance_bias"]["max_distance"] == L["mixer"]["bias_max"]
        else:
            assert b.mixer["tau"] == L["mixer"]["tau"]
        if L["mlp"] and L["mlp"]["kind"] == "moe":
            assert b.feed_forward["score"] == "softmax_chosen" and b.feed_forward["router_bias"] is True
    # one schedule entry per layer run, the loop's first layer names the pass
    runs = pb.layer_order(cfg)
    assert [e.layer for e in spec.schedule] == [r["layer"] for r in runs]
    assert [None if e.before is None else e.before[1] for e in spec.schedule] == [r["pass"] for r in runs]
    assert all(e.cache_of is None for e in spec.schedule)
    # every tensor finds its place and none is left over, whatever the checkpoint's own two sizes are
    bound = bind_tensors(spec, pb.random_tensors(cfg, seed, **sizes))
    assert "embedding.weight" in bound and "lm_head.weight" in bound
    if cfg["loop"]:
        assert tuple(bound["loop.step"].shape) == (cfg["loop"]["times"], cfg["width"])


def test_every_pass_has_a_cache_of_its_own():
    spec = spec_from_config(cb.MBD_A)
    plan = CachePlan(spec, [build_block(b) for b in spec.blocks])
    paged = [need for need, _ in plan.paged_groups]
    assert PagedNeed(2, 16, None, 0, None) in paged and PagedNeed(1, 32, None, 0, None) in paged
    states = [need for need, _ in plan.state_entries]
    assert states.count(StateNeed((2, 24, 16), "float32")) == 2            # heads x value size x key size, layers 0 and 3
    # layers 1 and 2 run twice: four paged entries in all
    assert sum(len(entries) for _, entries in plan.paged_groups) == 4
    spec = spec_from_config(cb.MBD_ONLY_STATE)
    plan = CachePlan(spec, [build_block(b) for b in spec.blocks])
    assert len(plan.state_entries) == 3 and not plan.paged_groups          # the looped layer twice, then the last one


def test_refusals_name_the_key():
    def broken(change):
        cfg = copy.deepcopy(cb.MBD_A)
        change(cfg)
        with pytest.raises(GessoError) as e:
            MabidraConfig.from_json(cfg)
        return str(e.value)
    assert "type" in broken(lambda c: c["layers"][0].update(type="mamba"))
    assert "tau" in broken(lambda c: c["layers"][0]["mixer"].update(tau=0.0))
    assert "kv_heads" in broken(lambda c: c["layers"][1]["mixer"].update(kv_heads=3))
    assert "kind" in broken(lambda c: c["layers"][0]["mlp"].update(kind="glu"))
    assert "experts" in broken(lambda c: c["layers"][1]["mlp"]["router"].update(top=7))
    assert "q_temp" in broken(lambda c: c["layers"][1]["mixer"].pop("q_temp"))
    assert "bias_max" in broken(lambda c: c["layers"][1]["mixer"].pop("bias_max"))
    assert "groups" in broken(lambda c: c["norm"].update(groups=5))
    assert "loop" in broken(lambda c: c["loop"].update(stop=9))
    assert "eps" in broken(lambda c: c.update(norm={}))
    cfg, seed, sizes = cb.MBD["a"]
    tensors = pb.random_tensors(cfg, seed, **sizes)
    del tensors["l1.mix.pb"]
    tensors["l0.mix.rel"] = torch.zeros(4, 2)                              # a recurrence has no distance table
    tensors["l2.mix.a1"] = tensors["l0.mix.a1"]
    with pytest.raises(GessoError) as e:
        bind_tensors(spec_from_config(cfg), tensors)
    assert "l1.mix.pb" in str(e.value) and "l0.mix.rel" in str(e.value)
    # the two matrices of the decay's projection must agree on the rank, whatever it is
    tensors = pb.random_tensors(cfg, seed, **sizes)
    tensors["l0.mix.a1"] = torch.zeros(sizes["decay_rank"] + 1, cfg["width"], dtype=torch.bfloat16)
    spec = spec_from_config(cfg)
    bound = bind_tensors(spec, tensors)
    blk = build_block(spec.blocks[0])
    with pytest.raises(GessoError):
        blk.mixer.bind({k[len("layers.0.mixer."):]: v for k, v in bound.items() if k.startswith("layers.0.mixer.")}, None)


def test_distance_rows_and_temperature():
    # half of the rows are the distances themselves; further ones share rows that widen; from the limit on the last
    for rows, limit in ((12, 40.0), (6, 9.5), (32, 1000.0), (2, 3.0), (20, 33.0)):
        n_max = int(math.ceil(limit)) + 5
        got = distance_rows(n_max, rows, limit).tolist()
        want = [pb.distance_bucket(n, rows, limit) for n in range(n_max + 1)]
        assert got == want
        assert got[:rows // 2] == list(range(rows // 2)) and got[rows // 2] == rows // 2
        assert all(a <= b for a, b in zip(got, got[1:])) and got[int(math.ceil(limit))] == rows - 1 == got[-1]
    assert pb.distance_bucket(11, 12, 40.0) == 6 + int(math.log(11 / 6) / math.log(40 / 6) * 6)
    assert pb.query_temperature(0, 0.5, 4) == 1.0 and pb.query_temperature(2, 0.5, 4) == 1.0
    assert pb.query_temperature(3, 0.5, 4) == 1.0 + 0.5 * math.log(2) == pb.query_temperature(6, 0.5, 4)
    assert pb.query_temperature(7, 0.5, 4) == 1.0 + 0.5 * math.log(3)


def test_plain_attention_forms_agree_and_nothing_is_normalized():
    T, H, G, D = 45, 4, 2, 8
    q, k = torch.randn(T, H, D, dtype=pb.F64), torch.randn(T, G, D, dtype=pb.F64)
    v = torch.randn(T, G, 5, dtype=pb.F64)
    rel, hb = torch.randn(10, H, dtype=pb.F64), torch.randn(H, dtype=pb.F64)
    a = pb.sigmoid_attend(q, k, v, 0.3, rel, hb, 30.0, 2)
    b = pb.sigmoid_attend_fast(q, k, v, 0.3, rel, hb, 30.0, 2)
    assert torch.allclose(a, b, atol=1e-12)
    # zero scores and a zero table: every visible key weighs one half, so position i sums (i + 1) / 2 values of one
    ones = torch.ones(T, 1, 1, dtype=pb.F64)
    out = pb.sigmoid_attend(torch.zeros(T, 1, D, dtype=pb.F64), k[:, :1], ones, 1.0, torch.zeros(10, 1, dtype=pb.F64),
                            torch.zeros(1, dtype=pb.F64), 30.0, 1).view(T)
    assert torch.allclose(out, (torch.arange(T, dtype=pb.F64) + 1) / 2)
    # a table that opens exactly one row: only keys at the distances of that row count
    rel = torch.full((10, 1), -80.0, dtype=pb.F64)
    rel[7] = 80.0
    out = pb.sigmoid_attend(torch.zeros(T, 1, D, dtype=pb.F64), k[:, :1], ones, 1.0, rel, torch.zeros(1, dtype=pb.F64),
                            30.0, 1).view(T)
    for i in range(T):
        n = sum(1 for j in range(i + 1) if pb.distance_bucket(i - j, 10, 30.0) == 7)
        assert abs(float(out[i]) - n) < 1e-9


def test_plain_recurrence_activation_and_router():
    T, H, D, Dv = 9, 1, 3, 2
    q, k, v = torch.randn(T, H, D, dtype=pb.F64), torch.randn(T, H, D, dtype=pb.F64), torch.randn(T, H, Dv, dtype=pb.F64)
    alpha = torch.rand(T, H, D, dtype=pb.F64)
    o, S = pb.gla_recurrence(q, k, v, alpha)
    for t in range(T):           # the sum form: key s reaches t through the product of the decays behind it
        want = sum((q[t, 0] * k[s, 0] * alpha[s + 1:t + 1, 0].prod(dim=0)).sum() * v[s, 0] for s in range(t + 1))
        assert torch.allclose(o[t, 0], want, atol=1e-12)
    o2, S2 = pb.gla_recurrence(q[5:], k[5:], v[5:], alpha[5:], state=pb.gla_recurrence(q[:5], k[:5], v[:5], alpha[:5])[1])
    assert torch.allclose(o2, o[5:], atol=1e-12) and torch.allclose(S2, S, atol=1e-12)
    z = torch.tensor([-3.0, -1e-9, 0.0, 1e-9, 2.0], dtype=pb.F64)
    y = pb.xielu(z, 0.3, -0.2)
    sp = lambda a: math.log(1 + math.exp(a))
    assert abs(float(y[4]) - (sp(0.3) * 4 + 1)) < 1e-12 and float(y[2]) == 0.0
    assert abs(float(y[0]) - ((0.5 + sp(-0.2)) * (math.exp(-3) + 2) - 1.5)) < 1e-12
    assert abs(float(y[1]) - float(y[3])) < 1e-8                               # continuous at zero
    P = {"mlp.router": torch.eye(4, dtype=pb.F64), "mlp.router.b": torch.tensor([0.0, 0.0, 5.0, 0.0], dtype=pb.F64)}
    idx, w = pb.route(torch.tensor([[3.0, 1.0, -1.0, 2.0]], dtype=pb.F64), P, 2)
    assert idx[0].tolist() == [2, 0] and torch.allclose(w[0], torch.softmax(torch.tensor([4.0, 3.0], dtype=pb.F64), 0))
    assert abs(float(w.sum()) - 1.0) < 1e-12
