"""Mabidra on the device against the plain implementation: every mechanism alone (with inputs made so that a far key
that is lost, a distance that reads the wrong row of the table, a decay of the wrong channel or a lost state shows),
then whole models under four ways of cutting and batching, pages and slots used again, long decoding, and
generation through the session."""
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import configs_mabidra as cb
import plain_mabidra as pb
import trace_tools as tt

pytestmark = pytest.mark.gpu

DEV = "cuda"
# the error of a logits row: root mean square of the difference (its mean taken off) over that of the row
TOL = {"float32": 5e-5, "bfloat16": 0.04}
# bfloat16 rounding grows with the layer runs a token passes (configuration c: nine, with eight-head attention under a
# strong temperature and no normalization over the keys), and float32 rounding with how narrow the normed parts are
# (a read-out or a sublayer's output that happens to be small is divided by its own size): the random configurations
# and c are held to wider limits; an error of logic is of order one in both.
TOL_OF = {("c", "bfloat16"): 0.15}
TOL_RANDOM = {"float32": 2e-4, "bfloat16": 0.06}


def tol_of(name, dtype):
    return TOL_OF.get((name, dtype), TOL[dtype])
LENGTHS = {"a": [7, 130, 1, 64, 33, 97, 2, 65], "b": [40, 1, 23, 64, 150, 5, 17, 50], "c": [48, 3, 150, 31, 80]}
CLEAR_MARGIN = 0.15


def row_error(got, ref):
    d = np.asarray(got, dtype=np.float64) - np.asarray(ref, dtype=np.float64)
    r = np.asarray(ref, dtype=np.float64)
    return float(np.sqrt(np.mean((d - d.mean()) ** 2)) / np.sqrt(np.mean((r - r.mean()) ** 2)))


def compare(rows, ref, tol, what, margins=None):
    """Every row within ``tol``.  With ``margins`` (bfloat16 runs): a row whose routing in the plain model hangs on
    less than the run's rounding can move is not held to ``tol``; of the others nine in ten must be within it
    and their median within a third of it."""
    errs = []
    for (rid, pos), row in sorted(rows.items()):
        assert np.isfinite(row).all(), f"{what}: request {rid} position {pos}: non-finite logits"
        e = row_error(row, ref[rid][pos])
        if margins is None:
            assert e <= tol, f"{what}: request {rid} position {pos} of {len(ref[rid])}: error {e:.3e} > {tol:.1e} (first bad place)"
        elif float(margins[rid][pos]) >= CLEAR_MARGIN:
            errs.append(e)
    if margins is not None:
        errs = np.sort(np.asarray(errs))
        assert len(errs) >= len(rows) // 3, f"{what}: too few rows with a clear routing"
        inside = float((errs <= tol).mean())
        assert inside >= 0.9 and errs[len(errs) // 2] <= tol / 3, \
            f"{what}: {inside:.2%} of {len(errs)} rows within {tol}, median {errs[len(errs) // 2]:.3e}"


@pytest.fixture(scope="module")
def mbd_dirs(tmp_path_factory):
    out = {}
    for name, (cfg, seed, sizes) in cb.MBD.items():
        d = str(tmp_path_factory.mktemp(f"mbd_{name}"))
        pb.write_model(d, cfg, seed, **sizes)
        out[name] = d
    return out


@pytest.fixture(scope="module")
def plain(mbd_dirs):
    models = {n: pb.PlainMabidra.from_dir(d) for n, d in mbd_dirs.items()}
    cache, margins = {}, {}

    def get(name):
        if name not in cache:
            reqs = tt.make_requests(cb.MBD[name][0]["vocab"], LENGTHS[name], seed=90 + len(name))
            cache[name] = (reqs, [models[name].logits(t).numpy() for t in reqs])
            margins[name] = [models[name].margins(t).numpy() for t in reqs]
        return cache[name]
    get.models = models
    get.margins = lambda name, dtype: margins[name] if dtype == "bfloat16" else None
    return get


@pytest.fixture(scope="module")
def loaded(mbd_dirs):
    import gesso_b200
    cache = {}

    def get(name, dtype):
        if (name, dtype) not in cache:
            cache[(name, dtype)] = gesso_b200.load(mbd_dirs[name], dtype=dtype, max_positions=1024)
        return cache[(name, dtype)]
    return get


SCHEDULES = {
    "whole": lambda reqs: tt.trace_whole(reqs),
    "tail_decode": lambda reqs: tt.trace_tail_decode(reqs, tail=60),     # decoded tokens pass the distance tables' ends
    "portions": lambda reqs: tt.trace_portions(reqs),
    "mixed": lambda reqs: tt.trace_mixed(reqs, seed=5),
}


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


def segments(lens):
    """Flat-axis metadata of a step whose segments have these lengths."""
    seg = torch.cat([torch.full((n,), i) for i, n in enumerate(lens)]).to(torch.int32).to(DEV)
    start = i32(np.concatenate([[0], np.cumsum(lens)]).tolist())
    return seg, start


# ---- mechanisms alone ------------------------------------------------------------------------------------
@pytest.mark.parametrize("width,groups,rows", [(64, 2, 5), (48, 1, 37), (512, 4, 300), (96, 6, 70), (30, 3, 9), (256, 256, 4),
                                               (1024, 4, 33), (2048, 4, 9), (2048, 2, 5), (768, 2, 7)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("delta_dtype", [torch.float32, torch.bfloat16])
def test_group_norm_of_the_delta_then_of_the_stream(width, groups, rows, out_dtype, delta_dtype):
    """``h += norm(delta + bias)`` and ``norm(h)`` in one pass; groups of uneven sizes of magnitude (one group a
    thousand times the others) so that a statistic taken over the whole row, or over the wrong part, shows."""
    from gesso_b200 import ops
    eps = 1e-5
    h = torch.randn(rows, width, device=DEV)
    delta = torch.randn(rows, width, device=DEV)
    delta[:, :width // groups] *= 1000.0
    delta = delta.to(delta_dtype)
    bias = torch.randn(width, device=DEV)
    w_post = (1 + 0.3 * torch.randn(width, device=DEV))
    w_pre = (1 + 0.3 * torch.randn(width, device=DEV))
    h64 = h.double().cpu() + pb.group_norm(delta.double().cpu() + bias.double().cpu(), w_post.double().cpu(), groups, eps)
    want = pb.group_norm(h64, w_pre.double().cpu(), groups, eps)
    got = ops.add_group_rmsnorm(h, delta, bias, ops.GroupRmsParams(w_post, eps, groups), ops.GroupRmsParams(w_pre, eps, groups),
                                out_dtype)
    tol = 2e-5 if delta_dtype == torch.float32 else 1e-4      # a bfloat16 delta is exact; its sum with the bias is float32
    assert (h.double().cpu() - h64).abs().max() <= tol * h64.abs().max()
    otol = 2e-5 if out_dtype == torch.float32 else 8e-3
    assert (got.double().cpu() - want).abs().max() <= otol * want.abs().max()
    # only some rows, and the stream stays
    before = h.clone()
    pick = i32([rows - 1, 0])
    some = ops.add_group_rmsnorm(h, None, None, None, ops.GroupRmsParams(w_pre, eps, groups), out_dtype, rows=pick)
    assert torch.equal(h, before)
    assert (some.double().cpu() - want[[rows - 1, 0]]).abs().max() <= otol * want.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_streams_side_by_side_and_the_pass_vector(dtype):
    from gesso_b200 import ops
    a, b = torch.randn(37, 50, device=DEV), torch.randn(37, 50, device=DEV)
    both = ops.concat_cast(a, b, dtype)
    assert torch.equal(both, torch.cat([a, b], dim=1).to(dtype))
    v = torch.randn(50, device=DEV)
    want = a + v
    assert torch.equal(ops.rows_add_vector(a, v), want)


def _pages(k, v, page_size, order):
    T, G, D = k.shape
    n = (T + page_size - 1) // page_size
    kp = torch.full((len(order) + 1, G, page_size, D), float("nan"), dtype=k.dtype, device=k.device)
    vp = torch.full((len(order) + 1, G, v.shape[2], page_size), float("nan"), dtype=k.dtype, device=k.device)
    for p in range(n):
        lo, hi = p * page_size, min(T, (p + 1) * page_size)
        kp[order[p], :, :hi - lo] = k[lo:hi].transpose(0, 1)
        vp[order[p], :, :, :hi - lo] = v[lo:hi].permute(1, 2, 0)
    bt = torch.full((1, len(order)), -1, dtype=torch.int32, device=k.device)
    bt[0, :n] = torch.tensor(order[:n], dtype=torch.int32)
    return kp, vp, bt


def _bias_by_distance(rel, hb, n_max, bias_max):
    """[heads, n_max + 1]: the table's row of every distance plus the per-head number, by the plain bucket rule."""
    rows = [pb.distance_bucket(n, rel.shape[0], bias_max) for n in range(n_max + 1)]
    return (rel[rows] + hb[None, :]).t().contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,Vd,B,bias_max,every", [(4, 2, 16, 24, 12, 40.0, 8), (3, 3, 10, 40, 6, 9.5, 1),
                                                       (8, 1, 64, 64, 32, 250.0, 64), (2, 1, 96, 32, 20, 33.0, 50),
                                                       (1, 1, 48, 48, 2, 500.0, 7), (6, 2, 128, 128, 16, 128.0, 100),
                                                       (4, 2, 32, 32, 10, 64.0, 3), (12, 1, 96, 96, 8, 300.0, 128),
                                                       (32, 2, 64, 64, 6, 20.0, 16)])
def test_sigmoid_attention_far_keys_table_rows_and_temperature(H, G, D, Vd, B, bias_max, every, dtype):
    """One sequence of 300 positions in pages handed out of order, free pages full of NaN.  Head 0 is quiet (a per-head
    number of -12 closes every key) except for keys made to stand out: the first token, a token hundreds back and the
    query's own, so a far key that is lost, or weights normalized over the keys, change the result by a lot.  The last
    head's table is a wall: rows up to one in the widening half are open, the next ones shut, so a distance that reads
    the neighbouring row shows at the wall's edge.  The temperature steps inside the sequence.  Queries run as one
    portion and one by one."""
    from gesso_b200 import ops
    T, page, scale, coef = 300, 16, 0.21, 0.4
    q = torch.randn(T, H, D, device=DEV)
    k = torch.randn(T, G, D, device=DEV)
    v = torch.randn(T, G, Vd, device=DEV)
    rel = torch.randn(B, H, device=DEV)
    hb = torch.randn(H, device=DEV) - 1.0
    hb[0] = -12.0
    wall = min(B - 2, B // 2 + 1)
    rel[wall + 1:, H - 1] = -40.0
    probes = (T - 1, 200, 77)
    for i in probes:
        temp = pb.query_temperature(i, coef, every)
        for n, j in enumerate((0, max(0, i - 170), i)):
            u = q[i, 0] / q[i, 0].norm()
            k[j, 0] = u * (20.0 + 3 * n) / (scale * temp * float(q[i, 0].norm()))
    q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
    gate = torch.randn(T, H + 3, device=DEV).to(dtype)[:, 1:H + 1]          # a view into wider rows
    order = [7, 12, 2, 9, 0, 14, 4, 1, 18, 8, 3, 16, 6, 5, 11, 10, 13, 15, 17]
    kp, vp, bt = _pages(k, v, page, order)
    temps = torch.tensor([pb.query_temperature(p, coef, every) for p in range(T)], dtype=pb.F64)
    q64 = q.double().cpu() * temps[:, None, None]
    want = pb.sigmoid_attend_fast(q64, k.double().cpu(), v.double().cpu(), scale, rel.double().cpu(), hb.double().cpu(),
                                  bias_max, H // G)
    lone = pb.sigmoid_attend(q64[:12], k.double().cpu()[:12], v.double().cpu()[:12], scale, rel.double().cpu(),
                             hb.double().cpu(), bias_max, H // G)
    assert torch.allclose(lone, want[:12], atol=1e-9)
    want = (want * torch.sigmoid(gate.double().cpu())[:, :, None]).reshape(T, H * Vd)
    # the quiet head's probes are carried by the keys that stand out
    for i in probes:
        assert want[i, :Vd].abs().max() > 0.3 * torch.sigmoid(gate[i, 0].double().cpu())
    table = _bias_by_distance(rel, hb, int(math.ceil(bias_max)), bias_max)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    seg = torch.zeros(T, dtype=torch.int32, device=DEV)
    got = ops.sigmoid_attention_generic(q, kp, vp, bt, pos, seg, scale, table, coef, every, gate).double().cpu()
    err = (got - want).abs().max(dim=1).values / want.abs().max()
    assert err.max() <= tol, f"portion: {float(err.max()):.3e} first at {int((err > tol).nonzero()[0]) if (err > tol).any() else -1}"
    for i in probes + (0, 1, 15, 16, B // 2, wall + 3, min(T - 2, int(bias_max)), min(T - 1, int(bias_max) + 1)):
        got = ops.sigmoid_attention_generic(q[i:i + 1].contiguous(), kp, vp, bt, pos[i:i + 1], seg[:1], scale, table, coef,
                                            every, gate[i:i + 1]).double().cpu()
        err = (got[0] - want[i]).abs().max() / want.abs().max()
        assert err <= tol, f"single token at {i}: {float(err):.3e}"
    if dtype == torch.bfloat16 and D == Vd and ops.fast_attention_takes(D, page, H, G):
        # the tensor-core kernels: the whole sequence as one portion, a portion that starts inside a page and a tile,
        # and single tokens with the keys in one piece and cut into several
        def tiles_of(n):
            return i32([0] * ((n + 63) // 64)), i32(list(range(0, n, 64)))
        for first in (0, 100, 293):
            n = T - first
            tile_seg, tile_q0 = tiles_of(n)
            got = ops.sigmoid_prefill_attention(q[first:].contiguous(), kp, vp, bt, i32([0, n]), i32([first]), tile_seg,
                                                tile_q0, scale, table, coef, every, gate[first:]).double().cpu()
            err = (got - want[first:]).abs().max(dim=1).values / want.abs().max()
            assert err.max() <= tol, (f"tensor-core portion from {first}: {float(err.max()):.3e} first at "
                                      f"{first + int((err > tol).nonzero()[0])}")
        for i in probes + (0, 1, 15, 16, B // 2, wall + 3, min(T - 2, int(bias_max)), min(T - 1, int(bias_max) + 1)):
            for splits in (1, 3):
                got = ops.sigmoid_decode_attention(q[i:i + 1].contiguous(), kp, vp, bt, pos[i:i + 1], scale, splits, None,
                                                   None, table, coef, every, gate[i:i + 1]).double().cpu()
                err = (got[0] - want[i]).abs().max() / want.abs().max()
                assert err <= tol, f"tensor-core single token at {i}, {splits} pieces: {float(err):.3e}"
        got = ops.sigmoid_prefill_attention(q, kp, vp, bt, i32([0, T]), i32([0]), *tiles_of(T), scale).double().cpu()
        bare = pb.sigmoid_attend_fast(q.double().cpu(), k.double().cpu(), v.double().cpu(), scale,
                                      torch.zeros(2, H, dtype=pb.F64), torch.zeros(H, dtype=pb.F64), 4.0, H // G)
        assert (got - bare.reshape(T, H * Vd)).abs().max() <= tol * bare.abs().max()
    # no table, no temperature, no gate: every weight is the sigmoid of the scaled product
    plainest = pb.sigmoid_attend_fast(q.double().cpu(), k.double().cpu(), v.double().cpu(), scale,
                                      torch.zeros(2, H, dtype=pb.F64), torch.zeros(H, dtype=pb.F64), 4.0, H // G)
    got = ops.sigmoid_attention_generic(q, kp, vp, bt, pos, seg, scale).double().cpu()
    assert (got - plainest.reshape(T, H * Vd)).abs().max() <= tol * plainest.abs().max()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,Dv,tau", [(2, 16, 24, 4.0), (3, 40, 8, 1.0), (1, 64, 64, 16.0), (2, 128, 20, 8.0),
                                        (1, 200, 33, 2.0), (4, 7, 5, 32.0), (2, 128, 128, 16.0), (2, 64, 256, 4.0)])
def test_gated_recurrence_portions_and_single_tokens(H, D, Dv, tau, dtype):
    """Decays per key channel and token: channel 0 of head 0 forgets nothing (a logit of +30) and carries the first
    token, made large, to the last of 300 positions; channel 1 forgets everything (-30 under any tau here) although it
    holds the largest keys, so a decay that lands on the wrong channel or on the value axis shows.  The same rows run as
    one portion, token by token, and in uneven portions beside another request; the state slot carries everything."""
    from gesso_b200 import ops
    T = 300
    stride = 2 * H * D + H * Dv + (16 if Dv >= 128 else 11)       # rows on 16-byte boundaries, and not
    q_scale = float(D) ** -0.5
    rows = [torch.randn(T, stride, device=DEV).to(dtype) for _ in range(2)]
    zs = [(2.0 + 3.0 * torch.randn(T, H * D, device=DEV)) for _ in range(2)]
    zb = torch.randn(H * D, device=DEV)
    for r in range(2):
        zs[r][:, 0] = 30.0 - zb[0]
        zs[r][:, 1] = -30.0 * tau - zb[1]
        rows[r][:, H * D + 1] = 5.0                           # large keys on the channel that forgets
    rows[0][0, H * D] = 4.0                                    # the first token's key on the channel that keeps
    rows[0][0, 2 * H * D:2 * H * D + Dv] = 6.0                 # and its values stand out
    want, last = [], []
    for r in range(2):
        x = rows[r].double().cpu()
        qq = x[:, :H * D].view(T, H, D) * q_scale
        kk = x[:, H * D:2 * H * D].view(T, H, D)
        vv = x[:, 2 * H * D:2 * H * D + H * Dv].view(T, H, Dv)
        alpha = torch.sigmoid(zs[r].double().cpu() + zb.double().cpu()).pow(1.0 / tau).view(T, H, D)
        o, S = pb.gla_recurrence(qq, kk, vv, alpha)
        want.append(o.reshape(T, H * Dv))
        last.append(S.transpose(1, 2))                          # the engine keeps [heads, value size, key size]
    tol = 3e-5 if dtype == torch.float32 else 2e-2

    def check(got, r, what):
        err = (got - want[r]).abs().max() / want[r].abs().max()
        assert err <= tol, f"{what}: {float(err):.3e}"
    state = torch.full((3, H, Dv, D), float("nan"), device=DEV)
    state[0].zero_()
    check(ops.gated_linear_attention(rows[0], zs[0], zb, tau, q_scale, state, i32([0, T]), i32([0]), 1, H, D, Dv).double().cpu(),
          0, "one portion")
    assert (state[0].double().cpu() - last[0]).abs().max() <= tol * last[0].abs().max()
    state[2].zero_()
    out = [ops.gated_linear_attention(rows[0][t:t + 1], zs[0][t:t + 1].contiguous(), zb, tau, q_scale, state, i32([0, 1]),
                                      i32([2]), 1, H, D, Dv) for t in range(T)]
    check(torch.cat(out).double().cpu(), 0, "token by token")
    assert (state[2].double().cpu() - last[0]).abs().max() <= tol * last[0].abs().max()
    state[0].zero_()
    state[1].zero_()
    cuts = [1, 2, 17, 1, 64, 3, 100, 2, 45, 65]
    assert sum(cuts) == T
    got, at = [[], []], 0
    for kk_, n in enumerate(cuts):
        order = [0, 1] if kk_ % 2 else [1, 0]
        both = torch.cat([rows[r][at:at + n] for r in order])
        zboth = torch.cat([zs[r][at:at + n] for r in order]).contiguous()
        _, start = segments([n, n])
        y = ops.gated_linear_attention(both, zboth, zb, tau, q_scale, state, start, i32([1 if r == 0 else 0 for r in order]),
                                       2, H, D, Dv)
        for j, r in enumerate(order):
            got[r].append(y[j * n:(j + 1) * n].double().cpu())
        at += n
    for r in range(2):
        check(torch.cat(got[r]), r, f"portions, request {r}")
    # by 64-token tiles side by side: one portion from an empty state, then two requests' uneven portions, the later
    # ones from the state the earlier ones left
    def tiles_of(lens):
        return (i32([s for s, n in enumerate(lens) for _ in range(0, n, 64)]),
                i32([x for n in lens for x in range(0, n, 64)]))
    state[0].zero_()
    check(ops.gated_linear_attention(rows[0], zs[0], zb, tau, q_scale, state, i32([0, T]), i32([0]), 1, H, D, Dv,
                                     *tiles_of([T])).double().cpu(), 0, "one portion by tiles")
    assert (state[0].double().cpu() - last[0]).abs().max() <= tol * last[0].abs().max()
    state[0].zero_()
    state[1].zero_()
    got, at = [[], []], [0, 0]
    for lens in ([130, 64], [1, 171], [169, 65]):
        both = torch.cat([rows[r][at[r]:at[r] + n] for r, n in enumerate(lens)])
        zboth = torch.cat([zs[r][at[r]:at[r] + n] for r, n in enumerate(lens)]).contiguous()
        _, start = segments(lens)
        y = ops.gated_linear_attention(both, zboth, zb, tau, q_scale, state, start, i32([1, 0]), 2, H, D, Dv, *tiles_of(lens))
        got[0].append(y[:lens[0]].double().cpu())
        got[1].append(y[lens[0]:].double().cpu())
        at = [at[0] + lens[0], at[1] + lens[1]]
    assert at == [T, T]
    for r in range(2):
        check(torch.cat(got[r]), r, f"portions by tiles, request {r}")
    assert (state[1].double().cpu() - last[0]).abs().max() <= tol * last[0].abs().max()
    assert (state[0].double().cpu() - last[1]).abs().max() <= tol * last[1].abs().max()
    # without a bias vector
    state[0].zero_()
    y = ops.gated_linear_attention(rows[0], zs[0] + zb, None, tau, q_scale, state, i32([0, T]), i32([0]), 1, H, D, Dv)
    check(y.double().cpu(), 0, "bias folded into the logits")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_a_silu_gate_and_xielu(dtype):
    """The recurrence's read-out normed head by head (one head a thousand times the others, so a statistic over the
    whole row shows) and gated by silu of a view into wider rows; xIELU on both sides of zero, at zero, and where
    exp(z) - 1 - z cancels."""
    from gesso_b200 import ops
    N, H, Dv, eps = 41, 3, 20, 1e-5
    o = torch.randn(N, H * Dv, device=DEV)
    o[:, :Dv] *= 1000.0
    w = 1 + 0.3 * torch.randn(Dv, device=DEV)
    wide = torch.randn(N, H * Dv + 9, device=DEV).to(dtype)
    gate = wide[:, 4:4 + H * Dv]
    got = ops.head_gated_rmsnorm(o, w, eps, gate, H, dtype, gate_act="silu").double().cpu()
    want = pb.head_norm(o.double().cpu().view(N, H, Dv), w.double().cpu(), eps).reshape(N, H * Dv) * pb.silu(gate.double().cpu())
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    assert (got - want).abs().max() <= tol * want.abs().max()
    z = torch.cat([torch.linspace(-12, 6, 1001), torch.tensor([0.0, -0.0, 1e-4, -1e-4, -1e-3, -30.0, 17.0])]).to(DEV).to(dtype)
    for p, q in ((0.3, -0.2), (-2.0, 1.5), (0.0, 0.0)):
        got = ops.xielu(z, torch.tensor([p, q], device=DEV)).double().cpu()
        want = pb.xielu(z.double().cpu(), p, q)
        if dtype == torch.float32:
            assert (got - want).abs().max() <= 2e-6 * want.abs().max() and float(got[1001]) == 0.0
            small = (z.double().cpu().abs() <= 1e-3)
            assert ((got - want)[small].abs() <= 1e-6 * z.double().cpu()[small].abs() + 1e-12).all()   # no cancellation
        else:
            assert ((got - want).abs() <= 8e-3 * want.abs() + 1e-30).all()


@pytest.mark.parametrize("E,top", [(6, 2), (4, 4), (16, 3), (5, 1), (12, 5)])
def test_router_weighs_by_the_softmax_over_the_chosen(E, top):
    """The bias decides: without it expert 0 would never be chosen.  The weights sum to one whatever the other logits
    are (a softmax over all experts would not)."""
    from gesso_b200 import ops
    N, W = 77, 48
    x = torch.randn(N, W, device=DEV)
    wr = torch.randn(E, W, device=DEV) * 0.3
    wr[0] = 0.0
    b = torch.randn(E, device=DEV)
    b[0] = 50.0
    idx, w = ops.moe_route(x, wr, None, top, 1, 1, score="softmax_chosen", logit_bias=b)
    P = {"mlp.router": wr.double().cpu(), "mlp.router.b": b.double().cpu()}
    widx, ww = pb.route(x.double().cpu(), P, top)
    assert torch.equal(idx.cpu().long(), widx) and (idx[:, 0] == 0).all()
    assert (w.double().cpu() - ww).abs().max() <= 1e-5
    assert (w.sum(dim=1) - 1).abs().max() <= 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,W,F,E,top", [(5, 64, 24, 6, 2), (70, 96, 20, 4, 4), (300, 128, 32, 16, 3), (33, 72, 100, 5, 1)])
def test_squared_relu_experts_pairwise_and_grouped(T, W, F, E, top, dtype):
    from gesso_b200 import ops
    x = torch.randn(T, W, device=DEV).to(dtype)
    up = (torch.randn(E, F, W, device=DEV) / math.sqrt(W)).to(dtype)
    down = (torch.randn(E, W, F, device=DEV) / math.sqrt(F)).to(dtype)
    z = torch.randn(T, E, device=DEV)
    vals, idx = torch.topk(z, top, dim=-1)
    w = torch.softmax(vals, dim=-1).contiguous()
    idx = idx.to(torch.int32).contiguous()
    P = {f"mlp.e{e}.up": up[e].double().cpu() for e in range(E)}
    P.update({f"mlp.e{e}.down": down[e].double().cpu() for e in range(E)})
    want = torch.zeros(T, W, dtype=pb.F64)
    xd = x.double().cpu()
    for t in range(T):
        for e, g in zip(idx[t].tolist(), w[t].tolist()):
            want[t] += g * (pb.relu2(xd[t] @ P[f"mlp.e{e}.up"].T) @ P[f"mlp.e{e}.down"].T)
    tol = 3e-5 if dtype == torch.float32 else 2e-2
    got = ops.moe_experts_pairs(x, up, down, idx, w, act="relu2").double().cpu()
    assert (got - want).abs().max() <= tol * want.abs().max()
    if ops.moe_grouped_takes(x, up, down, top, "relu2"):
        got = ops.moe_experts_grouped(x, up, down, idx, w, act="relu2").double().cpu()
        assert (got - want).abs().max() <= tol * want.abs().max()


# ---- whole models ------------------------------------------------------------------------------------------
def test_layer_streams_float32(loaded, plain):
    """The stream after every layer run, in float32: a hook on the blocks copies the stream and adds what the run
    left pending (a looped layer counts every time it runs)."""
    from gesso_b200 import ops
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.trace import make_engine
    for name in cb.MBD:
        model = loaded(name, "float32")
        toks = tt.make_requests(cb.MBD[name][0]["vocab"], [29], seed=3)[0]
        want = plain.models[name].stream(toks)
        eng = make_engine(model, 64, use_graphs=False)
        seen, olds = [], []
        for blk in model.blocks:
            old = blk.forward
            olds.append(old)

            def hooked(h, pending, ctx, cache, old=old):
                out = old(h, pending, ctx, cache)
                s = h.clone()
                ops.flush_pending(s, out)
                seen.append(s.double().cpu())
                return out
            blk.forward = hooked
        try:
            eng.admit("r")
            eng.step([StepEntry("r", toks, [len(toks) - 1])])
        finally:
            for blk, old in zip(model.blocks, olds):
                blk.forward = old
        eng.release("r")
        assert len(seen) == len(want) == len(pb.layer_order(cb.MBD[name][0]))
        for i, (a, b) in enumerate(zip(seen, want)):
            assert (a - b).abs().max() <= 2e-5 * b.abs().max(), f"{name}: layer run {i}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", list(SCHEDULES))
@pytest.mark.parametrize("name", list(cb.MBD))
def test_replay_matches_plain(name, schedule, dtype, loaded, plain, tmp_path):
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES[schedule](reqs)
    model = loaded(name, dtype)
    tt.run_in_process(model, tb, max_tokens, str(tmp_path))
    rows = tt.read_rows(tb, str(tmp_path), model.vocab_size)
    compare(rows, ref, tol_of(name, dtype), f"{name}/{schedule}/{dtype}", plain.margins(name, dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("schedule", ["whole", "portions", "mixed"])
@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_recurrence_by_tiles_in_the_engine(name, schedule, dtype, loaded, plain, tmp_path, monkeypatch):
    """With the threshold lowered, every step whose longest portion has 65 tokens or more runs the recurrence by
    64-token tiles (tile sums, scan, tile outputs) instead of token after token: portions that start from the state
    an earlier portion left, beside single tokens of other requests, on slots that are used again."""
    from gesso_b200 import ops
    monkeypatch.setattr(ops, "GLA_CHUNK_MIN_TOKENS", 65)
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES[schedule](reqs)
    model = loaded(name, dtype)
    tt.run_in_process(model, tb, max_tokens, str(tmp_path))
    rows = tt.read_rows(tb, str(tmp_path), model.vocab_size)
    compare(rows, ref, tol_of(name, dtype), f"tiles {name}/{schedule}/{dtype}", plain.margins(name, dtype))


@pytest.mark.parametrize("sizes", [(2,), (3, 2), (2, 2, 2, 5), (64, 2, 63), (16, 17, 15, 2)])
def test_portions_of_every_size_float32(sizes, loaded, plain, tmp_path):
    """Portions down to two tokens, and cuts on and beside page borders, give the logits of whole prompts."""
    reqs, ref = plain("a")
    tb, max_tokens = tt.trace_portions(reqs, sizes=sizes)
    model = loaded("a", "float32")
    tt.run_in_process(model, tb, max_tokens, str(tmp_path))
    compare(tt.read_rows(tb, str(tmp_path), model.vocab_size), ref, TOL["float32"], f"portions {sizes}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(cb.MBD))
def test_pages_and_slots_used_again(name, dtype, loaded, plain, tmp_path):
    """Every free page and slot filled with NaN before a mixed replay on a pool made for the live requests only,
    with graphs off and on: a recurrence that reads the state the slot's last owner left, or a key of a page's last
    owner, gives NaN."""
    reqs, ref = plain(name)
    tb, max_tokens = SCHEDULES["mixed"](reqs)
    model = loaded(name, dtype)
    for graphs in (False, True):
        d = tmp_path / f"g{int(graphs)}"
        tt.run_in_process(model, tb, max_tokens, str(d), prepare=tt.poison_free_memory, use_graphs=graphs)
        compare(tt.read_rows(tb, str(d), model.vocab_size), ref, tol_of(name, dtype), f"poisoned {name}/{dtype}",
                plain.margins(name, dtype))


def test_schedules_agree_float32(loaded, plain, tmp_path):
    reqs, _ = plain("a")
    model = loaded("a", "float32")
    got = {}
    for sched, make in SCHEDULES.items():
        tb, max_tokens = make(reqs)
        tt.run_in_process(model, tb, max_tokens, str(tmp_path / sched))
        got[sched] = tt.read_rows(tb, str(tmp_path / sched), model.vocab_size)
    for sched, rows in got.items():
        for key, row in rows.items():
            assert row_error(row, got["whole"][key]) <= 2e-5, (sched, key)


@pytest.mark.parametrize("name", ["a", "c"])
def test_long_decoding(name, loaded, plain):
    """Token by token far past the end of every distance table and over many temperature steps; the states carry
    on, and every key stays visible (there is no window: no page is given back before the request ends)."""
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.engine import Engine
    model = loaded(name, "float32")
    toks = tt.make_requests(cb.MBD[name][0]["vocab"], [330], seed=9)[0]
    want = plain.models[name].logits(toks).numpy()
    eng = Engine(model, max_positions=512, page_size=16, num_pages=22, max_requests=2)
    eng.admit("r")
    eng.step([StepEntry("r", toks[:40], [])])
    for p in range(40, 330):
        lg = eng.step([StepEntry("r", [toks[p]], [0])])
        if p % 37 == 0 or p > 320:
            assert row_error(lg[0].cpu().numpy(), want[p]) <= TOL["float32"], p
    assert max(eng.cache.pages_in_use()) == 21
    eng.release("r")
    eng.cache.check_invariants()
    assert all(n == 0 for n in eng.cache.pages_in_use())


@pytest.mark.parametrize("name", list(cb.MBD))
def test_greedy_generation_through_the_session(name, loaded, plain):
    import gesso_b200
    model = loaded(name, "float32")
    s = gesso_b200.Session(model, context_length=256, page_size=16, max_batch=4)
    prompts = tt.make_requests(cb.MBD[name][0]["vocab"], [9, 1, 60, 2], seed=21)
    for p in prompts:
        assert s.generate(p, max_new_tokens=6) == plain.models[name].greedy(p, 6)
    res = s.run_batch([gesso_b200.BatchRequest(p, max_new_tokens=6) for p in prompts])
    for p, r in zip(prompts, res):
        assert list(r.ids) == plain.models[name].greedy(p, 6)
    assert all(n == 0 for n in s.engine.cache.pages_in_use())


def random_mabidra_config(seed):
    """Seeded random configurations: any order of the two mixers, any head layout, values wider and narrower than
    keys, distance tables that end inside and beyond the prompts, temperatures that step often and never,
    feed-forwards of both kinds and none, any number of norm groups, a loop anywhere (or none) of one to three
    passes.  Returns the configuration, the sizes only the checkpoint decides, and the prompt lengths."""
    import random
    r = random.Random(seed)
    groups = r.choice([1, 2, 3, 4, 6])
    bias_rows = r.choice([2, 4, 7, 12, 32])
    width = groups * r.choice([8, 10, 16, 24])
    n_layers = r.randint(1, 4)

    def mlp():
        kind = r.choice(["dense", "moe", "moe", None])
        if kind is None:
            return None
        if kind == "dense":
            return cb.dense(r.choice([8, 24, 50, 64]))
        experts = r.randint(2, 9)
        return cb.moe(r.choice([8, 12, 40]), experts, r.randint(1, experts))
    layers = []
    for i in range(n_layers):
        if r.random() < 0.45:
            layers.append(cb.gla(r.randint(1, 4), r.choice([4, 7, 16, 33, 64]), r.choice([4, 9, 16, 32, 70]),
                                 r.choice([1.0, 2.0, 7.5, 16.0]), mlp()))
        else:
            g = r.randint(1, 3)
            layers.append(cb.attention(g * r.randint(1, 4), g, r.choice([2, 6, 16, 32, 64, 130]),
                                       r.choice([2, 6, 16, 32, 64, 130]), r.choice([0.1, 0.25, 0.5]),
                                       r.choice([x for x in (3.5, 12, 40, 129, 1000) if x > bias_rows // 2]),
                                       r.choice([0.0, 0.2, 0.6]),
                                       r.choice([1, 5, 16, 64, 1000]), mlp()))
    loop = None
    if r.random() < 0.7:
        start = r.randint(0, n_layers - 1)
        loop = {"start": start, "stop": r.randint(start + 1, n_layers), "times": r.randint(1, 3)}
    cfg = cb.config(r.randint(40, 300), width, r.choice([0.5, 1.0, 3.0]), r.choice([1e-5, 1e-6]), groups, layers, loop)
    sizes = {"decay_rank": r.choice([1, 3, 8, 16]), "bias_rows": bias_rows}
    return cfg, sizes, [r.randint(1, 140) for _ in range(5)]


@pytest.mark.parametrize("seed", [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 13, 15, 17])
def test_random_configuration_replays_like_plain(seed, tmp_path):
    import gesso_b200
    cfg, sizes, lengths = random_mabidra_config(seed)
    d = str(tmp_path / "model")
    pb.write_model(d, cfg, seed, **sizes)
    plain_model = pb.PlainMabidra.from_dir(d)
    reqs = tt.make_requests(cfg["vocab"], lengths, seed=seed)
    ref = [plain_model.logits(t).numpy() for t in reqs]
    margins = [plain_model.margins(t).numpy() for t in reqs] if seed % 2 else None      # bfloat16 for every other seed
    for dtype in ("float32", "bfloat16") if margins is not None else ("float32",):
        model = gesso_b200.load(d, dtype=dtype, max_positions=256)
        for name, make in SCHEDULES.items():
            tb, max_tokens = make(reqs)
            out = str(tmp_path / f"{dtype}_{name}")
            tt.run_in_process(model, tb, max_tokens, out)
            compare(tt.read_rows(tb, out, cfg["vocab"]), ref, TOL_RANDOM[dtype], f"seed {seed} {name} {dtype} {cfg}",
                    margins if dtype == "bfloat16" else None)
        del model


@pytest.mark.parametrize("which", ["MBD_ONLY_STATE", "MBD_ONLY_PAGES", "MBD_ONE_PASS"])
def test_stacks_of_one_kind_of_cache_and_a_loop_of_one_pass(which, tmp_path):
    """A model without any pages, one without any state and one whose loop runs once go through the same engine, in
    both run types."""
    import gesso_b200
    cfg = getattr(cb, which)
    d = str(tmp_path / "model")
    pb.write_model(d, cfg, 4, decay_rank=3, bias_rows=8)
    plain_model = pb.PlainMabidra.from_dir(d)
    reqs = tt.make_requests(cfg["vocab"], [33, 1, 70, 18], seed=8)
    ref = [plain_model.logits(t).numpy() for t in reqs]
    for dtype in ("float32", "bfloat16"):
        model = gesso_b200.load(d, dtype=dtype, max_positions=256)
        for name, make in SCHEDULES.items():
            tb, max_tokens = make(reqs)
            out = str(tmp_path / f"{dtype}_{name}")
            tt.run_in_process(model, tb, max_tokens, out)
            compare(tt.read_rows(tb, out, cfg["vocab"]), ref, TOL[dtype], f"{which} {name} {dtype}")
        del model


def test_layer_widths_of_a_real_model():
    """Width 1,024, 16 heads of 64, recurrences of 8 heads of 64 x 128, 16 experts, the middle layers run twice: a
    prompt of 1,300 tokens takes the paths that only large steps take.  Cut into portions the float32 engine gives
    the same logits as in one step; the bfloat16 engine agrees with the float32 one within rounding (bfloat16 matrix
    products through eight layer runs leave the median row between one and two hundredths; single rows may sit on a
    router's close call, and the last bit of an attention weight decides which)."""
    import gesso_b200
    from gesso_b200.engine.batch import StepEntry
    from gesso_b200.engine.trace import make_engine
    moe = cb.moe(512, 16, 4)
    layers = [cb.gla(8, 64, 128, 16.0, cb.dense(2048)),
              cb.attention(16, 4, 64, 64, 0.125, 512, 0.3, 256, moe),
              cb.attention(16, 2, 64, 64, 0.125, 2000, 0.1, 100, cb.dense(2048)),
              cb.gla(8, 64, 128, 8.0, moe)]
    cfg = cb.config(1024, 1024, 1.0, 1e-6, 4, layers, loop={"start": 1, "stop": 3, "times": 2})
    T = 1300
    toks = tt.make_requests(1024, [T], seed=1)[0]
    want = list(range(0, T, 37)) + [T - 1]
    res = {}
    for dtype in ("float32", "bfloat16"):
        model = gesso_b200.random_model(cfg, seed=0, dtype=dtype, max_positions=2048, style="fan_in")
        for mode, cuts in (("whole", [T]), ("portions", [1100, 2, 64, 100, 1, 1, 30, 2])):
            eng = make_engine(model, 2048)
            eng.admit("a")
            rows, at = [], 0
            for c in cuts:
                w = [p - at for p in want if at <= p < at + c]
                lg = eng.step([StepEntry("a", toks[at:at + c], w)])
                if w:
                    rows.append(lg.float().cpu().numpy().copy())
                at += c
            eng.check_status()
            eng.release("a")
            res[(dtype, mode)] = np.concatenate(rows, 0)
        del model
        torch.cuda.empty_cache()
    ref = res[("float32", "whole")]
    errs = lambda a: np.array([row_error(x, y) for x, y in zip(a, ref)])
    assert np.isfinite(ref).all() and errs(res[("float32", "portions")]).max() <= 2e-5
    for mode in ("whole", "portions"):
        e = errs(res[("bfloat16", mode)])
        assert np.median(e) <= 0.02 and np.percentile(e, 80) <= 0.04, (mode, float(np.median(e)), float(e.max()))


def test_trace_program_on_a_model_folder(mbd_dirs, plain, tmp_path):
    reqs, ref = plain("b")
    tb, max_tokens = tt.trace_mixed(reqs, seed=2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    p = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", mbd_dirs["b"], "--dtype", "bfloat16",
                        "--out", str(out), "--max-tokens", str(max_tokens)], input=tb.text(), capture_output=True, text=True,
                       timeout=900)
    assert p.returncode == 0, p.stderr[-2000:]
    compare(tt.read_rows(tb, str(out), cb.MBD_B["vocab"]), ref, TOL["bfloat16"], "trace program b/mixed",
            plain.margins("b", "bfloat16"))
