"""Tiny Mabidra configurations of the tests.  They differ in every size and option."""


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def gla(heads, dim, vdim, tau, mlp):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "mlp": mlp}


def attention(heads, kv, dim, vdim, scale, bias_max, coef, every, mlp):
    return {"type": "attention", "mlp": mlp,
            "mixer": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": bias_max,
                      "q_temp": {"coef": coef, "every": every}}}


def config(vocab, width, scale, eps, groups, layers, loop=None):
    return {"architecture": "Mabidra", "vocab": vocab, "width": width, "embedding": {"scale": scale},
            "norm": {"eps": eps, "groups": groups}, "loop": loop, "layers": layers}


# both mixers, both feed-forwards and a layer without one; the loop runs the two attention layers twice (it starts
# behind the first layer and ends before the last); distance tables that end well inside the prompts; a query
# temperature that steps every 8 positions; values wider than keys in the recurrence.
MBD_A = config(131, 64, 0.7, 1e-5, 2, [
    gla(2, 16, 24, 4.0, dense(80)),
    attention(4, 2, 16, 16, 0.3, 40, 0.4, 8, moe(24, 6, 2)),
    attention(2, 1, 32, 32, 0.2, 100, 0.2, 50, dense(40)),
    gla(2, 16, 24, 8.0, None),
], loop={"start": 1, "stop": 3, "times": 2})

# sizes that are no multiples of 8 or powers of two; one norm group; embedding scale one; as many kv heads as heads;
# values wider than keys in attention and narrower in the recurrence; tau one (the decay is the sigmoid itself);
# a temperature that steps at every position; a distance limit that is no whole number; every expert chosen;
# no loop.
MBD_B = config(257, 96, 1.0, 1e-6, 1, [
    attention(3, 3, 10, 40, 0.4, 9.5, 0.25, 1, moe(20, 4, 4)),
    gla(3, 40, 8, 1.0, moe(20, 5, 1)),
    attention(1, 1, 48, 24, 0.15, 300, 0.0, 7, dense(72)),
])

# sizes the tensor-core paths take (heads of 32 and 64 with values as wide, widths in multiples of 16, many (token,
# expert) pairs); the loop is the whole stack, three times; eight query heads on one kv head.
MBD_C = config(300, 128, 0.5, 1e-6, 4, [
    attention(4, 2, 64, 64, 0.125, 64, 0.3, 32, moe(32, 16, 3)),
    gla(2, 64, 64, 16.0, moe(32, 16, 3)),
    attention(8, 1, 32, 32, 0.18, 33, 0.5, 16, dense(96)),
], loop={"start": 0, "stop": 3, "times": 3})

# a loop of one pass over one layer in the middle (the re-entry mix still happens once); stacks with states only and
# with pages only
MBD_ONE_PASS = config(90, 48, 2.0, 1e-5, 3, [
    gla(1, 24, 8, 2.0, dense(32)), attention(2, 2, 8, 8, 0.35, 20, 0.1, 4, None), gla(3, 8, 16, 3.0, None),
], loop={"start": 1, "stop": 2, "times": 1})
MBD_ONLY_STATE = config(90, 48, 1.5, 1e-6, 2, [gla(3, 8, 16, 2.0, dense(32)), gla(1, 24, 8, 32.0, None)],
                        loop={"start": 0, "stop": 1, "times": 2})
MBD_ONLY_PAGES = config(90, 48, 0.8, 1e-6, 6, [attention(2, 1, 8, 12, 0.3, 25, 0.3, 3, None),
                                                attention(6, 3, 16, 24, 0.2, 70, 0.0, 1, dense(64))])

# name -> (config, seed, {sizes the checkpoint alone decides})
MBD = {"a": (MBD_A, 31, {"decay_rank": 5, "bias_rows": 12}), "b": (MBD_B, 32, {"decay_rank": 1, "bias_rows": 6}),
       "c": (MBD_C, 33, {"decay_rank": 16, "bias_rows": 20})}
