"""
Small Nipizen configurations for the tests, as config.json dictionaries.  They differ from one another
in every size and in the order of layers: widths and head counts that are not powers of two, key and
value sizes that differ (and, once, agree), rotation over part of a head and over all of it, with and
without YaRN rescaling, fewer q/k heads than value heads in the delta rule, convolutions of 2, 3 and
4 taps, experts with top 1, 2 and 3, a layer without a feed-forward, a model of matrix memories only.
"""


def attention(heads, kv_heads, dim, vdim, scale, rot_dims, base=10000.0, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": rot}


def delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def parallel(left, right, left_scale, right_scale):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}}


def mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def moe(experts, top, ff):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}


def model(vocab, width, eps, layers):
    return {"architecture": "Nipizen", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}


# every mechanism; odd sizes; a layer without a feed-forward
MIXED = model(300, 96, 1e-5, [
    (parallel(attention(4, 2, 24, 40, 0.2, 16, base=5000.0, scaling=(4.0, 64, 16.0, 2.0)), delta(4, 2, 20, 24, 3, 10, 6), 0.7, 1.3),
     moe(6, 2, 40)),
    (mlstm(3, 24, 40, 10.0), moe(5, 3, 24)),
    (parallel(attention(3, 3, 16, 16, 0.3, 16), delta(2, 1, 40, 8, 2, 5, 12), 1.5, 0.4), None),
    (mlstm(1, 72, 24, 15.0), moe(4, 1, 32)),
])

# matrix memories only: the model needs state slots, no page
RECURRENT = model(211, 64, 1e-6, [
    (mlstm(2, 24, 40, 6.0), moe(4, 2, 48)),
    (mlstm(4, 8, 16, 20.0), None),
])

# sizes the bfloat16 kernels for a few tokens and the tensor-core attention take (widths that are multiples of
# 32, keys and values of 64 channels a head on pages of 64 tokens)
WIDE = model(512, 128, 1e-6, [
    (parallel(attention(4, 2, 64, 64, 0.125, 32, scaling=(8.0, 128, 32.0, 1.0)), delta(4, 4, 32, 32, 4, 16, 16), 1.0, 1.0),
     moe(8, 2, 64)),
    (mlstm(2, 64, 64, 15.0), moe(8, 1, 96)),
    (parallel(attention(2, 1, 32, 96, 0.18, 8), delta(2, 2, 64, 64, 4, 8, 8), 0.5, 2.0), moe(3, 3, 32)),
])

# heads of 128 channels, three query heads a key/value head (the tensor-core attention's other head size)
GROUPED = model(257, 128, 1e-5, [
    (parallel(attention(6, 2, 128, 128, 0.09, 64, scaling=(2.0, 256, 16.0, 4.0)), delta(2, 2, 32, 32, 4, 8, 8), 0.9, 1.1), moe(4, 2, 32)),
])

WEIGHTS = {"std": 0.08, "unit_std": 0.25}
