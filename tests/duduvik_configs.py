"""
Small Duduvik configurations for the tests, as config.json dictionaries.  They differ from one another
in every size and in the order of layers: widths and head counts that are not powers of two, key and
value sizes that differ, a rotation over part of a head, several windows (shorter and longer than a
cache page), experts with top 1, 2 and 3, with and without a shared expert, a layer without a
feed-forward, a model without any attention layer, and an embedding scale of one.
"""


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, window, scale, base=10000.0):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
                      "mask": {"size": window}, "scale": scale, "rot": {"base": base, "dims": rot_dim}}}


def gla(heads, dim, vdim, tau, decay_rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "decay_rank": decay_rank}}


def retention(heads, dim, vdim, decay, rot_dims, base=10000.0):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay,
                                           "rot": {"base": base, "dims": rot_dims}}}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, limit, shared=None):
    out = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def model(vocab, width, scale, eps, layers):
    return {"architecture": "Duduvik", "vocab": vocab, "width": width, "embedding": {"scale": scale}, "norm": {"eps": eps},
            "layers": [dict(mixer, mlp=mlp) for mixer, mlp in layers]}


# every mechanism, windows of 21 (inside one 16-token page and a bit) and 50, a layer without feed-forward
MIXED = model(300, 96, 7.0, 1e-5, [
    (gla(2, 24, 40, 8.0, 12), moe(6, 3, 40, 2.0, shared=(56, 0.75))),
    (latent(3, 16, 8, 24, 40, 48, 21, 0.2), dense(136)),
    (retention(3, 32, 16, [0.9, 0.97, 0.995], 16, base=5000.0), None),
    (latent(2, 24, 12, 8, 24, 36, 50, 0.15, base=777.0), moe(5, 1, 24, 1.25)),
    (gla(3, 16, 16, 3.0, 5), dense(80)),
])

# no attention layer at all: the model needs state slots only, no page
RECURRENT = model(211, 64, 1.0, 1e-6, [
    (retention(2, 24, 40, [0.75, 0.9990234375], 24), moe(4, 2, 48, 1.0, shared=(32, 3.0))),
    (gla(1, 40, 72, 20.0, 8), None),
])

# attention only, odd sizes: cache rows of 44 elements, a window of 5, one head, one expert choice of two
LATENT_ONLY = model(150, 72, 3.0, 1e-5, [
    (latent(5, 12, 4, 20, 28, 40, 5, 0.3), moe(2, 1, 16, 0.5, shared=(24, 1.5))),
    (latent(1, 40, 16, 40, 16, 24, 33, 0.11, base=100.0), dense(100)),
])

# sizes the bfloat16 kernels for a few tokens take (widths that are multiples of 32)
WIDE = model(512, 128, 4.0, 1e-6, [
    (latent(4, 32, 32, 32, 64, 64, 70, 0.125), dense(256)),
    (gla(2, 64, 64, 16.0, 32), moe(8, 2, 64, 1.5, shared=(96, 1.0))),
    (retention(4, 32, 64, [0.96875, 0.984375, 0.9921875, 0.99609375], 32, base=1000000.0), dense(192)),
])

WEIGHTS = {"std": 0.08, "unit_std": 0.25}
