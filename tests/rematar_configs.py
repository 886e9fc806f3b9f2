"""Tiny Rematar configurations for tests: config.json dicts that differ in every size, constant and layer order."""


def ssm(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, window=None, base=10000.0, dims=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if dims is not None:
        m["rot"] = {"base": base, "dims": dims}
    return m


def layer(kind, mixer, ff, weights_of=None):
    out = {"type": kind, "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}
    if weights_of is not None:
        out["weights_of"] = weights_of
    return out


_SA = ssm(6, 16, 24, 3, 3, 3)
_LA = latent(4, 16, 8, 24, 40, 48, 14.0, window=20, dims=8)
# Attention first, then recurrences; two layers that run with earlier layers' tensors (one of each kind); three heads
# to a group, three normed parts, three taps; a window a little longer than a page; a stream weight of 2.
R_A = {"architecture": "Rematar", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "postln_alpha": 2.0,
       "embedding": {"scale": 4.0}, "layers": [
           layer("latent_attention", _LA, 160),
           layer("mamba2", _SA, 160),
           layer("mamba2", _SA, 160, weights_of=1),
           layer("latent_attention", _LA, 160, weights_of=0),
       ]}

# Sizes that defeat every vector path (a width that is no multiple of 8, odd head sizes, an odd vocabulary), one group
# for five heads, two taps, one normed part, a window shorter than a page, a rotation that leaves a part of the rotated
# piece unturned, a layer without a feed-forward, no stream weight and no embedding scale.
R_B = {"architecture": "Rematar", "vocab": 257, "width": 100, "norm": {"eps": 3e-5}, "layers": [
    layer("mamba2", ssm(5, 20, 12, 1, 2, 1), 172),
    layer("latent_attention", latent(3, 20, 12, 28, 36, 44, 9.0, window=7, base=500.0, dims=8), None),
    layer("mamba2", ssm(5, 20, 12, 1, 2, 1), None),
]}

# What another model may make equal or 1: a group per head, a single tap (nothing of the convolution is kept), a
# window no request reaches, a layer without a window and one without a rotation, value size equal to the key size,
# a chain of three layers on one set of tensors.
R_C = {"architecture": "Rematar", "vocab": 320, "width": 64, "norm": {"eps": 1e-6}, "postln_alpha": 0.5,
       "embedding": {"scale": 0.25}, "layers": [
           layer("mamba2", ssm(4, 8, 16, 4, 1, 2), 72),
           layer("latent_attention", latent(2, 32, 16, 32, 24, 32, 20.0, window=500, base=1e6, dims=16), 72),
           layer("latent_attention", latent(2, 32, 16, 32, 24, 32, 20.0, base=1e6, dims=16), 72),
           layer("latent_attention", latent(5, 8, 4, 8, 16, 24, 25.0, window=33), None),
           layer("mamba2", ssm(4, 8, 16, 4, 1, 2), 72, weights_of=0),
           layer("mamba2", ssm(4, 8, 16, 4, 1, 2), 72, weights_of=4),
       ]}

# Wide pieces: a state of 128 rows and heads of 64 channels, five taps, a latent wider than a block of threads, a
# window of exactly four pages.
R_D = {"architecture": "Rematar", "vocab": 272, "width": 128, "norm": {"eps": 1e-5}, "postln_alpha": 3.0,
       "embedding": {"scale": 11.0}, "layers": [
           layer("mamba2", ssm(2, 64, 128, 1, 5, 4), 96),
           layer("latent_attention", latent(2, 64, 32, 64, 72, 320, 6.0, window=64, dims=32), 96),
           layer("mamba2", ssm(3, 48, 40, 3, 4, 1), None),
       ]}

REMATAR = {"ra": (R_A, 41), "rb": (R_B, 42), "rc": (R_C, 43), "rd": (R_D, 44)}
