"""Tiny Todupel configurations for tests: config.json dicts that differ in every size, constant and layer order."""


def _mixer(heads, kv_heads, dim, vdim, scale=None, softcap=None, diff=0.4, q_temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "diff": diff}
    if scale is not None:
        m["scale"] = scale
    if softcap is not None:
        m["softcap"] = softcap
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _layer(mixer, ff):
    return {"type": "attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


# Two groups of two heads, values twice as wide as a map, the third layer reads the first layer's keys and values;
# a temperature that changes every 8 positions and a cap low enough to bend the scores.
T_A = {"architecture": "Todupel", "vocab": 300, "width": 96, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(4, 2, 16, 32, 0.25, 6.0, 0.3, (0.5, 8)), 160),
    _layer(_mixer(4, 2, 16, 32, 0.25, 6.0, 0.3, (0.5, 8)), 160),
    _layer(_mixer(4, 2, 16, 32, 0.25, 6.0, 0.3, (0.5, 8), kv_from=0), 160),
]}

# Three heads to a key/value head, values narrower than a map, a layer without a feed-forward, layers that differ
# from one another in every constant, a temperature step of 5 (no power of two).
T_B = {"architecture": "Todupel", "vocab": 257, "width": 80, "norm": {"eps": 3e-5}, "layers": [
    _layer(_mixer(6, 2, 48, 16, 0.2, 3.0, 0.6, (0.7, 5)), 112),
    _layer(_mixer(3, 1, 32, 48, 0.3, 20.0, 0.2, (0.1, 13)), None),
    _layer(_mixer(6, 2, 48, 16, 0.15, 40.0, 0.55, (1.0, 3), kv_from=0), 64),
]}

# One head per key/value head, maps and values of one size (64: the widest tile paths), no cap and no temperature
# (keys left out), the default scale, two chains of layers that share keys and values, eps of another size.
T_C = {"architecture": "Todupel", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    _layer(_mixer(2, 2, 64, 64), 136),
    _layer(_mixer(2, 2, 64, 64, kv_from=0), 136),
    _layer(_mixer(2, 2, 64, 64), 136),
    _layer(_mixer(2, 2, 64, 64, kv_from=2), None),
]}

# Sizes that defeat every vector path: a width, map size, value size and inner width that are no multiples of 8, an
# odd vocabulary, five heads on one key/value head, a single layer.
T_D = {"architecture": "Todupel", "vocab": 301, "width": 100, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(5, 1, 20, 36, 0.22, 8.0, 0.45, (0.4, 7)), 172),
]}

# Wide heads: maps and values of 128, eight heads on two key/value heads.
T_E = {"architecture": "Todupel", "vocab": 272, "width": 64, "norm": {"eps": 1e-5}, "layers": [
    _layer(_mixer(8, 2, 128, 128, 0.09, 30.0, 0.35, (0.25, 16)), 96),
    _layer(_mixer(8, 2, 128, 128, 0.09, 30.0, 0.35, (0.25, 16), kv_from=0), 96),
]}

TODUPEL = {"ta": (T_A, 21), "tb": (T_B, 22), "tc": (T_C, 23), "td": (T_D, 24), "te": (T_E, 25)}
