"""A plain, slow Todupel for tests: whole sequences in float64 with NumPy, one function per mechanism.

It shares no code with `dynalm_b200`: it reads config.json and model.safetensors by itself. Notation: n tokens,
H query heads in G groups (one key/value head per group), two score maps per head, d = per-map query/key size,
e = value size. Every function takes and returns arrays; `PlainTodupel.logits` strings them together, and
`PlainTodupel.logits_stepwise` runs the same model one token at a time from explicit per-layer lists of past keys
and values, so that the whole-sequence functions are checked against a second reading of the same equations.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Sequence

import numpy as np


def read_tensors(path: str) -> Dict[str, np.ndarray]:
    """A safetensors file: 8-byte little-endian header length, JSON header, data. Floats come back as float64."""
    with open(path, "rb") as f:
        raw = f.read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    data = raw[8 + hlen:]
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        lo, hi = e["data_offsets"]
        buf = data[lo:hi]
        if e["dtype"] == "F32":
            a = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif e["dtype"] == "BF16":
            a = (np.frombuffer(buf, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        elif e["dtype"] == "I32":
            a = np.frombuffer(buf, dtype="<i4").copy()
        else:
            raise ValueError(f"dtype {e['dtype']} of {name}")
        out[name] = a.reshape(e["shape"])
    return out


# --------------------------------------------------------------------------------------------
# mechanisms
# --------------------------------------------------------------------------------------------

def rms_norm(x: np.ndarray, eps: float, weight: Optional[np.ndarray] = None) -> np.ndarray:
    """x / sqrt(mean(x^2) + eps) over the last axis, times `weight` when there is one."""
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y * weight if weight is not None else y


def query_temperature(positions: np.ndarray, coef: float, every: int) -> np.ndarray:
    """The factor a query at position p is multiplied by: 1 + coef * ln(floor((p + 1) / every) + 1)."""
    return 1.0 + coef * np.log(np.floor((positions + 1) / every) + 1.0)


def capped(scores: np.ndarray, cap: float) -> np.ndarray:
    """cap * tanh(scores / cap); cap 0 means none."""
    return cap * np.tanh(scores / cap) if cap else scores


def causal_softmax(scores: np.ndarray, q_pos: np.ndarray, k_pos: np.ndarray) -> np.ndarray:
    """Softmax over the keys j with k_pos[j] <= q_pos[i], row by row; scores [queries, keys]."""
    seen = k_pos[None, :] <= q_pos[:, None]
    s = np.where(seen, scores, -np.inf)
    s = s - s.max(axis=-1, keepdims=True)
    w = np.exp(s)
    return w / w.sum(axis=-1, keepdims=True)


def diff_lambda(lq1, lk1, lq2, lk2, init: float) -> float:
    return math.exp(float(np.dot(lq1, lk1))) - math.exp(float(np.dot(lq2, lk2))) + init


def diff_combine(a1: np.ndarray, a2: np.ndarray, lam: float, init: float, eps: float) -> np.ndarray:
    """The two maps' outputs of one head -> the head's output: difference, unit RMS over the values, (1 - init)."""
    return rms_norm(a1 - lam * a2, eps) * (1.0 - init)


def map_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, q_pos, k_pos, scale: float, cap: float) -> np.ndarray:
    """One score map of one head: q [nq, d], k [nk, d], v [nk, e] -> [nq, e]."""
    return causal_softmax(capped((q @ k.T) * scale, cap), q_pos, k_pos) @ v


def relu2_mlp(h: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    z = np.maximum(h @ up.T, 0.0)
    return (z * z) @ down.T


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------

class PlainTodupel:
    def __init__(self, folder: str):
        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_tensors(os.path.join(folder, "model.safetensors"))
        self.eps = float(self.cfg["norm"]["eps"])
        self.vocab = int(self.cfg["vocab"])

    # -- per layer -------------------------------------------------------------------------
    def queries(self, i: int, h: np.ndarray, positions: np.ndarray) -> np.ndarray:
        """[n, H, 2, d]: projected, normalised per head and map, scaled by the temperature of the position."""
        m = self.cfg["layers"][i]["mixer"]
        q = (h @ self.w[f"l{i}.mix.q"].T).reshape(len(h), m["heads"], 2, m["dim"])
        q = rms_norm(q, self.eps, self.w[f"l{i}.mix.q.norm"])
        t = m.get("q_temp")
        if t:
            q = q * query_temperature(positions, t["coef"], t["every"])[:, None, None, None]
        return q

    def keys_values(self, i: int, h: np.ndarray):
        """([n, G, 2, d] normalised keys, [n, G, e] values) of a layer that has projections of its own."""
        m = self.cfg["layers"][i]["mixer"]
        g = m.get("kv_heads", m["heads"])
        k = (h @ self.w[f"l{i}.mix.k"].T).reshape(len(h), g, 2, m["dim"])
        v = (h @ self.w[f"l{i}.mix.v"].T).reshape(len(h), g, m.get("vdim", m["dim"]))
        return rms_norm(k, self.eps, self.w[f"l{i}.mix.k.norm"]), v

    def attend(self, i: int, q: np.ndarray, k: np.ndarray, v: np.ndarray, q_pos, k_pos) -> np.ndarray:
        """q [nq, H, 2, d] over k [nk, G, 2, d], v [nk, G, e] -> [nq, H * e]."""
        m = self.cfg["layers"][i]["mixer"]
        heads, groups = m["heads"], m.get("kv_heads", m["heads"])
        init = float(m.get("diff", 0.0))
        scale = float(m.get("scale", m["dim"] ** -0.5))
        cap = float(m.get("softcap", 0.0))
        p = f"l{i}.mix."
        lam = diff_lambda(self.w[p + "lq1"], self.w[p + "lk1"], self.w[p + "lq2"], self.w[p + "lk2"], init)
        out = []
        for hd in range(heads):
            g = hd // (heads // groups)
            a1 = map_attention(q[:, hd, 0], k[:, g, 0], v[:, g], q_pos, k_pos, scale, cap)
            a2 = map_attention(q[:, hd, 1], k[:, g, 1], v[:, g], q_pos, k_pos, scale, cap)
            out.append(diff_combine(a1, a2, lam, init, self.eps))
        return np.concatenate(out, axis=-1)

    def layer(self, i: int, x: np.ndarray, q_pos: np.ndarray, kv: dict, k_pos: np.ndarray) -> np.ndarray:
        """x [n, width] at positions q_pos -> the layer's output. `kv[j]` = (keys, values) of every position in
        k_pos that layer j has seen; a layer with projections of its own appends to its entry first."""
        spec = self.cfg["layers"][i]
        h = rms_norm(x, self.eps, self.w[f"l{i}.norm1"])
        src = spec["mixer"].get("kv_from")
        if src is None:
            k_new, v_new = self.keys_values(i, h)
            if i in kv:
                kv[i] = (np.concatenate([kv[i][0], k_new]), np.concatenate([kv[i][1], v_new]))
            else:
                kv[i] = (k_new, v_new)
            src = i
        k, v = kv[src]
        mix = self.attend(i, self.queries(i, h, q_pos), k, v, q_pos, k_pos) @ self.w[f"l{i}.mix.o"].T
        ff = 0.0
        if spec.get("mlp"):
            ff = relu2_mlp(rms_norm(x, self.eps, self.w[f"l{i}.norm2"]), self.w[f"l{i}.mlp.up"], self.w[f"l{i}.mlp.down"])
        return x + (mix + ff)

    def head(self, x: np.ndarray) -> np.ndarray:
        return rms_norm(x, self.eps, self.w["final.norm"]) @ self.w["head"].T

    # -- whole sequences ---------------------------------------------------------------------
    def hidden(self, tokens: Sequence[int], per_layer: Optional[list] = None) -> np.ndarray:
        x = self.w["embed"][np.asarray(tokens, dtype=np.int64)]
        pos = np.arange(len(tokens))
        kv: dict = {}
        for i in range(len(self.cfg["layers"])):
            x = self.layer(i, x, pos, kv, pos)
            if per_layer is not None:
                per_layer.append(x.copy())
        return x

    def logits(self, tokens: Sequence[int]) -> np.ndarray:
        """[n, vocab]: the logits after every token of the sequence."""
        return self.head(self.hidden(tokens))

    def logits_stepwise(self, tokens: Sequence[int]) -> np.ndarray:
        """The same, one token at a time over growing lists of past keys and values."""
        kv: dict = {}
        rows = []
        for p, tok in enumerate(tokens):
            x = self.w["embed"][np.asarray([tok])]
            for i in range(len(self.cfg["layers"])):
                x = self.layer(i, x, np.asarray([p]), kv, np.arange(p + 1))
            rows.append(self.head(x)[0])
        return np.stack(rows)

    def greedy(self, prompt: Sequence[int], n: int) -> List[int]:
        seq = list(prompt)
        for _ in range(n):
            seq.append(int(np.argmax(self.logits(seq)[-1])))
        return seq[len(prompt):]
