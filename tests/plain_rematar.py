"""A plain, slow Rematar for tests: float64 NumPy, one function per mechanism.

It shares no code with `dynalm_b200`: it reads config.json and model.safetensors by itself. `PlainRematar.logits`
runs whole sequences; `PlainRematar.logits_stepwise` runs the same model one token at a time from explicit
per-layer state (the recurrent matrix and the last convolution inputs of a state-space layer, the cached latents and
rotated keys of an attention layer), so that the whole-sequence functions are checked against a second reading of
the same equations.

Notation. n tokens, width W. State-space mixer: H heads of P channels each, N state rows, G groups of heads that
share B and C, K taps. Latent attention: H heads, d unrotated and r rotated query/key sizes, e value size, R latent
size, window w.
"""

from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional

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
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y * weight if weight is not None else y


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: np.ndarray) -> np.ndarray:
    return z / (1.0 + np.exp(-z))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z: np.ndarray) -> np.ndarray:
    return np.logaddexp(0.0, z)


def dense_mlp(h: np.ndarray, up: np.ndarray, down: np.ndarray) -> np.ndarray:
    return gelu_tanh(h @ up.T) @ down.T


def sum_then_norm(x: np.ndarray, y: np.ndarray, alpha: float, eps: float, weight: np.ndarray,
                  layer_scale: Optional[np.ndarray] = None) -> np.ndarray:
    """The norm after the sum: norm(alpha * x + s * y) * weight, s the per-channel scale of the sublayer's result."""
    return rms_norm(alpha * x + (y * layer_scale if layer_scale is not None else y), eps, weight)


def causal_conv(u: np.ndarray, taps: np.ndarray, bias: np.ndarray, before: Optional[np.ndarray] = None) -> np.ndarray:
    """Per-channel causal convolution. u [n, C]; taps [C, K], the last column is the current token's; `before`
    [K - 1, C] are the inputs in front of u (zeros at the start of a sequence)."""
    n, C = u.shape
    K = taps.shape[1]
    front = np.zeros((K - 1, C)) if before is None else before
    full = np.concatenate([front, u], axis=0)
    out = np.tile(bias, (n, 1)).astype(np.float64)
    for k in range(K):
        out += full[k:k + n] * taps[:, k]
    return out


def ssm_scan(x: np.ndarray, dt: np.ndarray, B: np.ndarray, C: np.ndarray, a_log: np.ndarray, D: np.ndarray,
             state: Optional[np.ndarray] = None):
    """The recurrence of every head. x [n, H, P], dt [n, H] (after softplus), B and C [n, H, N] (already spread
    from groups to heads), state [H, N, P] or None for zeros. Returns (y [n, H, P], the state after the last token)."""
    n, H, P = x.shape
    N = B.shape[-1]
    S = np.zeros((H, N, P)) if state is None else state.copy()
    y = np.zeros((n, H, P))
    rate = np.exp(a_log)
    for t in range(n):
        decay = np.exp(-rate * dt[t])                                       # [H]
        S = decay[:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = np.einsum("hnp,hn->hp", S, C[t]) + D[:, None] * x[t]
    return y, S


def gated_group_norm(y: np.ndarray, z: np.ndarray, parts: int, eps: float, weight: np.ndarray) -> np.ndarray:
    """y * silu(z), then each of `parts` equal pieces of the row divided by its own root mean square, times weight."""
    n, inner = y.shape
    g = (y * silu(z)).reshape(n, parts, inner // parts)
    return rms_norm(g, eps).reshape(n, inner) * weight


def rotate_pairs(v: np.ndarray, positions: np.ndarray, dims: int, base: float) -> np.ndarray:
    """Rotary positions in the interleaved layout on the first `dims` of the last axis: (v[2i], v[2i+1]) turned by
    positions * base^(-2i/dims). v [n, ..., >= dims]; the rest passes unchanged."""
    out = v.copy()
    i = np.arange(dims // 2)
    freq = base ** (-2.0 * i / dims)
    shape = (len(positions),) + (1,) * (v.ndim - 2) + (dims // 2,)
    ang = (positions[:, None].astype(np.float64) * freq[None, :]).reshape(shape)
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * np.cos(ang) - b * np.sin(ang)
    out[..., 1:dims:2] = b * np.cos(ang) + a * np.sin(ang)
    return out


def window_sink_softmax(scores: np.ndarray, q_pos: np.ndarray, k_pos: np.ndarray, window: int,
                        sink: Optional[float]) -> np.ndarray:
    """Row by row over the keys j with 0 <= q_pos[i] - k_pos[j] < window (window 0: all earlier keys); the
    denominator also holds exp(sink), which has no key and no value."""
    gap = q_pos[:, None] - k_pos[None, :]
    seen = (gap >= 0) & ((gap < window) if window > 0 else True)
    s = np.where(seen, scores, -np.inf)
    top = s.max(axis=-1, keepdims=True)
    if sink is not None:
        top = np.maximum(top, sink)
    w = np.exp(s - top)
    den = w.sum(axis=-1, keepdims=True)
    if sink is not None:
        den = den + np.exp(sink - top)
    return w / den


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------

class PlainRematar:
    def __init__(self, folder: str):
        with open(os.path.join(folder, "config.json")) as f:
            self.cfg = json.load(f)
        self.w = read_tensors(os.path.join(folder, "model.safetensors"))
        self.eps = float(self.cfg["norm"]["eps"])
        self.alpha = float(self.cfg.get("postln_alpha", 1.0))
        self.vocab = int(self.cfg["vocab"])
        self.layers = self.cfg["layers"]

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses."""
        while "weights_of" in self.layers[i] and self.layers[i]["weights_of"] is not None:
            i = int(self.layers[i]["weights_of"])
        return i

    def t(self, i: int, name: str) -> Optional[np.ndarray]:
        return self.w.get(f"l{self.owner(i)}.{name}")

    # -- state-space mixer -----------------------------------------------------------------
    def ssm_split(self, i: int, h: np.ndarray):
        m = self.layers[i]["mixer"]
        H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
        inner = H * P
        p = h @ self.t(i, "mix.in").T
        z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
        return z, xbc, dt

    def ssm_mixer(self, i: int, h: np.ndarray, state=None):
        """state: None (start of a sequence) or (S [H, N, P], the last K - 1 convolution inputs [K - 1, C])."""
        m = self.layers[i]["mixer"]
        H, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
        inner, n = H * P, len(h)
        z, xbc, dt = self.ssm_split(i, h)
        before = None if state is None else state[1]
        act = silu(causal_conv(xbc, self.t(i, "mix.conv"), self.t(i, "mix.conv.b"), before))
        front = np.zeros((K - 1, xbc.shape[1])) if before is None else before
        kept = np.concatenate([front, xbc], axis=0)[-(K - 1):] if K > 1 else np.zeros((0, xbc.shape[1]))
        x = act[:, :inner].reshape(n, H, P)
        per = H // G
        B = np.repeat(act[:, inner:inner + G * N].reshape(n, G, N), per, axis=1)
        C = np.repeat(act[:, inner + G * N:].reshape(n, G, N), per, axis=1)
        dt = softplus(dt + self.t(i, "mix.dt_bias"))
        y, S = ssm_scan(x, dt, B, C, self.t(i, "mix.A_log"), self.t(i, "mix.D"), None if state is None else state[0])
        g = gated_group_norm(y.reshape(n, inner), z, m["norm_groups"], self.eps, self.t(i, "mix.norm"))
        return g @ self.t(i, "mix.o").T, (S, kept)

    # -- latent attention -------------------------------------------------------------------
    def latent_queries(self, i: int, h: np.ndarray, positions: np.ndarray) -> np.ndarray:
        """[n, H, d + r], the last r of every head rotated."""
        m = self.layers[i]["mixer"]
        H, d, r = m["heads"], m["dim"], m["rot_dim"]
        cq = rms_norm(h @ self.t(i, "mix.dq").T, self.eps, self.t(i, "mix.dq.norm"))
        q = (cq @ self.t(i, "mix.uq").T).reshape(len(h), H, d + r)
        rot = m.get("rot") or {}
        if r and rot.get("dims", 0):
            q[..., d:] = rotate_pairs(q[..., d:], positions, int(rot["dims"]), float(rot["base"]))
        return q

    def latent_cached(self, i: int, h: np.ndarray, positions: np.ndarray):
        """What a token leaves behind: (latent [n, R], rotated shared key part [n, r])."""
        m = self.layers[i]["mixer"]
        R, r = m["kv_rank"], m["rot_dim"]
        p = h @ self.t(i, "mix.dkv").T
        c = rms_norm(p[:, :R], self.eps, self.t(i, "mix.dkv.norm"))
        kr = p[:, R:R + r]
        rot = m.get("rot") or {}
        if r and rot.get("dims", 0):
            kr = rotate_pairs(kr, positions, int(rot["dims"]), float(rot["base"]))
        return c, kr

    def latent_attend(self, i: int, h: np.ndarray, q: np.ndarray, q_pos: np.ndarray, c: np.ndarray, kr: np.ndarray,
                      k_pos: np.ndarray) -> np.ndarray:
        m = self.layers[i]["mixer"]
        H, d, r, e, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
        window = int((m.get("mask") or {}).get("size", 0))
        k = (c @ self.t(i, "mix.uk").T).reshape(len(c), H, d)
        v = (c @ self.t(i, "mix.uv").T).reshape(len(c), H, e)
        sink = self.t(i, "mix.sink")
        heads = []
        for a in range(H):
            s = (q[:, a, :d] @ k[:, a].T + q[:, a, d:] @ kr.T) * float(m["scale"])
            w = window_sink_softmax(s, q_pos, k_pos, window, None if sink is None else float(sink[a]))
            heads.append(w @ v[:, a])
        out = np.concatenate(heads, axis=-1)
        gate = self.t(i, "mix.g")
        if gate is not None:
            out = out * sigmoid(h @ gate.T)
        return out @ self.t(i, "mix.o").T

    def latent_mixer(self, i: int, h: np.ndarray, positions: np.ndarray, state=None):
        """state: None or (latents so far, rotated key parts so far, their positions)."""
        q = self.latent_queries(i, h, positions)
        c, kr = self.latent_cached(i, h, positions)
        if state is not None:
            c, kr, k_pos = np.concatenate([state[0], c]), np.concatenate([state[1], kr]), np.concatenate([state[2], positions])
        else:
            k_pos = positions
        return self.latent_attend(i, h, q, positions, c, kr, k_pos), (c, kr, k_pos)

    # -- a layer, the model --------------------------------------------------------------------
    def layer(self, i: int, x: np.ndarray, positions: np.ndarray, state=None):
        kind = self.layers[i]["type"]
        if kind == "mamba2":
            y, state = self.ssm_mixer(i, x, state)
        elif kind == "latent_attention":
            y, state = self.latent_mixer(i, x, positions, state)
        else:
            raise ValueError(kind)
        x = sum_then_norm(x, y, self.alpha, self.eps, self.t(i, "norm1"), self.t(i, "ls1"))
        if self.layers[i].get("mlp"):
            f = dense_mlp(x, self.t(i, "mlp.up"), self.t(i, "mlp.down"))
            x = sum_then_norm(x, f, self.alpha, self.eps, self.t(i, "norm2"), self.t(i, "ls2"))
        return x, state

    def embed(self, tokens) -> np.ndarray:
        return self.w["embed"][np.asarray(tokens)] * float((self.cfg.get("embedding") or {}).get("scale", 1.0))

    def head(self, x: np.ndarray) -> np.ndarray:
        return rms_norm(x, self.eps, self.w["final.norm"]) @ self.w["head"].T

    def hidden(self, tokens, keep: Optional[List[np.ndarray]] = None) -> np.ndarray:
        x = self.embed(tokens)
        pos = np.arange(len(tokens))
        for i in range(len(self.layers)):
            x, _ = self.layer(i, x, pos)
            if keep is not None:
                keep.append(x.copy())
        return x

    def logits(self, tokens) -> np.ndarray:
        return self.head(self.hidden(tokens))

    def logits_stepwise(self, tokens, portions: Optional[List[int]] = None) -> np.ndarray:
        """The same, fed in portions (default: one token at a time), every layer going on from its own state."""
        portions = portions or [1] * len(tokens)
        states = [None] * len(self.layers)
        rows, at = [], 0
        for n in portions:
            x = self.embed(tokens[at:at + n])
            pos = np.arange(at, at + n)
            for i in range(len(self.layers)):
                x, states[i] = self.layer(i, x, pos, states[i])
            rows.append(self.head(x))
            at += n
        return np.concatenate(rows)
