"""The Todupel configuration: config.json -> TodupelConfig.

A Todupel config.json lists its layers one by one; every layer carries the sizes and constants of its own mixer
and feed-forward, so two layers of one model may differ in all of them:

    {"architecture": "Todupel", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "diff",
                           "q_temp": {"coef", "every"}, "kv_from": j (optional)},
                 "mlp": {"kind": "dense", "ff": F} or null}, ...]}

Nothing here has a default that stands for a model's value except where a key may be left out to switch a
mechanism off (softcap, q_temp) or where the design fixes the value (scale defaults to dim ** -0.5).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from ..errors import Corrupt, InvalidArgument, NotFound, Unsupported
from .reader import KeyReader

DEFAULT_CONTEXT = 131072      # the design has no positional limit; block tables are sized for this unless told otherwise


@dataclass(frozen=True)
class TodupelMixer:
    heads: int
    kv_heads: int
    dim: int                     # per-head, per-map query/key size
    vdim: int                    # per-head value size
    scale: float
    softcap: float               # 0: none
    diff: float                  # the constant of lambda, and 1 - diff scales the head's output
    temp_coef: float
    temp_every: int              # 0: no query temperature
    kv_from: Optional[int]       # the layer whose keys and values this one reads, or None


@dataclass(frozen=True)
class TodupelMLP:
    kind: str
    ff: int


@dataclass(frozen=True)
class TodupelLayer:
    type: str
    mixer: TodupelMixer
    mlp: Optional[TodupelMLP]


@dataclass(frozen=True)
class TodupelConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[TodupelLayer, ...]
    context: int = DEFAULT_CONTEXT

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.context

    @classmethod
    def from_dict(cls, obj: Mapping[str, Any]) -> "TodupelConfig":
        top = KeyReader(obj)
        vocab, width = top.int("vocab"), top.int("width")
        if vocab <= 0 or width <= 0:
            raise InvalidArgument("config.json: vocab and width must be positive")
        norm = top.object_or_none("norm")
        eps = norm.float_or("eps", 1e-6) if norm is not None else 1e-6
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise NotFound("config.json: missing 'layers' (a list with one entry per layer)")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw, f"config.json: layers[{i}]")
            kind = lr.str_or("type", "attention")
            if kind != "attention":
                raise Unsupported(f"config.json: layers[{i}] has a mixer of type '{kind}'; this design has 'attention'")
            mr = lr.object_or_none("mixer")
            if mr is None:
                raise NotFound(f"config.json: layers[{i}] has no 'mixer'")
            heads, dim = mr.int("heads"), mr.int("dim")
            kv_heads = mr.int_or("kv_heads", heads)
            vdim = mr.int_or("vdim", dim)
            if min(heads, kv_heads, dim, vdim) <= 0 or heads % kv_heads:
                raise InvalidArgument(f"config.json: layers[{i}]: heads {heads}, kv_heads {kv_heads}, dim {dim}, vdim {vdim}")
            temp = mr.object_or_none("q_temp")
            temp_coef = temp.float_or("coef", 0.0) if temp is not None else 0.0
            temp_every = temp.int_or("every", 0) if temp is not None else 0
            if temp_every < 0:
                raise InvalidArgument(f"config.json: layers[{i}]: q_temp.every must not be negative")
            kv_from = mr.int("kv_from") if mr.has("kv_from") else None
            if kv_from is not None and not 0 <= kv_from < i:
                raise InvalidArgument(f"config.json: layers[{i}] reads keys and values of layer {kv_from}, which is not earlier")
            mixer = TodupelMixer(heads, kv_heads, dim, vdim, mr.float_or("scale", dim ** -0.5), mr.float_or("softcap", 0.0),
                                 mr.float_or("diff", 0.0), temp_coef, temp_every if temp_coef != 0.0 else 0, kv_from)
            mlp = None
            pr = lr.object_or_none("mlp")
            if pr is not None:
                mlp = TodupelMLP(pr.str_or("kind", "dense"), pr.int("ff"))
                if mlp.kind != "dense":
                    raise Unsupported(f"config.json: layers[{i}] has a feed-forward of kind '{mlp.kind}'; this design has 'dense'")
                if mlp.ff <= 0:
                    raise InvalidArgument(f"config.json: layers[{i}]: ff must be positive")
            layers.append(TodupelLayer(kind, mixer, mlp))
        for i, layer in enumerate(layers):
            j = layer.mixer.kv_from
            if j is None:
                continue
            src = layers[j].mixer
            if src.kv_from is not None:
                raise InvalidArgument(f"config.json: layers[{i}] reads keys and values of layer {j}, which has none of its own")
            if (src.kv_heads, src.dim, src.vdim) != (layer.mixer.kv_heads, layer.mixer.dim, layer.mixer.vdim):
                raise Corrupt(f"config.json: layers[{i}] and layer {j}, whose keys and values it reads, differ in "
                              f"kv_heads, dim or vdim")
        return cls(vocab, width, eps, tuple(layers), top.int_or("context", DEFAULT_CONTEXT))
