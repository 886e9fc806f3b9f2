"""The Rematar configuration: config.json -> RematarConfig.

A Rematar config.json lists its layers one by one. A layer is a state-space mixer ("mamba2") or latent attention
("latent_attention"), each with its own sizes, followed by a dense feed-forward or none; a layer may run with the
tensors of an earlier layer (`weights_of`) while keeping a cache or state of its own:

    {"architecture": "Rematar", "vocab": V, "width": W, "norm": {"eps": e}, "postln_alpha": a,
     "embedding": {"scale": s},
     "layers": [{"type": "mamba2",
                 "mixer": {"heads", "vdim", "state", "groups", "conv", "norm_groups"},
                 "mlp": {"kind": "dense", "ff": F} or null, "weights_of": j (optional)},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale",
                           "rot": {"base", "dims"}, "mask": {"size"}}, ...}]}

Where a key may be left out a mechanism is switched off (no window without `mask`, no rotation without `rot`, an
alpha and an embedding scale of 1); no default stands for a model's value.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from ..errors import Corrupt, InvalidArgument, NotFound, Unsupported
from .reader import KeyReader

DEFAULT_CONTEXT = 131072      # the design has no positional limit; block tables are sized for this unless told otherwise


@dataclass(frozen=True)
class RematarSSM:
    heads: int
    vdim: int                    # channels per head
    state: int                   # rows of a head's recurrent matrix
    groups: int                  # groups of heads that share B and C
    conv: int                    # taps of the short convolution
    norm_groups: int             # equal parts of the gated output that are normed each by itself


@dataclass(frozen=True)
class RematarLatent:
    heads: int
    dim: int                     # unrotated query/key size per head
    rot_dim: int                 # rotated query/key size per head (the key's is shared by all heads)
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int                # how many of the rot_dim dimensions are turned (0: none)
    window: int                  # 0: all earlier keys


@dataclass(frozen=True)
class RematarMLP:
    kind: str
    ff: int


@dataclass(frozen=True)
class RematarLayer:
    type: str
    mixer: Union[RematarSSM, RematarLatent]
    mlp: Optional[RematarMLP]
    weights_of: Optional[int]    # the layer whose tensors this one runs with, chains resolved; None: its own


@dataclass(frozen=True)
class RematarConfig:
    vocab: int
    width: int
    norm_eps: float
    alpha: float
    embedding_scale: float
    layers: Tuple[RematarLayer, ...]
    context: int = DEFAULT_CONTEXT

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def max_position_embeddings(self) -> int:
        return self.context

    @classmethod
    def from_dict(cls, obj: Mapping[str, Any]) -> "RematarConfig":
        top = KeyReader(obj)
        vocab, width = top.int("vocab"), top.int("width")
        if vocab <= 0 or width <= 0:
            raise InvalidArgument("config.json: vocab and width must be positive")
        norm = top.object_or_none("norm")
        eps = norm.float_or("eps", 1e-6) if norm is not None else 1e-6
        emb = top.object_or_none("embedding")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise NotFound("config.json: missing 'layers' (a list with one entry per layer)")
        layers = []
        for i, raw in enumerate(raw_layers):
            lr = KeyReader(raw, f"config.json: layers[{i}]")
            kind = lr.str_or("type", None)
            mr = lr.object_or_none("mixer")
            if mr is None:
                raise NotFound(f"config.json: layers[{i}] has no 'mixer'")
            if kind == "mamba2":
                mixer = RematarSSM(mr.int("heads"), mr.int("vdim"), mr.int("state"), mr.int_or("groups", 1),
                                   mr.int("conv"), mr.int_or("norm_groups", 1))
                if min(mixer.heads, mixer.vdim, mixer.state, mixer.groups, mixer.conv, mixer.norm_groups) <= 0:
                    raise InvalidArgument(f"config.json: layers[{i}]: every size of the mixer must be positive")
                if mixer.heads % mixer.groups:
                    raise InvalidArgument(f"config.json: layers[{i}]: {mixer.heads} heads do not divide into {mixer.groups} groups")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise InvalidArgument(f"config.json: layers[{i}]: {mixer.heads * mixer.vdim} channels do not divide "
                                          f"into {mixer.norm_groups} normed parts")
            elif kind == "latent_attention":
                dim, rot_dim = mr.int("dim"), mr.int_or("rot_dim", 0)
                rot = mr.object_or_none("rot")
                mask = mr.object_or_none("mask")
                mixer = RematarLatent(mr.int("heads"), dim, rot_dim, mr.int_or("vdim", dim), mr.int("q_rank"),
                                      mr.int("kv_rank"), mr.float_or("scale", (dim + rot_dim) ** -0.5),
                                      rot.float_or("base", 10000.0) if rot is not None else 10000.0,
                                      rot.int_or("dims", rot_dim) if rot is not None else 0,
                                      mask.int_or("size", 0) if mask is not None else 0)
                if min(mixer.heads, mixer.dim, mixer.vdim, mixer.q_rank, mixer.kv_rank) <= 0 or mixer.rot_dim < 0:
                    raise InvalidArgument(f"config.json: layers[{i}]: every size of the mixer must be positive")
                if mixer.rot_dims < 0 or mixer.rot_dims > mixer.rot_dim or mixer.rot_dims % 2:
                    raise InvalidArgument(f"config.json: layers[{i}]: rot.dims {mixer.rot_dims} must be even and at "
                                          f"most rot_dim {mixer.rot_dim}")
                if mixer.window < 0:
                    raise InvalidArgument(f"config.json: layers[{i}]: mask.size must not be negative")
            else:
                raise Unsupported(f"config.json: layers[{i}] has a mixer of type '{kind}'; this design has 'mamba2' "
                                  f"and 'latent_attention'")
            mlp = None
            pr = lr.object_or_none("mlp")
            if pr is not None:
                mlp = RematarMLP(pr.str_or("kind", "dense"), pr.int("ff"))
                if mlp.kind != "dense":
                    raise Unsupported(f"config.json: layers[{i}] has a feed-forward of kind '{mlp.kind}'; this design has 'dense'")
                if mlp.ff <= 0:
                    raise InvalidArgument(f"config.json: layers[{i}]: ff must be positive")
            source = lr.int("weights_of") if lr.has("weights_of") else None
            if source is not None:
                if not 0 <= source < i:
                    raise InvalidArgument(f"config.json: layers[{i}] runs with the tensors of layer {source}, which is not earlier")
                first = layers[source]
                if (first.type, first.mixer, first.mlp) != (kind, mixer, mlp):
                    raise Corrupt(f"config.json: layers[{i}] and layer {source}, whose tensors it runs with, differ")
                if first.weights_of is not None:
                    source = first.weights_of
            layers.append(RematarLayer(kind, mixer, mlp, source))
        return cls(vocab, width, eps, top.float_or("postln_alpha", 1.0),
                   emb.float_or("scale", 1.0) if emb is not None else 1.0, tuple(layers),
                   top.int_or("context", DEFAULT_CONTEXT))
