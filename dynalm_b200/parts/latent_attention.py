"""Attention whose keys and values are projections of a cached latent: the "latent_attention" mixer.

Per token the layer's input h gives a query latent and a key/value latent:

    c_q = rmsnorm(dq h) * dq_norm,   q = uq c_q                  H heads of [d unrotated | r rotated] numbers
    c   = rmsnorm((dkv h)[:R]) * dkv_norm,   k_rot = (dkv h)[R:]    one rotated key part of r numbers for all heads
    k_h = uk_h c,  v_h = uv_h c                                    (d and e numbers per head)
    s   = scale * (q_h[:d] . k_h + rot(q_h[d:]) . rot(k_rot))
    p   = exp(s) / (sum over the window of exp(s) + exp(sink_h))   the sink has no key and no value
    out = o( concat_h(sum p v_h) * sigmoid(g h) )

Only c and rot(k_rot) are cached, as one record per token, and the attention runs on the records themselves: since
q_h . uk_h c = (uk_h^T q_h) . c, every head gets a "wide" query [uk_h^T q_h | rot(q_h[d:])] of R + r numbers that is
scored against the records, the softmax weights sum the records' latents, and uv_h is applied to that sum. The two
per-head products are block-diagonal (ops.head_linear). The window (0: every earlier key) also tells the cache
manager which pages may be given back.

All sizes and constants come from the spec: num_heads, head_dim (d), rot_dim (r), value_dim (e), q_rank, kv_rank (R),
scale, window, eps, position (a PositionSpec of kind "rotary_interleaved", or None); the sinks and the output gate are
there when the model has their tensors.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import POSITIONS, CacheSpec, TensorDecl, register_mixer


@register_mixer("latent_attention")
class LatentAttention:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        H, d, r, e = spec.num_heads, spec.head_dim, spec.rot_dim, spec.value_dim
        return {
            "dq": TensorDecl((spec.q_rank, spec.width)),
            "dq_norm": TensorDecl((spec.q_rank,), role="vector", init="around_one"),
            "uq": TensorDecl((H * (d + r), spec.q_rank)),
            "dkv": TensorDecl((spec.kv_rank + r, spec.width)),
            "dkv_norm": TensorDecl((spec.kv_rank,), role="vector", init="around_one"),
            "uk": TensorDecl((H * d, spec.kv_rank)),
            "uv": TensorDecl((H * e, spec.kv_rank)),
            "sink": TensorDecl((H,), role="vector", required=False, init="bias"),
            "gate": TensorDecl((H * e, spec.width), required=False),
            "o": TensorDecl((spec.width, H * e)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        H, d, r, e, R = spec.num_heads, spec.head_dim, spec.rot_dim, spec.value_dim, spec.kv_rank
        if R > 1024 or R + r > 8192:
            raise Unsupported(f"latent_attention: a latent of {R} numbers has no kernel (1,024 at most)")
        self.spec = spec
        self.rt = runtime
        self.has_gate = "gate" in tensors
        # one product for everything that reads the layer's input: [query latent | latent | key part | gate]
        down = [tensors["dq"], tensors["dkv"]] + ([tensors["gate"]] if self.has_gate else [])
        self.w_down = torch.cat(down, dim=0).contiguous()
        self.dq_norm, self.dkv_norm = tensors["dq_norm"], tensors["dkv_norm"]
        self.w_uq = tensors["uq"]
        self.w_uk = tensors["uk"].reshape(H, d, R).contiguous()                          # [H, in = d, out = R] as stored
        self.w_uv = tensors["uv"].reshape(H, e, R).transpose(1, 2).contiguous()          # [H, in = R, out = e]
        self.sink = tensors.get("sink")
        self.w_o = tensors["o"]
        self.eps = float(spec.eps)
        pos = spec.get("position")
        self.position = POSITIONS.get(pos.kind)(pos, runtime) if pos is not None else None
        if self.position is not None and not getattr(self.position, "interleaved", False):
            raise Unsupported(f"latent_attention: position encoding '{pos.kind}' has no kernel here (rotary_interleaved has)")
        self.rot = self.position.rotary_dim if self.position is not None else 0
        self.freq = self.position.frequencies if self.position is not None else None

    def first_weights(self) -> torch.Tensor:
        return self.w_down

    def step_plans(self) -> list:
        """The query tiles of the step, for the tensor-core kernel (kernels/latent_attention.py)."""
        from ..kernels import latent_attention as fast
        return [fast.tile_plan(self.spec)] if fast.flash_applies(self.spec, self.rt.dtype) else []

    def graph_key(self, ctx) -> tuple:
        from ..kernels import latent_attention as fast
        return (("latent_parts", fast.key_parts(ctx, self.spec)),) if fast.flash_applies(self.spec, self.rt.dtype) else ()

    def cache_spec(self) -> Optional[CacheSpec]:
        s = self.spec
        return CacheSpec(kind="pages", entry_shape=(s.kv_rank + s.rot_dim,), tensors=1, window=int(s.get("window", 0)))

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] in the compute dtype -> [rows, width] (or split-K partial sums of it)."""
        s, rt = self.spec, self.rt
        if not owns_cache:
            raise Unsupported("latent_attention: every run of the layer writes records of its own")
        H, d, r, e, R = s.num_heads, s.head_dim, s.rot_dim, s.value_dim, s.kv_rank
        rows = x.shape[0]
        (records,) = cache.arrays
        down = rt.buffer("latent_down", (rows, self.w_down.shape[0]))
        linear(x, self.w_down, down)
        cq = rt.buffer("latent_cq", (rows, s.q_rank))
        ops.latent_prep(down, s.q_rank, R, r, self.rot, self.dq_norm, self.dkv_norm, self.eps, self.freq, ctx.positions,
                        ctx.row_slot, cache.block_table, records, cache.page_size, cq)
        q = rt.buffer("latent_q", (rows, H * (d + r)))
        linear(cq, self.w_uq, q)
        wide = rt.buffer("latent_wide_q", (rows, H * (R + r)))
        ops.head_linear(q, d + r, d, self.w_uk, wide, R + r)
        if r:
            ops.rotate_pairs(q, d + r, d, wide, R + r, R, r, self.rot, self.freq, ctx.positions, H)
        mixed = rt.buffer("latent_mixed", (rows, H * R))
        self.attend(wide, cache, ctx, mixed)
        heads = rt.buffer("latent_heads", (rows, H * e))
        gate = down[:, s.q_rank + R + r:] if self.has_gate else None
        ops.head_linear(mixed, R, R, self.w_uv, heads, e, gate, e)
        return linear_partial(heads, self.w_o, rt, "mixer_out")

    def attend(self, wide: torch.Tensor, cache, ctx, out: torch.Tensor) -> None:
        s = self.spec
        (records,) = cache.arrays
        from ..kernels import latent_attention as fast
        if fast.attend(wide, cache, ctx, out, s, self.sink, self.rt):
            return
        ops.latent_attention(wide, records, cache.block_table, ctx.positions, ctx.row_slot, self.sink, out, s.num_heads,
                             s.kv_rank, s.rot_dim, cache.page_size, float(s.scale), int(s.get("window", 0)))
