"""Differential attention over a paged cache: the "diff_attention" mixer.

Every head has two score maps. Each map is a causal softmax attention of its own (its own slice of the query and
of the key, `head_dim` wide) over the same values (`value_dim` wide), and the head's output is their difference:

    q, k  <- per-unit RMS norm (one weight for all query units, one for all key units; a unit = one map of one head)
    q     <- q * (1 + temp_coef * ln(floor((p + 1) / temp_every) + 1))        at position p, when temp_every > 0
    s_m   = scale * q_m . k_m;   s_m <- softcap * tanh(s_m / softcap) when softcap > 0;   a_m = softmax(s_m) V
    o     = a_1 - lambda * a_2;  o <- o / sqrt(mean(o^2) + eps) * (1 - lambda_init)
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init                     (one number per layer)

then the output projection over the concatenated heads. There is no rotation: positions enter through the causal
mask and the query temperature only. Query head h reads KV head h / (heads / kv_heads). The cache keeps one record
per token, [keys of all KV heads, both maps, normalised | values of all KV heads]; a layer may read the records
another layer wrote (`own_kv` False: it has no key and value tensors and makes queries only).

All sizes and constants come from the spec: num_heads, num_kv_heads, head_dim, value_dim, scale, softcap,
lambda_init, temp_coef, temp_every, eps, own_kv.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import CacheSpec, TensorDecl, register_mixer


@register_mixer("diff_attention")
class DiffAttention:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row counts (and graph_key) only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        qw = spec.num_heads * 2 * spec.head_dim
        kw = spec.num_kv_heads * 2 * spec.head_dim
        vw = spec.num_kv_heads * spec.value_dim
        d = (spec.head_dim,)
        out = {
            "q": TensorDecl((qw, spec.width)),
            "q_norm": TensorDecl(d, role="vector", init="around_one"),
            "lq1": TensorDecl(d, role="vector", init="bias"),
            "lk1": TensorDecl(d, role="vector", init="bias"),
            "lq2": TensorDecl(d, role="vector", init="bias"),
            "lk2": TensorDecl(d, role="vector", init="bias"),
            "o": TensorDecl((spec.width, spec.num_heads * spec.value_dim)),
        }
        if spec.get("own_kv", True):
            out.update({
                "k": TensorDecl((kw, spec.width)),
                "v": TensorDecl((vw, spec.width)),
                "k_norm": TensorDecl(d, role="vector", init="around_one"),
            })
        return out

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        if not (0 < spec.head_dim <= 256 and 0 < spec.value_dim <= 256):
            raise Unsupported(f"diff_attention: head_dim {spec.head_dim} and value_dim {spec.value_dim} must be at most 256")
        if spec.num_heads % spec.num_kv_heads:
            raise Unsupported(f"diff_attention: {spec.num_heads} heads do not divide into {spec.num_kv_heads} KV heads")
        self.spec = spec
        self.rt = runtime
        self.own_kv = bool(spec.get("own_kv", True))
        self.q_width = spec.num_heads * 2 * spec.head_dim
        self.k_width = spec.num_kv_heads * 2 * spec.head_dim
        self.v_width = spec.num_kv_heads * spec.value_dim
        self.out_width = spec.num_heads * spec.value_dim
        if self.own_kv:
            self.w_qkv = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
            self.k_norm = tensors["k_norm"]
        else:
            self.w_qkv = tensors["q"]
            self.k_norm = None
        self.q_norm = tensors["q_norm"]
        self.w_o = tensors["o"]
        # lambda is a function of the layer's weights alone: worked out once, in float32, and kept on the device so
        # that kernels read it through a pointer (layers of equal spec then differ in their tensors only)
        dot1 = (tensors["lq1"].float() * tensors["lk1"].float()).sum()
        dot2 = (tensors["lq2"].float() * tensors["lk2"].float()).sum()
        self.lam = (torch.exp(dot1) - torch.exp(dot2) + torch.tensor(float(spec.lambda_init), dtype=torch.float32,
                                                                       device=dot1.device)).reshape(1).contiguous()
        self.out_scale = 1.0 - float(spec.lambda_init)
        self.eps = float(spec.eps)

    def first_weights(self) -> torch.Tensor:
        return self.w_qkv

    def step_plans(self) -> list:
        """The query tiles of the step, for the prompt kernel (kernels/diff_attention.py)."""
        from ..kernels import diff_attention as fast
        return fast.step_plans()

    def graph_key(self, ctx) -> tuple:
        from ..kernels import diff_attention as fast
        return (("diff_splits", fast.split_count(ctx.num_tokens, self.spec.num_heads, self.spec.num_kv_heads, ctx.max_kv_len)),)

    def cache_spec(self) -> Optional[CacheSpec]:
        """One record per token: the normalised keys of every KV head and map, then the values."""
        if not self.own_kv:
            return None
        return CacheSpec(kind="pages", entry_shape=(self.k_width + self.v_width,), tensors=1)

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] normed input in the compute dtype -> [rows, width]."""
        s, rt = self.spec, self.rt
        rows = x.shape[0]
        if owns_cache != self.own_kv:
            raise Unsupported("diff_attention: a layer with key and value tensors owns its cache, one without reads another's")
        (records,) = cache.arrays
        if records.shape[-1] != self.k_width + self.v_width:
            raise Unsupported("diff_attention: the cache it reads was written with other head counts or sizes")
        # a layer that reads another layer's records makes queries only
        qkv = rt.buffer("diff_qkv", (rows, self.q_width + self.k_width + self.v_width)) if owns_cache else \
            rt.buffer("diff_q", (rows, self.q_width))
        linear(x, self.w_qkv, qkv)
        ops.qk_norm_cache_write(qkv, ctx.positions, ctx.row_slot, cache.block_table, records, 0, self.k_width,
                                self.q_norm, self.k_norm, self.eps, float(s.get("temp_coef", 0.0)),
                                int(s.get("temp_every", 0)), 2 * s.num_heads, 2 * s.num_kv_heads, s.head_dim,
                                self.v_width, cache.page_size, write_cache=owns_cache)
        attn = rt.buffer("diff_attn_out", (rows, self.out_width))
        self.attend(qkv, cache, ctx, attn)
        return linear_partial(attn, self.w_o, rt, "mixer_out")

    def attend(self, qkv: torch.Tensor, cache, ctx, out: torch.Tensor) -> None:
        s = self.spec
        (records,) = cache.arrays
        from ..kernels import diff_attention as fast
        if fast.attend(qkv, cache, ctx, out, s, self.lam, self.out_scale, self.eps, self.rt):
            return
        ops.diff_attention(qkv, records, 0, self.k_width, cache.block_table, ctx.positions, ctx.row_slot, out,
                           s.num_heads, s.num_kv_heads, s.head_dim, s.value_dim, cache.page_size, float(s.scale),
                           float(s.get("softcap", 0.0)), self.lam, self.out_scale, self.eps)
