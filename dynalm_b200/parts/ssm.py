"""A state-space mixer with a matrix state per head: the "ssd" mixer.

One projection of the layer's input gives, per token, a gate z, the inputs x of H heads of P channels, and B and C
(N numbers each for every one of G groups of heads) and a raw step size per head. x, B and C pass a short causal
convolution over the last `taps` tokens (per channel, with a bias) and silu. Then, per head h (group h / (H / G)):

    dt  = softplus(dt_raw + dt_bias_h)
    S_h <- exp(-exp(a_log_h) dt) S_h + dt B x_h^T          (N x P, starts at zero)
    y_h = S_h^T C + d_h x_h

and the mixer's output is o(norm_parts(y * silu(z)) * norm), the gated row normed in `norm_groups` equal parts, each
by its own root mean square. Nothing is cached per token: a request keeps one row of a float32 state array, [S of
every head | the last taps - 1 inputs of the convolution], which the cache manager hands out zeroed.

All sizes come from the spec: num_heads, head_dim (P), state (N), groups, taps, norm_groups, eps.
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import Unsupported
from ..kernels import linear, ops
from ..kernels.gemm import linear_partial
from .base import CacheSpec, TensorDecl, register_mixer


@register_mixer("ssd")
class StateSpaceMixer:
    replay_safe = True     # all device work goes through the recorded launches of kernels/ops.py (engine/launch_memo.py)
    graph_safe = True      # launches depend on row and request counts only

    @staticmethod
    def declare(spec) -> Dict[str, TensorDecl]:
        H, P, N, G = spec.num_heads, spec.head_dim, spec.state, spec.groups
        inner, channels = H * P, H * P + 2 * G * N
        return {
            "in_proj": TensorDecl((2 * inner + 2 * G * N + H, spec.width)),
            "conv": TensorDecl((channels, spec.taps), role="vector", init="bias"),
            "conv_bias": TensorDecl((channels,), role="vector", init="bias"),
            "dt_bias": TensorDecl((H,), role="vector", init="bias"),
            "a_log": TensorDecl((H,), role="vector", init="bias"),
            "d": TensorDecl((H,), role="vector", init="around_one"),
            "norm": TensorDecl((inner,), role="vector", init="around_one"),
            "o": TensorDecl((spec.width, inner)),
        }

    def __init__(self, spec, tensors: Dict[str, torch.Tensor], runtime):
        H, P, N, G = spec.num_heads, spec.head_dim, spec.state, spec.groups
        if H % G:
            raise Unsupported(f"ssd: {H} heads do not divide into {G} groups")
        if (H * P) % spec.norm_groups:
            raise Unsupported(f"ssd: {H * P} channels do not divide into {spec.norm_groups} normed parts")
        if N > 1024:
            raise Unsupported(f"ssd: a state of {N} rows has no kernel (1,024 at most)")
        self.spec = spec
        self.rt = runtime
        self.inner = H * P
        self.channels = self.inner + 2 * G * N
        self.w_in = tensors["in_proj"]
        self.taps = tensors["conv"].t().contiguous()          # [taps, channels]: neighbouring channels in neighbouring words
        self.conv_bias = tensors["conv_bias"]
        self.dt_bias, self.a_log, self.d = tensors["dt_bias"], tensors["a_log"], tensors["d"]
        self.norm = tensors["norm"]
        self.w_o = tensors["o"]
        self.eps = float(spec.eps)
        self.keep_off = H * N * P                          # where a slot's kept convolution inputs begin

    def first_weights(self) -> torch.Tensor:
        return self.w_in

    def step_plans(self) -> list:
        """The segments that long portions are cut into, for the recurrence (kernels/ops.SsmSegmentPlan)."""
        return [ops.SSM_SEGMENTS]

    def cache_spec(self) -> Optional[CacheSpec]:
        s = self.spec
        return CacheSpec(kind="state", state_shape=(self.keep_off + (s.taps - 1) * self.channels,), dtype="float32")

    def forward(self, x: torch.Tensor, ctx, cache, owns_cache: bool = True) -> torch.Tensor:
        """x: [rows, width] in the compute dtype -> [rows, width] (or split-K partial sums of it)."""
        s, rt = self.spec, self.rt
        if not owns_cache or cache is None or cache.kind != "state":
            raise Unsupported("ssd: every run of the layer keeps a state of its own")
        (state,) = cache.arrays
        rows = x.shape[0]
        H, P, N, G = s.num_heads, s.head_dim, s.state, s.groups
        proj = rt.buffer("ssd_proj", (rows, 2 * self.inner + 2 * G * N + H))
        linear(x, self.w_in, proj)
        u = rt.buffer("ssd_conv", (rows, self.channels))
        ops.ssm_conv(proj, self.inner, self.channels, self.taps, self.conv_bias, state, self.keep_off, ctx.positions,
                     ctx.row_request, ctx.row_slot, ctx.pos_start, u)
        ops.ssm_conv_keep(proj, self.inner, self.channels, s.taps, state, self.keep_off, ctx.q_start, ctx.state_slots,
                          ctx.num_requests)
        y = rt.buffer("ssd_y", (rows, self.inner), torch.float32)
        planned = ctx.extras.get(ops.SSM_SEGMENTS.name)
        scratch = seg_decay = None
        if planned is not None and planned[1][0]:
            # (sized once for the most segments a step of the runtime's size can have; shared by all layers of these sizes)
            most = ops.SSM_SEGMENTS.most_segments(rt.max_tokens)
            scratch = rt.flat(f"ssd_segment_states_{self.keep_off}", most * self.keep_off)
            seg_decay = rt.flat(f"ssd_segment_decays_{H}", most * H)
        ops.ssm_scan(u, proj, self.inner + self.channels, self.dt_bias, self.a_log, self.d, state, ctx.q_start,
                     ctx.state_slots, y, ctx.num_requests, H, P, N, G, planned, scratch, seg_decay)
        g = rt.buffer("ssd_gated", (rows, self.inner))
        ops.gated_group_norm(y, proj, self.norm, self.eps, s.norm_groups, g)
        return linear_partial(g, self.w_o, rt, "mixer_out")
