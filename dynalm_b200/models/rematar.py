"""The Rematar architecture: config.json -> RematarConfig -> ModelPlan.

A decoder whose layers norm AFTER the sum: x <- norm1(alpha x + s1 * mixer(x)), x <- norm2(alpha x + s2 * ffn(x)),
s1 and s2 per-channel scales; both sublayers read x itself (block kind "post_norm", norm kind "rms_after_sum"). The
mixer of a layer is a state-space recurrence (parts/ssm.py, kind "ssd") or latent attention with a sliding window
(parts/latent_attention.py); the feed-forward is ungated with the tanh form of GELU (parts/mlp.py, kind "mlp"), or
absent. A layer may run with the tensors of an earlier layer: in the run order that is the earlier layer named
again, with a cache or state of its own. Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.ls1`, `l<i>.ls2`,
`l<i>.mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}` or `l<i>.mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,sink,g,o}`,
`l<i>.mlp.{up,down}`, `final.norm`, `head`.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

from ..config.plan import (BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan, NormSpec,
                           PositionSpec)
from ..config.rematar import RematarConfig, RematarLatent, RematarSSM
from ..registry import register_architecture


class RematarArchitecture:
    name = "Rematar"
    model_types = ("rematar",)

    def read_config(self, obj: Mapping[str, Any]) -> RematarConfig:
        return RematarConfig.from_dict(obj)

    def plan(self, cfg: RematarConfig, present: Optional[set] = None) -> ModelPlan:
        """`present`: names of the tensors in the model folder, when known: the per-channel scales, the sinks and
        the output gate are taken when the file has them (all of them when no listing is given)."""
        has = (lambda n: n in present) if present is not None else (lambda n: True)
        layers, order, ignorable, block_of = [], [], [], {}
        for i, layer in enumerate(cfg.layers):
            if layer.weights_of is not None:
                order.append(LayerRun(block_of[layer.weights_of]))
                continue
            p, m = f"l{i}.", layer.mixer
            if isinstance(m, RematarSSM):
                names = {k: p + "mix." + f for k, f in (("in_proj", "in"), ("conv", "conv"), ("conv_bias", "conv.b"),
                                                        ("dt_bias", "dt_bias"), ("a_log", "A_log"), ("d", "D"),
                                                        ("norm", "norm"), ("o", "o"))}
                mixer = MixerSpec("ssd", cfg.width, names, num_heads=m.heads, head_dim=m.vdim, state=m.state,
                                  groups=m.groups, taps=m.conv, norm_groups=m.norm_groups, eps=cfg.norm_eps)
            else:
                assert isinstance(m, RematarLatent)
                names = {k: p + "mix." + f for k, f in (("dq", "dq"), ("dq_norm", "dq.norm"), ("uq", "uq"), ("dkv", "dkv"),
                                                        ("dkv_norm", "dkv.norm"), ("uk", "uk"), ("uv", "uv"), ("o", "o"))}
                for local, f in (("sink", "sink"), ("gate", "g")):
                    if has(p + "mix." + f):
                        names[local] = p + "mix." + f
                position = PositionSpec("rotary_interleaved", head_dim=m.rot_dim, rotary_dim=m.rot_dims,
                                        theta=m.rot_base) if m.rot_dims > 0 else None
                mixer = MixerSpec("latent_attention", cfg.width, names, num_heads=m.heads, head_dim=m.dim,
                                  rot_dim=m.rot_dim, value_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale,
                                  window=m.window, eps=cfg.norm_eps, position=position)

            def after_sum(norm: str, scale: str) -> NormSpec:
                tensors = {"weight": p + norm}
                if has(p + scale):
                    tensors["delta_scale"] = p + scale
                return NormSpec("rms_after_sum", cfg.width, cfg.norm_eps, tensors, alpha=cfg.alpha)

            parts = dict(mixer=mixer, mixer_norm=after_sum("norm1", "ls1"))
            if layer.mlp is not None:
                parts["ffn"] = FeedForwardSpec("mlp", cfg.width, {"up": p + "mlp.up", "down": p + "mlp.down"},
                                               inner=layer.mlp.ff, activation="gelu_tanh")
                parts["ffn_norm"] = after_sum("norm2", "ls2")
            else:
                ignorable += [p + "norm2", p + "ls2"]      # a layer without a feed-forward may still carry them
            block_of[i] = len(layers)
            layers.append(BlockSpec("post_norm", **parts))
            order.append(LayerRun(block_of[i]))
        plan = ModelPlan(
            embedding=EmbeddingSpec(cfg.vocab, cfg.width, cfg.embedding_scale, {"weight": "embed"}),
            layers=layers, order=order,
            final_norm=NormSpec("rms", cfg.width, cfg.norm_eps, {"weight": "final.norm"}),
            head=HeadSpec(cfg.vocab, cfg.width, False, 1.0, {"weight": "head"}),
            context_length=cfg.context, ignorable=tuple(ignorable))
        plan.validate()
        return plan


register_architecture(RematarArchitecture())
