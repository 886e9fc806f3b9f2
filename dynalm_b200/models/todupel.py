"""The Todupel architecture: config.json -> TodupelConfig -> ModelPlan.

A decoder of parallel blocks, x <- x + (mixer(norm1(x)) + mlp(norm2(x))): the mixer is differential attention
without a rotation (parts/diff_attention.py), the feed-forward an ungated one with a squared ReLU (parts/mlp.py,
kind "mlp"), or none. A layer may read the keys and values another layer cached; in the run order that is an
entry with `cache_of`. Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,k,v,o,q.norm,k.norm,lq1,lk1,
lq2,lk2}`, `l<i>.mlp.{up,down}`, `final.norm`, `head`.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

from ..config.plan import BlockSpec, EmbeddingSpec, FeedForwardSpec, HeadSpec, LayerRun, MixerSpec, ModelPlan, NormSpec
from ..config.todupel import TodupelConfig
from ..registry import register_architecture


class TodupelArchitecture:
    name = "Todupel"
    model_types = ("todupel",)

    def read_config(self, obj: Mapping[str, Any]) -> TodupelConfig:
        return TodupelConfig.from_dict(obj)

    def plan(self, cfg: TodupelConfig, present: Optional[set] = None) -> ModelPlan:
        layers, order, ignorable = [], [], []
        for i, layer in enumerate(cfg.layers):
            p, m = f"l{i}.", layer.mixer
            own_kv = m.kv_from is None
            names = {"q": p + "mix.q", "q_norm": p + "mix.q.norm", "o": p + "mix.o", "lq1": p + "mix.lq1",
                     "lk1": p + "mix.lk1", "lq2": p + "mix.lq2", "lk2": p + "mix.lk2"}
            if own_kv:
                names.update({"k": p + "mix.k", "v": p + "mix.v", "k_norm": p + "mix.k.norm"})
            parts = dict(
                mixer_norm=NormSpec("rms", cfg.width, cfg.norm_eps, {"weight": p + "norm1"}),
                mixer=MixerSpec("diff_attention", cfg.width, names, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                head_dim=m.dim, value_dim=m.vdim, scale=m.scale, softcap=m.softcap, lambda_init=m.diff,
                                temp_coef=m.temp_coef, temp_every=m.temp_every, eps=cfg.norm_eps, own_kv=own_kv))
            if layer.mlp is not None:
                parts["ffn_norm"] = NormSpec("rms", cfg.width, cfg.norm_eps, {"weight": p + "norm2"})
                parts["ffn"] = FeedForwardSpec("mlp", cfg.width, {"up": p + "mlp.up", "down": p + "mlp.down"},
                                               inner=layer.mlp.ff, activation="relu2")
            else:
                ignorable.append(p + "norm2")      # a layer without a feed-forward may still carry its second norm
            layers.append(BlockSpec("parallel", **parts))
            order.append(LayerRun(i, cache_of=m.kv_from))
        plan = ModelPlan(
            embedding=EmbeddingSpec(cfg.vocab, cfg.width, 1.0, {"weight": "embed"}),
            layers=layers, order=order,
            final_norm=NormSpec("rms", cfg.width, cfg.norm_eps, {"weight": "final.norm"}),
            head=HeadSpec(cfg.vocab, cfg.width, False, 1.0, {"weight": "head"}),
            context_length=cfg.context, ignorable=tuple(ignorable))
        plan.validate()
        return plan


register_architecture(TodupelArchitecture())
