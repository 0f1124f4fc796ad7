"""``Pemorax`` as a spec: the one file that knows this architecture.

A plain token embedding; every layer a ``pre_post_norm`` block (an RMS norm ahead of and behind each sublayer) whose
mixer is ``side_by_side``: ``window_attention`` (short convolution, interleaved rotary positions that may be
frequency-scaled, capped scores, a window that keeps the first tokens, a sink, a sigmoid gate) beside
``retention`` (rotate-half positions, a decay per head, unit norm per head, silu gate), their outputs normed and
averaged; the feed-forward is ``gelu_mlp``, ``routed_experts`` or absent; a last RMS norm and an output head.
Every distinct set of rotary parameters is one position table, shared by the layers that use it.  Tensor names:
``embed``, ``l<i>.{norm1,norm1b,norm2,norm2b}``, ``l<i>.mix.{left,right}.*``, ``l<i>.mix.{left,right}.out``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

import json

from ..config.model_config import PemoraxConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20      # the design has no longest sequence; this bounds the engine's bookkeeping


def build_pemorax_spec(cfg: PemoraxConfig) -> ModelSpec:
    h, eps = cfg.width, cfg.norm_eps
    positions, by_params = {}, {}

    def position_of(rot) -> str:
        """The name of the table for these rotary parameters (None if nothing rotates)."""
        if not rot["dims"]:
            return None
        key = json.dumps(rot, sort_keys=True)
        if key not in by_params:
            by_params[key] = f"rot{len(by_params)}"
            positions[by_params[key]] = PartSpec("rotary", dict(rotary_dim=rot["dims"], theta=rot["base"],
                                                                scaling=rot["scaling"]))
        return by_params[key]

    norm = lambda leaf: PartSpec("rmsnorm", dict(weight_name=leaf, hidden=h, eps=eps))
    layers = []
    for i, layer in enumerate(cfg.layers):
        l, r = layer.mixer["left"], layer.mixer["right"]
        mask = l["mask"] or {}
        left = dict(kind="window_attention", position=position_of(l["rot"]), out="left.out", params=dict(
            name="mix.left", hidden=h, heads=l["heads"], kv_heads=l["kv_heads"], dim=l["dim"], vdim=l["vdim"],
            conv=l["conv"], rot_dims=l["rot"]["dims"], rot_layout="interleaved", scale=l["scale"], softcap=l["softcap"],
            window=mask.get("size"), keep_first=mask.get("keep_first", 0), sink=True, gate=True))
        right = dict(kind="retention", position=position_of(r["rot"]), out="right.out", params=dict(
            name="mix.right", hidden=h, heads=r["heads"], dim=r["dim"], vdim=r["vdim"], decay=list(r["decay"]),
            rot_dims=r["rot"]["dims"], rot_layout="half", eps=eps))
        parts = dict(mixer_norm=norm("norm1"), mixer_post_norm=norm("norm1b"),
                     mixer=PartSpec("side_by_side", dict(name="mix", hidden=h, eps=eps, branches=[left, right])))
        if layer.mlp is not None:
            parts.update(feed_forward_norm=norm("norm2"), feed_forward_post_norm=norm("norm2b"))
            if layer.mlp["kind"] == "dense":
                parts["feed_forward"] = PartSpec("gelu_mlp", dict(name="mlp", hidden=h, intermediate=layer.mlp["ff"]))
            else:
                parts["feed_forward"] = PartSpec("routed_experts", dict(name="mlp", hidden=h, intermediate=layer.mlp["ff"],
                                                                        experts=layer.mlp["experts"], top=layer.mlp["top"]))
        layers.append(LayerSpec(prefix=f"l{i}", arrangement="pre_post_norm", parts=parts, position=None))
    return ModelSpec(
        architecture=PemoraxConfig.ARCHITECTURE, hidden_size=h, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=h, weight_name="embed")),
        final_norm=PartSpec("rmsnorm", dict(weight_name="final.norm", hidden=h, eps=eps)),
        lm_head=PartSpec("linear_head", dict(weight_name="head", vocab=cfg.vocab, hidden=h, tied_to=None)),
        positions=positions, layers=layers, schedule=[Run(i) for i in range(len(layers))])


register_architecture(PemoraxConfig.ARCHITECTURE, PemoraxConfig, build_pemorax_spec, model_type=PemoraxConfig.MODEL_TYPE)
