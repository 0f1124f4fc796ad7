"""``Kunonex`` as a spec: the one file that knows this architecture.

The embedding adds sinusoidal positions and norms; every layer is a parallel
block (one layer norm, a token-shifted mixer beside a PolyNorm feed-forward
that may be absent, one sum); mixers are ``mingru`` or ``latent_attention`` as
config.json lists them layer by layer; a stretch of layers may run several
times in a row on the same weights, every pass with caches and states of its
own and with a ``loop_entry`` junction ahead of it; a final layer norm and an
output head whose logits are scaled.  Tensor names: ``embed``, ``embed.norm``,
``loop.in``, ``loop.step``, ``l<i>.{norm1,shift}``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.model_config import ConfigError, KunonexConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20      # the design has no longest sequence; this bounds the engine's bookkeeping


def build_kunonex_spec(cfg: KunonexConfig) -> ModelSpec:
    h, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "mingru":
            mixer = PartSpec("mingru", dict(name="mix", hidden=h, width=m["width"]))
        elif layer.type == "latent_attention":
            mixer = PartSpec("latent_attention", dict(name="mix", hidden=h, heads=m["heads"], dim=m["dim"], vdim=m["vdim"],
                                                      kv_rank=m["kv_rank"], q_rank=m["q_rank"], scale=m["scale"], eps=eps))
        else:
            raise ConfigError(f"layer {i}: unknown mixer type '{layer.type}'")
        parts = dict(norm=PartSpec("layernorm", dict(weight_name="norm1", hidden=h, eps=eps)),
                     shift=PartSpec("token_shift", dict(weight_name="shift", hidden=h)), mixer=mixer)
        if layer.ff:
            parts["feed_forward"] = PartSpec("polynorm", dict(name="mlp", hidden=h, intermediate=layer.ff, eps=eps))
        layers.append(LayerSpec(prefix=f"l{i}", arrangement="parallel", parts=parts, position=None))
    n = len(layers)
    if cfg.loop_times:
        entry = n                    # the junction ahead of every pass is one more "layer" of the spec
        layers.append(LayerSpec(prefix="loop", arrangement="junction", parts=dict(junction=PartSpec("loop_entry", dict(
            hidden=h, passes=cfg.loop_times, in_name="loop.in", step_name="loop.step")))))
        schedule = [Run(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            schedule.append(Run(entry, params={"pass": t}))
            schedule += [Run(i, params={"pass": t}) for i in range(cfg.loop_start, cfg.loop_stop)]
        schedule += [Run(i) for i in range(cfg.loop_stop, n)]
    else:
        schedule = [Run(i) for i in range(n)]
    return ModelSpec(
        architecture=KunonexConfig.ARCHITECTURE, hidden_size=h, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("sinusoid_norm_embedding", dict(vocab=cfg.vocab, hidden=h, eps=eps, base=10000.0,
                                                           table="embed", norm_weight="embed.norm")),
        final_norm=PartSpec("layernorm", dict(weight_name="final.norm", hidden=h, eps=eps)),
        lm_head=PartSpec("linear_head", dict(weight_name="head", vocab=cfg.vocab, hidden=h, tied_to=None,
                                             scale=cfg.logit_scale)),
        positions={}, layers=layers, schedule=schedule)


register_architecture(KunonexConfig.ARCHITECTURE, KunonexConfig, build_kunonex_spec, model_type=KunonexConfig.MODEL_TYPE)
