"""``Tekosun`` as a spec: the one file that knows this architecture.

A token embedding times a constant; every layer a ``post_norm`` block (the sublayers read the stream itself, an RMS
norm sits behind each) whose mixer is ``mamba2``, ``general_delta`` or ``window_attention`` (with the norm over the
whole query and key projections, rotate-half positions that may be frequency-scaled by wavelength bands, a unit norm
on every value head, an optional window, and the blend of the values with those of the first layer that asks for
it); the feed-forward is ``routed_experts`` (squared relu, a softmax router over all experts, a shared expert) or
absent; a last RMS norm and an output head.  Every distinct set of rotary parameters is one position table, shared
by the layers that use it.  Tensor names: ``embed``, ``l<i>.{norm1,norm2}``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import json

from ..config.model_config import TekosunConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20      # the design has no longest sequence; this bounds the engine's bookkeeping


def build_tekosun_spec(cfg: TekosunConfig) -> ModelSpec:
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
    layers, mixing_seen = [], False
    for i, layer in enumerate(cfg.layers):
        m, position = layer.mixer, None
        if layer.type == "mamba2":
            mixer = PartSpec("mamba2", dict(name="mix", hidden=h, heads=m["heads"], vdim=m["vdim"], state=m["state"],
                                            groups=m["groups"], conv=m["conv"], norm_groups=m["norm_groups"], eps=eps))
        elif layer.type == "general_delta":
            mixer = PartSpec("general_delta", dict(name="mix", hidden=h, heads=m["heads"], dim=m["dim"],
                                                   decay_rank=m["decay_rank"], eps=eps))
        else:
            position = position_of(m["rot"])
            v_mix = None
            if m["v_mix"]:
                v_mix, mixing_seen = ("blend" if mixing_seen else "first"), True
            mixer = PartSpec("window_attention", dict(
                name="mix", hidden=h, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], conv=0,
                rot_dims=m["rot"]["dims"], rot_layout="half", scale=m["scale"], softcap=None, window=m["window"],
                keep_first=0, sink=False, gate=False, qk_norm=True, v_norm=True, v_mix=v_mix, eps=eps))
        parts = dict(mixer=mixer, mixer_post_norm=norm("norm1"))
        if layer.mlp is not None:
            f = layer.mlp
            parts.update(feed_forward_post_norm=norm("norm2"), feed_forward=PartSpec("routed_experts", dict(
                name="mlp", hidden=h, intermediate=f["ff"], experts=f["experts"], top=f["top"], activation="relu2",
                route="all", scale=f["scale"], router_bias=False, shared=f["shared_ff"])))
        layers.append(LayerSpec(prefix=f"l{i}", arrangement="post_norm", parts=parts, position=position))
    return ModelSpec(
        architecture=TekosunConfig.ARCHITECTURE, hidden_size=h, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=h, weight_name="embed", scale=cfg.embedding_scale)),
        final_norm=PartSpec("rmsnorm", dict(weight_name="final.norm", hidden=h, eps=eps)),
        lm_head=PartSpec("linear_head", dict(weight_name="head", vocab=cfg.vocab, hidden=h, tied_to=None)),
        positions=positions, layers=layers, schedule=[Run(i) for i in range(len(layers))])


register_architecture(TekosunConfig.ARCHITECTURE, TekosunConfig, build_tekosun_spec, model_type=TekosunConfig.MODEL_TYPE)
