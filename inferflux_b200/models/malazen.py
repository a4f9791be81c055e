"""``Malazen`` as a spec: the one file that knows this architecture.

A plain token embedding; every layer a ``prenorm`` block whose norms are ``group_rmsnorm`` (the row normed in
``norm.groups`` equal parts).  A layer's mixer is ``side_by_side`` with ``combine="weighted"``:
``window_attention`` without window or rotation (biases, a query temperature that grows with the logarithm of the
position, a toll on the score that grows with the logarithm of the distance) beside ``gated_linear_attention`` (a
decay per key channel from a narrow projection, a normed and silu-gated output), summed with the two factors the
configuration gives; or it is ``latent_attention`` with a direct query projection, a rotated key part shared by
the heads (neighbouring pairs, frequencies optionally stretched), a window and a learned sink per head.  The
feed-forward is ``clamped_glu`` or absent.  A stretch of layers may run several times in a row on the same
weights, every pass with caches and states of its own; ahead of every pass but the first an ``add_embedding``
junction adds the embedding's output to the stream.  A last ``group_rmsnorm`` and an output head that is the
embedding table.  Every distinct set of rotary parameters is one position table, shared by the layers that use
it.  Tensor names: ``embed``, ``l<i>.{norm1,norm2}``, ``l<i>.mix.{left,right}.*`` or ``l<i>.mix.*``,
``l<i>.mlp.*``, ``final.norm``.
"""
from __future__ import annotations

import json

from ..config.model_config import ConfigError, MalazenConfig
from ..config.registry import register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20      # the design has no longest sequence; this bounds the engine's bookkeeping
GLU_ALPHA, GLU_SHIFT = 1.702, 1.0       # the feed-forward's two constants: g * sigmoid(1.702 g) * (u + 1)


def build_malazen_spec(cfg: MalazenConfig) -> ModelSpec:
    h, eps, groups = cfg.width, cfg.norm_eps, cfg.norm_groups
    positions, by_params = {}, {}

    def position_of(rot) -> str:
        """The name of the table for these rotary parameters (None if nothing rotates)."""
        if not rot or not rot["dims"]:
            return None
        key = json.dumps(rot, sort_keys=True)
        if key not in by_params:
            by_params[key] = f"rot{len(by_params)}"
            positions[by_params[key]] = PartSpec("rotary", dict(rotary_dim=rot["dims"], theta=rot["base"],
                                                                scaling=rot["scaling"]))
        return by_params[key]

    norm = lambda leaf: PartSpec("group_rmsnorm", dict(weight_name=leaf, hidden=h, eps=eps, groups=groups))
    layers = []
    for i, layer in enumerate(cfg.layers):
        m, position = layer.mixer, None
        if layer.type == "parallel":
            l, r = m["left"], m["right"]
            left = dict(kind="window_attention", position=None, out=None, params=dict(
                name="mix.left", hidden=h, heads=l["heads"], kv_heads=l["kv_heads"], dim=l["dim"], vdim=l["vdim"], conv=0,
                rot_dims=0, scale=l["scale"], softcap=None, window=None, keep_first=0, sink=False, gate=False, bias=True,
                q_temp=l["q_temp"], distance_toll=True))
            right = dict(kind="gated_linear_attention", position=None, out=None, params=dict(
                name="mix.right", hidden=h, heads=r["heads"], dim=r["dim"], vdim=r["vdim"], tau=r["tau"], eps=eps))
            mixer = PartSpec("side_by_side", dict(name="mix", hidden=h, eps=eps, combine="weighted",
                                                  scales=[m["left_scale"], m["right_scale"]], branches=[left, right]))
        elif layer.type == "latent_attention":
            position = position_of(m["rot"])
            mixer = PartSpec("latent_attention", dict(
                name="mix", hidden=h, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], kv_rank=m["kv_rank"], q_rank=0,
                scale=m["scale"], eps=eps, gate=False, rot_dim=m["rot_dim"], window=m["window"], sink=True))
        else:
            raise ConfigError(f"layer {i}: unknown mixer type '{layer.type}'")
        parts = dict(mixer_norm=norm("norm1"), mixer=mixer)
        if layer.mlp is not None:
            parts.update(feed_forward_norm=norm("norm2"), feed_forward=PartSpec("clamped_glu", dict(
                name="mlp", hidden=h, intermediate=layer.mlp["ff"], limit=layer.mlp["limit"], alpha=GLU_ALPHA,
                shift=GLU_SHIFT, bias=True)))
        layers.append(LayerSpec(prefix=f"l{i}", arrangement="prenorm", parts=parts, position=position))
    n = len(layers)
    if cfg.loop_times > 1:
        entry = n                    # the junction ahead of every later pass is one more "layer" of the spec
        layers.append(LayerSpec(prefix="loop", arrangement="junction", parts=dict(junction=PartSpec("add_embedding", {}))))
        schedule = [Run(i) for i in range(cfg.loop_start)]
        for t in range(cfg.loop_times):
            if t > 0:
                schedule.append(Run(entry, params={"pass": t}))
            schedule += [Run(i, params={"pass": t}) for i in range(cfg.loop_start, cfg.loop_stop)]
        schedule += [Run(i) for i in range(cfg.loop_stop, n)]
    else:
        schedule = [Run(i) for i in range(n)]
    return ModelSpec(
        architecture=MalazenConfig.ARCHITECTURE, hidden_size=h, vocab_size=cfg.vocab, max_position=MAX_POSITION,
        embedding=PartSpec("token_embedding", dict(vocab=cfg.vocab, hidden=h, weight_name="embed")),
        final_norm=PartSpec("group_rmsnorm", dict(weight_name="final.norm", hidden=h, eps=eps, groups=groups)),
        lm_head=PartSpec("linear_head", dict(weight_name="head", vocab=cfg.vocab, hidden=h, tied_to="embed")),
        positions=positions, layers=layers, schedule=schedule)


register_architecture(MalazenConfig.ARCHITECTURE, MalazenConfig, build_malazen_spec, model_type=MalazenConfig.MODEL_TYPE)
