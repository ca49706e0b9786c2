"""Revelix as a blueprint of parts.

A decoder of pre-norm layers whose norm is Dynamic Tanh (tanh(alpha x) * w + b:
no mean, no variance).  A layer's mixer is either *retention* - linear attention
with a constant decay per head, rotated q and k, a unit-RMS norm per head and a
SiLU gate - or two mixers side by side whose outputs are added with fixed
weights: softmax attention with biased, convolved projections, an interleaved
rotation with stretched frequencies, capped scores, a window that keeps the
first positions, a keyless term in the softmax denominator and heads whose
weights are mixed after the softmax; and a gated linear recurrence whose forget
gate also decides what is written.  The feed-forward is down(act(up x)) with a
two-parameter activation, or absent.  The logits are the final norm's output
times the embedding table, times a constant.  Tensor names: ``embed``,
``l<i>.norm1`` / ``.norm2`` (+ ``.b``, ``.alpha``), ``l<i>.mix.*`` (``.left.*``
and ``.right.*`` in a parallel layer), ``l<i>.mlp.*``, ``final.norm``.
"""

from __future__ import annotations

from ..config.revelix import RevelixConfig
from ..engine.blueprint import LayerSpec, ModelBlueprint, PartSpec, RunSpec
from ..registry import register_architecture

# The configuration gives no longest sequence: the rotation tables are built for what the first cache asks for.
NO_POSITION_LIMIT = 1 << 30


def revelix_blueprint(cfg: RevelixConfig) -> ModelBlueprint:
    H = cfg.width
    positions = {}

    def rotation(rot):
        if rot is None:
            return None, 0
        name = rot.key()
        positions.setdefault(name, PartSpec("position", "rotary_scaled",
                                            dict(dims=rot.dims, base=rot.base, scaling=rot.scaling,
                                                 max_positions=NO_POSITION_LIMIT)))
        return name, rot.dims

    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        if L.type == "retention":
            rope, rot_dims = rotation(m.rot)
            mixer = PartSpec("mixer", "retention",
                             dict(hidden_size=H, n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, decay=list(m.decay),
                                  eps=cfg.norm_eps, position=rope, rot_dims=rot_dims), f"{p}.mix")
        else:
            a, r = m.left, m.right
            rope, rot_dims = rotation(a.rot)
            left = PartSpec("mixer", "conv_gated_attention",
                            dict(hidden_size=H, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim,
                                 taps=a.conv, scale=a.scale, position=rope, rot_dims=rot_dims, window=a.window,
                                 gate=False, bias=True, interleaved=True, softcap=a.softcap, keep_first=a.keep_first,
                                 sink=True, talk=True), f"{p}.mix.left")
            right = PartSpec("mixer", "gated_linear_recurrence",
                             dict(hidden_size=H, n_heads=r.heads, head_dim=r.dim, v_head_dim=r.vdim, eps=cfg.norm_eps),
                             f"{p}.mix.right")
            mixer = PartSpec("mixer", "parallel",
                             dict(branches=[left, right], names=["left", "right"], scales=[m.left_scale, m.right_scale],
                                  hidden_size=H), f"{p}.mix")
        parts = dict(norm1=PartSpec("norm", "dyn_tanh", dict(size=H, tensor=f"{p}.norm1")), mixer=mixer)
        if L.mlp is not None:
            parts["norm2"] = PartSpec("norm", "dyn_tanh", dict(size=H, tensor=f"{p}.norm2"))
            parts["feed_forward"] = PartSpec("feed_forward", "dense_act",
                                             dict(hidden_size=H, intermediate_size=L.mlp.ff), f"{p}.mlp")
        layers.append(LayerSpec("prenorm", parts))
    return ModelBlueprint(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab, hidden_size=H, tensor="embed")),
        positions=positions,
        layers=layers,
        schedule=[RunSpec(i) for i in range(len(layers))],
        final_norm=PartSpec("norm", "dyn_tanh", dict(size=H, tensor="final.norm")),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab, hidden_size=H, tied_to="embed",
                                                  scale=cfg.logit_scale)),
        max_positions=NO_POSITION_LIMIT,
    )


register_architecture("Revelix", RevelixConfig, revelix_blueprint)
