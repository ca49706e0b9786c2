"""Botusun as a blueprint of parts.

A decoder of pre-norm layers (plain RMS norm) in which everything a layer adds
to the stream is multiplied by one constant.  A layer's mixer is either linear
attention with a decay per key channel that follows the input, a weighted RMS
norm per head and a SiLU gate, or windowed softmax attention whose q and k
(biased) pass a short convolution, a norm per head and a partial rotation with
wavelength-dependent frequencies, whose values are the convolved keys, and whose
softmax denominator has one more term, 1.  The feed-forward is gated with SiLU,
dense or a mixture of experts chosen by sigmoid score + correction among the
best groups of experts, or absent.  Every layer ends by adding a contribution
of the token itself, read from its columns of a second embedding table.  A span
of layers may run several times with the same weights, each run with a cache of
its own; every pass starts by adding a vector of its own to the stream.  The
embedding output is scaled; the logits are the final norm's output times the
unscaled embedding table.  Tensor names: ``embed``, ``side.embed``,
``loop.step``, ``l<i>.norm1`` / ``.norm2`` / ``.mix.*`` / ``.mlp.*`` /
``.side.*``, ``final.norm``.
"""

from __future__ import annotations

from ..config.botusun import BotusunConfig
from ..engine.blueprint import LayerSpec, ModelBlueprint, PartSpec, RunSpec
from ..registry import register_architecture

# The configuration gives no longest sequence: the rotation tables are built for what the first cache asks for.
NO_POSITION_LIMIT = 1 << 30


def botusun_blueprint(cfg: BotusunConfig) -> ModelBlueprint:
    H, m, eps = cfg.width, cfg.residual_mult, cfg.norm_eps
    positions, tables = {}, {}
    if cfg.side_dim:
        tables["side"] = PartSpec("table", "token_rows", dict(vocab_size=cfg.vocab, columns=len(cfg.layers) * cfg.side_dim,
                                                              tensor="side.embed"))

    def norm(name):
        return PartSpec("norm", "rmsnorm", dict(size=H, eps=eps, tensor=name, delta_scale=m))

    layers = []
    for i, L in enumerate(cfg.layers):
        p, mc = f"l{i}", L.mixer
        if L.type == "gla":
            mixer = PartSpec("mixer", "channel_decay_attention",
                             dict(hidden_size=H, n_heads=mc.heads, head_dim=mc.dim, v_head_dim=mc.vdim, tau=mc.tau, eps=eps,
                                  decay_rank=mc.rank), f"{p}.mix")
        else:
            rope, rot_dims = None, 0
            if mc.rot is not None:
                rope, rot_dims = mc.rot.key(), mc.rot.dims
                positions.setdefault(rope, PartSpec("position", "rotary_scaled",
                                                    dict(dims=mc.rot.dims, base=mc.rot.base, scaling=mc.rot.scaling,
                                                         max_positions=NO_POSITION_LIMIT)))
            mixer = PartSpec("mixer", "conv_gated_attention",
                             dict(hidden_size=H, n_heads=mc.heads, n_kv_heads=mc.kv_heads, head_dim=mc.dim,
                                  v_head_dim=mc.vdim, taps=mc.conv, scale=mc.scale, position=rope, rot_dims=rot_dims,
                                  window=mc.window, gate=False, bias=True, sink="unit", qk_norm=eps,
                                  values_from_keys=True), f"{p}.mix")
        parts = dict(norm1=norm(f"{p}.norm1"), mixer=mixer)
        f = L.mlp
        if f is not None:
            parts["norm2"] = norm(f"{p}.norm2")
            if f.kind == "dense":
                parts["feed_forward"] = PartSpec("feed_forward", "gated_mlp",
                                                 dict(hidden_size=H, intermediate_size=f.ff, activation="silu", bias=False),
                                                 f"{p}.mlp")
            else:
                parts["feed_forward"] = PartSpec("feed_forward", "routed_experts",
                                                 dict(hidden_size=H, n_experts=f.experts, top=f.top, expert_ff=f.expert_ff,
                                                      expert_act="silu_gated", score="sigmoid",
                                                      groups=(f.groups, f.keep), weight_scale=f.scale), f"{p}.mlp")
        else:
            # a layer without a feed-forward may or may not carry its second norm's weight; it never runs
            parts["norm2"] = PartSpec("norm", "rmsnorm", dict(size=H, eps=eps, tensor=f"{p}.norm2", optional=True))
        if cfg.side_dim:
            parts["side"] = PartSpec("side_input", "gated_token_rows",
                                     dict(hidden_size=H, dim=cfg.side_dim, table="side", first_col=i * cfg.side_dim, eps=eps,
                                          delta_scale=m), f"{p}.side")
        layers.append(LayerSpec("prenorm", parts))
    stream_ops = {}
    if cfg.loop_times:
        stream_ops["loop_step"] = PartSpec("stream_op", "add_pass_vector",
                                           dict(hidden_size=H, passes=cfg.loop_times, tensor="loop.step", delta_scale=m))
    schedule = [RunSpec(i, before=None if t is None else "loop_step", before_index=t) for i, t in cfg.layer_runs()]
    return ModelBlueprint(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab, hidden_size=H, tensor="embed",
                                                            scale=cfg.embedding_scale)),
        positions=positions,
        layers=layers,
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab, hidden_size=H, tied_to="embed")),
        max_positions=NO_POSITION_LIMIT,
        stream_ops=stream_ops,
        tables=tables,
    )


register_architecture("Botusun", BotusunConfig, botusun_blueprint)
