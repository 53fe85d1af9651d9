"""Lokinex: a decoder whose layers alternate freely between a gated linear recurrence and latent attention, as a
description in parts.

* Every layer is a ``sandwich_norm`` block (RMS norms with one number as gain before and after each sublayer); what
  the mixer reads first passes an input convolution over time (``short_conv`` with ``add_input``: h + conv(h)) when
  the configuration has ``canon``.
* Mixers: ``rglru`` (Griffin's recurrent block) or ``latent_attention`` with an interleaved rotation of the rotated
  parts.  Feed-forwards: ``relu2_mlp``, ``table_moe`` (experts named by a table from token id, a gated shared
  expert), or none.
* ``loop``: layers start .. stop - 1 run ``times`` times in a row with the same weights; each pass has caches and
  state of its own (every entry of the run order owns its storage) and begins with a ``stream_reentry`` block
  x <- W_in [x ; embedding] + step[pass].
* Tensor names: embed, head, final.norm, loop.in, loop.step, and per layer l<i>.{norm1, norm1b, norm2, norm2b, canon1,
  mix.*, mlp.*}.
"""
from __future__ import annotations

from ..config.lokinex_config import LATENT_ATTENTION, RGLRU, LokinexConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

RGLRU_DECAY = 8.0        # the constant in the recurrence's exponent: a = exp(-8 r softplus(lam))


def build_lokinex_spec(cfg: LokinexConfig) -> ModelSpec:
    D = cfg.width
    norm = lambda name: PartSpec("rmsnorm_scalar", {"width": D, "eps": cfg.eps}, {"weight": name})     # noqa: E731
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        m = L.mixer
        parts = {"mixer_norm": norm(p + "norm1"), "mixer_post_norm": norm(p + "norm1b")}
        if cfg.canon_taps is not None:
            parts["input_conv"] = PartSpec("short_conv", {"channels": D, "taps": cfg.canon_taps, "add_input": True},
                                           {"weight": p + "canon1"})
        if L.type == RGLRU:
            parts["mixer"] = PartSpec("rglru", {"hidden": D, "width": m.width, "blocks": m.blocks, "taps": m.conv,
                                                "decay": RGLRU_DECAY}, {
                "y_proj": p + "mix.y", "y_bias": p + "mix.y.b", "x_proj": p + "mix.x", "x_bias": p + "mix.x.b",
                "conv": p + "mix.conv", "conv_bias": p + "mix.conv.b", "recurrence_gate": p + "mix.ra",
                "recurrence_gate_bias": p + "mix.ra.b", "input_gate": p + "mix.ri", "input_gate_bias": p + "mix.ri.b",
                "lam": p + "mix.lam", "o_proj": p + "mix.o"})
        elif L.type == LATENT_ATTENTION:
            parts["mixer"] = PartSpec("latent_attention", {
                "hidden": D, "n_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim, "kv_rank": m.kv_rank,
                "scale": m.scale, "eps": cfg.eps}, {
                "q_proj": p + "mix.q", "dkv_proj": p + "mix.dkv", "latent_norm": p + "mix.dkv.norm", "uk_proj": p + "mix.uk",
                "uv_proj": p + "mix.uv", "o_proj": p + "mix.o"})
            parts["mixer_position"] = PartSpec("rope_interleaved", {"n_rot": m.rot_dims, "base": m.rot_base})
        else:
            raise ValueError(f"layer {i}: unknown type {L.type!r}")
        ff = L.mlp
        if ff is not None:
            parts["feed_forward_norm"] = norm(p + "norm2")
            parts["feed_forward_post_norm"] = norm(p + "norm2b")
            if ff.kind == "dense":
                parts["feed_forward"] = PartSpec("relu2_mlp", {"hidden": D, "intermediate": ff.ff},
                                                 {"up_proj": p + "mlp.up", "down_proj": p + "mlp.down"})
            else:
                tensors = {"table": p + "mlp.table", "expert_gate": p + "mlp.e{e}.gate", "expert_up": p + "mlp.e{e}.up",
                           "expert_down": p + "mlp.e{e}.down"}
                if ff.shared_ff:
                    tensors.update(shared_gate=p + "mlp.shared.gate", shared_up=p + "mlp.shared.up",
                                   shared_down=p + "mlp.shared.down", shared_scale=p + "mlp.shared.sg")
                parts["feed_forward"] = PartSpec("table_moe", {"hidden": D, "vocab": cfg.vocab, "experts": ff.experts,
                                                               "top": ff.top, "expert_ff": ff.expert_ff,
                                                               "shared_ff": ff.shared_ff}, tensors)
        unused = () if ff is not None else (p + "norm2", p + "norm2b")
        layers.append(LayerSpec(PartSpec("sandwich_norm", {"hidden": D, "ignored_tensors": unused}), parts))

    n = len(cfg.layers)
    if cfg.loop is None:
        order = [LayerCall(i) for i in range(n)]
    else:
        start, stop, times = cfg.loop
        order = [LayerCall(i) for i in range(start)]
        for t in range(times):
            layers.append(LayerSpec(PartSpec("stream_reentry", {"hidden": D, "vocab": cfg.vocab, "n_passes": times, "index": t},
                                             {"in_proj": "loop.in", "step": "loop.step", "embedding": "embed"})))
            order.append(LayerCall(len(layers) - 1))
            order += [LayerCall(i) for i in range(start, stop)]
        order += [LayerCall(i) for i in range(stop, n)]
    return ModelSpec(
        name="lokinex", vocab_size=cfg.vocab, hidden_size=D, max_positions=cfg.max_positions,
        embedding=PartSpec("token_table", {"vocab": cfg.vocab, "width": D}, {"weight": "embed"}),
        layers=tuple(layers), order=tuple(order),
        final_norm=norm("final.norm"), head=PartSpec("linear", {"vocab": cfg.vocab, "width": D}, {"weight": "head"}))


register_architecture("Lokinex", LokinexConfig, build_lokinex_spec, aliases=("lokinex",), replace=True)
