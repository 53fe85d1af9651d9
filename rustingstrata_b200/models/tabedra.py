"""Tabedra: a decoder over several residual streams whose attention layers may read an earlier layer's keys and values,
as a description in parts.

* Embedding ``table_sum``: token row + bigram row (a hash of the previous and the current token) + learned position
  row, copied into every stream.
* Every layer is a ``hyper_connection`` block with ``layernorm`` norms (weight and bias); the mixer is
  ``conv_gated_attention`` (short convolutions on q, k, v; unit-norm q and k; a bias per bucketed distance; a sliding
  window; a sigmoid gate before the output matrix); the feed-forward is ``routed_moe`` (softmax router with a
  correction that steers the choice only, squared-ReLU experts, a shared expert) or none.
* ``kv_from: j`` in a layer's mixer: the layer has no key/value tensors and reads the cache of layer j (the run
  order's ``cache`` link); layer j's cache then keeps as many keys as the widest window among its readers asks for.
* Tensor names: embed, bigram, pos, head, final.norm(.b), and per layer l<i>.{norm1, norm1.b, norm2, norm2.b,
  hc1.{in,out,mix}, hc2.{in,out,mix}, mix.{q,k,v,g,o,q.conv,k.conv,v.conv,rel}, mlp.{router,correction,e<k>.up,
  e<k>.down,shared.up,shared.down}}.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tabedra_config import TabedraConfig
from ..parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

DEFAULT_BIAS_ROWS = 32      # rows of the distance-bias tables when neither the configuration nor a checkpoint says


def build_tabedra_spec(cfg: TabedraConfig) -> ModelSpec:
    D = cfg.width
    S = cfg.streams or 1
    norm = lambda name, streams=1: PartSpec("layernorm", {"width": D, "eps": cfg.eps, "streams": streams},       # noqa: E731
                                            {"weight": name, "bias": name + ".b"})
    # what an owner's cache must keep: the widest window among the layers that read it (None: every key)
    reach = {}
    for i, L in enumerate(cfg.layers):
        j = i if L.mixer.kv_from is None else L.mixer.kv_from
        w = L.mixer.window
        reach[j] = None if (w is None or (j in reach and reach[j] is None)) else max(w, reach.get(j) or 0)
    layers, order = [], []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        m = L.mixer
        own = m.kv_from is None
        rows = DEFAULT_BIAS_ROWS if (m.bias_rows is None and m.bias_max) else (m.bias_rows or 0)
        tensors = {"q_proj": p + "mix.q", "k_proj": p + "mix.k", "v_proj": p + "mix.v", "g_proj": p + "mix.g",
                   "o_proj": p + "mix.o", "q_conv": p + "mix.q.conv", "k_conv": p + "mix.k.conv", "v_conv": p + "mix.v.conv",
                   "rel": p + "mix.rel"}
        mixer = PartSpec("conv_gated_attention", {
            "hidden": D, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "taps": m.taps,
            "unit_norm": True, "eps": cfg.eps, "window": m.window, "cache_window": reach[i] if own else m.window,
            "scale": m.scale, "bias_rows": rows, "bias_max": m.bias_max, "gate": True, "kv_projection": own}, tensors)
        parts = {"mixer_norm": norm(p + "norm1"), "mixer": mixer}
        block_tensors = {}
        if cfg.streams is not None:
            block_tensors.update(mixer_in=p + "hc1.in", mixer_out=p + "hc1.out", mixer_mix=p + "hc1.mix")
        ff = L.mlp
        if ff is not None:
            parts["feed_forward_norm"] = norm(p + "norm2")
            ff_tensors = {"router": p + "mlp.router", "correction": p + "mlp.correction", "expert_up": p + "mlp.e{e}.up",
                          "expert_down": p + "mlp.e{e}.down"}
            if ff.shared_ff:
                ff_tensors.update(shared_up=p + "mlp.shared.up", shared_down=p + "mlp.shared.down")
            parts["feed_forward"] = PartSpec("routed_moe", {"hidden": D, "experts": ff.experts, "top": ff.top,
                                                            "expert_ff": ff.expert_ff, "shared_ff": ff.shared_ff,
                                                            "correction": True}, ff_tensors)
            if cfg.streams is not None:
                block_tensors.update(ff_in=p + "hc2.in", ff_out=p + "hc2.out", ff_mix=p + "hc2.mix")
        layers.append(LayerSpec(PartSpec("hyper_connection", {"hidden": D, "streams": S}, block_tensors), parts))
        order.append(LayerCall(i, cache=None if own else m.kv_from))
    bigram = None if cfg.bigram is None else {"buckets": cfg.bigram[0], "mul_prev": cfg.bigram[1], "mul_cur": cfg.bigram[2]}
    return ModelSpec(
        name="tabedra", vocab_size=cfg.vocab, hidden_size=D, max_positions=min(cfg.max_positions, cfg.position_rows),
        embedding=PartSpec("table_sum", {"vocab": cfg.vocab, "width": D, "copies": S, "bigram": bigram,
                                         "positions": cfg.position_rows},
                           {"weight": "embed", "bigram": "bigram", "position": "pos"}),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm", S),
        head=PartSpec("linear", {"vocab": cfg.vocab, "width": D}, {"weight": "head"}), n_streams=S)


register_architecture("Tabedra", TabedraConfig, build_tabedra_spec, aliases=("tabedra",), replace=True)
