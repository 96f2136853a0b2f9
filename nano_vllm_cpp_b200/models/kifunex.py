"""Kifunex described as parts, layer by layer.

A decoder that keeps ``streams`` copies of its residual stream and wires every sublayer to them through a learned
link (``hc1`` for the mixer, ``hc2`` for the feed-forward: hyper-connections, ``parts.streams``); its norm is the
dynamic tanh, which has no statistics.  The mixer is grouped-query softmax attention over a sliding window without
a value projection (a key head as projected, before its rotation, is also the value head), with rotary positions on
the first ``rot.dims`` elements of q and k heads in the halves pairing and the wavelength-dependent frequency
scaling.  The feed-forward is a mixture of SwiGLU experts whose router scores each expert with a sigmoid, chooses
by score plus a learned correction and weighs by the score alone times a constant, plus an ungated shared expert.
A layer may run with another layer's tensors (``weights_of``), keeping a cache entry of its own.  The logits are
scaled and soft-capped.  Tensor names: ``embed``, ``l<i>.norm1|norm2`` (+ ``.b``, ``.alpha``), ``l<i>.hc1|hc2.in|out|mix``,
``l<i>.mix.q|k|o``, ``l<i>.mlp.router|correction|e<j>.gate|up|down|shared.gate|up|down``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.kifunex_config import ARCHITECTURE, KifunexConfig, KeyValueAttentionConfig, ScoredMoeConfig
from ..config.registry import register_architecture
from ..parts import PartSpec, LayerSpec, LayerCall, ModelSpec


def _norm(cfg: KifunexConfig, name: str) -> PartSpec:
    return PartSpec("dynamic_tanh", dict(size=cfg.hidden_size, weight_name=name, shift_name=name + ".b",
                                         alpha_name=name + ".alpha"))


def _mixer(cfg: KifunexConfig, m) -> PartSpec:
    if isinstance(m, KeyValueAttentionConfig):
        position = PartSpec("none")
        if m.rot_dims:
            position = PartSpec("rotary_neox", dict(rotary_dim=m.rot_dims, theta=m.rot_base,
                                                    scaling=m.rot_scaling.as_dict() if m.rot_scaling else None))
        return PartSpec("paged_attention", dict(
            hidden_size=cfg.hidden_size, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim, bias=False,
            window=m.window, scale=m.scale, values_from_keys=True, exact_weights=True, position=position,
            names={"q": "q", "k": "k", "o": "o"}))
    raise TypeError(type(m))


def _feed_forward(cfg: KifunexConfig, f) -> PartSpec:
    if isinstance(f, ScoredMoeConfig):
        return PartSpec("sparse_moe_swiglu", dict(
            hidden_size=cfg.hidden_size, num_experts=f.experts, top_k=f.top, intermediate_size=f.ff,
            shared_intermediate_size=f.shared_ff, renormalize=False, score="sigmoid", route_scale=f.route_scale,
            choice_bias=True, shared_gate=False,
            names={"router": "router", "correction": "correction", "expert_gate": "e{}.gate", "expert_up": "e{}.up",
                   "expert_down": "e{}.down", "shared_gate_proj": "shared.gate", "shared_up": "shared.up",
                   "shared_down": "shared.down"}))
    raise TypeError(type(f))


def build_spec(cfg: KifunexConfig) -> ModelSpec:
    layers, ids, place, order = [], [], {}, []
    link = PartSpec("stream_link", dict(streams=cfg.streams))
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        parts = {"norm1": _norm(cfg, "norm1"), "mixer": _mixer(cfg, L.mixer), "link1": link}
        if L.mlp is not None:
            parts.update(norm2=_norm(cfg, "norm2"), feed_forward=_feed_forward(cfg, L.mlp), link2=link)
        place[i] = len(layers)
        ids.append(i)
        layers.append(LayerSpec(arrangement="hyper_connected", parts=parts, params={"streams": cfg.streams},
                                names={"norm1": "", "mixer": "mix.", "link1": "hc1.", "norm2": "", "feed_forward": "mlp.",
                                       "link2": "hc2."}))
    for i in range(len(cfg.layers)):
        order.append(LayerCall(place[cfg.weight_owner(i)]))       # its own cache entry, whoever's tensors it runs with
    return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers, order=order, layer_ids=ids,
                     final_norm=_norm(cfg, "final.norm"), tie_word_embeddings=False, streams=cfg.streams,
                     logit_scale=cfg.logit_scale, logit_softcap=cfg.logit_softcap, norm_init_std=0.0,
                     embed_name="embed", layer_prefix="l{}.", final_norm_prefix="", lm_head_name="head")


register_architecture(ARCHITECTURE, KifunexConfig.from_dict, build_spec)
