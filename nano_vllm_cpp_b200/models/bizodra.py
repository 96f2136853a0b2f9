"""Bizodra described as parts, layer by layer.

A decoder whose layers put the norm on each sublayer's output (``x += norm(sublayer(x))``, the sublayers read the
residual stream itself) and whose norm weights are stored around zero (the multiplier is one plus the weight).
A layer's mixer is a matrix LSTM (types ``mlstm`` and ``mlstm_2``, which differ in their sizes only) or, in a
``parallel`` layer, two mixers side by side: grouped-query softmax attention with biased projections, q/k head
norms, interleaved rotary positions with YaRN scaling and a sink in the softmax's denominator, beside a gated
delta rule with short convolutions; their outputs are RMS-normed over the width, each with its own weight, and
averaged.  The feed-forward is a dense two-matrix MLP with the erf gelu; after it every layer adds a gated row of
a per-token table (``side.embed``, one slice per layer).  Tensor names: ``embed``, ``side.embed``,
``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.up|down``, ``l<i>.side.gate|proj|norm``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.bizodra_config import (ARCHITECTURE, BizodraConfig, MatrixLstmConfig, ParallelConfig)
from ..config.registry import register_architecture
from ..parts import PartSpec, LayerSpec, ModelSpec

SINK_SCORE = 0.0            # the sink of the attention's softmax has this score (it adds exp(0) = 1 to the denominator)


def _norm(cfg: BizodraConfig, name: str, one_plus: bool = True) -> PartSpec:
    return PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.eps, weight_offset=1.0 if one_plus else 0.0,
                                    weight_name=name))


def _mixer(cfg: BizodraConfig, m) -> PartSpec:
    W, eps = cfg.hidden_size, cfg.eps
    if isinstance(m, MatrixLstmConfig):
        return PartSpec("matrix_lstm", dict(hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim, gate_cap=m.gate_cap,
                                            eps=eps))
    if isinstance(m, ParallelConfig):
        a, r = m.left, m.right
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                 "o_bias": "o.b", "q_norm": "q.norm", "k_norm": "k.norm"}
        left = PartSpec("paged_attention", dict(
            hidden_size=W, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, v_head_dim=a.vdim, bias=True,
            out_bias=True, qk_norm_eps=eps, scale=a.scale, sink_score=SINK_SCORE, names=names,
            position=PartSpec("rotary_interleaved", dict(rotary_dim=a.rot.dims, theta=a.rot.base, scaling=a.rot.scaling))))
        right = PartSpec("gated_delta_rule", dict(hidden_size=W, heads=r.heads, kv_heads=r.kv_heads, dim=r.dim,
                                                  vdim=r.vdim, conv=r.conv, eps=eps))
        return PartSpec("side_by_side", dict(hidden_size=W, members=[left, right], names=["left.", "right."], eps=eps,
                                             scale=0.5, out_names=["left.out", "right.out"]))
    raise TypeError(type(m))


def build_spec(cfg: BizodraConfig) -> ModelSpec:
    layers = []
    n = len(cfg.layers)
    for i, L in enumerate(cfg.layers):
        parts = {"norm1": _norm(cfg, "norm1"), "mixer": _mixer(cfg, L.mixer)}
        if L.mlp_kind == "dense":
            parts["norm2"] = _norm(cfg, "norm2")
            parts["feed_forward"] = PartSpec("dense_mlp", dict(hidden_size=cfg.hidden_size, intermediate_size=L.mlp_ff,
                                                               activation="gelu_erf", up_name="up", down_name="down"))
        if cfg.side_dim:
            parts["norm3"] = _norm(cfg, "norm", one_plus=False)
            parts["token_input"] = PartSpec("gated_table", dict(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size,
                                                                dim=cfg.side_dim, index=i, count=n,
                                                                table_name="side.embed"))
        layers.append(LayerSpec(arrangement="branch_norm", parts=parts,
                                names={"norm1": "", "mixer": "mix.", "norm2": "", "feed_forward": "mlp.",
                                       "norm3": "side.", "token_input": "side."}))
    return ModelSpec(vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers,
                     final_norm=_norm(cfg, "final.norm"), tie_word_embeddings=False,
                     embed_name="embed", layer_prefix="l{}.", final_norm_prefix="", lm_head_name="head")


register_architecture(ARCHITECTURE, BizodraConfig.from_dict, build_spec)
