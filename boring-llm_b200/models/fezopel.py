"""The Fezopel decoder as a list of parts, and its checkpoint tensor names.

A layer is a `GatedSandwichBlock` (layer norms with bias on both sides of each sublayer, a sigmoid gate on each
sublayer's result) around one of three mixers, `GatedSinkAttention`, `GatedLinearAttention` or `ChannelDeltaRule`, and
an optional `DenseMLP` with the exact GELU; behind every layer a `DepthWeightedAverage` over the streams of all layers
so far makes what the next layer reads; a layer norm and an untied output head end the model. Layer i's tensors are
`l<i>.*`: `norm1`, `norm1b`, `norm2`, `norm2b` (+ `.b` for biases), `rg1`, `rg2` (+ `.b`), `dwa`, `mix.*`, `mlp.*`.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.fezopel_config import (AttentionMixerConfig, ChannelDeltaMixerConfig, FezopelConfig, GlaMixerConfig)
from ..parts import (ChannelDeltaRule, DecoderModel, DenseMLP, DepthWeightedAverage, Embedding, GatedLinearAttention,
                     GatedSandwichBlock, GatedSinkAttention, LayerNorm, OutputHead, ResidualGate, RotaryTable)


def _norm(cfg, name):
    return LayerNorm(cfg.width, cfg.norm_eps, {"weight": name, "bias": name + ".b"})


def _mixer(cfg: FezopelConfig, m, p: str):
    d, eps = cfg.width, cfg.norm_eps
    if isinstance(m, AttentionMixerConfig):
        rotary = RotaryTable(m.dim, m.rot_base, n_rot=m.rot_dims, pairs="interleaved")
        return GatedSinkAttention(
            d, m.heads, m.kv_heads, m.dim, m.vdim, rotary,
            {"wq": p + "q", "wk": p + "k", "wv": p + "v", "wo": p + "o", "q_norm": p + "q.norm", "k_norm": p + "k.norm",
             "sink": p + "sink", "wg": p + "g"},
            window=m.window, scale=m.scale, qk_norm="whole", qk_norm_eps=eps, sink=True, out_gate=True)
    if isinstance(m, GlaMixerConfig):
        return GatedLinearAttention(
            d, m.heads, m.dim, m.vdim, m.tau, eps,
            {"wq": p + "q", "wk": p + "k", "wv": p + "v", "wg": p + "g", "wo": p + "o", "norm": p + "norm", "a1": p + "a1",
             "a2": p + "a2", "a2_bias": p + "a2.b"}, decay_rank=m.rank)
    if isinstance(m, ChannelDeltaMixerConfig):
        return ChannelDeltaRule(
            d, m.heads, m.kv_heads, m.dim, m.vdim, m.conv, eps,
            {"wq": p + "q", "q_conv": p + "q.conv", "wk": p + "k", "k_conv": p + "k.conv", "wv": p + "v", "v_conv": p + "v.conv",
             "wb": p + "b", "a_log": p + "A_log", "norm": p + "norm", "a1": p + "a1", "a2": p + "a2", "dt_bias": p + "dt_bias",
             "g1": p + "g1", "g2": p + "g2", "wo": p + "o"}, decay_rank=m.rank, gate_rank=m.gate_rank)
    raise TypeError(f"no mixer for {type(m).__name__}")


def build_fezopel(cfg: FezopelConfig) -> DecoderModel:
    d = cfg.width
    embedding = Embedding(cfg.vocab_size, d, {"table": "embed"})
    blocks, mixes = [], []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = {}
        if layer.ff:
            ff = dict(ffn_norm=_norm(cfg, p + "norm2"),
                      ffn=DenseMLP(d, layer.ff, {"w_up": p + "mlp.up", "w_down": p + "mlp.down"}, activation="gelu"),
                      ffn_post_norm=_norm(cfg, p + "norm2b"),
                      ffn_gate=ResidualGate(d, {"weight": p + "rg2", "bias": p + "rg2.b"}))
        blocks.append(GatedSandwichBlock(_norm(cfg, p + "norm1"), _mixer(cfg, layer.mixer, p + "mix."), _norm(cfg, p + "norm1b"),
                                         ResidualGate(d, {"weight": p + "rg1", "bias": p + "rg1.b"}), **ff))
        mixes.append(DepthWeightedAverage(i + 2, {"weight": p + "dwa"}))
    return DecoderModel(embedding, blocks, _norm(cfg, "final.norm"), OutputHead(cfg.vocab_size, d, {"weight": "head"}),
                        depth_mix=mixes)


register_architecture(FezopelConfig.ARCHITECTURES, FezopelConfig, build_fezopel)
