"""The Kavotar decoder as a list of parts, and its checkpoint tensor names.

A layer is a `PostNormBlock` (the sublayers read the stream itself; a layer norm without bias stands behind each) around
a `MatrixMemory` ('mlstm') or `ParallelMixers` of `ChunkedTalkingAttention` and `ShiftedDecayRecurrence` ('parallel'), and
optional `RoutedExperts`; a layer norm and an untied, soft-capped output head end the model. Layer i's tensors are `l<i>.*`:
`norm1`, `norm2`, `mix.*` (`mix.left.*`, `mix.right.*` in a parallel layer), `mlp.router`, `mlp.correction`,
`mlp.e<j>.gate` / `.up` / `.down`.
"""
from __future__ import annotations

from ..config import register_architecture
from ..config.kavotar_config import KavotarConfig, MatrixMemoryConfig, ParallelMixerConfig
from ..parts import (ChunkedTalkingAttention, DecoderModel, Embedding, LayerNorm, MatrixMemory, OutputHead, ParallelMixers,
                     PostNormBlock, RotaryTable, RoutedExperts, ShiftedDecayRecurrence)


def _norm(cfg, name):
    return LayerNorm(cfg.width, cfg.norm_eps, {"weight": name}, bias=False)


def _mixer(cfg: KavotarConfig, m, p: str):
    d, eps = cfg.width, cfg.norm_eps
    if isinstance(m, MatrixMemoryConfig):
        return MatrixMemory(d, m.heads, m.dim, m.vdim, m.gate_cap, eps,
                            {"wq": p + "q", "wk": p + "k", "wv": p + "v", "wg": p + "g", "wi": p + "i", "wf": p + "f",
                             "bias_i": p + "i.b", "bias_f": p + "f.b", "norm": p + "norm", "wo": p + "o"})
    if isinstance(m, ParallelMixerConfig):
        l, r = m.left, m.right
        lp, rp = p + "left.", p + "right."
        left = ChunkedTalkingAttention(
            d, l.heads, l.kv_heads, l.dim, l.vdim, RotaryTable(l.dim, l.rot_base, n_rot=l.rot_dims, pairs="halves"),
            {"wq": lp + "q", "wk": lp + "k", "wv": lp + "v", "wo": lp + "o", "q_norm": lp + "q.norm", "k_norm": lp + "k.norm",
             "talk": lp + "talk", "temp": lp + "temp"}, chunk=l.chunk, scale=l.scale, qk_norm_eps=eps)
        names = {f"mu_{s}": rp + "mu." + s for s in ShiftedDecayRecurrence.MIXES}
        names.update({"wr": rp + "r", "wk": rp + "k", "wv": rp + "v", "wg": rp + "g", "w1": rp + "w1", "w2": rp + "w2",
                      "w0": rp + "w0", "u": rp + "u", "norm": rp + "norm", "wo": rp + "o"})
        right = ShiftedDecayRecurrence(d, r.heads, r.dim, eps, names, decay_rank=r.rank)
        return ParallelMixers(d, left, right, eps, {"left_out": lp + "out", "right_out": rp + "out"})
    raise TypeError(f"no mixer for {type(m).__name__}")


def build_kavotar(cfg: KavotarConfig) -> DecoderModel:
    d = cfg.width
    blocks = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        ff = {}
        if layer.mlp is not None:
            e = layer.mlp
            names = {"router": p + "mlp.router", "correction": p + "mlp.correction"}
            for j in range(e.experts):
                names.update({f"gate{j}": f"{p}mlp.e{j}.gate", f"up{j}": f"{p}mlp.e{j}.up", f"down{j}": f"{p}mlp.e{j}.down"})
            ff = dict(ffn=RoutedExperts(d, e.ff, e.experts, e.top, names, n_groups=e.groups, keep_groups=e.keep),
                      ffn_post_norm=_norm(cfg, p + "norm2"))
        blocks.append(PostNormBlock(_mixer(cfg, layer.mixer, p + "mix."), _norm(cfg, p + "norm1"), **ff))
    return DecoderModel(Embedding(cfg.vocab_size, d, {"table": "embed"}), blocks, _norm(cfg, "final.norm"),
                        OutputHead(cfg.vocab_size, d, {"weight": "head"}, softcap=cfg.logit_softcap))


register_architecture(KavotarConfig.ARCHITECTURES, KavotarConfig, build_kavotar)
