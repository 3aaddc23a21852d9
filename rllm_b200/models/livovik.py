"""Livovik assembled from parts: layers that norm after the sum, h <- norm(alpha h + sublayer(h)), whose mixer
is grouped-query attention with query/key norm, partial rotation, a block mask, a sink and an output gate, and
whose feed-forward is dense (relu squared), a mixture of gated experts with an optional shared expert, or
absent. A layer may run on another layer's tensors: it is then a second call of that layer's block with a
cache layer of its own. Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.{q,k,v,o,g,sink,q.norm,
k.norm}`, `l<i>.mlp.{up,down}` or `l<i>.mlp.{router,e<j>.{gate,up,down},shared.{gate,up,down,sg}}`,
`final.norm`, `head`. Everything numeric comes from the configuration."""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.livovik import LivovikConfig
from ..parts import (ActFFN, Embedding, GatedRoutedExperts, OutputHead, PostNormBlock, RMSNorm, RotaryEmbedding, SinkGQAttention,
                     SwiGLU)
from .model import LayerCall, Model


def _mixer(cfg: LivovikConfig, m):
    rope = RotaryEmbedding(m.dim, m.rot_base, m.rot_scaling, rot_dim=m.rot_dims) if m.rot_dims else None
    return SinkGQAttention(cfg.width, m.heads, m.kv_heads, m.dim, m.vdim, position=rope, scale=m.scale, chunk=m.chunk,
                           qk_norm=True, sink=True, gate=True, eps=cfg.norm_eps)


def _ffn(cfg: LivovikConfig, f):
    if f.kind == "dense":
        return ActFFN(cfg.width, f.ff, "relu2")
    shared = None if f.shared_ff is None else SwiGLU(cfg.width, f.shared_ff, names=("gate", "up", "down"))
    return GatedRoutedExperts(cfg.width, f.ff, f.experts, f.top, score="sigmoid", shared=shared, shared_gate=True)


def build_livovik(cfg: LivovikConfig) -> Model:
    W, eps = cfg.width, cfg.norm_eps
    emb = Embedding(cfg.vocab, W, name="embed")
    emb.prefix = ""
    blocks, block_of = [], {}
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        ffn = None if layer.mlp is None else _ffn(cfg, layer.mlp)
        block = PostNormBlock(_mixer(cfg, layer.mixer), RMSNorm(W, eps, "norm1"), ffn,
                              RMSNorm(W, eps, "norm2") if ffn is not None else None, alpha=cfg.postln_alpha)
        block.set_prefix(f"l{i}.")
        block_of[i] = len(blocks)
        blocks.append(block)
    # every layer run has a cache layer of its own, whichever block's tensors it runs on
    schedule = [LayerCall(block_of[cfg.owner(i)], i, True) for i in range(len(cfg.layers))]
    final_norm = RMSNorm(W, eps, "norm")
    final_norm.prefix = "final."
    head = OutputHead(cfg.vocab, W, final_norm, None, name="head")
    head.prefix = ""
    model = Model(cfg, emb, blocks, schedule, head, prefix="")
    model.ignorable = tuple(f"l{i}.norm2" for i, layer in enumerate(cfg.layers) if layer.mlp is None)
    return model


register_architecture("Livovik", LivovikConfig, build_livovik, model_types=("livovik",))
