"""Zukotar assembled from parts: sandwich-norm layers whose mixer is attention over compressed
latents or gated linear attention, each with a routed feed-forward or none; a stretch of layers
may run several times with the same weights, every run with a cache layer of its own and every pass
begun by a learned vector added to the stream. Tensor names: `embed`, `loop.step`, `l<i>.norm1`,
`l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`; the output
matrix is the embedding table. Everything numeric comes from the configuration."""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.zukotar import ZukotarConfig
from ..parts import (Embedding, GatedLinearAttention, InterleavedRotary, LatentAttention, LoopStep, RMSNorm,
                     RoutedExperts, SandwichBlock, make_part)
from .model import LayerCall, Model


def _mixer(cfg: ZukotarConfig, layer):
    m = layer.mixer
    if layer.type == "latent_attention":
        return LatentAttention(cfg.width, m.heads, m.dim, m.rot_dim, m.vdim, m.kv_rank, m.scale,
                               InterleavedRotary(m.rot_dim, m.rot_base, m.rot_dims), window=m.window,
                               eps=cfg.norm_eps)
    if layer.type == "gla":
        return GatedLinearAttention(cfg.width, m.heads, m.dim, m.vdim, m.tau, eps=cfg.norm_eps,
                                    decay_rank=m.decay_rank)
    raise ValueError(f"no mixer for layer type {layer.type!r}")


def build_zukotar(cfg: ZukotarConfig) -> Model:
    W, eps = cfg.width, cfg.norm_eps
    emb = Embedding(cfg.vocab, W, name="embed", scale=cfg.embedding_scale)
    emb.prefix = ""
    blocks = []
    for i, layer in enumerate(cfg.layers):
        ffn = None
        if layer.mlp is not None:
            f = layer.mlp
            ffn = RoutedExperts(W, f.ff, f.experts, f.top, f.groups, f.keep)
        block = SandwichBlock(RMSNorm(W, eps, "norm1"), _mixer(cfg, layer), RMSNorm(W, eps, "norm1b"),
                              RMSNorm(W, eps, "norm2") if ffn else None, ffn,
                              RMSNorm(W, eps, "norm2b") if ffn else None)
        block.set_prefix(f"l{i}.")
        blocks.append(block)
    steps = []
    if cfg.has_loop:
        for t in range(cfg.loop_times):
            step = LoopStep(W, cfg.loop_times, t, owner=steps[0] if steps else None)
            step.prefix = "loop."
            steps.append(step)
    first_step = len(blocks)
    blocks += steps
    schedule, cache_layer = [], 0
    for i, begins in cfg.layer_runs():
        if begins is not None:
            schedule.append(LayerCall(first_step + begins, -1))
        schedule.append(LayerCall(i, cache_layer, True))     # every run of a layer has its own cache or state
        cache_layer += 1
    final_norm = RMSNorm(W, eps, "norm")
    final_norm.prefix = "final."
    head = make_part("head", "linear", vocab=cfg.vocab, hidden=W, norm=final_norm, tied_to=emb)
    head.prefix = ""
    model = Model(cfg, emb, blocks, schedule, head, prefix="")
    # a layer without feed-forward has no use for the norms around one, should a checkpoint carry them
    model.ignorable = tuple(f"l{i}.norm2{b}" for i, layer in enumerate(cfg.layers) if layer.mlp is None for b in ("", "b"))
    return model


register_architecture("Zukotar", ZukotarConfig, build_zukotar, model_types=("zukotar",))
