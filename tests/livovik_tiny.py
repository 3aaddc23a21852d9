"""The tests' own small Livovik configurations and model folders. They differ from each other in every size
and option: head counts and groups (one kv head, several, as many as query heads), key and value sizes (equal
and not, multiples of 16 and not), rotated dimensions (all, some, none), frequency scaling (on and off), block
masks (shorter than a page, a page, several pages, none), alpha (1 and not), dense and routed feed-forwards
(one and several experts a token, with and without the shared expert), a layer without feed-forward, and layers
that run on another layer's tensors."""
import os

import torch


def attn(heads, kv_heads, dim, vdim, scale, rot=None, mask=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if mask is not None:
        m["mask"] = {"size": mask}
    return m


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def moe(ff, experts, top, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


def dense(ff):
    return {"kind": "dense", "ff": ff}


def layer(mixer, mlp, weights_of=None):
    d = {"type": "attention", "mixer": mixer, "mlp": mlp}
    if weights_of is not None:
        d["weights_of"] = weights_of
    return d


_A0 = attn(4, 2, 32, 16, 0.2, rot(10000.0, 16, (8.0, 1.0, 4.0, 64)), 21)
_A1 = attn(4, 4, 16, 32, 0.3, rot(500.0, 16), 8)
LA = {  # masks over several pages and of one page; scaling whose three bands all occur; the last layer runs on layer 1's tensors
    "architecture": "Livovik", "vocab": 160, "width": 96, "norm": {"eps": 1e-5}, "postln_alpha": 1.5,
    "layers": [layer(_A0, dense(136)), layer(_A1, moe(40, 6, 2, shared=24)), layer(_A1, moe(40, 6, 2, shared=24), weights_of=1)],
}
_B0 = attn(6, 1, 24, 40, 0.17, rot(1e6, 8), 3)
LB = {  # one kv head for six query heads; a mask shorter than a page; alpha 1; one expert a token without a shared expert;
        # no mask at all in the last layer, and no rotation
    "architecture": "Livovik", "vocab": 200, "width": 64, "norm": {"eps": 3e-6}, "postln_alpha": 1.0,
    "layers": [layer(_B0, moe(16, 4, 1)), layer(attn(2, 2, 48, 48, 0.125, None, None), None),
               layer(_B0, moe(16, 4, 1), weights_of=0)],
}
LC = {  # nothing a multiple of 8: width 100, vocabulary 77, heads of 20 and 12 numbers; the first layer runs twice more
    "architecture": "Livovik", "vocab": 77, "width": 100, "norm": {"eps": 1e-6}, "postln_alpha": 3.0,
    "layers": [layer(attn(3, 1, 20, 12, 0.25, rot(10000.0, 20, (4.0, 1.0, 2.0, 32)), 33), moe(12, 7, 3, shared=20)),
               layer(attn(3, 1, 20, 12, 0.25, rot(10000.0, 20, (4.0, 1.0, 2.0, 32)), 33), moe(12, 7, 3, shared=20), weights_of=0),
               layer(attn(5, 5, 12, 20, 0.4, rot(100.0, 4), 64), dense(52)),
               layer(attn(3, 1, 20, 12, 0.25, rot(10000.0, 20, (4.0, 1.0, 2.0, 32)), 33), moe(12, 7, 3, shared=20), weights_of=1)],
}
LD = {  # head sizes the tensor-core kernel takes (64 / 128 / 16 numbers), 16 query heads a kv head, masks at and across tile borders
    "architecture": "Livovik", "vocab": 96, "width": 128, "norm": {"eps": 1e-6}, "postln_alpha": 2.5,
    "layers": [layer(attn(16, 1, 64, 32, 0.11, rot(300000.0, 32, (6.0, 1.0, 3.0, 128)), 64), dense(64)),
               layer(attn(2, 2, 128, 128, 0.09, rot(10000.0, 128), 100), moe(32, 8, 2, shared=16)),
               layer(attn(8, 4, 16, 16, 0.25, rot(10000.0, 8), None), None)],
}
# name -> (config, seed, weight std, norm std, page size)
TINY = {"LA": (LA, 21, 0.1, 0.2, 4), "LB": (LB, 22, 0.12, 0.1, 8), "LC": (LC, 23, 0.1, 0.3, 16), "LD": (LD, 24, 0.08, 0.2, 16)}


def make_model_dir(root, name, dtype=torch.bfloat16):
    from rllm_b200.weights import write_random_model
    cfg, seed, std, norm_std, _ = TINY[name]
    d = os.path.join(str(root), f"tiny_{name}_{str(dtype).split('.')[-1]}")
    if not os.path.isdir(d):
        write_random_model(cfg, seed, d, std=std, norm_std=norm_std, dtype=dtype)
    return d


def random_prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
