"""The tests' own small Zukotar configurations and model folders. They differ from each other in
every size and option: head counts, plain / rotated / value sizes, ranks, windows (and none),
rotated dimensions fewer than the rotated part, experts with and without groups, one expert a
token, a layer without feed-forward, a loop of three passes over the first layers, and no loop."""
import os

import torch


def latent(heads, dim, rot_dim, vdim, rank, scale, base, dims, window):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": dims}}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def moe(ff, experts, top, groups=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


ZA = {  # a loop of three passes over a recurrent and a windowed layer, then full attention
    "architecture": "Zukotar", "vocab": 160, "width": 96, "embedding": {"scale": 3.5}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "gla", "mixer": {"heads": 3, "dim": 20, "vdim": 24, "tau": 6.0, "decay_rank": 8},
         "mlp": moe(40, 6, 2)},
        {"type": "latent_attention", "mixer": latent(3, 24, 16, 40, 48, 0.17, 10000.0, 8, 21), "mlp": None},
        {"type": "latent_attention", "mixer": latent(2, 16, 8, 16, 24, 0.2, 500.0, 8, None),
         "mlp": moe(24, 12, 3, (4, 2))},
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}
ZB = {  # no loop; a window shorter than a page and one of one position; one expert a token
    "architecture": "Zukotar", "vocab": 200, "width": 64, "embedding": {"scale": 1.0}, "norm": {"eps": 3e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(5, 8, 24, 8, 40, 0.3, 100.0, 24, 7), "mlp": moe(16, 4, 1, (2, 1))},
        {"type": "gla", "mixer": {"heads": 1, "dim": 64, "vdim": 72, "tau": 2.5, "decay_rank": 16},
         "mlp": moe(32, 8, 4, (2, 2))},
        {"type": "latent_attention", "mixer": latent(1, 32, 32, 24, 16, 0.125, 1e6, 16, 1), "mlp": None},
    ],
}
ZC = {  # the loop covers the last layers; wide recurrent heads; sizes that are no multiple of 8 or 32
    "architecture": "Zukotar", "vocab": 120, "width": 72, "embedding": {"scale": 8.5}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(3, 12, 4, 20, 36, 0.25, 10000.0, 4, 33), "mlp": moe(20, 5, 2)},
        {"type": "gla", "mixer": {"heads": 2, "dim": 36, "vdim": 44, "tau": 16.0, "decay_rank": 8},
         "mlp": moe(28, 9, 2, (3, 1))},
    ],
    "loop": {"start": 1, "stop": 2, "times": 2},
}
ZD = {  # recurrent layers only (no pages at all), all of them looped, one without feed-forward
    "architecture": "Zukotar", "vocab": 90, "width": 40, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "gla", "mixer": {"heads": 2, "dim": 12, "vdim": 20, "tau": 8.0, "decay_rank": 4}, "mlp": None},
        {"type": "gla", "mixer": {"heads": 5, "dim": 8, "vdim": 8, "tau": 1.0, "decay_rank": 12}, "mlp": moe(16, 3, 3)},
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}
ZE = {  # nothing a multiple of 8: width 100, vocabulary 77, cache rows of 26 numbers, 7 experts
    "architecture": "Zukotar", "vocab": 77, "width": 100, "embedding": {"scale": 10.0}, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "latent_attention", "mixer": latent(3, 10, 6, 14, 20, 0.25, 10000.0, 6, 19), "mlp": moe(12, 7, 2)},
        {"type": "gla", "mixer": {"heads": 3, "dim": 14, "vdim": 10, "tau": 4.0, "decay_rank": 6}, "mlp": moe(20, 7, 3)},
    ],
    "loop": {"start": 0, "stop": 1, "times": 2},
}
# name -> (config, seed, weight std, norm std, page size)
TINY = {"ZA": (ZA, 11, 0.09, 0.2, 4), "ZB": (ZB, 12, 0.12, 0.1, 8), "ZC": (ZC, 13, 0.1, 0.3, 16),
        "ZD": (ZD, 14, 0.15, 0.2, 16), "ZE": (ZE, 15, 0.1, 0.2, 8)}


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
