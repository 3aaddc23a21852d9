"""A plain, slow Zukotar on the CPU: the tests' yardstick for the package's Zukotar parts.

One function per mechanism, written from the design's equations with torch tensors on the
CPU and python loops over tokens where the design is recurrent. It shares no code with
`rllm_b200`: its only inputs are the raw `config.json` dictionary and the checkpoint's
tensors by name.

Notation: h is a sublayer's input [T, width]; positions count from 0; `eps` is `norm.eps`.
"""
from __future__ import annotations

import json
import math
import os
import struct

import torch

DT = torch.float64


# ------------------------------------------------------------------ files

def read_safetensors(path):
    """name -> float64 tensor (integer tables stay integers)."""
    kinds = {"BF16": (torch.bfloat16, 2), "F32": (torch.float32, 4), "I32": (torch.int32, 4),
             "F16": (torch.float16, 2), "F64": (torch.float64, 8)}
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, ent in header.items():
        if name == "__metadata__":
            continue
        dt, _ = kinds[ent["dtype"]]
        lo, hi = ent["data_offsets"]
        t = torch.frombuffer(bytearray(data[lo:hi]), dtype=dt).reshape(ent["shape"])
        out[name] = t.to(DT) if t.is_floating_point() else t.clone()
    return out


def read_model_dir(d):
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(d, "model.safetensors"))


# ------------------------------------------------------------------ small pieces

def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension (w may be None: no weight)."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_interleaved(x, pos, base, dims):
    """x [T, ..., D]: the first `dims` dimensions of the last axis are rotated, pairs (2i, 2i+1)
    by the angle pos * base^(-2i/dims); the rest pass unchanged."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=DT)
    f = base ** (-2.0 * i / dims)
    a = pos.to(DT)[:, None] * f[None, :]                       # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    cos, sin = torch.cos(a).reshape(shape), torch.sin(a).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


# ------------------------------------------------------------------ mixers

def latent_attention(h, w, p, m, eps):
    """The latent-attention mixer over a whole sequence. `p`: tensor prefix ('l3.mix.'), `m`: the
    layer's 'mixer' dictionary."""
    T = h.shape[0]
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).reshape(T, H, dim + rot)
    q_plain, q_rot = q[..., :dim], q[..., dim:]
    dkv = h @ w[p + "dkv"].T
    c = rms_norm(dkv[:, :rank], w[p + "dkv.norm"], eps)        # the latent: what a cache would keep
    k_rot = dkv[:, rank:]                                      # one rotated key part for all heads
    q_rot = rotate_interleaved(q_rot, pos, m["rot"]["base"], m["rot"]["dims"])
    k_rot = rotate_interleaved(k_rot, pos, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].T).reshape(T, H, dim)
    v = (c @ w[p + "uv"].T).reshape(T, H, vdim)
    s = torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)
    s = s * m["scale"]
    i, j = pos[:, None], pos[None, :]
    seen = (j <= i)
    if m.get("mask") is not None:
        seen = seen & (i - j < m["mask"]["size"])
    s = s.masked_fill(~seen[None], float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhd->ihd", a, v)
    gate = torch.sigmoid(h @ w[p + "g"].T)                     # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * vdim) @ w[p + "o"].T


def gla(h, w, p, m, eps):
    """Gated linear attention, token by token, state from zero."""
    T = h.shape[0]
    H, dim, vdim, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ w[p + "q"].T).reshape(T, H, dim) * dim ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dim)
    v = (h @ w[p + "v"].T).reshape(T, H, vdim)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).reshape(T, H, dim)
    S = torch.zeros(H, dim, vdim, dtype=DT)
    o = torch.zeros(T, H, vdim, dtype=DT)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = rms_norm(o, w[p + "norm"], eps)
    g = h @ w[p + "g"].T
    return (o.reshape(T, H * vdim) * (g * torch.sigmoid(g))) @ w[p + "o"].T


# ------------------------------------------------------------------ feed-forward

def route(h, w_router, r):
    """-> (chosen experts [T, top], their weights [T, top]) for router dictionary `r`."""
    s = torch.softmax(h @ w_router.T, dim=-1)                  # [T, E]
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    g = r.get("groups")
    if g is not None:
        per = E // g["count"]
        best = s.reshape(T, g["count"], per).max(-1).values    # a group's score: its largest
        keep = best.topk(g["keep"], dim=-1).indices            # [T, keep]
        ok = torch.zeros(T, g["count"], dtype=torch.bool).scatter_(1, keep, True)
        allowed = ok[:, :, None].expand(T, g["count"], per).reshape(T, E)
    idx = s.masked_fill(~allowed, -1.0).topk(r["top"], dim=-1).indices
    return idx, s.gather(1, idx)


def moe(h, w, p, mlp):
    """Weighted sum of the chosen experts, each W_down relu(W_up h)^2."""
    idx, wt = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros(h.shape[0], w[p + "e0.down"].shape[0], dtype=DT)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), wt[t]):
            a = torch.relu(w[p + f"e{e}.up"] @ h[t]) ** 2
            out[t] += s * (w[p + f"e{e}.down"] @ a)
    return out


# ------------------------------------------------------------------ the model

MIXERS = {"latent_attention": latent_attention, "gla": gla}


def layer_runs(cfg):
    """[(layer index, pass number or None if the layer begins no pass)] in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t if i == loop["start"] else None))
    return runs + [(i, None) for i in range(loop["stop"], n)]


def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of a whole sequence; with `keep_layers` also the residual stream after
    every layer run."""
    ids = torch.as_tensor(ids, dtype=torch.long)
    eps = cfg["norm"]["eps"]
    x = w["embed"][ids] * cfg["embedding"]["scale"]
    seen = []
    for i, begins in layer_runs(cfg):
        L, p = cfg["layers"][i], f"l{i}."
        if begins is not None:
            x = x + w["loop.step"][begins]
        y = MIXERS[L["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.", L["mixer"], eps)
        x = x + rms_norm(y, w[p + "norm1b"], eps)
        if L.get("mlp") is not None:
            y = moe(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", L["mlp"])
            x = x + rms_norm(y, w[p + "norm2b"], eps)
        seen.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(seen)) if keep_layers else logits
