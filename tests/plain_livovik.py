"""The Livovik design written out plainly: one function per mechanism, float64 on the CPU, whole
sequences at a time, no cache. It shares no code with the package; the package's kernels, cache
and step function are measured against it.

A model is (cfg, weights): cfg the design's config.json as a dict, weights a dict name -> float64
tensor with the design's tensor names (`embed`, `l<i>.norm1`, `l<i>.mix.q`, ..., `final.norm`, `head`).
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np
import torch

F64 = torch.float64
DT = F64


def read_safetensors(path):
    """name -> float64 tensor (integer tables stay integers): 8-byte length, JSON header, raw bytes."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        raw = data[a:b]
        if e["dtype"] == "BF16":
            bits = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy()).to(F64)
        elif e["dtype"] == "F32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<f4").copy()).to(F64)
        elif e["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(raw, dtype="<i4").copy())
        else:
            raise ValueError(f"{name}: dtype {e['dtype']}")
        out[name] = t.reshape(e["shape"])
    return out


def read_model_dir(d):
    with open(os.path.join(d, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(d, "model.safetensors"))


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last dimension."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotary_frequencies(dims, base, scaling=None):
    """f_i = base^(-2i/dims), i < dims/2; with `scaling` {factor, low, high, original} the three
    wavelength bands: short waves kept, long waves divided by the factor, a blend between."""
    out = []
    for i in range(dims // 2):
        f = float(base) ** (-2.0 * i / dims)
        if scaling is not None:
            factor, low, high, orig = (float(scaling[k]) for k in ("factor", "low", "high", "original"))
            wave = 2.0 * math.pi / f
            if wave < orig / high:
                pass
            elif wave > orig / low:
                f = f / factor
            else:
                s = (orig / wave - low) / (high - low)
                f = (1.0 - s) * f / factor + s * f
        out.append(f)
    return out


def rotate(x, positions, freqs):
    """x [T, heads, dim]: of the first 2 * len(freqs) dimensions of every head, dimension i pairs with
    i + len(freqs); the pair (u, v) at position p turns by the angle p * f_i. The rest passes."""
    n = len(freqs)
    if n == 0:
        return x.clone()
    ang = torch.tensor(positions, dtype=F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :n], x[..., n:2 * n]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * n:]], dim=-1)


def visible(i, j, mask):
    """Does position i see position j? Causal always; `mask` {"size": n} keeps only the positions of
    i's own block of n positions counted from the start of the sequence."""
    if j > i:
        return False
    if mask is not None and i // int(mask["size"]) != j // int(mask["size"]):
        return False
    return True


def softmax_with_sink(scores, allowed, sink):
    """Row-wise weights exp(s_j) / (exp(sink) + sum over allowed j of exp(s_j)); the sink has no value."""
    s = scores.masked_fill(~allowed, -math.inf)
    m = torch.maximum(s.max(-1, keepdim=True).values, torch.full_like(s[..., :1], float(sink)))
    e = torch.exp(s - m)
    return e / (e.sum(-1, keepdim=True) + torch.exp(float(sink) - m))


def attention_mixer(h, w, m, eps, positions=None):
    """The attention mixer over a whole sequence. h [T, width]; w: the mixer's tensors by their short
    names (q, k, v, q.norm, k.norm, sink, g, o); m: the layer's `mixer` object of the configuration."""
    T = h.shape[0]
    H, G, D, V = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    positions = list(range(T)) if positions is None else positions
    q = (h @ w["q"].T).view(T, H, D)
    k = (h @ w["k"].T).view(T, G, D)
    v = (h @ w["v"].T).view(T, G, V)
    q, k = rms_norm(q, w["q.norm"], eps), rms_norm(k, w["k.norm"], eps)
    rot = m.get("rot")
    if rot is not None:
        f = rotary_frequencies(int(rot["dims"]), rot["base"], rot.get("scaling"))
        q, k = rotate(q, positions, f), rotate(k, positions, f)
    allowed = torch.tensor([[visible(positions[i], positions[j], m.get("mask")) for j in range(T)] for i in range(T)])
    gate = torch.sigmoid(h @ w["g"].T)                     # [T, H]
    out = torch.zeros(T, H, V, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * float(m["scale"])
        p = softmax_with_sink(s, allowed, w["sink"][hd])
        out[:, hd] = (p @ v[:, g]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * V) @ w["o"].T


def dense_ffn(h, w):
    """W_down relu(W_up h)^2."""
    return torch.relu(h @ w["up"].T) ** 2 @ w["down"].T


def gated_expert(h, w, prefix=""):
    """W_down (silu(W_gate h) * (W_up h))."""
    a = h @ w[prefix + "gate"].T
    return (a * torch.sigmoid(a) * (h @ w[prefix + "up"].T)) @ w[prefix + "down"].T


def route(h, w_router, top):
    """-> (chosen experts [T, top], their weights): scores sigmoid(W_router h), the `top` largest,
    the scores themselves as weights."""
    s = torch.sigmoid(h @ w_router.T)
    wt, idx = torch.topk(s, top, dim=-1)
    return idx, wt


def moe_ffn(h, w, mlp):
    """Sum over a token's chosen experts of expert(weight * h), plus, if there is one, the shared
    expert's output times sigmoid(W_sg h)."""
    experts, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    idx, wt = route(h, w["router"], top)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(idx[t].tolist(), wt[t].tolist()):
            out[t] += gated_expert(s * h[t:t + 1], w, f"e{e}.")[0]
    if mlp.get("shared") is not None:
        out = out + gated_expert(h, w, "shared.") * torch.sigmoid(h @ w["shared.sg"].T)
    assert experts == sum(1 for k in w if k.endswith(".gate") and k.startswith("e"))
    return out


def sub(weights, prefix):
    return {k[len(prefix):]: v for k, v in weights.items() if k.startswith(prefix)}


def layer_forward(x, cfg, weights, i, positions=None):
    """x <- norm1(alpha x + mixer(x)); x <- norm2(alpha x + ff(x)); a layer with `weights_of` j runs on
    layer j's tensors."""
    L = cfg["layers"][i]
    src = i
    while cfg["layers"][src].get("weights_of") is not None:       # the layer that owns the tensors
        src = cfg["layers"][src]["weights_of"]
    eps, alpha = float(cfg["norm"]["eps"]), float(cfg["postln_alpha"])
    pre = f"l{src}."
    if L["type"] != "attention":
        raise ValueError(L["type"])
    x = rms_norm(alpha * x + attention_mixer(x, sub(weights, pre + "mix."), L["mixer"], eps, positions),
                 weights[pre + "norm1"], eps)
    mlp = L.get("mlp")
    if mlp is not None:
        w = sub(weights, pre + "mlp.")
        y = dense_ffn(x, w) if mlp["kind"] == "dense" else moe_ffn(x, w, mlp)
        x = rms_norm(alpha * x + y, weights[pre + "norm2"], eps)
    return x


def forward(cfg, weights, tokens, collect=None):
    """Logits [T, vocab] of one sequence from position 0. `collect`: a list that receives the stream after
    every layer."""
    x = weights["embed"][torch.tensor(tokens)]
    for i in range(len(cfg["layers"])):
        x = layer_forward(x, cfg, weights, i)
        if collect is not None:
            collect.append(x.clone())
    return rms_norm(x, weights["final.norm"], float(cfg["norm"]["eps"])) @ weights["head"].T
