"""Gated linear attention as a mixer part: a recurrence over a per-request state.

Per head, with h the mixer's input: q = W_q h * dim^-1/2, k = W_k h (`dim` key channels), v = W_v h
(`vdim`), a decay per key channel alpha = sigmoid(z)^(1/tau) with z = W_a2 (W_a1 h) + b, and
    S_t = diag(alpha_t) S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t.
Each head's o is RMS-normed over vdim with one weight of size vdim shared by the heads; the heads are
concatenated, multiplied by silu(W_g h) and projected by W_o. The state S starts at zero, is float32
and lives in a state slot of the cache manager (`StateSpec`), carried from step to step; decays,
the recurrence and the norm are float, the projections run in the run dtype. The width of the
decay's bottleneck (rows of W_a1) is a size of the checkpoint, not of the configuration: it is taken
from the tensor unless `decay_rank` is given (random-weights mode).
"""
from __future__ import annotations

import torch

from .base import Param, Part, Source, StateSpec, register_part


class GatedLinearAttention(Part):
    graph_safe = True
    takes_deferred = True
    returns_output = True

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, tau: float, eps: float = 1e-6,
                 decay_rank: int | None = None):
        self.hidden, self.heads, self.dim, self.vdim = hidden, heads, dim, vdim
        self.tau, self.eps, self.decay_rank = float(tau), float(eps), decay_rank
        self.chunk = 128         # tokens per chunk of a long portion
        self.w_in = self.w_a2 = self.b_a2 = self.w_norm = self.w_o = None

    def params(self):
        H, W, r = self.heads, self.hidden, -1 if self.decay_rank is None else self.decay_rank
        return [Param("w_in", (Source("q", (H * self.dim, W)), Source("k", (H * self.dim, W)),
                               Source("v", (H * self.vdim, W)), Source("g", (H * self.vdim, W)),
                               Source("a1", (r, W)))),
                Param("w_a2", (Source("a2", (H * self.dim, r)),)),
                Param("b_a2", (Source("a2.b", (H * self.dim,)),), role="vector"),
                Param("w_norm", (Source("norm", (self.vdim,), init="norm"),), role="vector"),
                Param("w_o", (Source("o", (W, H * self.vdim)),))]

    def cache_spec(self):
        return StateSpec((("S", (self.heads, self.dim, self.vdim), torch.float32),))

    def finalize(self, device, dtype):
        self._b_f32 = self.b_a2.float().contiguous()
        self._norm_f32 = self.w_norm.float().contiguous()
        self._a1_off = 2 * self.heads * (self.dim + self.vdim)
        if self.w_a2.shape[1] != self.w_in.shape[0] - self._a1_off:
            raise ValueError(f"{self.prefix}a1 has {self.w_in.shape[0] - self._a1_off} rows, a2 takes {self.w_a2.shape[1]}")

    def forward(self, x, ctx, cache, residual=None):
        be = ctx.backend
        H, d, v = self.heads, self.dim, self.vdim
        proj = be.linear(x, self.w_in)                                   # [T, q | k | v | gate | a1]
        z = be.linear_f32(proj[:, self._a1_off:], self.w_a2)             # float decay logits [T, H * dim]
        alpha = be.gla_decay(z, self._b_f32, self.tau)                   # in place
        # long portions are cut into chunks that run side by side (the host knows a step's longest portion;
        # inside a decode graph it is one token)
        chunk = self.chunk if not ctx.graph_safe and ctx.max_q_len >= 3 * self.chunk else 0
        o = be.gla_scan(proj, 0, H * d, 2 * H * d, alpha, d ** -0.5, H, d, v, ctx.cu_q, ctx.num_seqs,
                        ctx.state_slots, cache.state["S"], chunk)
        att = be.gla_finish(o, self._norm_f32, self.eps, proj, 2 * H * d + H * v)
        if residual is None:
            return be.linear_f32(att, self.w_o)
        be.linear_residual(att, self.w_o, residual)
        return None


register_part("mixer", "gla", GatedLinearAttention)
