"""Mixers with a decaying matrix state per head (linear attention).  Per request and head

    S_t = diag(a_t) S_(t-1) + k_t v_t^T        S: [dim, vdim], fp32, zero at the request's start
                                               (kept transposed, [vdim, dim], in the request's state slot)
    o_t = S_t^T q_t

`lightning_attention`: q, k, v = silu(h W), a_t one constant factor per head; the heads' outputs are
normed together (RMS over all heads x vdim, weight of that size), multiplied by sigmoid(h W_g) and
projected.  `gated_linear_attention`: q = h W_q / sqrt(dim), k, v plain, a_t = sigmoid(z_t)^(1/tau) per key
channel with z = (h W_a1) W_a2 + b (a low-rank gate); every head's output is normed on its own (RMS over
vdim, one weight of size vdim for all heads), multiplied by silu(h W_g) and projected.

Both keep the state in a slot of the cache manager (`StateNeed`), run prompts, portions and single
tokens through one kernel that continues the state exactly, and fold `out_scale` into the last fp32
value before it is rounded for the output projection.  Decays, their logarithms, the state, the
read-out and the norms are fp32; the projections run in the activation dtype.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import Mixer, StateNeed, WeightDecl, register_mixer


class _LinearAttention(Mixer):
    def cache_need(self):
        # S transposed, [value column][key channel]: a thread of the kernel owns channels of one column
        return StateNeed(shape=(self.H, self.dv, self.dk), dtype="float32")

    def _project(self, h, w):
        out = torch.empty((h.shape[0], w.shape[0]), dtype=self.act_dtype, device=h.device)
        ops.linear(h, w, out)
        return out


@register_mixer("lightning_attention")
class LightningAttention(_LinearAttention):
    def __init__(self, d_model: int, heads: int, dim: int, vdim: int, decay, norm_eps: float, out_scale: float = 1.0):
        self.d, self.H, self.dk, self.dv = int(d_model), int(heads), int(dim), int(vdim)
        self.decay = [float(x) for x in decay]
        if len(self.decay) != self.H:
            raise ValueError(f"lightning_attention: {len(self.decay)} decay factors for {self.H} heads")
        self.eps, self.out_scale = float(norm_eps), float(out_scale)

    def weight_decls(self):
        H, dk, dv, d = self.H, self.dk, self.dv, self.d
        return {"q": WeightDecl((H * dk, d)), "k": WeightDecl((H * dk, d)), "v": WeightDecl((H * dv, d)),
                "g": WeightDecl((H * dv, d)), "o": WeightDecl((d, H * dv)),
                "norm": WeightDecl((H * dv,), role="vector", init="norm")}

    def bind(self, weights, act_dtype):
        super().bind(weights, act_dtype)
        # one product for q | k | v | g
        self.w_in = torch.cat([weights["q"], weights["k"], weights["v"], weights["g"]], dim=0).contiguous()
        self.wo, self.norm_w = weights["o"], weights["norm"]
        self.head_decay = torch.tensor(self.decay, dtype=torch.float32, device=self.wo.device)
        self.w = {"o": self.wo, "norm": self.norm_w}

    def forward(self, ctx, cache, h, residual, reads_only=False):
        if reads_only:
            raise ValueError("a lightning_attention layer cannot run on another layer's state")
        H, dk, dv = self.H, self.dk, self.dv
        T = h.shape[0]
        p = self._project(h, self.w_in)
        q, k, v, g = p[:, :H * dk], p[:, H * dk:2 * H * dk], p[:, 2 * H * dk:2 * H * dk + H * dv], p[:, 2 * H * dk + H * dv:]
        o = torch.empty((T, H * dv), dtype=torch.float32, device=h.device)
        ops.linear_attention(q, k, v, cache.state, ctx.slot_of_row, ctx.cu_q, o, H, dk, dv,
                             head_decay=self.head_decay, silu=True)
        y = torch.empty((T, H * dv), dtype=self.act_dtype, device=h.device)
        ops.gated_group_norm(o, g, self.norm_w, self.eps, H * dv, y, gate_act=ops.GATE_SIGMOID, out_scale=self.out_scale)
        ops.linear(y, self.wo, residual, accumulate=True)


@register_mixer("gated_linear_attention")
class GatedLinearAttention(_LinearAttention):
    def __init__(self, d_model: int, heads: int, dim: int, vdim: int, tau: float, gate_rank: int, norm_eps: float,
                 out_scale: float = 1.0):
        self.d, self.H, self.dk, self.dv = int(d_model), int(heads), int(dim), int(vdim)
        self.tau, self.rank = float(tau), int(gate_rank)
        self.eps, self.out_scale = float(norm_eps), float(out_scale)

    def weight_decls(self):
        H, dk, dv, d, r = self.H, self.dk, self.dv, self.d, self.rank
        return {"q": WeightDecl((H * dk, d)), "k": WeightDecl((H * dk, d)), "v": WeightDecl((H * dv, d)),
                "g": WeightDecl((H * dv, d)), "o": WeightDecl((d, H * dv)),
                "a1": WeightDecl((r, d)), "a2": WeightDecl((H * dk, r)),
                "a2_bias": WeightDecl((H * dk,), role="vector"),
                "norm": WeightDecl((dv,), role="vector", init="norm")}

    def bind(self, weights, act_dtype):
        super().bind(weights, act_dtype)
        # one product for q | k | v | g | a1 (the gate's first, narrow factor)
        self.w_in = torch.cat([weights["q"], weights["k"], weights["v"], weights["g"], weights["a1"]], dim=0).contiguous()
        self.wa2, self.bias = weights["a2"], weights["a2_bias"]
        self.wo, self.norm_w = weights["o"], weights["norm"]
        self.w = {"o": self.wo}

    def forward(self, ctx, cache, h, residual, reads_only=False):
        if reads_only:
            raise ValueError("a gated_linear_attention layer cannot run on another layer's state")
        H, dk, dv, r = self.H, self.dk, self.dv, self.rank
        T = h.shape[0]
        p = self._project(h, self.w_in)
        o0, o1, o2, o3 = H * dk, 2 * H * dk, 2 * H * dk + H * dv, 2 * H * dk + 2 * H * dv
        q, k, v, g, a1 = p[:, :o0], p[:, o0:o1], p[:, o1:o2], p[:, o2:o3], p[:, o3:o3 + r]
        z = torch.empty((T, H * dk), dtype=torch.float32, device=h.device)
        ops.linear(a1, self.wa2, z)
        o = torch.empty((T, H * dv), dtype=torch.float32, device=h.device)
        ops.linear_attention(q, k, v, cache.state, ctx.slot_of_row, ctx.cu_q, o, H, dk, dv,
                             gate=z, gate_bias=self.bias, tau=self.tau, q_scale=dk ** -0.5)
        y = torch.empty((T, H * dv), dtype=self.act_dtype, device=h.device)
        ops.gated_group_norm(o, g, self.norm_w, self.eps, dv, y, gate_act=ops.GATE_SILU, out_scale=self.out_scale)
        ops.linear(y, self.wo, residual, accumulate=True)
