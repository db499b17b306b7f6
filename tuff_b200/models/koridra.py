"""Koridra as a `ModelSpec`.

A decoder whose layers norm after the sum (`postnorm` block with the configuration's alpha): token
embedding plus a learned position vector; per layer a mixer and, unless the layer has none, a dense
SwiGLU feed-forward; a final norm and an untied head.  Two kinds of layer:

  "lightning"  `lightning_attention`: linear attention with one constant decay per head.
  "parallel"   `parallel_mixers` of
               left:  `gqa_attention` whose values are its keys as projected, with a norm over the whole
                      q and k projections, YaRN-scaled rotation of interleaved pairs on the first
                      rot.dims elements of a head, keys seen within the query's chunk of positions only,
                      and a zero-score sink in the softmax;
               right: `gated_linear_attention` (a decay per key channel from a low-rank gate),
               summed with the configuration's two weights.

Checkpoint tensor names: `embed`, `pos`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.{gate,up,down}`,
`final.norm`, `head`; a parallel layer's branches live under `l<i>.mix.left.*` and `l<i>.mix.right.*`.
"""
from __future__ import annotations

from dataclasses import replace

from ..config.koridra import ARCHITECTURE, KoridraConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec

# The inner width of a decay gate is the one size that config.json does not give: a checkpoint's tensor shape
# does (`refine_config`), and a model made without a file takes `gate_rank` from its configuration or this.
DEFAULT_GATE_RANK = 16


def _left(d, eps, L, scale, p):
    pos = None
    if L.rot_dims:
        s = L.rot_scaling
        pos = PartSpec("rope_yarn", dict(
            head_dim=L.dim, theta=L.rot_base, rotary_dim=L.rot_dims, pairing="interleaved",
            **({} if s is None else dict(factor=s.factor, original=s.original, fast=s.fast, slow=s.slow))))
    return PartSpec(
        "gqa_attention",
        dict(d_model=d, num_heads=L.heads, num_kv_heads=L.kv_heads, head_dim=L.dim, qk_norm_eps=eps,
             qk_norm_span="projection", values="keys", position_encoding=pos, scale=L.scale, chunk=L.chunk,
             sink=0.0, out_scale=scale),
        {"q_proj": p + "q", "k_proj": p + "k", "out_proj": p + "o", "q_layernorm": p + "q.norm",
         "k_layernorm": p + "k.norm"})


def _right(d, eps, R, scale, p):
    rank = R.gate_rank if R.gate_rank is not None else DEFAULT_GATE_RANK
    return PartSpec(
        "gated_linear_attention",
        dict(d_model=d, heads=R.heads, dim=R.dim, vdim=R.vdim, tau=R.tau, gate_rank=rank, norm_eps=eps, out_scale=scale),
        {"q": p + "q", "k": p + "k", "v": p + "v", "g": p + "g", "o": p + "o", "a1": p + "a1", "a2": p + "a2",
         "a2_bias": p + "a2.b", "norm": p + "norm"})


def koridra_spec(cfg: KoridraConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        m = l.mixer
        if l.type == "lightning":
            mixer = PartSpec("lightning_attention",
                             dict(d_model=d, heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay), norm_eps=eps),
                             {n: f"{p}mix.{n}" for n in ("q", "k", "v", "g", "o", "norm")})
        else:
            left = _left(d, eps, m.left, m.left_scale, p + "mix.left.")
            right = _right(d, eps, m.right, m.right_scale, p + "mix.right.")
            mixer = PartSpec("parallel_mixers", dict(branches={"left": left, "right": right}),
                             {**{f"left.{k}": v for k, v in left.tensors.items()},
                              **{f"right.{k}": v for k, v in right.tensors.items()}})
        ffn = ffn_norm = None
        if l.ff is not None:
            ffn = PartSpec("swiglu", dict(d_model=d, ffn_dim=l.ff),
                           {"w1": p + "mlp.gate", "w3": p + "mlp.up", "w2": p + "mlp.down"})
            ffn_norm = PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": p + "norm2"})
        layers.append(LayerSpec(mixer=mixer, ffn=ffn, ffn_norm=ffn_norm,
                                mixer_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": p + "norm1"}),
                                block=PartSpec("postnorm", dict(alpha=cfg.postln_alpha))))
    return ModelSpec(
        architecture=ARCHITECTURE, d_model=d, vocab_size=cfg.vocab,
        embedding=PartSpec("token_position_embedding", dict(vocab_size=cfg.vocab, d_model=d, max_positions=cfg.max_positions),
                           {"weight": "embed", "positions": "pos"}),
        layers=layers,
        final_norm=PartSpec("rmsnorm", dict(dim=d, eps=eps), {"weight": "final.norm"}),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, d_model=d), {"weight": "head"}),
        max_context=cfg.max_positions)


def refine_config(cfg: KoridraConfig, shapes) -> KoridraConfig:
    """Sizes that only a checkpoint's tensor shapes give: the inner width of each decay gate (rows of
    `l<i>.mix.right.a1`).  `shapes`: tensor name -> shape."""
    layers = list(cfg.layers)
    for i, l in enumerate(layers):
        name = f"l{i}.mix.right.a1"
        if l.type == "parallel" and name in shapes and len(shapes[name]) == 2:
            right = replace(l.mixer.right, gate_rank=int(shapes[name][0]))
            layers[i] = replace(l, mixer=replace(l.mixer, right=right))
    return replace(cfg, layers=tuple(layers))
