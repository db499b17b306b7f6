"""Small Koridra configurations for the tests, and model folders with weights large enough that every
mechanism shows in the logits.  They differ from one another in every size and option: layer order
(a parallel layer first / two of them / none but the last), layers without feed-forward, query and value
sizes that differ, key/value groups, rotated spans (half, whole, none), YaRN on and off, chunks that are
no multiple of a page, gate widths that the tensor-core product refuses (5), tau down to 1, alpha down
to 1, vocabularies and widths that are no multiple of 16."""
import json
import os

import numpy as np


def _lightning(heads, dim, vdim, decay, ff):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay),
                mlp=None if ff is None else dict(kind="dense", ff=ff))


def _parallel(left, right, ls, rs, ff):
    return dict(type="parallel", mixer=dict(left=left, right=right, left_scale=ls, right_scale=rs),
                mlp=None if ff is None else dict(kind="dense", ff=ff))


KOR_A = dict(
    architecture="Koridra", vocab=301, width=80, max_positions=400, norm=dict(eps=1e-5), postln_alpha=1.5,
    layers=[
        _parallel(dict(heads=4, kv_heads=2, dim=32, vdim=32, scale=0.25, mask=dict(size=24),
                       rot=dict(dims=16, base=10000.0, scaling=dict(factor=4.0, original=64, fast=16.0, slow=2.0))),
                  dict(heads=2, dim=24, vdim=40, tau=4.0, gate_rank=8), 0.7, 1.3, 160),
        _lightning(3, 16, 40, [0.5, 0.9, 0.995], 160),
        _lightning(2, 80, 24, [0.97, 0.8], None),
        _parallel(dict(heads=2, kv_heads=2, dim=48, vdim=48, scale=0.2, mask=dict(size=40),
                       rot=dict(dims=48, base=500.0)),
                  dict(heads=3, dim=16, vdim=16, tau=1.0, gate_rank=5), 1.0, 0.5, 200),
    ])

KOR_B = dict(
    architecture="Koridra", vocab=257, width=64, max_positions=300, norm=dict(eps=1e-6), postln_alpha=1.0,
    layers=[
        _lightning(4, 32, 32, [0.3, 0.7, 0.95, 1.0], 96),
        _lightning(1, 48, 72, [0.9], 128),
        _parallel(dict(heads=6, kv_heads=1, dim=16, vdim=16, scale=0.5, mask=dict(size=17), rot=dict(dims=0, base=10000.0)),
                  dict(heads=1, dim=40, vdim=24, tau=8.0, gate_rank=16), 0.5, 1.0, None),
    ])

# head size 64 for the tensor-core attention kernels, a chunk of one page and a half, a long-lived state
KOR_C = dict(
    architecture="Koridra", vocab=512, width=128, max_positions=600, norm=dict(eps=1e-5), postln_alpha=2.0,
    layers=[
        _lightning(2, 64, 128, [0.999, 0.9], 256),
        _parallel(dict(heads=4, kv_heads=2, dim=64, vdim=64, scale=0.125, mask=dict(size=96),
                       rot=dict(dims=32, base=1e6, scaling=dict(factor=8.0, original=128, fast=32.0, slow=1.0))),
                  dict(heads=2, dim=64, vdim=64, tau=16.0, gate_rank=24), 0.6, 1.1, 256),
    ])

# a width and a vocabulary that are no multiple of 8 (no tensor-core product takes them), head size 128 in the softmax
# branch (the TMA-fed attention kernels' other size), a chunk that is no multiple of anything, a gate width of 6
KOR_D = dict(
    architecture="Koridra", vocab=211, width=100, max_positions=256, norm=dict(eps=1e-5), postln_alpha=2.5,
    layers=[
        _parallel(dict(heads=2, kv_heads=1, dim=128, vdim=128, scale=0.09, mask=dict(size=50),
                       rot=dict(dims=64, base=1e4, scaling=dict(factor=2.0, original=32, fast=8.0, slow=1.0))),
                  dict(heads=2, dim=20, vdim=12, tau=2.0, gate_rank=6), 0.8, 0.9, 72),
        _lightning(2, 24, 36, [0.9, 0.99], 72),
    ])

CONFIGS = {"kor_a": (KOR_A, 11), "kor_b": (KOR_B, 12), "kor_c": (KOR_C, 13), "kor_d": (KOR_D, 14)}


def make_folder(tmp_path, name, gain=1.0):
    """A model folder whose matrices are N(0, gain / fan_in) (so that projections keep the size of their
    input and attention scores are far from uniform), norm weights 1 + N(0, 0.1), biases N(0, 1)."""
    import torch
    from tuff_b200.config.registry import config_from_dict
    from tuff_b200.models.model import Model
    from tuff_b200.weights import write_safetensors
    cfg, seed = CONFIGS[name]
    arch, typed = config_from_dict(cfg, name)
    rng = np.random.default_rng(seed)
    tensors = []
    for tname, decl in sorted(Model(arch.model_spec(typed)).expected_tensors().items()):
        if decl.init == "norm":
            a = 1.0 + 0.1 * rng.normal(size=decl.shape)
        elif decl.role == "vector":
            a = rng.normal(size=decl.shape)
        elif tname in ("embed", "pos"):
            a = rng.normal(size=decl.shape)
        else:
            a = rng.normal(size=decl.shape) * gain / np.sqrt(decl.shape[-1])
        tensors.append((tname, torch.tensor(a, dtype=torch.float32).to(torch.bfloat16)))
    folder = str(tmp_path / name)
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), tensors)
    return folder
