"""A plain, slow implementation of the Koridra decoder in NumPy float64: whole sequences, no cache,
token-by-token recurrences, one function per mechanism.  It shares no code with `tuff_b200` (it reads
config.json and the safetensors file with the standard library and NumPy alone) and is what the engine's
kernels, cache and batching are compared with.

Notation: h [T, d] is a sublayer's input; matrices are stored [out, in] and applied as h @ W.T.
"""
from __future__ import annotations

import json
import math
import os
import struct

import numpy as np


# ------------------------------------------------------------------ file reading
def read_config(model_dir):
    with open(os.path.join(model_dir, "config.json")) as f:
        return json.load(f)


def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        b, e = info["data_offsets"]
        if info["dtype"] == "BF16":
            a = (np.frombuffer(data[b:e], dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
        elif info["dtype"] == "F32":
            a = np.frombuffer(data[b:e], dtype=np.float32)
        else:
            raise ValueError(f"{name}: dtype {info['dtype']}")
        out[name] = a.astype(np.float64).reshape(info["shape"])
    return out


# ------------------------------------------------------------------ small functions
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def rms_norm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * w


def embedding(tokens, table, pos_table, first_position=0):
    """Token vector plus the learned vector of the token's position, unscaled."""
    t = np.asarray(tokens)
    return table[t] + pos_table[first_position:first_position + len(t)]


# ------------------------------------------------------------------ rotation
def yarn_frequencies(span, base, scaling=None):
    """(angular frequency of each of the span/2 pairs, factor on cos and sin)."""
    i = np.arange(span // 2, dtype=np.float64)
    f = base ** (-2.0 * i / span)
    if not scaling:
        return f, 1.0
    def pair_of(turns):
        return span * math.log(scaling["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(scaling["fast"])), 0)
    hi = min(math.ceil(pair_of(scaling["slow"])), span - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / scaling["factor"] * ramp + f * (1.0 - ramp), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate_interleaved(x, positions, span, freq, amplitude):
    """x [T, heads, dim]: within the first `span` elements of a head, (x[2i], x[2i+1]) turns by
    positions * freq[i]; cos and sin carry `amplitude`; the rest of the head passes."""
    out = x.copy()
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    c, s = np.cos(ang)[:, None, :] * amplitude, np.sin(ang)[:, None, :] * amplitude
    u, v = x[..., 0:span:2], x[..., 1:span:2]
    out[..., 0:span:2] = u * c - v * s
    out[..., 1:span:2] = v * c + u * s
    return out


# ------------------------------------------------------------------ softmax branch
def sink_softmax(scores, allowed, sink=0.0):
    """Row-wise exp(s_j) / (exp(sink) + sum_allowed exp(s_j)); disallowed places get 0."""
    s = np.where(allowed, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (np.exp(sink - m) + e.sum(axis=-1, keepdims=True))


def chunk_mask(T, chunk):
    i = np.arange(T)
    ok = i[None, :] <= i[:, None]
    if chunk:
        ok &= (i[None, :] // chunk) == (i[:, None] // chunk)
    return ok


def keys_as_values_attention(h, wq, wk, wo, q_norm, k_norm, m, eps):
    """The softmax branch: values are the keys as projected; q and k are normed over their whole
    projections, rotated, scored with m['scale'] inside the query's chunk, softmax with a zero sink."""
    T = h.shape[0]
    H, G, dim = m["heads"], m.get("kv_heads", m["heads"]), m["dim"]
    q, k = h @ wq.T, h @ wk.T
    v = k.reshape(T, G, dim)
    q = rms_norm(q, q_norm, eps).reshape(T, H, dim)
    k = rms_norm(k, k_norm, eps).reshape(T, G, dim)
    rot = m.get("rot")
    if rot and rot["dims"]:
        f, amp = yarn_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        q = rotate_interleaved(q, np.arange(T), rot["dims"], f, amp)
        k = rotate_interleaved(k, np.arange(T), rot["dims"], f, amp)
    ok = chunk_mask(T, (m.get("mask") or {}).get("size"))
    out = np.zeros((T, H, dim))
    for a in range(H):
        g = a // (H // G)
        p = sink_softmax((q[:, a] @ k[:, g].T) * m["scale"], ok)
        out[:, a] = p @ v[:, g]
    return out.reshape(T, H * dim) @ wo.T


# ------------------------------------------------------------------ recurrences
def decaying_state_scan(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv], decay [T, H, dk] (or broadcastable): per head
    S <- decay_t[:, None] * S + outer(k_t, v_t); o_t = S^T q_t, token by token from S = 0."""
    T, H, dk = k.shape
    dv = v.shape[2]
    decay = np.broadcast_to(decay, (T, H, dk))
    S = np.zeros((H, dk, dv))
    o = np.zeros((T, H, dv))
    for t in range(T):
        S = decay[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hkv,hk->hv", S, q[t])
    return o


def lightning_mixer(h, w, m, eps):
    """w: q, k, v, g, o, norm.  silu on q, k, v; one decay per head; the heads normed together;
    a sigmoid gate; the output projection."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w["q"].T).reshape(T, H, dk)
    k = silu(h @ w["k"].T).reshape(T, H, dk)
    v = silu(h @ w["v"].T).reshape(T, H, dv)
    o = decaying_state_scan(q, k, v, np.asarray(m["decay"], dtype=np.float64)[None, :, None])
    y = rms_norm(o.reshape(T, H * dv), w["norm"], eps) * sigmoid(h @ w["g"].T)
    return y @ w["o"].T


def gated_linear_branch(h, w, m, eps):
    """w: q, k, v, g, o, a1, a2, a2.b, norm.  A decay per key channel sigmoid(z)^(1/tau) from the
    low-rank gate z; every head normed on its own with one shared weight; a silu gate."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w["q"].T).reshape(T, H, dk) / math.sqrt(dk)
    k = (h @ w["k"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    decay = np.exp(np.log(sigmoid(z)) / m["tau"]).reshape(T, H, dk)
    o = decaying_state_scan(q, k, v, decay)
    y = rms_norm(o, w["norm"], eps).reshape(T, H * dv) * silu(h @ w["g"].T)
    return y @ w["o"].T


def dense_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


# ------------------------------------------------------------------ the model
class PlainKoridra:
    def __init__(self, model_dir):
        self.cfg = read_config(model_dir)
        self.w = read_safetensors(os.path.join(model_dir, "model.safetensors"))

    def sub(self, prefix):
        return {n[len(prefix):]: a for n, a in self.w.items() if n.startswith(prefix)}

    def mixer(self, i, h):
        L, eps = self.cfg["layers"][i], self.cfg["norm"]["eps"]
        m = L["mixer"]
        if L["type"] == "lightning":
            return lightning_mixer(h, self.sub(f"l{i}.mix."), m, eps)
        l = self.sub(f"l{i}.mix.left.")
        left = keys_as_values_attention(h, l["q"], l["k"], l["o"], l["q.norm"], l["k.norm"], m["left"], eps)
        right = gated_linear_branch(h, self.sub(f"l{i}.mix.right."), m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right

    def forward(self, tokens, layers_out=None):
        """Logits [T, vocab] of a whole sequence; `layers_out`: a list that receives the stream after each layer."""
        cfg, w = self.cfg, self.w
        eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
        x = embedding(tokens, w["embed"], w["pos"])
        for i, L in enumerate(cfg["layers"]):
            x = rms_norm(alpha * x + self.mixer(i, x), w[f"l{i}.norm1"], eps)
            if L.get("mlp") is not None:
                y = dense_ff(x, w[f"l{i}.mlp.gate"], w[f"l{i}.mlp.up"], w[f"l{i}.mlp.down"])
                x = rms_norm(alpha * x + y, w[f"l{i}.norm2"], eps)
            if layers_out is not None:
                layers_out.append(x.copy())
        return rms_norm(x, w["final.norm"], eps) @ w["head"].T
