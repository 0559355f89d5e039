"""Plain, slow Fiferax: whole sequences, dense masks, explicit loops over
tokens, no cache, float64, one function for each mechanism.  It shares no code
with ``airframe_b200`` (its own reading of config.json and of the tensors).

Notation: h is a sublayer's input [T, width]; W x means a weight stored
[out, in] applied to a vector; positions count from 0.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from plain_gemma2 import read_safetensors

F64 = torch.float64


def read_model_folder(folder, dtype=F64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    return cfg, read_safetensors(folder / "model.safetensors", dtype)


# ---------------------------------------------------------------- small pieces

def rms(x, eps, w=None):
    """x / sqrt(mean(x^2) + eps) over the last axis, times w when given."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


# ---------------------------------------------------------------- the mechanisms

def delta_rule(r, k, v, w, a, key_eps=1e-6):
    """The generalized delta rule of one sequence.  r, k, w, a [T, H, dk], v [T, H, dv].
    u = k / sqrt(|k|^2 + key_eps); S_t = diag(w_t) S - (a_t u_t)(u_t^T S) + k_t v_t^T with S the
    state before the token in both terms; o_t = S_t^T r_t.  Returns o [T, H, dv] and the last state."""
    T, H, dk = k.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=k.dtype)
    out = torch.zeros(T, H, dv, dtype=k.dtype)
    for t in range(T):
        for h in range(H):
            u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + key_eps)
            old = S[h]
            S[h] = w[t, h][:, None] * old - torch.outer(a[t, h] * u, u @ old) + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ r[t, h]
    return out, S


def general_delta(h, W, p, heads, dim, eps):
    T = h.shape[0]
    r = (h @ W[p + "r"].T).view(T, heads, dim)
    k = (h @ W[p + "k"].T).view(T, heads, dim)
    v = (h @ W[p + "v"].T).view(T, heads, dim)
    low = torch.tanh(h @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]
    w = torch.exp(-math.exp(-0.5) * sigmoid(low)).view(T, heads, dim)
    a = sigmoid(h @ W[p + "a"].T + W[p + "a.b"]).view(T, heads, dim)
    o, _ = delta_rule(r, k, v, w, a)
    o = rms(o, eps).reshape(T, heads * dim) * W[p + "norm"] * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def rotate_half(x, positions, base, dims):
    """x [T, heads, d]: element i < dims/2 pairs with i + dims/2; (a, b) -> (a cos - b sin, b cos + a sin)
    with the angle position * base^(-2i/dims); elements from dims on pass."""
    half = dims // 2
    if half == 0:
        return x
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    ang = positions.to(x.dtype)[:, None] * f[None]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def windowed_attention(q, k, v, scale, window):
    """q [T, H, d], k, v [T, G, d]; head h reads group h // (H / G); position i sees j with
    0 <= i - j < window; softmax of q.k * scale over the visible keys."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            out[i, h] = torch.softmax(s, dim=0) @ v[lo:i + 1, g]
    return out


def norm_rope_attention(h, W, p, m, eps):
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + "q"].T).view(T, H, d)
    k = (h @ W[p + "k"].T).view(T, G, d)
    v = k.clone()                                   # values: the raw key projection
    pos = torch.arange(T)
    q = rotate_half(rms(q, eps, W[p + "q.norm"]), pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half(rms(k, eps, W[p + "k.norm"]), pos, m["rot"]["base"], m["rot"]["dims"])
    o = windowed_attention(q, k, v, m["scale"], m["mask"]["size"])
    return o.reshape(T, H * d) @ W[p + "o"].T


def decay_linear_attention(q, k, v, decay):
    """q, k [T, H, dk], v [T, H, dv], decay [H]: S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t."""
    T, H, dk = k.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=k.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=k.dtype)
    for t in range(T):
        for h in range(H):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            out[t, h] = S[h].T @ q[t, h]
    return out


def lightning(h, W, p, m, eps):
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ W[p + "q"].T).view(T, H, dk)
    k = silu(h @ W[p + "k"].T).view(T, H, dk)
    v = silu(h @ W[p + "v"].T).view(T, H, dv)
    o = decay_linear_attention(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = rms(o.reshape(T, H * dv), eps, W[p + "norm"]) * sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def gated_recurrence(z, c):
    """z, c [T, n]: S_t = (1 - z_t) S_(t-1) + z_t c_t from S = 0; returns all S_t."""
    S = torch.zeros(z.shape[1], dtype=z.dtype)
    out = torch.zeros_like(z)
    for t in range(z.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * c[t]
        out[t] = S
    return out


def mingru(h, W, p):
    z = sigmoid(h @ W[p + "z"].T + W[p + "z.b"])
    u = h @ W[p + "x"].T + W[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, sigmoid(u))
    return (gated_recurrence(z, cand) * silu(h @ W[p + "g"].T)) @ W[p + "o"].T


def dense_mlp(h, W, p):
    return (gelu_tanh(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ---------------------------------------------------------------- the model

def mixer(h, cfg, W, i):
    layer, p, eps = cfg["layers"][i], f"l{i}.mix.", cfg["norm"]["eps"]
    m = layer["mixer"]
    if layer["type"] == "general_delta":
        return general_delta(h, W, p, m["heads"], m["dim"], eps)
    if layer["type"] == "mingru":
        return mingru(h, W, p)
    if layer["type"] == "parallel":
        return (m["left_scale"] * norm_rope_attention(h, W, p + "left.", m["left"], eps)
                + m["right_scale"] * lightning(h, W, p + "right.", m["right"], eps))
    raise ValueError(layer["type"])


def hidden_states(cfg, W, ids, per_layer=None):
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(ids)] * cfg["embedding"]["scale"]
    for i, layer in enumerate(cfg["layers"]):
        x = x + mixer(rms(x, eps, W[f"l{i}.norm1"]), cfg, W, i)
        if layer["mlp"] is not None:
            x = x + dense_mlp(rms(x, eps, W[f"l{i}.norm2"]), W, f"l{i}.mlp.")
        if per_layer is not None:
            per_layer.append(x.clone())
    return x


def logits(cfg, W, ids):
    x = hidden_states(cfg, W, ids)
    return rms(x, cfg["norm"]["eps"], W["final.norm"]) @ W["head"].T


def generate_greedy(cfg, W, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(logits(cfg, W, ids)[-1])))
    return ids[len(prompt):]
