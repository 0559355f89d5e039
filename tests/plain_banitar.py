"""Plain, slow Banitar: whole sequences, dense masks, no cache, float64, one
function for each mechanism.  It shares no code with ``airframe_b200`` (its own
reading of config.json and of the tensors).

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

def sigmoid(z):
    return 1.0 / (1.0 + torch.exp(-z))


def silu(z):
    return z * sigmoid(z)


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def tanh_norm(x, W, name):
    """The norm without statistics: tanh(alpha x) w + b."""
    return torch.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


# ---------------------------------------------------------------- rotations

def plain_frequencies(base, dims):
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def stretched_frequencies(base, dims, s):
    """Frequencies of which the slow ones are divided by ``factor`` and the fast ones kept, with a ramp
    in between, and the factor that cosines and sines are multiplied by."""
    factor, original, fast, slow = s["factor"], s["original"], s["fast"], s["slow"]

    def turn(t):
        return dims * math.log(original / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(fast)), 0)
    hi = min(math.ceil(turn(slow)), dims - 1)
    out = []
    for i, f in enumerate(plain_frequencies(base, dims)):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f / factor * ramp + f * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, pairs, magnitude=1.0):
    """x [T, heads, d]; the first 2 len(freqs) elements of a head are rotated, pair (a, b) becoming
    (a cos - b sin, b cos + a sin) * magnitude at angle position * frequency.  ``pairs`` 'half':
    element i with i + len(freqs); 'adjacent': 2i with 2i + 1."""
    n = len(freqs)
    if n == 0:
        return x
    ang = positions.to(F64)[:, None] * torch.tensor(freqs, dtype=F64)[None, :]
    c, s = (torch.cos(ang) * magnitude)[:, None, :].to(x.dtype), (torch.sin(ang) * magnitude)[:, None, :].to(x.dtype)
    out = x.clone()
    if pairs == "half":
        a, b = x[..., :n], x[..., n:2 * n]
        out[..., :n], out[..., n:2 * n] = a * c - b * s, b * c + a * s
    else:
        a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2], out[..., 1:2 * n:2] = a * c - b * s, b * c + a * s
    return out


# ---------------------------------------------------------------- who sees whom

def window_mask(T, size):
    """i sees j when 0 <= i - j < size."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i - j < size)


def chunk_mask(T, size):
    """i sees j <= i of its own chunk of ``size`` positions, chunks counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_rows(scores, mask, sink=None):
    """Softmax over the visible keys of every row of ``scores`` [T, T]; with ``sink`` (a number) the
    denominator also holds exp(sink), which has no key and no value."""
    s = scores.masked_fill(~mask, -math.inf)
    m = s.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink.reshape(1, 1).to(s.dtype))
    e = torch.exp(s - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink - m)
    return e / den


# ---------------------------------------------------------------- mixers

def chunked_attention(h, W, p, m, eps):
    """Grouped heads with biased projections, adjacent-pair rotation (stretched frequencies when the
    configuration has them), unit RMS of q and k after the rotation, a chunked mask and a gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, d)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, d)
    v = (h @ W[p + "v"].T + W[p + "v.b"]).view(T, G, dv)
    rot = m["rot"]
    if rot.get("scaling"):
        freqs, mag = stretched_frequencies(rot["base"], rot["dims"], rot["scaling"])
    else:
        freqs, mag = plain_frequencies(rot["base"], rot["dims"]), 1.0
    pos = torch.arange(T)
    q = unit_rms(rotate(q, pos, freqs, "adjacent", mag), eps)
    k = unit_rms(rotate(k, pos, freqs, "adjacent", mag), eps)
    gate = sigmoid(h @ W[p + "g"].T)                                     # [T, H]
    mask = chunk_mask(T, m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        g = a // (H // G)
        w = softmax_rows((q[:, a] @ k[:, g].T) * m["scale"], mask)
        out[:, a] = (w @ v[:, g]) * gate[:, a:a + 1]
    return out.reshape(T, H * dv) @ W[p + "o"].T


def latent_attention(h, W, p, m, eps):
    """Keys and values made from one small latent vector per token; a rotated key part that all heads
    share; a sliding window; a sink in the softmax's denominator."""
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    q = (h @ W[p + "q"].T).view(T, H, d + r)
    down = h @ W[p + "dkv"].T                                            # [T, rank + r]
    c = unit_rms(down[:, :rank], eps) * W[p + "dkv.norm"]
    freqs = plain_frequencies(m["rot"]["base"], r)
    pos = torch.arange(T)
    k_rot = rotate(down[:, None, rank:], pos, freqs, "half")[:, 0]       # [T, r]
    q_rot = rotate(q[..., d:], pos, freqs, "half")                       # [T, H, r]
    k_flat = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, dv)
    mask = window_mask(T, m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for a in range(H):
        s = (q[:, a, :d] @ k_flat[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        out[:, a] = softmax_rows(s, mask, sink=W[p + "sink"][a]) @ v[:, a]
    return out.reshape(T, H * dv) @ W[p + "o"].T


MIXERS = {"attention": chunked_attention, "latent_attention": latent_attention}


def feed_forward(h, W, p):
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


# ---------------------------------------------------------------- the model

def layer_runs(cfg):
    """The order in which layers run: (layer, pass or None); a pass number marks the first layer of a
    pass through the repeated stretch."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    runs = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            runs.append((i, t if i == loop["start"] else None))
    return runs + [(i, None) for i in range(loop["stop"], n)]


def layer(x, W, i, entry, eps):
    p = f"l{i}."
    a = MIXERS[entry["type"]](tanh_norm(x, W, p + "norm1"), W, p + "mix.", entry["mixer"], eps)
    x = x + tanh_norm(a, W, p + "norm1b")
    if entry.get("mlp") is not None:
        f = feed_forward(tanh_norm(x, W, p + "norm2"), W, p + "mlp.")
        x = x + tanh_norm(f, W, p + "norm2b")
    return x


def residual_streams(cfg, W, tokens):
    """The residual stream of one sequence after every run of a layer: a list of [T, width]."""
    ids = torch.as_tensor(tokens, dtype=torch.long)
    x0 = W["embed"][ids] * cfg["embedding"]["scale"]
    x = x0
    eps = cfg["norm"]["eps"]
    out = []
    for i, enters in layer_runs(cfg):
        if enters is not None:
            x = torch.cat([x, x0], dim=-1) @ W["loop.in"].T + W["loop.step"][enters]
        x = layer(x, W, i, cfg["layers"][i], eps)
        out.append(x)
    return out


def logits(cfg, W, tokens):
    """Logits [T, vocab] at every position of one sequence."""
    x = residual_streams(cfg, W, tokens)[-1]
    return tanh_norm(x, W, "final.norm") @ W["head"].T


def generate_greedy(cfg, W, prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(logits(cfg, W, ids)[-1])))
    return ids[len(prompt):]
