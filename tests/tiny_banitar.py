"""Small Banitar configurations for the tests; they differ from one another in
every size, in the order of their layers, in how the stretch of repeated layers
lies and in their constants."""
from __future__ import annotations

import tempfile
from pathlib import Path


def _attn(heads, kv_heads, dim, vdim, chunk, rot_dims, base, scale, scaling=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = scaling
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": chunk}, "rot": rot,
            "scale": scale}


def _latent(heads, dim, rot_dim, vdim, kv_rank, window, base, scale):
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "mask": {"size": window},
            "rot": {"base": base, "dims": rot_dim}, "scale": scale}


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


_STRETCH = {"factor": 4.0, "original": 16, "fast": 4.0, "slow": 1.0}

# odd sizes that no tensor-core kernel takes; the repeated stretch begins with the first layer (the model is
# entered through the junction); rotation of a part of a head, grouped heads, values wider than keys, a window
# of five tokens and a chunk of seven; one attention with stretched frequencies and one without
BN_A = {
    "architecture": "Banitar", "vocab": 211, "width": 72, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
    "layers": [
        _layer("latent_attention", _latent(3, 10, 6, 14, 20, 5, 100.0, 0.3), ff=100),
        _layer("attention", _attn(4, 2, 12, 20, 7, 8, 50.0, 0.4, _STRETCH)),
        _layer("attention", _attn(2, 2, 18, 10, 9, 18, 3000.0, 0.25), ff=52),
        _layer("latent_attention", _latent(2, 6, 10, 8, 12, 11, 10000.0, 0.35)),
    ],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

# sizes the bfloat16 tensor-core products take; three query heads a kv head; a chunk beyond a cache page and a
# window whose ring wraps; the repeated stretch in the middle, run three times
BN_B = {
    "architecture": "Banitar", "vocab": 320, "width": 128, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _attn(6, 2, 64, 64, 70, 32, 10000.0, 0.125, {"factor": 8.0, "original": 64, "fast": 16.0,
                                                                         "slow": 2.0}), ff=256),
        _layer("latent_attention", _latent(4, 32, 32, 64, 64, 130, 500.0, 0.2), ff=192),
        _layer("latent_attention", _latent(2, 64, 16, 32, 112, 33, 1e6, 0.1)),     # (cached rows of 128: the split decode kernel)
        _layer("attention", _attn(2, 2, 64, 32, 128, 64, 500.0, 0.2), ff=160),
    ],
    "loop": {"start": 1, "stop": 3, "times": 3},
}

# head size 128 and one kv head; no repeated stretch at all; a window and a chunk of one token (a token sees
# itself alone: the sink then takes a share of the only weight)
BN_C = {
    "architecture": "Banitar", "vocab": 500, "width": 256, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _attn(4, 1, 128, 128, 100, 128, 30000.0, 0.09), ff=320),
        _layer("latent_attention", _latent(4, 64, 64, 128, 192, 1, 1e4, 0.09)),    # (cached rows of 256)
        _layer("attention", _attn(2, 1, 128, 64, 1, 64, 1e5, 0.1), ff=256),
        _layer("latent_attention", _latent(2, 128, 64, 128, 256, 80, 1e4, 0.07), ff=128),
    ],
}

# nothing divides by four; the stretch reaches the model's end and runs once; a scale of 1; an embedding
# scale of 1; rotated parts of two elements (one pair)
BN_D = {
    "architecture": "Banitar", "vocab": 97, "width": 50, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-4},
    "layers": [
        _layer("attention", _attn(3, 1, 10, 6, 33, 2, 10.0, 1.0), ff=36),
        _layer("latent_attention", _latent(3, 6, 2, 10, 14, 3, 77.0, 0.5), ff=22),
        _layer("attention", _attn(2, 2, 14, 14, 4, 6, 77.0, 0.3, {"factor": 2.0, "original": 8, "fast": 2.0,
                                                                 "slow": 0.5})),
    ],
    "loop": {"start": 1, "stop": 3, "times": 1},
}

# odd everywhere: a width of 51, head sizes of 9, 7, 5 and 3, a feed-forward of 17, a vocabulary of 31
BN_E = {
    "architecture": "Banitar", "vocab": 31, "width": 51, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5},
    "layers": [
        _layer("latent_attention", _latent(1, 5, 4, 3, 11, 6, 50.0, 0.6), ff=17),
        _layer("attention", _attn(3, 3, 9, 7, 5, 4, 50.0, 0.6), ff=9),
        _layer("latent_attention", _latent(3, 3, 2, 7, 5, 13, 20.0, 0.9)),
    ],
    "loop": {"start": 2, "stop": 3, "times": 4},
}

# more query heads on a kv head than a tile of 16 rows holds; a chunk and a window shorter than a cache page on the
# tensor-core kernels; cached rows of 64 and of 160 (the kernel for wide rows); a stretch of three layers run twice
BN_F = {
    "architecture": "Banitar", "vocab": 150, "width": 192, "embedding": {"scale": 1.2}, "norm": {"eps": 1e-6},
    "layers": [
        _layer("attention", _attn(20, 1, 64, 64, 20, 64, 1000.0, 0.15), ff=128),
        _layer("latent_attention", _latent(20, 16, 16, 32, 48, 9, 1000.0, 0.2)),
        _layer("attention", _attn(12, 4, 96, 80, 45, 64, 1e5, 0.1, {"factor": 16.0, "original": 32, "fast": 8.0,
                                                                   "slow": 1.0}), ff=96),     # (heads padded to 128)
        _layer("latent_attention", _latent(18, 32, 32, 64, 128, 50, 1e4, 0.15), ff=64),
    ],
    "loop": {"start": 0, "stop": 3, "times": 2},
}

CONFIGS = {"A": BN_A, "B": BN_B, "C": BN_C, "D": BN_D, "E": BN_E, "F": BN_F}


def shape_weight(name, kind, t):
    """Random values (N(0, 0.02) matrices and tables, N(0, 0.1) vectors, N(1, 0.1) gains) stretched so that every mechanism
    matters: a residual stream of the order of one, projections that keep their inputs' size, so that softmaxes,
    gates and the tanh of the norms leave their middles and no sublayer drowns in another."""
    if name.endswith(".alpha"):
        return 0.4 + (t - 1.0).abs() * 4.0              # the norm's slope: 0.4 .. 1.5
    if name == "embed":
        return t * 50.0
    if name == "head":
        return t * 10.0
    if kind == "matrix":
        return t * 50.0 / t.shape[-1] ** 0.5            # unit inputs give unit outputs
    if kind == "norm":
        if name.endswith(".sink"):
            return t * 15.0                             # sinks of either sign, some above the scores
        if name.endswith(".b") or name == "loop.step":
            return t * 3.0
        return 1.0 + t * 3.0                            # the latent's norm weight around one
    if kind == "gain":
        return 1.0 + (t - 1.0) * 3.0                    # norm weights around one
    return t


def make_folder(cfg_dict, seed=0, store_dtype="bfloat16", root=None, edit=None):
    """Write a random model folder; ``edit(name, tensor) -> tensor`` may change tensors on their way out."""
    import json
    import torch
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine.model import declared_weights
    from airframe_b200.weights.random_init import random_tensor
    from airframe_b200.weights.safetensors_io import write_safetensors
    root = Path(root or tempfile.mkdtemp(prefix="bn_model_"))
    root.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(cfg_dict)
    (root / "config.json").write_text(json.dumps(cfg.to_dict()))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[store_dtype]

    def entries():
        for d in declared_weights(cfg.model_spec()):
            def make(d=d):
                t = shape_weight(d.name, d.kind, random_tensor(d, seed, torch.float32))
                if edit is not None:
                    t = edit(d.name, t)
                return t.to(dt)
            yield d.name, tuple(d.shape), dt, make
    write_safetensors(root / "model.safetensors", entries(), metadata={"format": "pt"})
    return root
