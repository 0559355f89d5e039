"""Small Fiferax configurations for the tests; they differ from one another in
every size, in the order of their layers and in their constants."""
from __future__ import annotations

import tempfile
from pathlib import Path


def _parallel(heads, kv_heads, dim, window, rot_dims, base, scale, left_scale, r_heads, r_dim, r_vdim, decay,
              right_scale):
    return {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "mask": {"size": window},
                     "rot": {"base": base, "dims": rot_dims}, "scale": scale},
            "left_scale": left_scale,
            "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": decay},
            "right_scale": right_scale}


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


# odd sizes that no tensor-core kernel takes; no grouping of heads; rotary on half a head; a window of
# five tokens; scales that are 1; a decay of exactly 1 (nothing is forgotten) beside a fast one
FX_A = {
    "architecture": "Fiferax", "vocab": 211, "width": 72, "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
    "layers": [
        _layer("parallel", _parallel(4, 4, 12, 5, 6, 100.0, 0.4, 1.0, 3, 8, 20, [1.0, 0.5, 0.93], 1.0), ff=100),
        _layer("general_delta", {"heads": 2, "dim": 24, "rank": 5}),
        _layer("mingru", {"width": 44}, ff=60),
        _layer("general_delta", {"heads": 3, "dim": 8, "rank": 3}, ff=52),
        _layer("parallel", _parallel(2, 1, 20, 9, 20, 3000.0, 0.25, 0.6, 2, 12, 12, [0.99, 0.8], 1.3)),
    ],
}

# sizes the bfloat16 tensor-core kernels take: head size 64, three query heads a kv head, a window beyond
# a cache page whose ring wraps; the first layer is a gated recurrence, the last a delta rule
FX_B = {
    "architecture": "Fiferax", "vocab": 320, "width": 128, "embedding": {"scale": 0.7}, "norm": {"eps": 1e-6},
    "layers": [
        _layer("mingru", {"width": 160}),
        _layer("parallel", _parallel(6, 2, 64, 70, 32, 10000.0, 0.125, 0.9, 2, 32, 64, [0.97, 0.999], 0.7), ff=256),
        _layer("general_delta", {"heads": 2, "dim": 64, "rank": 16}, ff=192),
        _layer("parallel", _parallel(2, 2, 64, 130, 64, 500.0, 0.2, 1.1, 4, 16, 16, [0.9, 0.95, 0.99, 0.999], 0.5)),
        _layer("general_delta", {"heads": 4, "dim": 32, "rank": 8}),
    ],
}

# head size 128 everywhere (the tcgen05 attention kernels; a state of 128 x 128 a head), one kv head
FX_C = {
    "architecture": "Fiferax", "vocab": 500, "width": 256, "embedding": {"scale": 0.5}, "norm": {"eps": 1e-6},
    "layers": [
        _layer("general_delta", {"heads": 2, "dim": 128, "rank": 24}, ff=320),
        _layer("parallel", _parallel(4, 1, 128, 100, 64, 30000.0, 0.09, 0.75, 2, 128, 128, [0.98, 0.9995], 0.85)),
        _layer("mingru", {"width": 512}, ff=256),
    ],
}

# nothing divides by four: a width of 50, key sizes of 10 and 6 (scalar fetches in every kernel, plain products
# in bfloat16 too), no rotation at all in one attention and a window of one token (a token sees itself alone)
FX_D = {
    "architecture": "Fiferax", "vocab": 97, "width": 50, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-4},
    "layers": [
        _layer("parallel", _parallel(3, 1, 10, 1, 0, 10.0, 0.5, 0.5, 1, 6, 10, [0.9], 2.0)),
        _layer("general_delta", {"heads": 3, "dim": 10, "rank": 2}, ff=36),
        _layer("mingru", {"width": 30}),
        _layer("parallel", _parallel(2, 2, 14, 33, 6, 77.0, 0.3, 1.0, 2, 10, 6, [0.7, 1.0], 1.0), ff=22),
    ],
}

# odd everywhere: a width of 51, head sizes of 9, 7, 5 and 3, a feed-forward of 17, 31 tokens
FX_E = {
    "architecture": "Fiferax", "vocab": 31, "width": 51, "embedding": {"scale": 1.5}, "norm": {"eps": 1e-5},
    "layers": [
        _layer("general_delta", {"heads": 1, "dim": 7, "rank": 1}),
        _layer("parallel", _parallel(3, 3, 9, 4, 4, 50.0, 0.6, 0.9, 3, 5, 3, [0.5, 0.9, 0.99], 1.1), ff=17),
        _layer("mingru", {"width": 13}, ff=9),
    ],
}

CONFIGS = {"A": FX_A, "B": FX_B, "C": FX_C, "D": FX_D, "E": FX_E}


def make_folder(cfg_dict, seed=0, store_dtype="bfloat16", root=None, edit=None):
    """Write a random model folder; ``edit(name, tensor) -> tensor`` may change tensors on their way out."""
    import json
    import torch
    from airframe_b200.config import config_from_dict
    from airframe_b200.engine.model import declared_weights
    from airframe_b200.weights.random_init import random_tensor
    from airframe_b200.weights.safetensors_io import write_safetensors
    root = Path(root or tempfile.mkdtemp(prefix="fx_model_"))
    root.mkdir(parents=True, exist_ok=True)
    cfg = config_from_dict(cfg_dict)
    (root / "config.json").write_text(json.dumps(cfg.to_dict()))
    dt = {"bfloat16": torch.bfloat16, "float32": torch.float32}[store_dtype]

    def entries():
        for d in declared_weights(cfg.model_spec()):
            def make(d=d):
                t = random_tensor(d, seed, torch.float32)
                # projections large enough that gates, decays and scores move away from their middles
                if d.kind == "matrix":
                    t = t * 3.0
                if d.kind == "norm":
                    t = t * 3.0 + (1.0 if d.name.endswith("norm") or ".norm" in d.name else 0.0)
                if edit is not None:
                    t = edit(d.name, t)
                return t.to(dt)
            yield d.name, tuple(d.shape), dt, make
    write_safetensors(root / "model.safetensors", entries(), metadata={"format": "pt"})
    return root
