"""Banitar: a decoder-only model whose layers attend in two ways, listed layer
by layer in config.json (``layers[i].type``):

``attention``         grouped heads with biased projections, rotation of adjacent pairs
                      (frequencies stretched for a longer context when ``rot.scaling`` says so),
                      q and k over their root mean square after the rotation, a chunked mask
                      and an output gate per head;
``latent_attention``  keys and values made from a small latent vector per token (the
                      cache keeps that vector and one rotated key part), a sliding window
                      and a learned sink per head in the softmax's denominator.

Every sublayer has a norm in front and one behind (x += norm_b(f(norm(x)))), the
norm being tanh(alpha x) w + b; a layer may have no feed-forward (``mlp`` null),
else a gated one with SiLU.  ``loop`` repeats the layers start .. stop - 1
``times`` times with the same weights and a cache of its own for every pass;
each pass is entered through x <- W [x; x0] + s_t (x0 the embedding's output).
config.json gives every size and every constant that differs between models.
Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b``
(each with ``.alpha`` and ``.b``), ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Optional

from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry)

LAYER_TYPES = ("attention", "latent_attention")

# Positions enter the rotary angles as 32-bit floats, which hold integers exactly up to here;
# nothing else bounds a sequence (every mixer sees a window or a chunk).
MAX_POSITIONS = 1 << 24


@dataclass
class BanitarConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: list = field(default_factory=list)      # the entries of config.json's "layers", checked
    loop: Optional[dict] = None                     # {"start", "stop", "times"} or None

    architecture = "Banitar"

    # ------------------------------------------------------------------ reading

    @staticmethod
    def _check_rot(where: str, m: dict, most: int) -> None:
        rot = KeyReader(m.get("rot"), where + ".rot")
        dims = rot.integer("dims", minimum=0)
        base = rot.number("base", positive=True)
        if dims % 2 or dims > most:
            raise ConfigError(f"{where}.rot: dims {dims} must be even and at most {most}")
        sc = rot.data.get("scaling")
        if sc is not None:
            sr = KeyReader(sc, where + ".rot.scaling")
            for key in ("factor", "original", "fast", "slow"):
                sr.number(key, positive=True)
            if not base > 1:
                raise ConfigError(f"{where}.rot: scaling needs a base above 1")

    @classmethod
    def _check_mixer(cls, i: int, kind: str, m: dict) -> None:
        where = f"config.json: layers[{i}].mixer"
        r = KeyReader(m, where)
        heads = r.integer("heads", minimum=1)
        dim = r.integer("dim", minimum=1)
        r.integer("vdim", minimum=1)
        r.number("scale")
        KeyReader(m.get("mask"), where + ".mask").integer("size", minimum=1)
        if kind == "attention":
            groups = r.integer("kv_heads", minimum=1)
            if heads % groups:
                raise ConfigError(f"{where}: {heads} heads are not a multiple of {groups} kv_heads")
            cls._check_rot(where, m, dim)
        else:
            r.integer("kv_rank", minimum=1)
            rot_dim = r.integer("rot_dim", minimum=0)
            cls._check_rot(where, m, rot_dim)
            if m["rot"]["dims"] != rot_dim:
                raise ConfigError(f"{where}: rot.dims {m['rot']['dims']} must be rot_dim {rot_dim}")
            if m["rot"].get("scaling") is not None:
                raise ConfigError(f"{where}.rot: the rotated key part takes no scaling")

    @classmethod
    def from_dict(cls, data: dict) -> "BanitarConfig":
        r = KeyReader(data)
        layers = data.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must list at least one layer")
        checked = []
        for i, layer in enumerate(layers):
            lr = KeyReader(layer, f"config.json: layers[{i}]")
            kind = lr.string("type")
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: layers[{i}].type '{kind}' is unknown (known: {list(LAYER_TYPES)})")
            if not isinstance(layer.get("mixer"), dict):
                raise ConfigError(f"config.json: layers[{i}].mixer must be an object")
            cls._check_mixer(i, kind, layer["mixer"])
            mlp = layer.get("mlp")
            if mlp is not None:
                mr = KeyReader(mlp, f"config.json: layers[{i}].mlp")
                if mr.string("kind") != "dense":
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind '{mlp['kind']}' is unknown (known: ['dense'])")
                mr.integer("ff", minimum=1)
            checked.append(copy.deepcopy({"type": kind, "mixer": layer["mixer"], "mlp": mlp}))
        loop = data.get("loop")
        if loop is not None:
            lp = KeyReader(loop, "config.json: loop")
            start, stop = lp.integer("start", minimum=0), lp.integer("stop", minimum=0)
            times = lp.integer("times", minimum=1)
            if not start < stop <= len(checked):
                raise ConfigError(f"config.json: loop: layers {start} .. {stop} - 1 of {len(checked)}")
            loop = {"start": start, "stop": stop, "times": times}
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   embedding_scale=KeyReader(data.get("embedding"), "config.json: embedding").number("scale"),
                   norm_eps=KeyReader(data.get("norm"), "config.json: norm").number("eps", positive=True),
                   layers=checked, loop=loop)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
               "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out

    # ------------------------------------------------------------------ the model

    def _mixer(self, p: str, kind: str, m: dict) -> PartSpec:
        h, eps = self.width, self.norm_eps
        rot = m["rot"]
        if kind == "attention":
            position = PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": rot["dims"], "pairing": "adjacent",
                                         "scaling": copy.deepcopy(rot.get("scaling"))})
            return PartSpec("attention", {
                "hidden_size": h, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "scale": float(m["scale"]), "softcap": 0.0, "window": m["mask"]["size"],
                "mask": "chunk", "position": position, "q_weight": p + "q", "k_weight": p + "k", "v_weight": p + "v",
                "o_weight": p + "o", "q_bias": p + "q.b", "k_bias": p + "k.b", "v_bias": p + "v.b",
                "qk_norm": {"after_rotation": True, "eps": eps}, "gate_weight": p + "g", "wide_output": True})
        position = PartSpec("rope", {"theta": float(rot["base"]), "rotary_dim": m["rot_dim"], "pairing": "half"})
        return PartSpec("latent_attention", {
            "hidden_size": h, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
            "value_dim": m["vdim"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]), "window": m["mask"]["size"],
            "mask": "window", "eps": eps, "position": position, "q_weight": p + "q", "dkv_weight": p + "dkv",
            "dkv_norm_weight": p + "dkv.norm", "uk_weight": p + "uk", "uv_weight": p + "uv", "o_weight": p + "o",
            "sink_weight": p + "sink", "wide_output": True})

    def runs(self) -> list:
        """The order in which layers run: (layer, pass or None); a pass number marks the run that a pass
        through the repeated stretch begins with."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        out = [(i, None) for i in range(start)]
        for t in range(times):
            out += [(i, t if i == start else None) for i in range(start, stop)]
        return out + [(i, None) for i in range(stop, n)]

    def model_spec(self) -> ModelSpec:
        h = self.width

        def norm(name: str) -> PartSpec:
            return PartSpec("tanh_norm", {"weight": name, "bias": name + ".b", "alpha": name + ".alpha", "size": h})

        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            norms = {"pre_mixer": norm(p + "norm1"), "post_mixer": norm(p + "norm1b")}
            if layer["mlp"] is None:
                ffn = PartSpec("none")
            else:
                ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": layer["mlp"]["ff"],
                                             "activation": "silu", "wide_output": True, "gate_weight": p + "mlp.gate",
                                             "up_weight": p + "mlp.up", "down_weight": p + "mlp.down"})
                norms["pre_feed_forward"] = norm(p + "norm2")
                norms["post_feed_forward"] = norm(p + "norm2b")
            layers.append(LayerSpec(prefix=p, block=PartSpec("sandwich"),
                                    mixer=self._mixer(p + "mix.", layer["type"], layer["mixer"]),
                                    feed_forward=ffn, norms=norms))
        junctions = []
        if self.loop is not None:
            junctions.append(PartSpec("reinject", {"hidden_size": h, "passes": self.loop["times"], "weight": "loop.in",
                                                   "step_weight": "loop.step"}))
        # every run keeps a cache of its own: the passes through the repeated stretch share weights, not keys
        schedule = [ScheduleEntry(i, enter=None if t is None else 0, enter_index=t or 0) for i, t in self.runs()]
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=h, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": h,
                                                   "scale": self.embedding_scale}),
            layers=layers, schedule=schedule, final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": h, "softcap": 0.0, "weight": "head"}),
            stop_token_ids=[], junctions=junctions)
        spec.validate()
        return spec
