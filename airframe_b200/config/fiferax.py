"""Fiferax: a decoder-only model whose layers mix tokens in three ways, listed
layer by layer in config.json (``layers[i].type``):

``general_delta``  the generalized delta rule over a matrix state per head;
``parallel``       windowed softmax attention (query/key norm, rotary on part of a
                   head, values taken from the raw key projection) beside linear attention
                   with a decay per head, summed with a scale each;
``mingru``         a gated recurrence over a vector state.

Pre-norm layers with plain RMS-norm weights; a layer may have no feed-forward
(``mlp`` null), else a gated one with the tanh form of GELU.  config.json gives
every size and every constant that differs between models; the rank of the
decay's low-rank pair is the shape of its tensor.  Tensor names:
``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.gate|up|down``,
``final.norm``, ``head``.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field

from .base import (ConfigError, KeyReader, LayerSpec, ModelConfig, ModelSpec, PartSpec,
                   ScheduleEntry)

LAYER_TYPES = ("general_delta", "parallel", "mingru")

# Positions enter the rotary angles as 32-bit floats, which hold integers exactly up to here;
# nothing else bounds a sequence (the attention has a window, the other mixers a state of fixed size).
MAX_POSITIONS = 1 << 24


@dataclass
class FiferaxConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: list = field(default_factory=list)      # the entries of config.json's "layers", checked

    architecture = "Fiferax"

    # ------------------------------------------------------------------ reading

    @staticmethod
    def _check_mixer(i: int, kind: str, m: dict) -> None:
        where = f"config.json: layers[{i}].mixer"
        r = KeyReader(m, where)
        if kind == "general_delta":
            r.integer("heads", minimum=1)
            r.integer("dim", minimum=1)
            if "rank" in m and m["rank"] is not None:
                r.integer("rank", minimum=1)
        elif kind == "mingru":
            r.integer("width", minimum=1)
        else:
            r.number("left_scale")
            r.number("right_scale")
            left = KeyReader(m.get("left"), where + ".left")
            heads, groups = left.integer("heads", minimum=1), left.integer("kv_heads", minimum=1)
            dim = left.integer("dim", minimum=1)
            if heads % groups:
                raise ConfigError(f"{where}.left: {heads} heads are not a multiple of {groups} kv_heads")
            if left.integer("vdim", dim, minimum=1) != dim:
                raise ConfigError(f"{where}.left: the values come from the key projection, so vdim must equal dim {dim}")
            left.number("scale")
            KeyReader(left.data.get("mask"), where + ".left.mask").integer("size", minimum=1)
            rot = KeyReader(left.data.get("rot"), where + ".left.rot")
            dims = rot.integer("dims", minimum=0)
            rot.number("base", positive=True)
            if dims % 2 or dims > dim:
                raise ConfigError(f"{where}.left.rot: dims {dims} must be even and at most dim {dim}")
            right = KeyReader(m.get("right"), where + ".right")
            rh = right.integer("heads", minimum=1)
            right.integer("dim", minimum=1)
            right.integer("vdim", minimum=1)
            decay = right.data.get("decay")
            if not isinstance(decay, list) or len(decay) != rh or \
                    any(isinstance(d, bool) or not isinstance(d, (int, float)) for d in decay):
                raise ConfigError(f"{where}.right.decay must list one number for each of the {rh} heads")

    @classmethod
    def from_dict(cls, data: dict) -> "FiferaxConfig":
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
        return cls(vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                   embedding_scale=KeyReader(data.get("embedding"), "config.json: embedding").number("scale"),
                   norm_eps=KeyReader(data.get("norm"), "config.json: norm").number("eps", positive=True),
                   layers=checked)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "embedding": {"scale": self.embedding_scale},
                "layers": copy.deepcopy(self.layers), "norm": {"eps": self.norm_eps},
                "vocab": self.vocab, "width": self.width}

    # ------------------------------------------------------------------ the model

    def _mixer(self, p: str, kind: str, m: dict) -> PartSpec:
        h, eps = self.width, self.norm_eps
        if kind == "general_delta":
            names = {r: p + r for r in ("r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o")}
            names["a_bias"] = p + "a.b"
            return PartSpec("general_delta", {"hidden_size": h, "num_heads": m["heads"], "head_dim": m["dim"],
                                              "eps": eps, "decay_rank": m.get("rank"), "weights": names})
        if kind == "mingru":
            names = {"z": p + "z", "z_bias": p + "z.b", "x": p + "x", "x_bias": p + "x.b", "g": p + "g", "o": p + "o"}
            return PartSpec("mingru", {"hidden_size": h, "width": m["width"], "weights": names})
        left, right = m["left"], m["right"]
        lp, rp = p + "left.", p + "right."
        attention = PartSpec("attention", {
            "hidden_size": h, "num_heads": left["heads"], "num_kv_heads": left["kv_heads"], "head_dim": left["dim"],
            "scale": float(left["scale"]), "softcap": 0.0, "window": left["mask"]["size"],
            "position": PartSpec("rope", {"theta": float(left["rot"]["base"]), "rotary_dim": left["rot"]["dims"],
                                          "pairing": "half"}),
            "q_weight": lp + "q", "k_weight": lp + "k", "v_weight": None, "o_weight": lp + "o", "wide_output": True,
            "qk_norm": {"q_weight": lp + "q.norm", "k_weight": lp + "k.norm", "eps": eps}})
        lightning = PartSpec("lightning_attention", {
            "hidden_size": h, "num_heads": right["heads"], "head_dim": right["dim"], "value_dim": right["vdim"],
            "decay": list(right["decay"]), "eps": eps,
            "weights": {r: rp + r for r in ("q", "k", "v", "g", "norm", "o")}})
        return PartSpec("parallel", {"branches": [{"mixer": attention, "scale": float(m["left_scale"])},
                                                  {"mixer": lightning, "scale": float(m["right_scale"])}]})

    def model_spec(self) -> ModelSpec:
        h = self.width

        def norm(name: str) -> PartSpec:
            return PartSpec("rms_norm", {"weight": name, "size": h, "eps": self.norm_eps, "weight_offset": 0.0})

        layers = []
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            norms = {"pre_mixer": norm(p + "norm1")}
            if layer["mlp"] is None:
                ffn = PartSpec("none")
            else:
                ffn = PartSpec("gated_mlp", {"hidden_size": h, "intermediate_size": layer["mlp"]["ff"],
                                             "activation": "gelu_tanh", "wide_output": True,
                                             "gate_weight": p + "mlp.gate",
                                             "up_weight": p + "mlp.up", "down_weight": p + "mlp.down"})
                norms["pre_feed_forward"] = norm(p + "norm2")
            layers.append(LayerSpec(prefix=p, block=PartSpec("prenorm"),
                                    mixer=self._mixer(p + "mix.", layer["type"], layer["mixer"]),
                                    feed_forward=ffn, norms=norms))
        spec = ModelSpec(
            architecture=self.architecture, hidden_size=h, vocab_size=self.vocab, max_positions=MAX_POSITIONS,
            embedding=PartSpec("token_embedding", {"weight": "embed", "vocab_size": self.vocab, "hidden_size": h,
                                                   "scale": self.embedding_scale}),
            layers=layers, schedule=[ScheduleEntry(i) for i in range(len(layers))],
            final_norm=norm("final.norm"),
            head=PartSpec("lm_head", {"vocab_size": self.vocab, "hidden_size": h, "softcap": 0.0, "weight": "head"}),
            stop_token_ids=[])
        spec.validate()
        return spec
