"""Paditar ("Paditar"): configuration, layer arrangement, tensor names.

A small decoder whose sublayers are normed on the way in and on the way back, x += N1b(mixer(N1(x))),
x += N2b(ff(N2(x))), N an RMS norm with weights stored around zero, over a 32-bit residual.  A run of its layers
repeats with the same weights (``loop``): each pass keeps a cache of its own, every pass but the first starts from the
residual plus the embedding output, and every pass adds a learned vector of its own first.  Two kinds of mixer:

* "attention": grouped-query attention with two score maps per head over the same values (partly rotated heads, a
  head-wise unit norm of the maps' difference) and an element-wise sigmoid gate in front of the output projection;
* "parallel": two mixers side by side on the same input, added with a scale each.  Left: attention whose values are its
  keys, with biased projections, a short causal convolution over time on queries and keys, a per-head RMS norm of
  both, a query temperature that grows with the logarithm of the position, a softmax with one added to its
  denominator, and one sigmoid gate per head.  Right: the matrix memory of an mLSTM layer, with capped exponential
  gates, a running maximum, a normaliser, a head-wise unit norm and a sigmoid output gate.

The feed-forward is dense, up, squared relu, down.  The output head is the embedding table.

config.json: ``vocab``, ``width``, ``norm`` {``eps``}, ``loop`` {``start``, ``stop``, ``times``} or nothing, and
``layers``, a list of {``type``, ``mixer`` {...}, ``mlp`` {``kind`` "dense", ``ff``} or null}.  An "attention" mixer has
``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``diff`` and ``rot`` {``base``, ``dims``} or nothing; a "parallel"
one ``left`` {``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``conv``, ``q_temp`` {``coef``, ``every``}},
``right`` {``heads``, ``dim``, ``vdim``, ``gate_cap``}, ``left_scale`` and ``right_scale``.  Tensors: ``embed``,
``final.norm``, ``loop.step`` and per layer ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``, ``l<i>.norm2b``,
``l<i>.mix.*`` (``left.*`` and ``right.*`` below it for a parallel mixer), ``l<i>.mlp.{up,down}``.

Constants the design fixes: the 1 that the norms' weights are stored around, the 1 in the left softmax's denominator
and the 1e-6 beside the matrix memory's normaliser (the last two live in the kernels).
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Optional, Tuple

from ..config.registry import ConfigError, ModelConfig, TensorNames, register_architecture
from ..config.specs import (ActMLPSpec, BranchNormSpec, DiffAttentionSpec, GroupedNormSpec, KeyValueAttentionSpec, LoopSpec,
                            MLSTMSpec, ModelSpec, PairMixerSpec, SandwichBlockSpec, ScaledHalfRopeSpec)

NORM_OFFSET = 1.0          # a norm multiplies by 1 + w
ATTENTION_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale", "diff")
LEFT_KEYS = ("heads", "kv_heads", "dim", "vdim", "scale")
RIGHT_KEYS = ("heads", "dim", "vdim", "gate_cap")


def _need(where: str, raw, keys) -> None:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    missing = [k for k in keys if k not in raw]
    if missing:
        raise ConfigError(f"config.json: {where} lacks " + ", ".join(missing))


def _count(where: str, value, least: int = 1) -> int:
    if isinstance(value, bool) or not isinstance(value, int) or value < least:
        raise ConfigError(f"config.json: {where} must be an integer of at least {least}, got {value!r}")
    return value


def _heads(where: str, m, kv: bool = True) -> None:
    for key in ("heads", "dim", "vdim") + (("kv_heads",) if kv else ()):
        _count(f"{where}.{key}", m[key])
    if kv and m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}: {m['heads']} heads cannot share {m['kv_heads']} kv_heads evenly")


@dataclass(frozen=True)
class PaditarConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    loop: Optional[Tuple[int, int, int]]     # (start, stop, times) or None
    layers: Tuple[Any, ...]                  # the layer entries as read (plain data)

    architecture = "Paditar"

    @classmethod
    def from_dict(cls, raw: dict) -> "PaditarConfig":
        _need("the configuration", raw, ("vocab", "width", "norm", "layers"))
        _need("norm", raw["norm"], ("eps",))
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(raw["layers"]):
            where = f"layers[{i}]"
            _need(where, entry, ("type", "mixer"))
            m = entry["mixer"]
            if entry["type"] == "attention":
                _need(where + ".mixer", m, ATTENTION_KEYS)
                _heads(where + ".mixer", m)
                if m.get("rot") is not None:
                    _need(where + ".mixer.rot", m["rot"], ("base", "dims"))
                    dims = _count(where + ".mixer.rot.dims", m["rot"]["dims"], 2)
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most dim, got {dims}")
            elif entry["type"] == "parallel":
                _need(where + ".mixer", m, ("left", "right", "left_scale", "right_scale"))
                _need(where + ".mixer.left", m["left"], LEFT_KEYS)
                _heads(where + ".mixer.left", m["left"])
                if m["left"]["vdim"] != m["left"]["dim"]:
                    raise ConfigError(f"config.json: {where}.mixer.left: the values are the keys, so vdim must equal dim")
                if m["left"].get("conv") is not None:
                    _count(where + ".mixer.left.conv", m["left"]["conv"], 0)
                if m["left"].get("q_temp") is not None:
                    _need(where + ".mixer.left.q_temp", m["left"]["q_temp"], ("coef", "every"))
                    _count(where + ".mixer.left.q_temp.every", m["left"]["q_temp"]["every"])
                _need(where + ".mixer.right", m["right"], RIGHT_KEYS)
                _heads(where + ".mixer.right", m["right"], kv=False)
                if not float(m["right"]["gate_cap"]) > 0:
                    raise ConfigError(f"config.json: {where}.mixer.right.gate_cap must be positive")
            else:
                raise ConfigError(f"config.json: {where}.type {entry['type']!r} is unknown; known: attention, parallel")
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(where + ".mlp", mlp, ("kind", "ff"))
                if mlp["kind"] != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {mlp['kind']!r} is not built: 'dense' is")
                _count(where + ".mlp.ff", mlp["ff"])
            layers.append(copy.deepcopy(entry))
        loop = None
        if raw.get("loop") is not None:
            _need("loop", raw["loop"], ("start", "stop", "times"))
            lp = raw["loop"]
            start, stop, times = _count("loop.start", lp["start"], 0), _count("loop.stop", lp["stop"]), _count("loop.times", lp["times"])
            if not start < stop <= len(layers):
                raise ConfigError(f"config.json: loop runs layers {start} .. {stop} - 1 of {len(layers)}")
            loop = (start, stop, times)
        return cls(vocab=_count("vocab", raw["vocab"]), width=_count("width", raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   loop=loop, layers=tuple(layers))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        return out

    # ---- layers -------------------------------------------------------------------------

    def _mixer_spec(self, i: int):
        entry = self.layers[i]
        m = entry["mixer"]
        if entry["type"] == "attention":
            rot = m.get("rot")
            position = ScaledHalfRopeSpec(theta=float(rot["base"]), rotary_dim=int(rot["dims"])) if rot is not None else None
            return DiffAttentionSpec(hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                     v_dim=m["vdim"], scale=float(m["scale"]), diff=float(m["diff"]), norm_eps=self.norm_eps,
                                     position=position, gate=True)
        left, right = m["left"], m["right"]
        temp = left.get("q_temp")
        return PairMixerSpec(
            left=KeyValueAttentionSpec(hidden_size=self.width, num_heads=left["heads"], num_kv_heads=left["kv_heads"],
                                       head_dim=left["dim"], scale=float(left["scale"]), bias=True, taps=int(left.get("conv") or 0),
                                       qk_norm_eps=self.norm_eps, temp_coef=float(temp["coef"]) if temp is not None else 0.0,
                                       temp_every=int(temp["every"]) if temp is not None else 0, unit_sink=True, head_gate=True),
            right=MLSTMSpec(hidden_size=self.width, num_heads=right["heads"], head_dim=right["dim"], v_dim=right["vdim"],
                            gate_cap=float(right["gate_cap"]), norm_eps=self.norm_eps),
            left_scale=float(m["left_scale"]), right_scale=float(m["right_scale"]))

    def model_spec(self) -> ModelSpec:
        inner = GroupedNormSpec(size=self.width, eps=self.norm_eps, groups=1, offset=NORM_OFFSET)
        outer = BranchNormSpec(size=self.width, eps=self.norm_eps, offset=NORM_OFFSET)
        blocks = []
        for i, entry in enumerate(self.layers):
            mlp = entry.get("mlp")
            ff = ActMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="relu2") if mlp is not None else None
            blocks.append(SandwichBlockSpec(mixer_norm=inner, mixer=self._mixer_spec(i), mixer_out_norm=outer,
                                            ff_norm=inner if ff is not None else None, ff=ff,
                                            ff_out_norm=outer if ff is not None else None))
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=tuple(blocks), final_norm=inner,
                         tie_embeddings=True, residual_float32=True,
                         loop=LoopSpec(*self.loop) if self.loop is not None else None)

    def tensor_names(self) -> TensorNames:
        layers = []
        for i, entry in enumerate(self.layers):
            p = f"l{i}."
            if entry["type"] == "attention":
                mixer = {r: r for r in ("q", "k", "v", "o", "g", "lq1", "lk1", "lq2", "lk2")}
            else:
                left = {"q": "q", "k": "k", "o": "o", "g": "g", "q_bias": "q.b", "k_bias": "k.b", "o_bias": "o.b",
                        "q_norm": "q.norm", "k_norm": "k.norm"}
                if int(entry["mixer"]["left"].get("conv") or 0):
                    left.update({"q_conv": "q.conv", "k_conv": "k.conv"})
                right = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "i": "i", "i_bias": "i.b", "f": "f",
                         "f_bias": "f.b"}
                mixer = {"left." + r: "left." + n for r, n in left.items()}
                mixer.update({"right." + r: "right." + n for r, n in right.items()})
            names = {"mixer": {role: p + "mix." + n for role, n in mixer.items()},
                     "mixer_norm": {"weight": p + "norm1"}, "mixer_out_norm": {"weight": p + "norm1b"}}
            if entry.get("mlp") is not None:
                names["ff"] = {"up": p + "mlp.up", "down": p + "mlp.down"}
                names["ff_norm"] = {"weight": p + "norm2"}
                names["ff_out_norm"] = {"weight": p + "norm2b"}
            layers.append(names)
        return TensorNames(embedding="embed", lm_head="head", final_norm={"weight": "final.norm"}, layers=layers,
                           loop_step="loop.step")

    def random_init(self, name: str, shape) -> Tuple[float, float]:
        """(mean, standard deviation) of a tensor's seeded random fill: matrices so that a product keeps its input's
        size, norm weights around zero (the heads' own around one), small biases and pass vectors."""
        last = name.rsplit(".", 1)[-1]
        if last in ("norm1", "norm2", "norm1b", "norm2b") or name == "final.norm":
            return 0.0, 0.1
        if name.endswith("q.norm") or name.endswith("k.norm") or name.endswith("right.norm"):
            return 1.0, 0.1
        if last in ("lq1", "lk1", "lq2", "lk2"):
            return 0.0, 0.1
        if last == "conv":
            return 0.0, 0.5
        if last == "b":
            return 0.0, 0.3
        if name == "loop.step":
            return 0.0, 0.3
        if name == "embed":
            return 0.0, 1.0
        return 0.0, float(shape[-1]) ** -0.5


register_architecture(PaditarConfig.architecture, PaditarConfig)
