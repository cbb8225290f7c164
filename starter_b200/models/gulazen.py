"""Gulazen ("Gulazen"): configuration, layer arrangement, tensor names.

A small decoder whose sublayers read the 32-bit residual itself and are normed on the way back:
x += ls1 * N1(mixer(x + conv(x))), x += ls2 * N2(ff(x)), N an RMS norm with weights stored around zero and ls a
learned vector per column.  The mixer ("attention") is grouped-query attention without rotation: an RMS norm over a
token's whole query (and key) projection, soft-capped scores that are mixed across heads by a learned table before
the softmax, a sliding window that keeps a sequence's first tokens visible, and a learned sink in the softmax's
denominator.  What the mixer reads first takes a short causal convolution over time.  The feed-forward is dense (up,
a two-sided activation with two learned numbers, down) or a mixture of gated experts chosen by their biased logits,
weighted by the softmax over the chosen logits, with a shared expert.  The embedded rows take a sinusoidal position
vector; the output head is the embedding table.

config.json: ``vocab``, ``width``, ``norm`` {``eps``}, ``canon`` {``taps``} and ``layers``, a list of
{``type`` "attention", ``mixer`` {``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``softcap``, ``mask``
{``size``, ``keep_first``}}, ``mlp`` {``kind`` "dense", ``ff``} or {``kind`` "moe", ``router`` {``experts``, ``top``},
``expert`` {``ff``}, ``shared`` {``ff``}} or null}.  Tensors: ``embed``, ``final.norm`` and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.ls1``, ``l<i>.ls2``, ``l<i>.canon1``, ``l<i>.mix.{q,k,v,o,q.norm,k.norm,talk,sink}``,
``l<i>.mlp.{up,down,act}`` or ``l<i>.mlp.{router,router.b,e<j>.{gate,up,down},shared.{gate,up,down}}``.

Constants the design fixes: the base 10000 of the position vector and the 1 that the norms' weights are stored around.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Tuple

from ..config.registry import ConfigError, ModelConfig, TensorNames, register_architecture
from ..config.specs import (ActMLPSpec, BranchNormSpec, CausalConvSpec, GatedMLPSpec, GroupedNormSpec, ModelSpec, MoESpec,
                            PostNormBlockSpec, SinusoidSpec, TalkingAttentionSpec)

POSITION_BASE = 10000.0    # column 2i of the position vector turns at 10000**(-2i / width)
NORM_OFFSET = 1.0          # a norm multiplies by 1 + w
MIXER_KEYS = {"attention": ("heads", "kv_heads", "dim", "vdim", "scale")}
COUNTS = ("heads", "kv_heads", "dim", "vdim")


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


@dataclass(frozen=True)
class GulazenConfig(ModelConfig):
    vocab: int
    width: int
    norm_eps: float
    taps: int                            # 0: nothing is convolved
    layers: Tuple[Any, ...]              # the layer entries as read (plain data)

    architecture = "Gulazen"

    @classmethod
    def from_dict(cls, raw: dict) -> "GulazenConfig":
        _need("the configuration", raw, ("vocab", "width", "norm", "layers"))
        _need("norm", raw["norm"], ("eps",))
        if not isinstance(raw["layers"], list) or not raw["layers"]:
            raise ConfigError("config.json: layers must be a list with at least one layer")
        taps = 0
        if raw.get("canon") is not None:
            _need("canon", raw["canon"], ("taps",))
            taps = _count("canon.taps", raw["canon"]["taps"])
        layers = []
        for i, entry in enumerate(raw["layers"]):
            _need(f"layers[{i}]", entry, ("type", "mixer"))
            kind = entry["type"]
            if kind not in MIXER_KEYS:
                raise ConfigError(f"config.json: layers[{i}].type {kind!r} is unknown; known: " + ", ".join(sorted(MIXER_KEYS)))
            m = entry["mixer"]
            _need(f"layers[{i}].mixer", m, MIXER_KEYS[kind])
            for key in COUNTS:
                _count(f"layers[{i}].mixer.{key}", m[key])
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: layers[{i}]: {m['heads']} heads cannot share {m['kv_heads']} kv_heads evenly")
            if m.get("softcap") is not None and not float(m["softcap"]) > 0:
                raise ConfigError(f"config.json: layers[{i}].mixer.softcap must be positive")
            if m.get("mask") is not None:
                _need(f"layers[{i}].mixer.mask", m["mask"], ("size",))
                _count(f"layers[{i}].mixer.mask.size", m["mask"]["size"])
                _count(f"layers[{i}].mixer.mask.keep_first", m["mask"].get("keep_first", 0), 0)
            mlp = entry.get("mlp")
            if mlp is not None:
                _need(f"layers[{i}].mlp", mlp, ("kind",))
                if mlp["kind"] == "dense":
                    _need(f"layers[{i}].mlp", mlp, ("ff",))
                    _count(f"layers[{i}].mlp.ff", mlp["ff"])
                elif mlp["kind"] == "moe":
                    _need(f"layers[{i}].mlp", mlp, ("router", "expert"))
                    _need(f"layers[{i}].mlp.router", mlp["router"], ("experts", "top"))
                    r = mlp["router"]
                    _count(f"layers[{i}].mlp.router.experts", r["experts"])
                    _count(f"layers[{i}].mlp.router.top", r["top"])
                    if r["top"] > r["experts"]:
                        raise ConfigError(f"config.json: layers[{i}].mlp.router chooses {r['top']} of {r['experts']}")
                    for part in ("expert", "shared"):
                        if mlp.get(part) is not None:
                            _need(f"layers[{i}].mlp.{part}", mlp[part], ("ff",))
                            _count(f"layers[{i}].mlp.{part}.ff", mlp[part]["ff"])
                else:
                    raise ConfigError(f"config.json: layers[{i}].mlp.kind {mlp['kind']!r} is not built: 'dense' and 'moe' are")
            layers.append(copy.deepcopy(entry))
        return cls(vocab=_count("vocab", raw["vocab"]), width=_count("width", raw["width"]), norm_eps=float(raw["norm"]["eps"]),
                   taps=taps, layers=tuple(layers))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": copy.deepcopy(list(self.layers)), "norm": {"eps": self.norm_eps},
               "vocab": self.vocab, "width": self.width}
        if self.taps:
            out["canon"] = {"taps": self.taps}
        return out

    # ---- layers -------------------------------------------------------------------------

    def _mixer_spec(self, i: int) -> TalkingAttentionSpec:
        m = self.layers[i]["mixer"]
        mask = m.get("mask")
        return TalkingAttentionSpec(hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                    v_dim=m["vdim"], scale=float(m["scale"]), qk_norm_eps=self.norm_eps,
                                    softcap=float(m["softcap"]) if m.get("softcap") is not None else None, talk=True, sink=True,
                                    window=int(mask["size"]) if mask is not None else None,
                                    keep_first=int(mask.get("keep_first", 0)) if mask is not None else 0)

    def _ff_spec(self, i: int):
        mlp = self.layers[i].get("mlp")
        if mlp is None:
            return None
        if mlp["kind"] == "dense":
            return ActMLPSpec(hidden_size=self.width, intermediate_size=int(mlp["ff"]), activation="xielu")

        def gated(part):
            return GatedMLPSpec(hidden_size=self.width, intermediate_size=int(part["ff"]), activation="silu")

        r = mlp["router"]
        return MoESpec(hidden_size=self.width, n_experts=int(r["experts"]), n_identity=0, top=int(r["top"]), route_scale=1.0,
                       expert=gated(mlp["expert"]), shared=gated(mlp["shared"]) if mlp.get("shared") is not None else None,
                       router_bias=True, correction=False, over_chosen=True)

    def model_spec(self) -> ModelSpec:
        norm = BranchNormSpec(size=self.width, eps=self.norm_eps, offset=NORM_OFFSET, layer_scale=True)
        conv = CausalConvSpec(size=self.width, taps=self.taps) if self.taps else None
        blocks = []
        for i in range(len(self.layers)):
            ff = self._ff_spec(i)
            blocks.append(PostNormBlockSpec(mixer=self._mixer_spec(i), mixer_norm=norm, conv=conv, ff=ff,
                                            ff_norm=norm if ff is not None else None))
        return ModelSpec(hidden_size=self.width, vocab_size=self.vocab, layers=tuple(blocks),
                         final_norm=GroupedNormSpec(size=self.width, eps=self.norm_eps, groups=1, offset=NORM_OFFSET),
                         tie_embeddings=True, residual_float32=True,
                         position_embedding=SinusoidSpec(size=self.width, base=POSITION_BASE))

    def tensor_names(self) -> TensorNames:
        layers = []
        for i, entry in enumerate(self.layers):
            p = f"l{i}."
            mixer = {"q": "q", "k": "k", "v": "v", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm", "talk": "talk", "sink": "sink"}
            names = {"mixer": {role: p + "mix." + n for role, n in mixer.items()},
                     "mixer_norm": {"weight": p + "norm1", "scale": p + "ls1"}}
            if self.taps:
                names["conv"] = {"weight": p + "canon1"}
            mlp = entry.get("mlp")
            if mlp is not None:
                if mlp["kind"] == "dense":
                    ff = {"up": "up", "down": "down", "act": "act"}
                else:
                    ff = {"router": "router", "router_bias": "router.b"}
                    for e in range(int(mlp["router"]["experts"])):
                        ff.update({f"e{e}_{r}": f"e{e}.{r}" for r in ("gate", "up", "down")})
                    if mlp.get("shared") is not None:
                        ff.update({"shared_" + r: "shared." + r for r in ("gate", "up", "down")})
                names["ff"] = {role: p + "mlp." + n for role, n in ff.items()}
                names["ff_norm"] = {"weight": p + "norm2", "scale": p + "ls2"}
            layers.append(names)
        return TensorNames(embedding="embed", lm_head="head", final_norm={"weight": "final.norm"}, layers=layers)

    def random_init(self, name: str, shape) -> Tuple[float, float]:
        """(mean, standard deviation) of a tensor's seeded random fill: matrices so that a product keeps its input's
        size, norm weights around zero, layer scales below one, a dense head table, a router that spreads."""
        last = name.rsplit(".", 1)[-1]
        if last == "talk":
            return 0.0, 0.35
        if last in ("ls1", "ls2"):
            return 0.5, 0.1
        if last in ("norm1", "norm2") or name == "final.norm":
            return 0.0, 0.1
        if name.endswith("q.norm") or name.endswith("k.norm"):
            return 1.0, 0.1
        if last == "sink":
            return 0.0, 1.0
        if last == "act":
            return 0.3, 0.5
        if last == "canon1":
            return 0.0, 0.3
        if last == "router":
            return 0.0, 2.0 * float(shape[-1]) ** -0.5
        if name.endswith("router.b"):
            return 0.0, 0.3
        if name == "embed":
            return 0.0, 1.0
        return 0.0, float(shape[-1]) ** -0.5


register_architecture(GulazenConfig.architecture, GulazenConfig)
