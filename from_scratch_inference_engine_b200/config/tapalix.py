"""Typed configuration of the Tapalix decoder, read from its own config.json keys.

A Tapalix model is a list of layers in which ONE layer norm (gain and bias) feeds both the mixer and
the feed-forward of a layer (x += mixer(h) + ff(h), h = norm(x)); a stretch of the layers may run
several times in a row with the same weights, each pass with its own cache, entered through a
product over [x; embedding output]; the embedding is scaled, the logits are scaled and capped:

    {"architecture": "Tapalix", "vocab": V, "width": W, "norm": {"eps": e},
     "embedding": {"scale": s}, "logit_scale": a, "logit_softcap": c,
     "loop": {"start": i, "stop": j, "times": n} | null,
     "layers": [{"type": "latent_attention" | "latent_attention_2", "mixer": {...},
                 "mlp": {...} | null}, ...]}

    latent_attention    heads, dim, rot_dim, vdim, kv_rank, scale,
                        rot {base, dims, scaling {factor, original, fast, slow} | null}
    latent_attention_2  heads, dim, vdim, kv_rank, scale      (no positions; a sigmoid gate on the heads)
    mlp                 kind "moe", expert {ff}, router {experts, top, scale, groups {count, keep}},
                        shared {ff} | null

Nothing here is fixed to one model: every size, the order of the layers and every constant come
from the file; the tensor names ('embed', 'head', 'loop.in', 'final.norm', 'final.norm.b',
'l<i>.norm1', 'l<i>.norm1.b', 'l<i>.mix.q', 'l<i>.mlp.e<j>.gate', 'l<i>.mlp.router', ...) are the
design's.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional

from .metulix import _integer
from .qwen2 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .zadepel import _number

MIXERS = ("latent_attention", "latent_attention_2")


def _scaling(where: str, rot: Mapping[str, Any]) -> Optional[Mapping[str, Any]]:
    scaling = rot.get("scaling")
    if scaling is None:
        return None
    if not isinstance(scaling, Mapping):
        raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
    for key in ("factor", "original", "fast", "slow"):
        if _number(where + ".rot.scaling", scaling, key) <= 0:
            raise ConfigError(f"config.json: {where}.rot.scaling.{key} must be positive")
    return scaling


@dataclass(frozen=True)
class TapalixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                      # the layer entries as read (dicts), checked
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: float = 0.0
    loop: Optional[tuple] = None       # (start, stop, times)
    eos_token_id: Optional[int] = None

    architecture = "Tapalix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "TapalixConfig":
        vocab = _integer("the model", data, "vocab")
        width = _integer("the model", data, "width")
        norm = data.get("norm")
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        embedding = data.get("embedding")
        if embedding is not None and not isinstance(embedding, Mapping):
            raise ConfigError("config.json: 'embedding' must be an object")
        scale = _number("embedding", embedding, "scale") if embedding and "scale" in embedding else 1.0
        logit_scale = _number("the model", data, "logit_scale") if data.get("logit_scale") is not None else 1.0
        softcap = _number("the model", data, "logit_softcap") if data.get("logit_softcap") is not None else 0.0
        loop = data.get("loop")
        if loop is not None:
            if not isinstance(loop, Mapping):
                raise ConfigError("config.json: 'loop' must be an object or null")
            loop = (_integer("loop", loop, "start", least=0), _integer("loop", loop, "stop", least=0),
                    _integer("loop", loop, "times", least=1))
        eos = data.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        config = cls(vocab, width, _number("norm", norm, "eps"), tuple(copy.deepcopy(list(layers))),
                     scale, logit_scale, softcap, loop, None if eos is None else int(eos))
        config.validate()
        return config

    def to_dict(self) -> Dict[str, Any]:
        data: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                                "width": self.width, "norm": {"eps": self.eps},
                                "embedding": {"scale": self.embedding_scale},
                                "logit_scale": self.logit_scale, "logit_softcap": self.logit_softcap,
                                "loop": None if self.loop is None else
                                {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]},
                                "layers": copy.deepcopy(list(self.layers))}
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # --------------------------------------------------------------- validation
    def validate(self) -> None:
        if self.eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if self.logit_softcap < 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        if self.loop is not None:
            start, stop, _ = self.loop
            if not start < stop <= len(self.layers):
                raise ConfigError(f"config.json: loop must name layers start < stop <= {len(self.layers)}, "
                                  f"got start {start}, stop {stop}")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, Mapping) or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with a 'mixer'")
            kind, mixer = layer.get("type"), layer["mixer"]
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design "
                                  f"({', '.join(MIXERS)})")
            where += ".mixer"
            for key in ("heads", "dim", "vdim", "kv_rank"):
                _integer(where, mixer, key)
            _number(where, mixer, "scale")
            if kind == "latent_attention":
                rope = _integer(where, mixer, "rot_dim", least=0)
                rot = mixer.get("rot")
                if rope and not isinstance(rot, Mapping):
                    raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims'")
                if rope:
                    if _number(where + ".rot", rot, "base") <= 1:
                        raise ConfigError(f"config.json: {where}.rot.base must exceed 1")
                    dims = _integer(where + ".rot", rot, "dims", least=0)
                    if dims % 2 or dims > rope:
                        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most "
                                          f"rot_dim ({rope})")
                    _scaling(where, rot)
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            where = f"layers[{index}].mlp"
            if not isinstance(mlp, Mapping) or mlp.get("kind") not in ("moe", "dense"):
                raise ConfigError(f"config.json: {where}.kind must be 'moe' or 'dense'")
            if mlp["kind"] == "dense":
                _integer(where, mlp, "ff")
                continue
            expert, router = mlp.get("expert"), mlp.get("router")
            if not isinstance(expert, Mapping) or not isinstance(router, Mapping):
                raise ConfigError(f"config.json: {where} needs 'expert' and 'router' objects")
            _integer(where + ".expert", expert, "ff")
            experts = _integer(where + ".router", router, "experts")
            top = _integer(where + ".router", router, "top")
            if top > experts:
                raise ConfigError(f"config.json: {where}.router.top exceeds the number of experts")
            if "scale" in router:
                _number(where + ".router", router, "scale")
            groups = router.get("groups")
            if groups is not None:
                if not isinstance(groups, Mapping):
                    raise ConfigError(f"config.json: {where}.router.groups must be an object or null")
                count = _integer(where + ".router.groups", groups, "count")
                keep = _integer(where + ".router.groups", groups, "keep")
                if experts % count or keep > count or top > keep * (experts // count):
                    raise ConfigError(f"config.json: {where}.router.groups: {experts} experts must divide "
                                      f"into {count} groups of which the {keep} kept hold at least "
                                      f"top = {top} experts")
            shared = mlp.get("shared")
            if shared is not None:
                if not isinstance(shared, Mapping):
                    raise ConfigError(f"config.json: {where}.shared must be an object or null")
                _integer(where + ".shared", shared, "ff")

    # --------------------------------------------------------------------- spec
    def _mixer(self, kind: str, mixer: Mapping[str, Any]) -> PartSpec:
        params = {"hidden_size": self.width, "heads": int(mixer["heads"]), "dim": int(mixer["dim"]),
                  "vdim": int(mixer["vdim"]), "rank": int(mixer["kv_rank"]),
                  "scale": float(mixer["scale"]), "eps": self.eps, "window": 0}
        rope = int(mixer.get("rot_dim", 0)) if kind == "latent_attention" else 0
        if rope:
            rot = mixer["rot"]
            common = {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "max_position": 0,
                      "pairing": "half"}
            scaling = rot.get("scaling")
            if scaling:
                position = PartSpec("yarn_rotary", dict(
                    common, factor=float(scaling["factor"]), original=float(scaling["original"]),
                    fast=float(scaling["fast"]), slow=float(scaling["slow"])))
            else:
                position = PartSpec("rotary", common)
        else:
            position = PartSpec("none", {})
        params.update(rope_dim=rope, position=position, gate=kind == "latent_attention_2")
        return PartSpec("latent_attention", params)

    def _feed_forward(self, mlp: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        plain = {"gate": "gate", "up": "up", "down": "down", "weight": "", "bias": ".b"}
        if mlp["kind"] == "dense":
            return PartSpec("gated_mlp", {"hidden_size": self.width, "intermediate_size": int(mlp["ff"]),
                                          "activation": "silu", "names": plain})
        router = mlp["router"]
        groups = router.get("groups") or {"count": 1, "keep": 1}
        shared = mlp.get("shared")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": int(mlp["expert"]["ff"]),
            "experts": int(router["experts"]), "top": int(router["top"]),
            "groups": int(groups["count"]), "keep": int(groups["keep"]),
            "scale": float(router.get("scale", 1.0)), "scores": "sigmoid", "normalise": True,
            "correction": True, "activation": "silu",
            "shared": None if shared is None else PartSpec("gated_mlp", {
                "hidden_size": self.width, "intermediate_size": int(shared["ff"]),
                "activation": "silu", "names": plain})})

    def build_spec(self) -> ModelSpec:
        """Lay the configuration out as parts: every layer is a `parallel` arrangement (one layer
        norm with gain and bias for both sublayers), its mixer a `latent_attention` (rotated pairs
        half a rotation apart with YaRN scaling; or without positions and with a sigmoid gate),
        its feed-forward `routed_experts` with a shared `gated_mlp`, or none.  The looped stretch
        appears in the run order once per pass, every call with a cache entry of its own, and the
        first call of each pass is entered through the `concat_embedding` inlet."""
        norm = PartSpec("layernorm", {"width": self.width, "eps": self.eps, "weight_name": "",
                                      "bias_name": ".b"})
        layers: List[LayerSpec] = []
        for index, layer in enumerate(self.layers):
            layers.append(LayerSpec(
                prefix=f"l{index}.", arrangement="parallel",
                mixer=self._mixer(layer["type"], layer["mixer"]),
                feed_forward=self._feed_forward(layer.get("mlp")),
                mixer_norm=norm, feed_forward_norm=None,
                mixer_name="mix.", feed_forward_name="mlp.", mixer_norm_name="norm1"))
        count = len(layers)
        inlets = ()
        if self.loop is None:
            schedule = [LayerCall(layer=i) for i in range(count)]
        else:
            start, stop, times = self.loop
            inlets = ((PartSpec("concat_embedding", {"hidden_size": self.width, "weight_name": "in"}),
                       "loop."),)
            schedule = [LayerCall(layer=i) for i in range(start)]
            for _ in range(times):
                schedule += [LayerCall(layer=i, inlet=0 if i == start else None)
                             for i in range(start, stop)]
            schedule += [LayerCall(layer=i) for i in range(stop, count)]
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_position=0, embedding_name="embed", head_name="head", final_norm=norm,
            final_norm_prefix="final.norm", layers=tuple(layers), schedule=tuple(schedule),
            embedding_scale=self.embedding_scale, logit_scale=self.logit_scale,
            logit_softcap=self.logit_softcap, inlets=inlets)
