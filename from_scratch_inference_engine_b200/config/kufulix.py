"""Typed configuration of the Kufulix decoder, read from its own config.json keys.

A Kufulix model is a list of pre-norm layers (x += mixer(N(x)); x += ff(N(x)), N an RMS norm whose
stored weight lies around zero: gain 1 + w) behind an embedding that passes through such a norm
itself, with capped logits; a layer may run another layer's tensors on a cache and state of its own:

    {"architecture": "Kufulix", "vocab": V, "width": W, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "parallel" | "attention", "mixer": {...}, "mlp": {...} | null,
                 "weights_of": j (optional)}, ...]}

    attention  heads, kv_heads, dim, vdim, scale, mask {size},
               rot {base, dims, scaling {factor, low, high, original} | null}
               (grouped-query attention with biases, keys visible inside the query's chunk of
               `mask.size` positions only, a sigmoid gate per head on the output)
    parallel   left {the keys of attention: here `mask.size` is a sliding window, and q and k are
               RMS-normed per head}, right {heads, vdim, state, groups, conv, norm_groups}
               (a state-space mixer), left_scale, right_scale
    mlp        kind "moe", expert {ff}, router {experts, top, identity, groups {count, keep} | null}

Nothing here is fixed to one model: every size, the order of the layers and every constant come
from the file; the tensor names ('embed', 'embed.norm', 'head', 'final.norm', 'l<i>.norm1',
'l<i>.mix.q', 'l<i>.mix.left.q.norm', 'l<i>.mix.right.in', 'l<i>.mlp.e<j>.up', 'l<i>.mlp.router', ...)
are the design's.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Mapping, Optional

from .metulix import _integer
from .qwen2 import ConfigError
from .spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from .zadepel import _number

MIXERS = ("parallel", "attention")


def _check_attention(where: str, mixer: Mapping[str, Any]) -> None:
    heads = _integer(where, mixer, "heads")
    kv_heads = _integer(where, mixer, "kv_heads") if "kv_heads" in mixer else heads
    if heads % kv_heads:
        raise ConfigError(f"config.json: {where}.heads must be a multiple of kv_heads")
    dim = _integer(where, mixer, "dim")
    if "vdim" in mixer:
        _integer(where, mixer, "vdim")
    _number(where, mixer, "scale")
    mask = mixer.get("mask")
    if mask is not None:            # absent or null: every earlier position is seen
        if not isinstance(mask, Mapping):
            raise ConfigError(f"config.json: {where}.mask must be an object with 'size', or null")
        _integer(where + ".mask", mask, "size")
    rot = mixer.get("rot")
    if rot is None:
        return
    if not isinstance(rot, Mapping):
        raise ConfigError(f"config.json: {where}.rot must be an object with 'base' and 'dims', or null")
    dims = _integer(where + ".rot", rot, "dims", least=0)
    if dims % 2 or dims > dim:
        raise ConfigError(f"config.json: {where}.rot.dims must be even and at most dim ({dim})")
    if dims and _number(where + ".rot", rot, "base") <= 1:
        raise ConfigError(f"config.json: {where}.rot.base must exceed 1")
    scaling = rot.get("scaling")
    if scaling is None:
        return
    if not isinstance(scaling, Mapping):
        raise ConfigError(f"config.json: {where}.rot.scaling must be an object or null")
    for key in ("factor", "low", "high", "original"):
        if _number(where + ".rot.scaling", scaling, key) <= 0:
            raise ConfigError(f"config.json: {where}.rot.scaling.{key} must be positive")


def _check_state_space(where: str, mixer: Mapping[str, Any]) -> None:
    heads = _integer(where, mixer, "heads")
    vdim = _integer(where, mixer, "vdim")
    _integer(where, mixer, "state")
    groups = _integer(where, mixer, "groups") if "groups" in mixer else 1
    _integer(where, mixer, "conv")
    parts = _integer(where, mixer, "norm_groups") if "norm_groups" in mixer else 1
    if heads % groups:
        raise ConfigError(f"config.json: {where}.heads must be a multiple of groups")
    if (heads * vdim) % parts:
        raise ConfigError(f"config.json: {where}: heads * vdim must divide into norm_groups equal parts")


def _check_mlp(where: str, mlp: Any) -> None:
    if not isinstance(mlp, Mapping) or mlp.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}.kind must be 'moe'")
    expert, router = mlp.get("expert"), mlp.get("router")
    if not isinstance(expert, Mapping) or not isinstance(router, Mapping):
        raise ConfigError(f"config.json: {where} needs 'expert' and 'router' objects")
    _integer(where + ".expert", expert, "ff")
    experts = _integer(where + ".router", router, "experts")
    top = _integer(where + ".router", router, "top")
    identity = _integer(where + ".router", router, "identity", least=0) if "identity" in router else 0
    routed = experts + identity
    if top > routed:
        raise ConfigError(f"config.json: {where}.router.top exceeds the number of experts")
    groups = router.get("groups")
    if groups is not None:
        if not isinstance(groups, Mapping):
            raise ConfigError(f"config.json: {where}.router.groups must be an object or null")
        count = _integer(where + ".router.groups", groups, "count")
        keep = _integer(where + ".router.groups", groups, "keep")
        if routed % count or keep > count or top > keep * (routed // count):
            raise ConfigError(f"config.json: {where}.router.groups: {routed} experts (identity ones "
                              f"included) must divide into {count} groups of which the {keep} kept "
                              f"hold at least top = {top}")


@dataclass(frozen=True)
class KufulixConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple                      # the layer entries as read (dicts), checked
    logit_softcap: float = 0.0
    eos_token_id: Optional[int] = None

    architecture = "Kufulix"

    # ------------------------------------------------------------------ reading
    @classmethod
    def from_dict(cls, data: Mapping[str, Any]) -> "KufulixConfig":
        vocab = _integer("the model", data, "vocab")
        width = _integer("the model", data, "width")
        norm = data.get("norm")
        if not isinstance(norm, Mapping) or "eps" not in norm:
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        layers = data.get("layers")
        if not isinstance(layers, (list, tuple)) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        softcap = _number("the model", data, "logit_softcap") if data.get("logit_softcap") is not None else 0.0
        eos = data.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        config = cls(vocab, width, _number("norm", norm, "eps"), tuple(copy.deepcopy(list(layers))),
                     softcap, None if eos is None else int(eos))
        config.validate()
        return config

    def to_dict(self) -> Dict[str, Any]:
        data: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab,
                                "width": self.width, "norm": {"eps": self.eps},
                                "logit_softcap": self.logit_softcap,
                                "layers": copy.deepcopy(list(self.layers))}
        if self.eos_token_id is not None:
            data["eos_token_id"] = self.eos_token_id
        return data

    # --------------------------------------------------------------- validation
    def source_of(self, index: int) -> int:
        """The layer whose tensors layer `index` runs (itself unless it names another)."""
        source = self.layers[index].get("weights_of")
        return index if source is None else int(source)      # (validate: that layer has its own)

    def validate(self) -> None:
        if self.eps < 0:
            raise ConfigError("config.json: norm.eps must not be negative")
        if self.logit_softcap < 0:
            raise ConfigError("config.json: logit_softcap must not be negative")
        for index, layer in enumerate(self.layers):
            where = f"layers[{index}]"
            if not isinstance(layer, Mapping) or not isinstance(layer.get("mixer"), Mapping):
                raise ConfigError(f"config.json: {where} must be an object with a 'mixer'")
            kind, mixer = layer.get("type"), layer["mixer"]
            if kind not in MIXERS:
                raise ConfigError(f"config.json: {where}.type '{kind}' is not a mixer of this design "
                                  f"({', '.join(MIXERS)})")
            if kind == "attention":
                _check_attention(where + ".mixer", mixer)
            else:
                for side, check in (("left", _check_attention), ("right", _check_state_space)):
                    if not isinstance(mixer.get(side), Mapping):
                        raise ConfigError(f"config.json: {where}.mixer.{side} must be an object")
                    check(f"{where}.mixer.{side}", mixer[side])
                for key in ("left_scale", "right_scale"):        # absent: 1
                    if key in mixer:
                        _number(where + ".mixer", mixer, key)
            if layer.get("mlp") is not None:
                _check_mlp(where + ".mlp", layer["mlp"])
            source = layer.get("weights_of")
            if source is None:
                continue
            if isinstance(source, bool) or not isinstance(source, int) or not 0 <= source < len(self.layers) \
                    or source == index:
                raise ConfigError(f"config.json: {where}.weights_of must name another layer")
            other = self.layers[source]
            if isinstance(other, Mapping) and other.get("weights_of") is not None:
                raise ConfigError(f"config.json: {where}.weights_of names layer {source}, which has no "
                                  f"tensors of its own")
            mine = {k: v for k, v in layer.items() if k != "weights_of"}
            theirs = {k: v for k, v in other.items() if k != "weights_of"} if isinstance(other, Mapping) else None
            if mine != theirs:
                raise ConfigError(f"config.json: {where} runs the tensors of layer {source} but "
                                  f"describes another layer")

    # --------------------------------------------------------------------- spec
    def _position(self, rot: Optional[Mapping[str, Any]]) -> PartSpec:
        if not rot or not int(rot["dims"]):
            return PartSpec("none", {})
        common = {"theta": float(rot["base"]), "rotary_dim": int(rot["dims"]), "max_position": 0,
                  "pairing": "half"}
        scaling = rot.get("scaling")
        if not scaling:
            return PartSpec("rotary", common)
        return PartSpec("llama3_rotary", dict(
            common, factor=float(scaling["factor"]), original=float(scaling["original"]),
            low=float(scaling["low"]), high=float(scaling["high"])))

    def _attention(self, mixer: Mapping[str, Any], windowed: bool) -> PartSpec:
        """`windowed`: the mask is a sliding window and q and k are normed per head (the left
        mixer of a parallel layer); else the mask is a chunk and the heads' outputs are gated."""
        size = int(mixer["mask"]["size"]) if mixer.get("mask") else 0
        return PartSpec("scaled_gqa_attention", {
            "hidden_size": self.width, "heads": int(mixer["heads"]),
            "kv_heads": int(mixer.get("kv_heads", mixer["heads"])),
            "dim": int(mixer["dim"]), "vdim": int(mixer.get("vdim", mixer["dim"])), "scale": float(mixer["scale"]),
            "position": self._position(mixer.get("rot")), "temperature": False, "value_mix": "none",
            "window": size if windowed else 0, "chunk": 0 if windowed else size,
            "qk_norm": windowed, "eps": self.eps, "head_gate": not windowed})

    def _state_space(self, mixer: Mapping[str, Any]) -> PartSpec:
        return PartSpec("state_space_duality", {
            "hidden_size": self.width, "heads": int(mixer["heads"]), "vdim": int(mixer["vdim"]),
            "state": int(mixer["state"]), "groups": int(mixer.get("groups", 1)), "taps": int(mixer["conv"]),
            "norm_groups": int(mixer.get("norm_groups", 1)), "eps": self.eps})

    def _mixer(self, kind: str, mixer: Mapping[str, Any]) -> PartSpec:
        if kind == "attention":
            return self._attention(mixer, windowed=False)
        return PartSpec("parallel_mixers", {
            "left": self._attention(mixer["left"], windowed=True),
            "right": self._state_space(mixer["right"]),
            "left_scale": float(mixer.get("left_scale", 1.0)),
            "right_scale": float(mixer.get("right_scale", 1.0))})

    def _feed_forward(self, mlp: Optional[Mapping[str, Any]]) -> Optional[PartSpec]:
        if mlp is None:
            return None
        router = mlp["router"]
        groups = router.get("groups") or {"count": 1, "keep": 1}
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": int(mlp["expert"]["ff"]),
            "experts": int(router["experts"]), "top": int(router["top"]),
            "identity": int(router.get("identity", 0)),
            "groups": int(groups["count"]), "keep": int(groups["keep"]), "group_score": "max",
            "scale": 1.0, "scores": "softmax", "normalise": True, "correction": True,
            "gated": False, "activation": "relu2", "shared": None})

    def build_spec(self) -> ModelSpec:
        """Lay the configuration out as parts: every layer is a `prenorm` arrangement of RMS norms
        with gain 1 + w, its mixer `scaled_gqa_attention` (chunked, gated heads) or
        `parallel_mixers` of a windowed `scaled_gqa_attention` with normed q and k beside a
        `state_space_duality`, its feed-forward `routed_experts` without gates and with identity
        experts, or none.  Only layers with tensors of their own become layers of the model; a
        layer that runs another's tensors is a second call of that layer in the run order, with
        its own cache entry and state."""
        def norm(name: str) -> PartSpec:
            return PartSpec("rmsnorm", {"width": self.width, "eps": self.eps, "weight_name": name,
                                        "one_plus": True})
        layers: List[LayerSpec] = []
        own: Dict[int, int] = {}           # layer of the configuration -> layer of the model
        for index, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            own[index] = len(layers)
            feed_forward = self._feed_forward(layer.get("mlp"))
            layers.append(LayerSpec(
                prefix=f"l{index}.", arrangement="prenorm",
                mixer=self._mixer(layer["type"], layer["mixer"]), feed_forward=feed_forward,
                mixer_norm=norm("norm1"), feed_forward_norm=norm("norm2"),
                mixer_name="mix.", feed_forward_name="mlp.", mixer_norm_name="",
                feed_forward_norm_name=""))
        schedule = [LayerCall(layer=own[self.source_of(index)]) for index in range(len(self.layers))]
        return ModelSpec(
            architecture=self.architecture, hidden_size=self.width, vocab_size=self.vocab,
            max_position=0, embedding_name="embed", head_name="head", final_norm=norm("norm"),
            final_norm_prefix="final.", layers=tuple(layers), schedule=tuple(schedule),
            logit_softcap=self.logit_softcap, embedding_norm=norm("norm"),
            embedding_norm_prefix="embed.")
