"""Typed configuration of the Bedarax decoder, read from its own config.json keys.

The design: token embedding followed by an RMS norm; pre-norm layers x += mixer(norm(x)),
x += ff(norm(x)) (the second half optional per layer); after every layer the stream that goes on is
a learned mix of the embedding output and all layers' results so far (a depth-weighted average).
Three kinds of mixer: attention without a rotation whose heads' scores are mixed before the
softmax, with a sliding window, values blended with those of the first such layer, and a gate per
head; a gated delta rule with one decay per head; and one with a decay per key channel and
low-rank decay and gate projections.  Two kinds of feed-forward: dense with the PolyNorm
activation, and routed experts with a softmax over the chosen.  Final norm and head.  Keys:

    architecture        "Bedarax"
    vocab, width        sizes; norm.eps: eps of every norm
    layers[i].type      "attention" | "delta" | "channel_delta"
    layers[i].mixer     attention: heads, kv_heads, dim, vdim, scale, mask {size} (absent: no
                        window), v_mix (true: values take part in the blend)
                        delta: heads, kv_heads, dim, vdim, conv
                        channel_delta: the same; the ranks of its low-rank pairs are the shapes of
                        the checkpoint's ``a1`` and ``g1`` (``a_rank``, ``g_rank`` may give them for
                        a model made from a configuration alone)
    layers[i].mlp       null, {kind: "dense", ff}, or {kind: "moe", expert {ff}, router {experts, top}}
    max_positions       optional bound on a sequence's length (default 2^20)

Tensor names: ``embed``, ``embed.norm``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.dwa``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, replace
from typing import Any, Mapping, Optional, Sequence, Tuple

from .base import ConfigError, ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule

ARCHITECTURE = "Bedarax"
MIXERS = ("attention", "delta", "channel_delta")
FEED_FORWARDS = ("dense", "moe")
DEFAULT_MAX_POSITIONS = 1 << 20
DEFAULT_RANK = 16


@dataclass(frozen=True)
class BedaraxLayer:
    type: str
    mixer: Mapping[str, Any]        # the mixer's object as config.json gives it (checked)
    mlp: Optional[Mapping[str, Any]]    # the feed-forward's object, or None
    # channel_delta: ranks of the decay's and the gate's projection pairs (None: not known yet)
    a_rank: Optional[int] = None
    g_rank: Optional[int] = None


@dataclass(frozen=True)
class BedaraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BedaraxLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "BedaraxConfig":
        r = ConfigReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            w = f"{where}.layers[{i}]"
            lr = ConfigReader(entry, w)
            kind = lr.string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{w}: unknown mixer type {kind!r} (known: {', '.join(MIXERS)})")
            mixer = entry.get("mixer")
            if not isinstance(mixer, Mapping):
                raise ConfigError(f"{w}: key 'mixer' must be an object")
            mlp = entry.get("mlp")
            if mlp is not None and not isinstance(mlp, Mapping):
                raise ConfigError(f"{w}: key 'mlp' must be an object or null")
            mr = ConfigReader(mixer, f"{w}.mixer")
            layers.append(BedaraxLayer(kind, dict(mixer), None if mlp is None else dict(mlp),
                                       mr.optional_integer("a_rank", minimum=1),
                                       mr.optional_integer("g_rank", minimum=1)))
        norm = data.get("norm") or {}
        cfg = cls(
            vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1),
            norm_eps=ConfigReader(norm, f"{where}.norm").number("eps", positive=True),
            layers=tuple(layers),
            max_positions=r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1),
            extra={k: v for k, v in data.items()},
        )
        cfg.plan()          # every key of every layer is read (and refused) here, not at the first step
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "BedaraxConfig":
        path = os.path.join(folder, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), where=path)

    def with_tensor_shapes(self, shapes: Mapping[str, Sequence[int]]) -> "BedaraxConfig":
        """The sizes that only a checkpoint's tensors give: the ranks of the low-rank pairs."""
        layers = []
        for i, layer in enumerate(self.layers):
            if layer.type == "channel_delta":
                a1, g1 = shapes.get(f"l{i}.mix.a1"), shapes.get(f"l{i}.mix.g1")
                layer = replace(layer,
                                a_rank=int(a1[0]) if a1 is not None and len(a1) == 2 else layer.a_rank,
                                g_rank=int(g1[0]) if g1 is not None and len(g1) == 2 else layer.g_rank)
            layers.append(layer)
        return replace(self, layers=tuple(layers))

    def to_dict(self) -> dict:
        layers = []
        for layer in self.layers:
            mixer = dict(layer.mixer)
            if layer.type == "channel_delta":
                mixer["a_rank"] = layer.a_rank or DEFAULT_RANK
                mixer["g_rank"] = layer.g_rank or DEFAULT_RANK
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.mlp is None else dict(layer.mlp)})
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "layers": layers}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ---- lowering to parts ----------------------------------------------------------
    def _mixer(self, i: int, layer: BedaraxLayer, first_value_layer: Optional[int]) -> PartSpec:
        w = f"config.layers[{i}].mixer"
        m = layer.mixer
        r = ConfigReader(m, w)
        heads = r.integer("heads", minimum=1)
        kv = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv != 0:
            raise ConfigError(f"{w}: heads {heads} is not a multiple of kv_heads {kv}")
        dim = r.integer("dim", minimum=1)
        vdim = r.integer("vdim", default=dim, minimum=1)
        if layer.type == "attention":
            window = 0
            if m.get("mask") is not None:
                window = ConfigReader(m["mask"], f"{w}.mask").integer("size", minimum=1)
            mix = "none"
            if r.boolean("v_mix", default=False):
                mix = "source" if first_value_layer == i else "blend"
            return PartSpec("talking_attention", dict(
                hidden_size=self.width, n_heads=heads, n_kv_heads=kv, head_dim=dim, value_dim=vdim,
                scale=r.number("scale"), window=window, talk=True, gate=True, value_mix=mix,
                tensor_prefix="mix."))
        channel = layer.type == "channel_delta"
        return PartSpec("gated_delta_rule", dict(
            hidden_size=self.width, n_heads=heads, n_kv_heads=kv, key_dim=dim, value_dim=vdim,
            conv=r.integer("conv", minimum=1), norm_eps=self.norm_eps,
            decay="channel" if channel else "head", gate="sigmoid" if channel else "silu",
            decay_rank=(layer.a_rank or DEFAULT_RANK) if channel else 0,
            gate_rank=(layer.g_rank or DEFAULT_RANK) if channel else 0, tensor_prefix="mix."))

    def _feed_forward(self, i: int, layer: BedaraxLayer) -> Optional[PartSpec]:
        if layer.mlp is None:
            return None
        w = f"config.layers[{i}].mlp"
        r = ConfigReader(layer.mlp, w)
        kind = r.string("kind")
        if kind not in FEED_FORWARDS:
            raise ConfigError(f"{w}: unknown kind {kind!r} (known: {', '.join(FEED_FORWARDS)})")
        if kind == "dense":
            return PartSpec("dense_mlp", {
                "hidden_size": self.width, "intermediate_size": r.integer("ff", minimum=1),
                "activation": "poly_norm", "norm_eps": self.norm_eps, "up_name": "mlp.up",
                "down_name": "mlp.down", "act_name": "mlp.act"})
        if not isinstance(layer.mlp.get("expert"), Mapping) or not isinstance(
                layer.mlp.get("router"), Mapping):
            raise ConfigError(f"{w}: a routed feed-forward needs the objects 'expert' and 'router'")
        router = ConfigReader(layer.mlp["router"], f"{w}.router")
        experts = router.integer("experts", minimum=1)
        top = router.integer("top", minimum=1)
        if top > experts:
            raise ConfigError(f"{w}.router: top {top} is more than the {experts} experts")
        return PartSpec("routed_experts", {
            "hidden_size": self.width,
            "intermediate_size": ConfigReader(layer.mlp["expert"], f"{w}.expert").integer("ff", minimum=1),
            "n_experts": experts, "top": top, "activation": "silu", "router_name": "mlp.router",
            "router_bias_name": "mlp.router.b", "expert_name": "mlp.e{e}"})

    def plan(self) -> ModelPlan:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps})
        # the first layer whose values take part in the blend gives them; later ones blend
        first_value_layer, value_width = None, None
        for i, layer in enumerate(self.layers):
            if layer.type == "attention" and layer.mixer.get("v_mix") is True:
                m = layer.mixer
                heads = m.get("heads")
                width = (m.get("kv_heads", heads), m.get("vdim", m.get("dim")))
                if first_value_layer is None:
                    first_value_layer, value_width = i, width
                elif width != value_width:
                    raise ConfigError(
                        f"config.layers[{i}].mixer: values of {width[0]} heads x {width[1]} cannot "
                        f"be blended with layer {first_value_layer}'s {value_width[0]} x {value_width[1]}")
        layers = []
        for i, layer in enumerate(self.layers):
            ffn = self._feed_forward(i, layer)
            layers.append(LayerSpec(
                prefix=f"l{i}.",
                block=PartSpec("pre_norm", {}),
                mixer=self._mixer(i, layer, first_value_layer),
                mixer_norm=norm.with_params(name="norm1", tensor_name="norm1"),
                feed_forward=ffn,
                feed_forward_norm=(norm.with_params(name="norm2", tensor_name="norm2")
                                   if ffn is not None else None),
            ))
        plan = ModelPlan(
            architecture=ARCHITECTURE,
            vocab_size=self.vocab,
            hidden_size=self.width,
            embedding_name="embed",
            head_name="head",
            final_norm=norm.with_params(name="final.norm", tensor_name="final.norm"),
            final_norm_prefix="",
            layers=layers,
            schedule=default_schedule(len(layers)),
            max_positions=self.max_positions,
            after_embedding=PartSpec("embedding_norm", {
                "width": self.width, "eps": self.norm_eps, "tensor_name": "embed.norm"}),
            after_layer=PartSpec("depth_average", {
                "width": self.width, "names": [f"l{i}.dwa" for i in range(len(layers))]}),
            model_part_prefix="",
            # a layer without a feed-forward has no use for a second norm, nor a layer outside the
            # blend of values for its weight
            ignorable_tensors=tuple(
                [f"l{i}.norm2" for i, layer in enumerate(self.layers) if layer.mlp is None] +
                [f"l{i}.mix.vmix" for i, layer in enumerate(self.layers)
                 if layer.type == "attention" and layer.mixer.get("v_mix") is not True]),
        )
        plan.validate()
        return plan
