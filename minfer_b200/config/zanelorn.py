"""Typed configuration of the Zanelorn decoder, read from its own config.json keys.

The design: token embedding times a constant; layers whose norms sit on the sublayers' outputs,
x += m norm(mixer(x)), x += m norm(ff(x)) (the second half optional), each followed by a per-layer
input looked up by token id; the mixer is retention (linear attention with a fixed decay per head,
rotated q and k, per-sequence state) or two mixers side by side, grouped attention (biases, q and k
normed per head, a linearly scaled partial rotation, a sliding window that keeps the first tokens,
an output gate) plus a selective scan, their outputs scaled and added; the feed-forward is dense
(erf gelu) or routed (softmax scores over all experts, a correction on the choice, experts without
weights that hand their input on, a clamped activation, a gated shared expert).  Final norm, head.
config.json keys:

    architecture        "Zanelorn"
    vocab, width        sizes; norm.eps: eps of every norm; residual_mult: m; embedding.scale
    token_side.dim      width of the per-layer token input (absent or null: none)
    layers[i].type      "retention" | "parallel"
    layers[i].mixer     retention: heads, dim, vdim, decay [heads], rot {base, dims}
                        parallel: left {heads, kv_heads, dim, vdim, scale, mask {size, keep_first},
                        rot {base, dims, scaling {factor}}}, right {inner, state, dt_rank, conv},
                        left_scale, right_scale
    layers[i].mlp       null, {kind: "dense", ff} or {kind: "moe", expert {ff, limit},
                        router {experts, identity, top}, shared {ff, limit} or null}
    max_positions       optional bound on a sequence's length (default 2^20)

Tensor names: ``embed``, ``side.embed``, ``final.norm``, ``head``, and per layer ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.side.{gate,proj,norm}``.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Any, Mapping, Optional, Tuple

from .base import ConfigError, ConfigReader, LayerSpec, ModelPlan, PartSpec, default_schedule

ARCHITECTURE = "Zanelorn"
MIXERS = ("retention", "parallel")
FEED_FORWARDS = ("dense", "moe")
DEFAULT_MAX_POSITIONS = 1 << 20


def _rotation(data: Optional[Mapping[str, Any]], where: str, head_width: int) -> Optional[PartSpec]:
    """The ``rot`` object of a mixer as a rotary part (None: no rotation); ``scaling.factor``
    divides every frequency."""
    if data is None:
        return None
    r = ConfigReader(data, where)
    dims = r.integer("dims", minimum=0)
    if dims == 0:
        return None
    if dims % 2 != 0 or dims > head_width:
        raise ConfigError(f"{where}: dims {dims} must be even and at most {head_width}")
    divide = 1.0
    if data.get("scaling") is not None:
        divide = ConfigReader(data["scaling"], f"{where}.scaling").number("factor", positive=True)
    return PartSpec("rotary", {"head_dim": head_width, "rotary_dim": dims,
                               "theta": r.number("base", positive=True),
                               "frequency_scale": 1.0 / divide, "style": "neox"})


@dataclass(frozen=True)
class ZanelornLayer:
    type: str
    mixer: Mapping[str, Any]        # the mixer's object as config.json gives it (checked)
    mlp: Optional[Mapping[str, Any]]


@dataclass(frozen=True)
class ZanelornConfig:
    vocab: int
    width: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    side_dim: int                   # 0: no per-layer token input
    layers: Tuple[ZanelornLayer, ...]
    max_positions: int = DEFAULT_MAX_POSITIONS
    extra: Mapping[str, Any] = field(default_factory=dict, compare=False)

    @classmethod
    def from_dict(cls, data: Mapping[str, Any], where: str = "config.json") -> "ZanelornConfig":
        r = ConfigReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(raw_layers):
            w = f"{where}.layers[{i}]"
            kind = ConfigReader(entry, w).string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{w}: unknown mixer type {kind!r} (known: {', '.join(MIXERS)})")
            if not isinstance(entry.get("mixer"), Mapping):
                raise ConfigError(f"{w}: key 'mixer' must be an object")
            mlp = entry.get("mlp")
            if mlp is not None:
                mlp_kind = ConfigReader(mlp, f"{w}.mlp").string("kind")
                if mlp_kind not in FEED_FORWARDS:
                    raise ConfigError(f"{w}.mlp: unknown kind {mlp_kind!r} "
                                      f"(known: {', '.join(FEED_FORWARDS)})")
            layers.append(ZanelornLayer(kind, dict(entry["mixer"]), None if mlp is None else dict(mlp)))
        side = data.get("token_side")
        cfg = cls(
            vocab=r.integer("vocab", minimum=1),
            width=r.integer("width", minimum=1),
            norm_eps=ConfigReader(data.get("norm") or {}, f"{where}.norm").number("eps", positive=True),
            residual_mult=r.number("residual_mult", default=1.0),
            embedding_scale=ConfigReader(data.get("embedding") or {}, f"{where}.embedding").number(
                "scale", default=1.0),
            side_dim=0 if side is None else ConfigReader(side, f"{where}.token_side").integer("dim", minimum=1),
            layers=tuple(layers),
            max_positions=r.integer("max_positions", default=DEFAULT_MAX_POSITIONS, minimum=1),
            extra={k: v for k, v in data.items()},
        )
        cfg.plan()          # every mixer's keys are read (and refused) here, not at the first step
        return cfg

    @classmethod
    def from_folder(cls, folder: str) -> "ZanelornConfig":
        path = os.path.join(folder, "config.json")
        with open(path, "r", encoding="utf-8") as f:
            return cls.from_dict(json.load(f), where=path)

    def to_dict(self) -> dict:
        out = {"architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
               "embedding": {"scale": self.embedding_scale},
               "layers": [{"type": layer.type, "mixer": dict(layer.mixer),
                           "mlp": None if layer.mlp is None else dict(layer.mlp)}
                          for layer in self.layers]}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            out["max_positions"] = self.max_positions
        return out

    # ---- lowering to parts ----------------------------------------------------------
    def _attention(self, m: Mapping[str, Any], w: str) -> PartSpec:
        r = ConfigReader(m, w)
        heads = r.integer("heads", minimum=1)
        kv = r.integer("kv_heads", default=heads, minimum=1)
        if heads % kv != 0:
            raise ConfigError(f"{w}: heads {heads} is not a multiple of kv_heads {kv}")
        dim = r.integer("dim", minimum=1)
        window = keep = 0
        if m.get("mask") is not None:
            mr = ConfigReader(m["mask"], f"{w}.mask")
            window = mr.integer("size", minimum=1)
            keep = mr.integer("keep_first", default=0, minimum=0)
        return PartSpec("qk_norm_attention", dict(
            hidden_size=self.width, norm_eps=self.norm_eps, n_heads=heads, n_kv_heads=kv,
            head_dim=dim, value_dim=r.integer("vdim", default=dim, minimum=1),
            scale=r.number("scale"), window=window, keep_first=keep, qk_norm=True,
            norm_scope="head", bias=True, gate=True,
            position=_rotation(m.get("rot"), f"{w}.rot", dim)))

    def _scan(self, m: Mapping[str, Any], w: str) -> PartSpec:
        r = ConfigReader(m, w)
        return PartSpec("selective_scan", dict(
            hidden_size=self.width, inner=r.integer("inner", minimum=1),
            n_state=r.integer("state", minimum=1), dt_rank=r.integer("dt_rank", minimum=1),
            conv=r.integer("conv", minimum=1)))

    def _mixer(self, i: int, layer: ZanelornLayer) -> PartSpec:
        w = f"config.layers[{i}].mixer"
        m = layer.mixer
        r = ConfigReader(m, w)
        if layer.type == "retention":
            heads = r.integer("heads", minimum=1)
            dim = r.integer("dim", minimum=1)
            decay = m.get("decay")
            if (not isinstance(decay, (list, tuple)) or len(decay) != heads
                    or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay)):
                raise ConfigError(f"{w}: key 'decay' must list one number per head ({heads})")
            return PartSpec("retention", dict(
                hidden_size=self.width, norm_eps=self.norm_eps, n_heads=heads, head_dim=dim,
                value_dim=r.integer("vdim", default=dim, minimum=1), decay=[float(d) for d in decay],
                position=_rotation(m.get("rot"), f"{w}.rot", dim), tensor_prefix="mix."))
        for side in ("left", "right"):
            if not isinstance(m.get(side), Mapping):
                raise ConfigError(f"{w}: key '{side}' must be an object")
        return PartSpec("parallel", dict(
            left=self._attention(m["left"], f"{w}.left"), right=self._scan(m["right"], f"{w}.right"),
            left_scale=r.number("left_scale", default=1.0),
            right_scale=r.number("right_scale", default=1.0), tensor_prefix="mix."))

    def _feed_forward(self, i: int, layer: ZanelornLayer) -> Optional[PartSpec]:
        if layer.mlp is None:
            return None
        w = f"config.layers[{i}].mlp"
        r = ConfigReader(layer.mlp, w)
        if layer.mlp["kind"] == "dense":
            return PartSpec("dense_mlp", {
                "hidden_size": self.width, "intermediate_size": r.integer("ff", minimum=1),
                "activation": "gelu", "up_name": "mlp.up", "down_name": "mlp.down"})
        for key in ("expert", "router"):
            if not isinstance(layer.mlp.get(key), Mapping):
                raise ConfigError(f"{w}: key '{key}' must be an object")
        er = ConfigReader(layer.mlp["expert"], f"{w}.expert")
        rr = ConfigReader(layer.mlp["router"], f"{w}.router")
        shared = None
        if layer.mlp.get("shared") is not None:
            sr = ConfigReader(layer.mlp["shared"], f"{w}.shared")
            shared = {"ff": sr.integer("ff", minimum=1), "limit": sr.number("limit", positive=True),
                      "name": "mlp.shared", "gate_name": "mlp.shared.sg"}
        experts = rr.integer("experts", minimum=1)
        identity = rr.integer("identity", default=0, minimum=0)
        top = rr.integer("top", minimum=1)
        if top > experts + identity:
            raise ConfigError(f"{w}.router: top {top} exceeds the {experts + identity} experts")
        return PartSpec("routed_experts", {
            "hidden_size": self.width, "intermediate_size": er.integer("ff", minimum=1),
            "n_experts": experts, "top": top, "activation": "clamped_swish",
            "limit": er.number("limit", positive=True), "scoring": "softmax_all",
            "identity": identity, "router_name": "mlp.router", "router_bias_name": None,
            "correction_name": "mlp.correction", "expert_name": "mlp.e{e}", "shared": shared})

    def plan(self) -> ModelPlan:
        norm = PartSpec("rms_norm", {"size": self.width, "eps": self.norm_eps})
        layers = []
        n = len(self.layers)
        for i, layer in enumerate(self.layers):
            ffn = self._feed_forward(i, layer)
            side = None
            if self.side_dim:
                side = {"hidden_size": self.width, "vocab_size": self.vocab, "dim": self.side_dim,
                        "offset": i * self.side_dim, "table_width": n * self.side_dim,
                        "eps": self.norm_eps, "table_name": "side.embed", "gate_name": "side.gate",
                        "proj_name": "side.proj", "norm_name": "side.norm"}
            layers.append(LayerSpec(
                prefix=f"l{i}.",
                block=PartSpec("output_norm", {"mult": self.residual_mult, "side": side}),
                mixer=self._mixer(i, layer),
                mixer_norm=norm.with_params(name="norm1", tensor_name="norm1"),
                feed_forward=ffn,
                feed_forward_norm=None if ffn is None else norm.with_params(name="norm2", tensor_name="norm2"),
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
            embedding_scale=self.embedding_scale,
            model_part_prefix="",
        )
        plan.validate()
        return plan
