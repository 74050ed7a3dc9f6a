"""The Zabutar configuration: a decoder whose layers are listed one by one, with learned
absolute positions, a short causal convolution in front of every sublayer and a norm on both
sides of it.

``config.json`` names the architecture in ``architecture`` and gives ``vocab``, ``width``,
``max_positions``, ``norm.eps``, ``canon.taps`` and ``layers``.  Per layer: ``type`` (which
mixer), the mixer's sizes and constants (``mixer``) and its feed-forward (``mlp``, or null).

A layer: x += norm1b(mixer(u1)), x += norm2b(ff(u2)), where u = y + conv(y), y = norm(x) and
conv a causal convolution over time with ``canon.taps`` taps per channel.  Every norm is an RMS
norm whose weight is stored as its distance from one.

Mixers:

* ``hgrn2`` - a gated linear recurrence: per head a 32-bit state [dim, vdim] whose rows the
  forget gate f scales while 1 - f writes the value into them; f is bounded below by a learned
  number per head and channel; the head's output is RMS-normalised;
* ``attention`` - grouped-query softmax attention without rotation, with a learned bias by
  (bucketed) distance and head; ``kv_from``: j makes the layer read layer j's keys and values.

Feed-forwards (``mlp.kind``): ``dense`` - down(xIELU(up(x))) with biases and two learned
numbers of the activation; ``moe`` - ``router.experts`` SiLU-gated units plus
``router.identity`` experts that hand their input on, softmax scores over all of them, a
correction added for the choice only, the choice limited to the best ``groups.keep`` of
``groups.count`` groups, weights renormalised and multiplied by ``router.scale``; a shared
unit that every token uses.

Tensor names: ``embed``, ``pos``, ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.canon1``,
``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.norm2b``, ``l<i>.canon2``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from .specs import (
    AttentionSpec,
    DenseMLPSpec,
    GatedMLPSpec,
    GatedRecurrenceSpec,
    LayerSpec,
    ModelSpec,
    NoPositionSpec,
    NormSpec,
    RoutedMLPSpec,
    RunSpec,
    SandwichConvSpec,
)
from .zofadra import _int, _number

RENORM_FLOOR = 1e-20             # added to the sum the chosen experts' scores are divided by
NORM_WEIGHT_OFFSET = 1.0         # norm weights are stored around zero

_BARE = (("weight", ""),)        # a norm's weight is stored under the norm's own name
_UNIT = (("gate_proj.weight", "gate"), ("up_proj.weight", "up"), ("down_proj.weight", "down"))
_DENSE = (("up_proj.weight", "up"), ("up_proj.bias", "up.b"), ("down_proj.weight", "down"),
          ("down_proj.bias", "down.b"))
_ATTENTION = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"))
_RECURRENCE = (("f.bias", "f.b"),)
_CONV = (("conv1", "canon1"), ("conv2", "canon2"))


@dataclass(frozen=True)
class ZabutarLayer:
    type: str
    mixer: dict
    mlp: dict | None


@dataclass(frozen=True)
class ZabutarConfig:
    vocab: int
    width: int
    eps: float
    taps: int
    max_positions: int
    layers: tuple

    architecture = "Zabutar"

    @classmethod
    def from_dict(cls, raw: dict) -> "ZabutarConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json 'layers' must be a non-empty list")
        eps = _number(raw.get("norm") or {}, "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        taps = _int(raw.get("canon") or {}, "taps", "canon")
        layers = []
        for index, item in enumerate(layers_raw):
            where = f"layers[{index}]"
            kind, mixer = item.get("type"), item.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind not in ("hgrn2", "attention"):
                raise ConfigError(f"{where}.type={kind!r}; known: attention, hgrn2")
            for key in ("heads", "dim", "vdim"):
                _int(mixer, key, f"{where}.mixer")
            if kind == "attention":
                _int(mixer, "kv_heads", f"{where}.mixer")
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.heads must be a multiple of kv_heads")
                _number(mixer, "scale", f"{where}.mixer")
                if _number(mixer, "bias_max", f"{where}.mixer") <= 1:
                    raise ConfigError(f"{where}.mixer.bias_max must be above 1")
                if mixer.get("bias_rows") is not None and _int(mixer, "bias_rows", f"{where}.mixer", 2) % 2:
                    raise ConfigError(f"{where}.mixer.bias_rows must be even")
                source = mixer.get("kv_from")
                if source is not None:
                    _int(mixer, "kv_from", f"{where}.mixer", 0)
                    if source >= index or layers[source].type != "attention" or layers[source].mixer.get("kv_from") is not None:
                        raise ConfigError(f"{where}.mixer.kv_from={source} must name an earlier attention layer "
                                          "with keys and values of its own")
                    other = layers[source].mixer
                    if any(other[key] != mixer[key] for key in ("kv_heads", "dim", "vdim")):
                        raise ConfigError(f"{where}.mixer: kv_heads, dim and vdim must equal those of layer {source}")
            mlp = item.get("mlp")
            if mlp is not None:
                style = mlp.get("kind", "dense")
                if style == "dense":
                    _int(mlp, "ff", f"{where}.mlp")
                elif style == "moe":
                    router = mlp.get("router") or {}
                    experts = _int(router, "experts", f"{where}.mlp.router")
                    identity = _int(router, "identity", f"{where}.mlp.router", 0) if router.get("identity") is not None else 0
                    top = _int(router, "top", f"{where}.mlp.router")
                    _number(router, "scale", f"{where}.mlp.router")
                    outputs, allowed = experts + identity, experts + identity
                    groups = router.get("groups")
                    if groups is not None:
                        count = _int(groups, "count", f"{where}.mlp.router.groups")
                        keep = _int(groups, "keep", f"{where}.mlp.router.groups")
                        if outputs % count or keep > count:
                            raise ConfigError(f"{where}.mlp.router.groups: {outputs} router outputs do not form "
                                              f"{count} equal groups of which {keep} are kept")
                        allowed = outputs // count * keep
                    if top > allowed:
                        raise ConfigError(f"{where}.mlp.router.top={top} is more than the {allowed} experts that can be chosen")
                    _int(mlp.get("expert") or {}, "ff", f"{where}.mlp.expert")
                    if mlp.get("shared") is not None:
                        _int(mlp["shared"], "ff", f"{where}.mlp.shared")
                else:
                    raise ConfigError(f"{where}.mlp.kind={style!r}; known: dense, moe")
            layers.append(ZabutarLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        return cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), eps=eps, taps=taps,
                   max_positions=_int(raw, "max_positions", "config"), layers=tuple(layers))

    # ------------------------------------------------------------------------------
    def _norm(self) -> NormSpec:
        return NormSpec(self.width, self.eps, rename=_BARE, weight_offset=NORM_WEIGHT_OFFSET)

    def _mixer_spec(self, layer: ZabutarLayer):
        m = layer.mixer
        # the rows of the bias table are the stored tensor's; a configuration made for random
        # weights, which has no tensor to read them from, may say them in ``bias_rows``
        bias_rows = m.get("bias_rows")
        if layer.type == "hgrn2":
            return GatedRecurrenceSpec(self.width, m["heads"], m["dim"], m["vdim"], self.eps, rename=_RECURRENCE)
        return AttentionSpec(
            hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], qk_norm=False,
            qk_norm_eps=self.eps, bias=False, scale=float(m["scale"]), position=NoPositionSpec(), window=None,
            v_head_dim=m["vdim"], rename=_ATTENTION, distance_bias_table=(bias_rows, float(m["bias_max"])),
            kv_projection=m.get("kv_from") is None,
        )

    def _unit_spec(self, raw: dict) -> GatedMLPSpec:
        return GatedMLPSpec(self.width, raw["ff"], "silu", rename=_UNIT)

    def _ffn_spec(self, mlp: dict):
        if mlp.get("kind", "dense") == "dense":
            return DenseMLPSpec(self.width, mlp["ff"], "xielu", bias=True, rename=_DENSE)
        router, shared = mlp["router"], mlp.get("shared")
        groups = router.get("groups")
        return RoutedMLPSpec(
            hidden_size=self.width, experts=router["experts"], top=router["top"], expert=self._unit_spec(mlp["expert"]),
            shared=None if shared is None else self._unit_spec(shared), score="softmax", renormalise=True,
            weight_on="output", shared_gate=False, identity=int(router.get("identity") or 0), correction=True,
            groups=None if groups is None else (int(groups["count"]), int(groups["keep"])),
            renorm_floor=RENORM_FLOOR, weight_scale=float(router["scale"]),
        )

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}"
            ffn = None if layer.mlp is None else self._ffn_spec(layer.mlp)
            layers.append(LayerSpec(
                input_norm=self._norm(), mixer=self._mixer_spec(layer),
                post_norm=None if ffn is None else self._norm(), ffn=ffn,
                names={"input_norm": f"{prefix}.norm1", "mixer": f"{prefix}.mix", "mixer_out_norm": f"{prefix}.norm1b",
                       "post_norm": f"{prefix}.norm2", "ffn": f"{prefix}.mlp", "ffn_out_norm": f"{prefix}.norm2b",
                       "conv": prefix},
                arrangement="sandwich_conv",
                options=SandwichConvSpec(self.taps, self._norm(), None if ffn is None else self._norm(), rename=_CONV),
            ))
            schedule.append(RunSpec(index, cache_of=layer.mixer.get("kv_from") if layer.type == "attention" else None))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers), schedule=tuple(schedule),
            final_norm=self._norm(), tie_embeddings=False, max_positions=self.max_positions, eos_token_ids=(),
            embed_name="embed", final_norm_name="final.norm", head_name="head", position_table_name="pos",
        )
