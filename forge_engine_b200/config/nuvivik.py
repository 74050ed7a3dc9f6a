"""The Nuvivik configuration: a decoder whose layers are listed one by one, every sublayer
reading the residual stream itself and normalised on its way back into it.

``config.json`` names the architecture in ``architecture`` and gives ``vocab``, ``width``,
``norm.eps``, ``embedding.scale``, ``logit_scale``, ``logit_softcap`` (optional) and ``layers``.
Per layer: ``type`` (which mixer), the mixer's sizes and constants (``mixer``) and its
feed-forward (``mlp``, or null).

A layer: x += norm1(mixer(x)), x += norm2(ff(x)), both RMS norms with a weight.  The embedding
is multiplied by ``embedding.scale``; the logits are head(final norm(x)) * ``logit_scale``,
then c tanh(. / c) with c = ``logit_softcap``.

Mixers (both causal with a sliding window of ``mask.size`` tokens, the query's own included;
without ``mask`` every earlier token is visible):

* ``attention`` - grouped-query attention: q, k, v with biases; the first ``rot.dims``
  elements of every head rotated (element i with i + dims / 2, base ``rot.base``, frequencies
  optionally stretched by wavelength: ``rot.scaling`` with ``factor``, ``low``, ``high``,
  ``original``); after the rotation q and k are divided by their root mean square per head (no
  weight); scores times ``scale``, capped by ``softcap`` tanh(. / ``softcap``) where given;
* ``latent_attention`` - queries through a normalised latent of ``q_rank``; keys and values
  expanded from a normalised latent of ``kv_rank`` plus one rotated key part of ``rot_dim``
  shared by the heads (only those two are cached); a learned sink per head in the softmax's
  denominator.

Feed-forwards (``mlp.kind``): ``dense`` - down(gelu_tanh(up(x))); ``moe`` -
``router.experts`` units down(relu(up(x))^2) of which a token uses ``router.top``, chosen by
the sigmoid of 32-bit router logits among the experts of the best ``groups.keep`` of
``groups.count`` groups of neighbours (a group is worth the sum of its two largest scores),
weighted by those scores as they are.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.*``, ``l<i>.norm2``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from dataclasses import dataclass

from ..errors import ConfigError
from .specs import (
    AttentionSpec,
    DenseMLPSpec,
    LatentAttentionSpec,
    LayerSpec,
    ModelSpec,
    NormSpec,
    OutputNormSpec,
    RotarySpec,
    RoutedMLPSpec,
    RunSpec,
)
from .zofadra import _int, _number

MAX_POSITIONS = 1 << 20          # rotary positions have no table; the cache bounds a request first

_BARE = (("weight", ""),)        # a norm's weight is stored under the norm's own name
_ATTENTION = (("q_proj.weight", "q"), ("k_proj.weight", "k"), ("v_proj.weight", "v"), ("o_proj.weight", "o"),
              ("q_proj.bias", "q.b"), ("k_proj.bias", "k.b"), ("v_proj.bias", "v.b"))
_UNIT = (("up_proj.weight", "up"), ("down_proj.weight", "down"))


@dataclass(frozen=True)
class NuvivikLayer:
    type: str
    mixer: dict
    mlp: dict | None


def _rotary(mixer: dict, where: str, dims_key_from: int | None = None) -> None:
    rot = mixer.get("rot")
    if not isinstance(rot, dict):
        raise ConfigError(f"{where}.rot must be an object")
    if _number(rot, "base", f"{where}.rot") <= 0:
        raise ConfigError(f"{where}.rot.base must be positive")
    dims = _int(rot, "dims", f"{where}.rot", 2)
    limit = mixer["dim"] if dims_key_from is None else dims_key_from
    if dims % 2 or dims > limit:
        raise ConfigError(f"{where}.rot.dims={dims} must be even and at most {limit}")
    scaling = rot.get("scaling")
    if scaling is not None:
        if not isinstance(scaling, dict):
            raise ConfigError(f"{where}.rot.scaling must be an object")
        values = {key: _number(scaling, key, f"{where}.rot.scaling") for key in ("factor", "low", "high", "original")}
        if values["factor"] <= 0 or values["original"] <= 0 or values["high"] <= values["low"]:
            raise ConfigError(f"{where}.rot.scaling needs factor > 0, original > 0 and high > low")


@dataclass(frozen=True)
class NuvivikConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    logit_softcap: float | None
    layers: tuple

    architecture = "Nuvivik"

    @classmethod
    def from_dict(cls, raw: dict) -> "NuvivikConfig":
        layers_raw = raw.get("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError("config.json 'layers' must be a non-empty list")
        eps = _number(raw.get("norm") or {}, "eps", "norm")
        if eps <= 0:
            raise ConfigError("norm.eps must be positive")
        layers = []
        for index, item in enumerate(layers_raw):
            where = f"layers[{index}]"
            kind, mixer = item.get("type"), item.get("mixer")
            if not isinstance(mixer, dict):
                raise ConfigError(f"{where}.mixer must be an object")
            if kind not in ("attention", "latent_attention"):
                raise ConfigError(f"{where}.type={kind!r}; known: attention, latent_attention")
            for key in ("heads", "dim", "vdim"):
                _int(mixer, key, f"{where}.mixer")
            _number(mixer, "scale", f"{where}.mixer")
            if mixer.get("mask") is not None:                    # no mask: every earlier token is visible
                _int(mixer["mask"], "size", f"{where}.mixer.mask")
            if kind == "attention":
                if mixer.get("kv_heads") is None:
                    mixer = dict(mixer, kv_heads=mixer["heads"])    # every query head with keys and values of its own
                _int(mixer, "kv_heads", f"{where}.mixer")
                if mixer["heads"] % mixer["kv_heads"]:
                    raise ConfigError(f"{where}.mixer.heads must be a multiple of kv_heads")
                if mixer.get("softcap") is not None and _number(mixer, "softcap", f"{where}.mixer") <= 0:
                    raise ConfigError(f"{where}.mixer.softcap must be positive")
                _rotary(mixer, f"{where}.mixer")
            else:
                for key in ("q_rank", "kv_rank"):
                    _int(mixer, key, f"{where}.mixer")
                _rotary(mixer, f"{where}.mixer", _int(mixer, "rot_dim", f"{where}.mixer", 2))
                if mixer["rot"]["dims"] != mixer["rot_dim"]:
                    raise ConfigError(f"{where}.mixer.rot.dims must equal rot_dim: the whole shared key part is rotated")
            mlp = item.get("mlp")
            if mlp is not None:
                style = mlp.get("kind", "dense")
                if style == "dense":
                    _int(mlp, "ff", f"{where}.mlp")
                elif style == "moe":
                    router = mlp.get("router") or {}
                    experts = _int(router, "experts", f"{where}.mlp.router")
                    top = _int(router, "top", f"{where}.mlp.router")
                    allowed = experts
                    groups = router.get("groups")
                    if groups is not None:
                        count = _int(groups, "count", f"{where}.mlp.router.groups")
                        keep = _int(groups, "keep", f"{where}.mlp.router.groups")
                        if experts % count or keep > count:
                            raise ConfigError(f"{where}.mlp.router.groups: {experts} experts do not form {count} equal "
                                              f"groups of which {keep} are kept")
                        allowed = experts // count * keep
                    if top > allowed:
                        raise ConfigError(f"{where}.mlp.router.top={top} is more than the {allowed} experts that can be chosen")
                    _int(mlp.get("expert") or {}, "ff", f"{where}.mlp.expert")
                else:
                    raise ConfigError(f"{where}.mlp.kind={style!r}; known: dense, moe")
            layers.append(NuvivikLayer(kind, dict(mixer), None if mlp is None else dict(mlp)))
        cap = raw.get("logit_softcap")
        if cap is not None and _number(raw, "logit_softcap", "config") <= 0:
            raise ConfigError("logit_softcap must be positive")
        return cls(vocab=_int(raw, "vocab", "config"), width=_int(raw, "width", "config"), eps=eps,
                   embedding_scale=_number(raw.get("embedding") or {"scale": 1.0}, "scale", "embedding"),
                   logit_scale=_number(raw, "logit_scale", "config") if raw.get("logit_scale") is not None else 1.0,
                   logit_softcap=None if cap is None else float(cap), layers=tuple(layers))

    # ------------------------------------------------------------------------------
    def _norm(self) -> NormSpec:
        return NormSpec(self.width, self.eps, rename=_BARE)

    @staticmethod
    def _position(rot: dict, size: int) -> RotarySpec:
        scaling = rot.get("scaling")
        return RotarySpec(
            head_dim=size, theta=float(rot["base"]), rotary_dim=int(rot["dims"]), interleaved=False, exact_frequencies=True,
            scaling=None if scaling is None else tuple(float(scaling[key]) for key in ("factor", "low", "high", "original")))

    def _mixer_spec(self, layer: NuvivikLayer):
        m = layer.mixer
        window = None if m.get("mask") is None else int(m["mask"]["size"])
        if layer.type == "attention":
            return AttentionSpec(
                hidden_size=self.width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"], qk_norm=True,
                qk_norm_eps=self.eps, bias=True, o_bias=False, scale=float(m["scale"]), position=self._position(m["rot"], m["dim"]),
                window=window, v_head_dim=m["vdim"], rename=_ATTENTION,
                softcap=None if m.get("softcap") is None else float(m["softcap"]),
                qk_norm_weight=False, qk_norm_after_rotation=True,
            )
        return LatentAttentionSpec(
            hidden_size=self.width, num_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_head_dim=m["vdim"],
            q_rank=m["q_rank"], kv_rank=m["kv_rank"], norm_eps=self.eps, scale=float(m["scale"]),
            position=self._position(m["rot"], m["rot_dim"]), window=window, sink=True,
        )

    def _ffn_spec(self, mlp: dict):
        if mlp.get("kind", "dense") == "dense":
            return DenseMLPSpec(self.width, mlp["ff"], "gelu_tanh", bias=False, rename=_UNIT)
        router = mlp["router"]
        groups = router.get("groups")
        return RoutedMLPSpec(
            hidden_size=self.width, experts=router["experts"], top=router["top"],
            expert=DenseMLPSpec(self.width, mlp["expert"]["ff"], "relu2", bias=False, rename=_UNIT),
            shared=None, score="sigmoid", renormalise=False, weight_on="output", shared_gate=False,
            groups=None if groups is None else (int(groups["count"]), int(groups["keep"])), group_score="top2",
        )

    def to_model_spec(self) -> ModelSpec:
        layers, schedule = [], []
        for index, layer in enumerate(self.layers):
            prefix = f"l{index}"
            ffn = None if layer.mlp is None else self._ffn_spec(layer.mlp)
            layers.append(LayerSpec(
                input_norm=None, mixer=self._mixer_spec(layer), post_norm=None, ffn=ffn,
                names={"mixer": f"{prefix}.mix", "mixer_out_norm": f"{prefix}.norm1", "ffn": f"{prefix}.mlp",
                       "ffn_out_norm": f"{prefix}.norm2"},
                arrangement="output_norm",
                options=OutputNormSpec(self._norm(), None if ffn is None else self._norm()),
            ))
            schedule.append(RunSpec(index))
        return ModelSpec(
            vocab_size=self.vocab, hidden_size=self.width, layers=tuple(layers), schedule=tuple(schedule),
            final_norm=self._norm(), tie_embeddings=False, max_positions=MAX_POSITIONS, eos_token_ids=(),
            embed_name="embed", final_norm_name="final.norm", head_name="head",
            embedding_scale=self.embedding_scale, logit_scale=self.logit_scale, logit_softcap=self.logit_softcap,
        )
