"""Typed descriptions of the parts a model is assembled from.

A *spec* is plain frozen data: every size and constant a part needs, nothing about
the model it sits in.  An architecture (see ``models/``) turns its ``config.json``
into a ``ModelSpec``; ``parts.build`` turns specs into parts.  A new kind of part
brings its own spec dataclass with a unique ``kind`` string and registers a builder
for it (``parts.registry``); nothing in this file has to change for that.
"""

from __future__ import annotations

from dataclasses import dataclass, field


def local_name(spec, canonical: str) -> str:
    """The name a part's tensor has in its checkpoint, relative to the part's prefix.
    ``spec.rename`` is a tuple of (canonical, stored) pairs; a stored name "" means that
    the tensor is called by the prefix alone."""
    return dict(getattr(spec, "rename", ()) or ()).get(canonical, canonical)


def join_name(prefix: str, local: str) -> str:
    """Checkpoint name of a part's tensor: ``prefix.local``, or ``prefix`` for local ""."""
    return f"{prefix}.{local}" if local else prefix


@dataclass(frozen=True)
class NormSpec:
    """RMS normalisation over the last ``size`` elements."""

    size: int
    eps: float
    kind: str = "rmsnorm"
    rename: tuple = ()
    # The checkpoint stores the weight's distance from this number: the rows are multiplied
    # by ``weight_offset`` + stored weight (0: the weight is stored as it is used).
    weight_offset: float = 0.0


@dataclass(frozen=True)
class LayerNormSpec:
    """(x - mean) / sqrt(variance + eps) * weight over the last ``size`` elements, the
    variance being the mean of the squared deviations; no bias."""

    size: int
    eps: float
    kind: str = "layernorm"
    rename: tuple = ()


@dataclass(frozen=True)
class RotarySpec:
    """Rotary position encoding: pairs element j with j + rotary_dim/2.

    ``theta`` is the base; ``rotary_dim`` is the number of leading elements of a
    head that are rotated (the whole head for Qwen3).
    """

    head_dim: int
    theta: float
    rotary_dim: int
    kind: str = "rope"
    # False: element j is paired with j + rotary_dim/2; True: element 2j with 2j + 1.
    interleaved: bool = False
    # None, or (factor, low, high, original): frequencies are stretched by wavelength
    # l = 2 pi / f.  Below original / high the frequency stays; above original / low it becomes
    # f / factor; between the two, with s = (original / l - low) / (high - low), it becomes
    # (1 - s) f / factor + s f.
    scaling: tuple | None = None
    # True: theta^(-2j / rotary_dim) is worked out in 64-bit and rounded once (always so with
    # ``interleaved`` or ``scaling``); False: in 32-bit throughout, as Qwen3's own code does.
    exact_frequencies: bool = False


@dataclass(frozen=True)
class NoPositionSpec:
    """No position encoding: queries and keys are used as they come."""

    kind: str = "none"


@dataclass(frozen=True)
class AttentionSpec:
    """Causal grouped-query attention.

    ``window`` is None for full attention, else the number of most recent keys
    (the query's own included) a query may look at.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    qk_norm: bool
    qk_norm_eps: float
    bias: bool
    scale: float
    position: object
    window: int | None = None
    kind: str = "gqa_attention"
    # Size of a value head where it differs from ``head_dim`` (None: the same).
    v_head_dim: int | None = None
    # "head": q and k are normalised head by head with weights of ``head_dim`` (when
    # ``qk_norm``); "whole": over all heads of the projection at once, with weights of the
    # projection's size.
    qk_norm_scope: str = "head"
    # None, or the base b of a bias on the distance: head h of H takes
    # b^(-(h + 1) / H) * (i - j) off the score of query i and key j (b = 2^8 gives the
    # slopes 2^(-8 (h + 1) / H)).
    distance_bias_base: float | None = None
    rename: tuple = ()
    # With a window: keys at positions below ``keep_first`` stay visible to every later query
    # (at their true positions), and their cache pages are never given back.
    keep_first: int = 0
    # None, or c: scores become c * tanh(score / c) before the softmax.
    softcap: float | None = None
    # None, or (coef, every): the scores of a query at position p are multiplied by
    # 1 + coef * ln(floor((p + 1) / every) + 1).
    query_temperature: tuple | None = None
    # True: head h's output is multiplied by sigmoid(w_h . x), x the mixer's input; the
    # checkpoint holds ``gate_proj.weight`` [heads, hidden].
    head_gate: bool = False
    # None, or a DifferentialSpec: every head has two score maps over the same values.
    differential: object = None
    # None, or (rows, far): a learned bias by distance and head, tensor ``rel`` [rows, heads].
    # Distance n = i - j uses row n below rows/2 and beyond that rows that widen
    # logarithmically: min(rows - 1, h + floor(ln(n / h) / ln(far / h) * (rows - h))), h = rows/2.
    # The bias is added to the scaled score (the scale does not multiply it).
    distance_bias_table: tuple | None = None
    # False: the layer has no key and value projections; it reads another run's cache
    # (``RunSpec.cache_of``) with queries, bias and output projection of its own.
    kv_projection: bool = True
    # With ``bias``: whether the output projection has one too (None: as q, k and v).
    o_bias: bool | None = None
    # False (per-head ``qk_norm`` only): q and k are divided by their root mean square and
    # multiplied by no learned weight; the checkpoint holds no norm tensors.
    qk_norm_weight: bool = True
    # True (per-head ``qk_norm`` only): the norm is taken of the rotated head, not before the rotation.
    qk_norm_after_rotation: bool = False


@dataclass(frozen=True)
class DifferentialSpec:
    """Two softmax maps per head, from two queries and two keys of ``head_dim`` each (a head's
    projection rows are [map 1, map 2]), over the same values: o = a1 - lambda a2 with
    lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + offset, one number for the layer from four
    vectors of ``head_dim`` in the checkpoint; then o / sqrt(mean(o^2) + eps) over the head's
    values, times (1 - offset)."""

    offset: float
    eps: float


@dataclass(frozen=True)
class LatentAttentionSpec:
    """Causal attention whose keys and values are expanded from one cached latent.

    Per head ``head_dim`` query/key elements that are not rotated and ``rot_dim`` that are;
    the rotated key part is one vector shared by all heads.  Cached per token: the
    normalised latent (``kv_rank``) and the rotated key part (``rot_dim``).  ``kv_from``
    None: the layer projects and caches its own latent; otherwise it reads the cache of
    the layer of that index.  ``position`` is a RotarySpec for the ``rot_dim`` part."""

    hidden_size: int
    num_heads: int
    head_dim: int
    rot_dim: int
    v_head_dim: int
    q_rank: int
    kv_rank: int
    norm_eps: float
    scale: float
    position: object
    kv_from: int | None = None
    kind: str = "latent_attention"
    rename: tuple = ()
    # None for full attention, else the number of most recent keys (the query's own included).
    window: int | None = None
    # True: tensor ``sink`` [heads]; exp(sink_h) joins the denominator of head h's softmax once,
    # with no key and no value, neither scaled nor capped.
    sink: bool = False


@dataclass(frozen=True)
class LinearRecurrenceSpec:
    """Linear attention with a fixed decay per head ("lightning" attention):
    S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with q, k, v = act(W x); the heads'
    outputs are RMS-normalised together, gated by sigmoid(W_g x) and projected."""

    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    decay: tuple
    norm_eps: float
    activation: str = "silu"
    kind: str = "linear_recurrence"
    rename: tuple = ()


@dataclass(frozen=True)
class GatedRecurrenceSpec:
    """Linear attention whose forget gate also decides what is written: per head a state
    S [head_dim, v_head_dim] with S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T, o_t = S_t^T q_t,
    q = silu(W_q x), v = W_v x and f = l + (1 - l) sigmoid(W_f x + b_f) for a learned lower
    bound l per head and channel.  Each head's output is RMS-normalised over its values with
    one weight vector shared by the heads, and the heads are projected by W_o."""

    hidden_size: int
    num_heads: int
    head_dim: int
    v_head_dim: int
    norm_eps: float
    kind: str = "gated_recurrence"
    rename: tuple = ()


@dataclass(frozen=True)
class DenseMLPSpec:
    """down(act(up(x) + b_up)) + b_down, no gate.  ``activation`` "xielu": with two learned
    numbers p, q (tensor ``act`` [2]) act(z) = softplus(p) z^2 + z / 2 above zero and
    (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 at and below it; "gelu_tanh":
    0.5 z (1 + tanh(sqrt(2 / pi) (z + 0.044715 z^3))); "relu2": max(z, 0)^2 (neither has tensors
    of its own)."""

    hidden_size: int
    intermediate_size: int
    activation: str = "xielu"
    bias: bool = True
    kind: str = "dense_mlp"
    rename: tuple = ()


@dataclass(frozen=True)
class GatedMLPSpec:
    """down(act(gate(x)) * up(x)) without biases."""

    hidden_size: int
    intermediate_size: int
    # "silu", "gelu_tanh", or "clamped_swish": g' sigmoid(slope g') (u' + 1) in place of
    # act(g) u, with g' = min(g, limit) and u' = clamp(u, -limit, limit)
    activation: str = "silu"
    kind: str = "gated_mlp"
    rename: tuple = ()
    limit: float | None = None
    slope: float = 1.0


@dataclass(frozen=True)
class RoutedMLPSpec:
    """A routed feed-forward: ``experts`` units (``expert``: a GatedMLPSpec, or a DenseMLPSpec
    without biases for units that have no gate; tensors
    ``e<i>.<name>``) of which every token uses the ``top`` with the largest router scores.
    ``score``: "sigmoid" or "softmax" of the router's 32-bit logits; ``renormalise``: the
    chosen scores are divided by their sum; ``weight_on`` "input": the unit runs on
    weight * x, "output": its result is multiplied.  ``shared`` (a GatedMLPSpec or None;
    tensors ``shared.<name>``) runs for every token and is added, times
    sigmoid(``shared.sg`` . x) when ``shared_gate``."""

    hidden_size: int
    experts: int
    top: int
    expert: object
    shared: object = None
    score: str = "sigmoid"
    renormalise: bool = False
    weight_on: str = "input"
    shared_gate: bool = False
    kind: str = "routed_mlp"
    rename: tuple = ()
    # The last ``identity`` outputs of the router (it has ``experts`` + ``identity``) stand
    # for experts without tensors whose output is their input.
    identity: int = 0
    # True: tensor ``correction`` [router outputs] is added to the scores for the choice of
    # experts only; the weights come from the scores without it.
    correction: bool = False
    # None, or (count, keep): the router's outputs form ``count`` equal groups of neighbours;
    # a group's mark is its largest choice score and only the ``keep`` best groups can be chosen.
    groups: tuple | None = None
    # With ``renormalise``: weights = scores / (sum + renorm_floor); always times weight_scale.
    renorm_floor: float = 0.0
    weight_scale: float = 1.0
    # What a group is worth: "max" - its largest choice score; "top2" - the sum of its two
    # largest (of its one, where a group is a single expert).
    group_score: str = "max"


@dataclass(frozen=True)
class LayerSpec:
    """One block: which norm, mixer and feed-forward it has and how they are wired.

    ``arrangement`` "pre_norm": h += mixer(norm1(h)); h += ffn(norm2(h)).
    ``names`` maps the roles (input_norm, mixer, post_norm, ffn) to the tensor-name
    prefix of this layer's weights in a checkpoint.
    """

    input_norm: object
    mixer: object
    post_norm: object
    ffn: object
    names: dict = field(default_factory=dict, hash=False, compare=False)
    arrangement: str = "pre_norm"
    # What an arrangement other than "pre_norm" needs to know (a frozen dataclass of its own).
    options: object = None


@dataclass(frozen=True)
class StreamMixSpec:
    """Options of the "stream_mix" arrangement: ``streams`` copies of the residual stream
    that every sublayer reads as a weighted sum and writes back through a mixing matrix
    (``learned`` True: weights ``in`` [streams], ``out`` [streams], ``mix`` [streams, streams]
    per sublayer in the checkpoint; False: one stream and the plain residual sum), the
    sublayer's output scaled by ``update_scale``."""

    streams: int = 1
    learned: bool = False
    update_scale: float = 1.0


@dataclass(frozen=True)
class SandwichConvSpec:
    """Options of the "sandwich_conv" arrangement: every sublayer's update is normalised
    again before it joins the residual stream (x += norm_b(sublayer(u))), and what a sublayer
    reads is u = y + conv(y), y the normalised stream and conv a causal convolution over time
    with ``taps`` taps per channel (tensors ``conv1`` / ``conv2`` [width, taps]; tap j weighs
    the input taps - 1 - j tokens back).  The last taps - 1 rows of y belong to a request's
    state, for both sublayers.  ``mixer_out_norm`` / ``ffn_out_norm``: the specs of the norms
    norm_b (roles of the same names; the second is None for a layer without feed-forward)."""

    taps: int
    mixer_out_norm: object = None
    ffn_out_norm: object = None
    rename: tuple = ()


@dataclass(frozen=True)
class OutputNormSpec:
    """Options of the "output_norm" arrangement: a sublayer reads the residual stream as it
    is and its output is normalised before it joins the stream, x += norm(sublayer(x)), for the
    mixer and then for the feed-forward.  ``mixer_out_norm`` / ``ffn_out_norm``: the specs of
    those norms (roles of the same names; the second is None for a layer without
    feed-forward).  The layer has no ``input_norm`` and no ``post_norm``."""

    mixer_out_norm: object = None
    ffn_out_norm: object = None


@dataclass(frozen=True)
class RunSpec:
    """One entry of the order in which layers run.

    ``layer`` indexes ``ModelSpec.layers`` (a layer may appear in several runs).
    ``cache_of`` is None when the run keeps a cache of its own, else the index of
    an earlier *run* whose cache it reads without writing.
    """

    layer: int
    cache_of: int | None = None
    # None, or (tensor name, row): that row of a [rows, hidden] tensor of the checkpoint is
    # added to the residual stream right before this run.
    shift: tuple | None = None


@dataclass(frozen=True)
class ModelSpec:
    """Everything needed to assemble a decoder-only language model from parts."""

    vocab_size: int
    hidden_size: int
    layers: tuple
    schedule: tuple
    final_norm: object
    tie_embeddings: bool
    max_positions: int
    eos_token_ids: tuple = ()
    embed_name: str = "model.embed_tokens.weight"
    final_norm_name: str = "model.norm"
    head_name: str = "lm_head.weight"
    embedding_scale: float = 1.0     # the embedding rows are multiplied by this
    residual_streams: int = 1        # copies of the residual stream (see StreamMixSpec)
    # tensors of the checkpoint that belong to no layer: (name, shape, role) each
    extra_tensors: tuple = ()
    # None, or the name of a tensor [max_positions, hidden]: row p is added to the embedding
    # of the token at position p.
    position_table_name: str | None = None
    # logits = head(x) * logit_scale, then (with a cap c) c * tanh(logits / c)
    logit_scale: float = 1.0
    logit_softcap: float | None = None
