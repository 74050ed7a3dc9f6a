"""Arrangement of norm, mixer and feed-forward in one block.

"pre_norm" is upstream's decoder layer (src/forge_engine/qwen3.py:241-261):
h += mixer(norm1(h)); h += ffn(norm2(h)).  The residual stream ``h`` is a 32-bit
tensor updated in place; the block returns its last update *unadded* so that the next
block's first norm (or the final norm) adds it in the same kernel that normalises.

"stream_mix" is the same pre-norm block over several copies of the residual stream that
learned weights mix (or over one, with the update scaled by a constant).  "sandwich_conv" has
a norm on both sides of every sublayer and a short convolution on its input; "output_norm" a
norm on the sublayer's output only, the sublayer reading the stream itself.
"""

from __future__ import annotations

import os

import torch

from ..ops import native
from .base import BuildContext, CacheView, WeightInfo, build_part, part_class, register_arrangement


class PreNormBlock:
    roles = ("input_norm", "mixer", "post_norm", "ffn")

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        """``weights[role]`` is the dict of that part's local tensors."""
        self.ctx = ctx
        self.input_norm = build_part(spec.input_norm, weights["input_norm"], ctx)
        self.mixer = build_part(spec.mixer, weights["mixer"], ctx)
        # a layer without a feed-forward is the first half alone: h += mixer(norm1(h))
        self.post_norm = self.ffn = None
        if spec.ffn is not None:
            self.post_norm = build_part(spec.post_norm, weights["post_norm"], ctx)
            self.ffn = build_part(spec.ffn, weights["ffn"], ctx)
        self._chain_parts = None

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """role -> {local name -> WeightInfo}"""
        return {role: part_class(getattr(spec, role)).weight_shapes(getattr(spec, role)) for role in cls.roles
                if getattr(spec, role) is not None}

    def cache_needs(self):
        return self.mixer.cache_needs()

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        planner = getattr(self.mixer, "plan_step", None)
        if planner is not None:
            planner(entries, page_size, plans)

    @property
    def graph_safe(self) -> bool:
        return all(getattr(part, "graph_safe", False)
                   for part in (self.input_norm, self.mixer, self.post_norm, self.ffn) if part is not None)

    def _chain(self):
        """What the one-kernel form of "output projection, norm, feed-forward" needs of this
        block's parts, or None: a mixer that can stop before its bias-free bfloat16 output
        projection, an RMS norm, and a gated feed-forward whose gate/up rows alternate in
        sixteens, all at sizes the kernel takes.  Worked out once."""
        if self._chain_parts is None:
            self._chain_parts = False
            o_proj = getattr(self.mixer, "o_proj", None)
            gate_up, down = getattr(self.ffn, "gate_up", None), getattr(self.ffn, "down", None)
            norm = self.post_norm
            usable = (self.ctx.dtype == torch.bfloat16 and hasattr(self.mixer, "attend")
                      and all(lin is not None and lin.bias is None and lin.weight.dtype == torch.bfloat16
                              for lin in (o_proj, gate_up, down))
                      and getattr(self.ffn, "block", 0) == 16 and getattr(self.ffn, "activation", None) == native.ACT_SILU
                      and hasattr(norm, "eps") and getattr(norm, "weight", None) is not None
                      and os.environ.get("FORGE_ENGINE_DECODE_CHAIN", "0") == "1")
            if usable:
                shapes = [(o_proj.out_features, o_proj.in_features, native.CHAIN_SRC_ACTIVATIONS, native.CHAIN_ADD),
                          (gate_up.out_features, gate_up.in_features, native.CHAIN_SRC_NORM, native.CHAIN_SILU_MUL),
                          (down.out_features, down.in_features, native.CHAIN_SRC_ACTIVATIONS, native.CHAIN_ADD)]
                if native.decode_chain_takes(shapes, 1):
                    self._chain_parts = (o_proj, norm, gate_up, down)
        return self._chain_parts or None

    def forward(self, h, pending, batch, cache: CacheView, shift=None):
        """``h`` 32-bit [N, hidden] (in place); ``pending`` the previous block's update or
        None; ``shift`` None or a 32-bit vector that is added to every row of ``h`` before
        anything else (in the first norm's kernel).  Returns this block's last update, still
        to be added (None when it has already been added)."""
        enter = (lambda: self.input_norm.add_forward(h, pending)) if shift is None else \
            (lambda: self.input_norm.add_forward(h, pending, shift=shift))
        chain = None
        if shift is None and self.ffn is not None and batch.n_tokens <= native.CHAIN_MAX_TOKENS and self.ctx.timer is None:
            chain = self._chain()
        if chain is not None:
            # few tokens: output projection (+= h), norm + gate/up with SiLU*mul and the down
            # projection (+= h) run as one persistent kernel whose weight stream never stops
            o_proj, norm, gate_up, down = chain
            normed = enter()
            heads = self.mixer.attend(normed, batch, cache)
            act = torch.empty((h.shape[0], gate_up.out_features // 2), dtype=torch.bfloat16, device=h.device)
            native.decode_chain(
                [dict(w=o_proj.weight, x=heads, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD),
                 dict(w=gate_up.weight, x=h, norm_w=norm.weight, eps=norm.eps, out=act,
                      src=native.CHAIN_SRC_NORM, epi=native.CHAIN_SILU_MUL),
                 dict(w=down.weight, x=act, out=h, src=native.CHAIN_SRC_ACTIVATIONS, epi=native.CHAIN_ADD)],
                h.shape[0], self.ctx.status)
            return None
        if self.ctx.timer is None:
            # a part that can add its update into the residual stream itself (in the epilogue of
            # its last projection) does so; the norm after it then only reads the stream
            normed = enter()
            adds = getattr(self.mixer, "forward_add", None)
            update = None if adds is not None and adds(normed, batch, cache, h) else self.mixer.forward(normed, batch, cache)
            if self.ffn is None:
                return update
            normed = self.post_norm.add_forward(h, update)
            adds = getattr(self.ffn, "forward_add", None)
            return None if adds is not None and adds(normed, h) else self.ffn.forward(normed)
        with self.ctx.section("input_norm"):
            normed = enter()
        with self.ctx.section("mixer"):
            update = self.mixer.forward(normed, batch, cache)
        if self.ffn is None:
            return update
        with self.ctx.section("post_norm"):
            normed = self.post_norm.add_forward(h, update)
        with self.ctx.section("ffn"):
            return self.ffn.forward(normed)


class StreamMixBlock:
    """Pre-norm sublayers over several copies of the residual stream.

    The stream ``h`` is 32-bit [N, S, hidden].  A sublayer (the mixer; then the feed-forward,
    if the layer has one) reads u = sum_s in[s] x_s through its norm and writes back
    x_t = sum_s mix[s, t] x_s + c out[t] y for all t at once, c being the spec's
    ``update_scale``.  With ``learned`` false there is one stream and in = out = mix = 1:
    the plain x += c y.  Adding a sublayer's output and normalising for the next one is one
    kernel launch; the block hands its last output on, unadded, as ``(y, mix, out, c)``, and
    ``close`` folds the last one of the model into the final norm of the summed streams."""

    roles = ("input_norm", "mixer", "post_norm", "ffn", "mix1", "mix2")

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.ctx = ctx
        self.options = spec.options
        self.scale = float(spec.options.update_scale)
        self.input_norm = build_part(spec.input_norm, weights["input_norm"], ctx)
        self.mixer = build_part(spec.mixer, weights["mixer"], ctx)
        self.ffn = self.post_norm = None
        if spec.ffn is not None:
            self.post_norm = build_part(spec.post_norm, weights["post_norm"], ctx)
            self.ffn = build_part(spec.ffn, weights["ffn"], ctx)
        self.coefficients = [(None, None, None), (None, None, None)]      # (in, out, mix) per sublayer
        if spec.options.learned:
            for index, role in enumerate(("mix1", "mix2")):
                if role in weights:
                    part = weights[role]
                    self.coefficients[index] = tuple(
                        part[key].to(device=ctx.device, dtype=torch.float32).contiguous() for key in ("in", "out", "mix"))

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """role -> {local name -> WeightInfo}"""
        streams = spec.options.streams
        mixing = {"in": WeightInfo((streams,), "norm"), "out": WeightInfo((streams,), "norm"),
                  "mix": WeightInfo((streams, streams), "identity")}
        shapes = {"input_norm": part_class(spec.input_norm).weight_shapes(spec.input_norm),
                  "mixer": part_class(spec.mixer).weight_shapes(spec.mixer)}
        if spec.options.learned:
            shapes["mix1"] = dict(mixing)
        if spec.ffn is not None:
            shapes["post_norm"] = part_class(spec.post_norm).weight_shapes(spec.post_norm)
            shapes["ffn"] = part_class(spec.ffn).weight_shapes(spec.ffn)
            if spec.options.learned:
                shapes["mix2"] = dict(mixing)
        return shapes

    def cache_needs(self):
        return self.mixer.cache_needs()

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        planner = getattr(self.mixer, "plan_step", None)
        if planner is not None:
            planner(entries, page_size, plans)

    @property
    def graph_safe(self) -> bool:
        parts = [self.input_norm, self.mixer] + ([self.post_norm, self.ffn] if self.ffn is not None else [])
        return all(getattr(part, "graph_safe", False) for part in parts)

    def _enter(self, h, pending, sublayer: int, norm):
        """Add what is pending, mix, and normalise the sublayer's input."""
        update, mix, out, scale = pending if pending is not None else (None, None, None, 1.0)
        normed = torch.empty((h.shape[0], h.shape[-1]), dtype=self.ctx.dtype, device=h.device)
        native.stream_mix_norm(h, update, scale, mix, out, self.coefficients[sublayer][0], norm.stream_kind,
                               norm.weight, norm.eps, normed)
        return normed

    def forward(self, h, pending, batch, cache: CacheView):
        with self.ctx.section("input_norm"):
            normed = self._enter(h, pending, 0, self.input_norm)
        with self.ctx.section("mixer"):
            update = self.mixer.forward(normed, batch, cache)
        pending = (update, self.coefficients[0][2], self.coefficients[0][1], self.scale)
        if self.ffn is None:
            return pending
        with self.ctx.section("post_norm"):
            normed = self._enter(h, pending, 1, self.post_norm)
        with self.ctx.section("ffn"):
            update = self.ffn.forward(normed)
        return (update, self.coefficients[1][2], self.coefficients[1][1], self.scale)

    def close(self, h, pending, final_norm, row_map):
        """The model's last step: what is pending is added, the streams are summed, and the
        final norm is taken - for the rows of ``row_map`` only, without writing the streams."""
        update, mix, out, scale = pending if pending is not None else (None, None, None, 1.0)
        normed = torch.empty((row_map.numel(), h.shape[-1]), dtype=self.ctx.dtype, device=h.device)
        native.stream_mix_norm(h, update, scale, mix, out, None, final_norm.stream_kind, final_norm.weight,
                               final_norm.eps, normed, row_map, write_streams=False)
        return normed


register_arrangement("pre_norm", PreNormBlock, replace=True)
register_arrangement("stream_mix", StreamMixBlock, replace=True)


class SandwichConvBlock:
    """Sublayers with a norm on both sides and a short causal convolution on their input.

    x += norm_b(sublayer(u)) with u = y + conv(y), y = norm(x): for the mixer, then for the
    feed-forward if the layer has one.  The residual stream ``h`` is 32-bit.  A sublayer's
    update is handed on unadded, with the norm that still has to be taken of it, and one kernel
    launch normalises it, adds it and normalises the stream for the next sublayer; the
    convolution runs on those 32-bit rows and rounds once, for the sublayer's projections.
    The last taps - 1 rows of y of either sublayer are the block's own state per request
    (``CacheNeeds.own_state`` [2, taps - 1, hidden]), its own also in a layer that reads
    another layer's keys and values."""

    roles = ("input_norm", "mixer", "mixer_out_norm", "post_norm", "ffn", "ffn_out_norm", "conv")

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        from ..config.specs import local_name

        self.ctx = ctx
        options = spec.options
        self.taps = int(options.taps)
        if not 1 <= self.taps <= native.CONV_MAX_TAPS:
            raise ValueError(f"a convolution of {self.taps} taps; the kernel takes 1 to {native.CONV_MAX_TAPS}")
        self.width = spec.input_norm.size
        self.input_norm = build_part(spec.input_norm, weights["input_norm"], ctx)
        self.mixer = build_part(spec.mixer, weights["mixer"], ctx)
        self.mixer_out_norm = build_part(options.mixer_out_norm, weights["mixer_out_norm"], ctx)
        self.post_norm = self.ffn = self.ffn_out_norm = None
        if spec.ffn is not None:
            self.post_norm = build_part(spec.post_norm, weights["post_norm"], ctx)
            self.ffn = build_part(spec.ffn, weights["ffn"], ctx)
            self.ffn_out_norm = build_part(options.ffn_out_norm, weights["ffn_out_norm"], ctx)
        # stored [hidden, taps]; the kernel reads a tap's weights side by side
        self.conv = [weights["conv"][local_name(options, key)].to(device=ctx.device, dtype=torch.float32).t().contiguous()
                     for key in (("conv1", "conv2") if spec.ffn is not None else ("conv1",))]

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """role -> {local name -> WeightInfo}"""
        from ..config.specs import local_name

        options = spec.options
        shape = WeightInfo((spec.input_norm.size, options.taps), "small")
        shapes = {"input_norm": part_class(spec.input_norm).weight_shapes(spec.input_norm),
                  "mixer": part_class(spec.mixer).weight_shapes(spec.mixer),
                  "mixer_out_norm": part_class(options.mixer_out_norm).weight_shapes(options.mixer_out_norm),
                  "conv": {local_name(options, "conv1"): shape}}
        if spec.ffn is not None:
            shapes["post_norm"] = part_class(spec.post_norm).weight_shapes(spec.post_norm)
            shapes["ffn"] = part_class(spec.ffn).weight_shapes(spec.ffn)
            shapes["ffn_out_norm"] = part_class(options.ffn_out_norm).weight_shapes(options.ffn_out_norm)
            shapes["conv"][local_name(options, "conv2")] = shape
        return shapes

    def cache_needs(self):
        import dataclasses

        from ..cache.manager import StateSpec

        needs = self.mixer.cache_needs()
        if self.taps > 1:
            needs = dataclasses.replace(needs, own_state=StateSpec((2, self.taps - 1, self.width), "float32"))
        return needs

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        planner = getattr(self.mixer, "plan_step", None)
        if planner is not None:
            planner(entries, page_size, plans)

    @property
    def graph_safe(self) -> bool:
        parts = [self.input_norm, self.mixer, self.mixer_out_norm]
        if self.ffn is not None:
            parts += [self.post_norm, self.ffn, self.ffn_out_norm]
        return all(getattr(part, "graph_safe", False) for part in parts)

    def _enter(self, h, pending, norm, sublayer: int, batch, cache: CacheView):
        """Add what is pending (normalised), normalise the stream, convolve: the sublayer's input."""
        update = out_norm = None
        if isinstance(pending, tuple):
            update, out_norm = pending
        elif pending is not None:
            h.add_(pending)              # a block of another arrangement handed a plain update on
        u = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        state = None if cache.own_state is None else cache.own_state[:, sublayer]
        if batch.max_new == 1 and batch.n_entries == h.shape[0]:
            # every entry brings one token: norms, sum and convolution in one launch
            native.add_normed_rmsnorm(h, update, None if out_norm is None else out_norm.weight, norm.weight, u,
                                      0.0 if out_norm is None else out_norm.eps, norm.eps,
                                      conv=(self.conv[sublayer], state, batch.slots))
            return u
        y = torch.empty(h.shape, dtype=torch.float32, device=h.device)
        native.add_normed_rmsnorm(h, update, None if out_norm is None else out_norm.weight, norm.weight, y,
                                  0.0 if out_norm is None else out_norm.eps, norm.eps)
        native.causal_conv_state(y, self.conv[sublayer], state, batch.slots, batch.cu_tokens, batch.token_entry, u,
                                 batch.n_entries)
        return u

    def forward(self, h, pending, batch, cache: CacheView):
        with self.ctx.section("input_norm"):
            u = self._enter(h, pending, self.input_norm, 0, batch, cache)
        with self.ctx.section("mixer"):
            update = self.mixer.forward(u, batch, cache)
        pending = (update, self.mixer_out_norm)
        if self.ffn is None:
            return pending
        with self.ctx.section("post_norm"):
            u = self._enter(h, pending, self.post_norm, 1, batch, cache)
        with self.ctx.section("ffn"):
            update = self.ffn.forward(u)
        return (update, self.ffn_out_norm)

    def close(self, h, pending, final_norm, row_map):
        """The model's last step: the pending update is normalised and added and the final norm
        taken, for the rows of ``row_map`` only and without writing the stream."""
        update, out_norm = pending if isinstance(pending, tuple) else (pending, None)
        normed = torch.empty((row_map.numel(), h.shape[-1]), dtype=self.ctx.dtype, device=h.device)
        if out_norm is None:
            return final_norm.add_forward(h, update, row_map=row_map)
        native.add_normed_rmsnorm(h, update, out_norm.weight, final_norm.weight, normed, out_norm.eps, final_norm.eps,
                                  row_map=row_map, write_residual=False)
        return normed


register_arrangement("sandwich_conv", SandwichConvBlock, replace=True)


class OutputNormBlock:
    """Sublayers that read the residual stream as it is and whose output is normalised before
    it joins the stream: x += norm_a(mixer(x)), then x += norm_b(ff(x)) if the layer has a
    feed-forward.  The stream ``h`` is 32-bit.  A sublayer's update is handed on unadded,
    together with the norm that still has to be taken of it; one kernel launch normalises it,
    adds it and writes the sum once more in the activation dtype, which is what the next
    sublayer's projections read (in the 32-bit engine an exact copy).  The model's last norm
    takes the pending update along through ``close``.  Updates are kept as the 32-bit sums of
    the sublayer's last projection where the part can give them."""

    roles = ("mixer", "mixer_out_norm", "ffn", "ffn_out_norm")

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.ctx = ctx
        options = spec.options
        self.mixer = build_part(spec.mixer, weights["mixer"], ctx)
        self.mixer_out_norm = build_part(options.mixer_out_norm, weights["mixer_out_norm"], ctx)
        self.ffn = self.ffn_out_norm = None
        if spec.ffn is not None:
            self.ffn = build_part(spec.ffn, weights["ffn"], ctx)
            self.ffn_out_norm = build_part(options.ffn_out_norm, weights["ffn_out_norm"], ctx)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        """role -> {local name -> WeightInfo}"""
        options = spec.options
        shapes = {"mixer": part_class(spec.mixer).weight_shapes(spec.mixer),
                  "mixer_out_norm": part_class(options.mixer_out_norm).weight_shapes(options.mixer_out_norm)}
        if spec.ffn is not None:
            shapes["ffn"] = part_class(spec.ffn).weight_shapes(spec.ffn)
            shapes["ffn_out_norm"] = part_class(options.ffn_out_norm).weight_shapes(options.ffn_out_norm)
        return shapes

    def cache_needs(self):
        return self.mixer.cache_needs()

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        planner = getattr(self.mixer, "plan_step", None)
        if planner is not None:
            planner(entries, page_size, plans)

    @property
    def graph_safe(self) -> bool:
        parts = [self.mixer, self.mixer_out_norm] + ([self.ffn, self.ffn_out_norm] if self.ffn is not None else [])
        return all(getattr(part, "graph_safe", False) for part in parts)

    def _enter(self, h, pending):
        """Add what is pending (normalised) and hand the stream on in the activation dtype."""
        update = out_norm = None
        if isinstance(pending, tuple):
            update, out_norm = pending
        elif pending is not None:
            h.add_(pending)              # a block of another arrangement handed a plain update on
        u = torch.empty(h.shape, dtype=self.ctx.dtype, device=h.device)
        native.add_normed_rmsnorm(h, update, None if out_norm is None else out_norm.weight, None, u,
                                  0.0 if out_norm is None else out_norm.eps, 0.0)
        return u

    def _mix(self, u, batch, cache):
        """The mixer's update, as the 32-bit sums of its output projection where it has one."""
        attend, o_proj = getattr(self.mixer, "attend", None), getattr(self.mixer, "o_proj", None)
        if attend is None or o_proj is None:
            return self.mixer.forward(u, batch, cache)
        heads = attend(u, batch, cache)
        with self.ctx.section("mixer.o_proj"):
            return o_proj(heads, out_dtype=torch.float32)

    def forward(self, h, pending, batch, cache: CacheView):
        with self.ctx.section("input_norm"):
            u = self._enter(h, pending)
        with self.ctx.section("mixer"):
            update = self._mix(u, batch, cache)
        pending = (update, self.mixer_out_norm)
        if self.ffn is None:
            return pending
        with self.ctx.section("post_norm"):
            u = self._enter(h, pending)
        with self.ctx.section("ffn"):
            update = self.ffn.forward(u)
        return (update, self.ffn_out_norm)

    def close(self, h, pending, final_norm, row_map):
        """The model's last step: the pending update is normalised and added and the final norm
        taken, for the rows of ``row_map`` only and without writing the stream."""
        update, out_norm = pending if isinstance(pending, tuple) else (pending, None)
        if out_norm is None:
            return final_norm.add_forward(h, update, row_map=row_map)
        normed = torch.empty((row_map.numel(), h.shape[-1]), dtype=self.ctx.dtype, device=h.device)
        native.add_normed_rmsnorm(h, update, out_norm.weight, final_norm.weight, normed, out_norm.eps, final_norm.eps,
                                  row_map=row_map, write_residual=False)
        return normed


register_arrangement("output_norm", OutputNormBlock, replace=True)
