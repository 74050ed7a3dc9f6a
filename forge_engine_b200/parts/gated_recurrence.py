"""Linear attention whose forget gate also decides what is written (a gated linear recurrence).

q = silu(W_q x) [heads x dim], v = W_v x [heads x vdim], and per head and channel a forget
gate f = l + (1 - l) sigmoid(W_f x + b_f) that a learned lower bound l keeps away from zero.
Per head the state S [dim, vdim] follows S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T (there is no
key: what the gate lets go of, the value fills) and the output is o_t = S_t^T q_t, divided by
its root mean square over the head's values and multiplied by a weight vector all heads share.
The heads are then projected.  The state is 32-bit, starts at zero and lives in the request's
state slot between steps; q, f and v are one fused projection whose 32-bit sums the recurrence
kernel reads: activations, gates and the output's norm are taken there, in 32-bit.
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheNeeds, StateSpec
from ..config.specs import local_name
from ..ops import native
from .base import BuildContext, CacheView, Mixer, WeightInfo, register_part
from .linear import Linear, fused_rows


class GatedRecurrence(Mixer):
    graph_safe = True      # the state is indexed on the device, by the batch's slots

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.spec, self.ctx = spec, ctx
        self.h, self.dk, self.dv = spec.num_heads, spec.head_dim, spec.v_head_dim
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        qk, v = self.h * self.dk, self.h * self.dv
        self.proj = Linear(fused_rows(weights, [name("q"), name("f"), name("v")], [qk, qk, v]), status=ctx.status)
        vector = lambda key: weights[name(key)].to(device=ctx.device, dtype=torch.float32).reshape(-1).contiguous()  # noqa: E731
        self.f_bias, self.lower, self.norm = vector("f.bias"), vector("lower"), vector("norm")
        self.o_proj = Linear(weights[name("o")], status=ctx.status)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        qk, v, w = spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim, spec.hidden_size
        return {
            name("q"): WeightInfo((qk, w)),
            name("f"): WeightInfo((qk, w)),
            name("f.bias"): WeightInfo((qk,), "bias"),
            name("lower"): WeightInfo((qk,), "bias"),
            name("v"): WeightInfo((v, w)),
            name("norm"): WeightInfo((spec.v_head_dim,), "norm"),
            name("o"): WeightInfo((w, v)),
        }

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(state=StateSpec((self.h, self.dk, self.dv), "float32"))

    def mix(self, x, batch, cache: CacheView):
        """Everything but the output projection: the normalised heads [N, heads * vdim]."""
        qk = self.h * self.dk
        with self.ctx.section("mixer.projection"):
            proj = self.proj(x, out_dtype=torch.float32)
        mixed = torch.empty((x.shape[0], self.h * self.dv), dtype=self.ctx.dtype, device=x.device)
        with self.ctx.section("mixer.recurrence"):
            native.gated_recurrence(proj, 0, qk, 2 * qk, self.f_bias, self.lower, self.norm, self.spec.norm_eps,
                                    cache.state, batch.slots, batch.cu_tokens, mixed, batch.n_entries, self.ctx.status,
                                    max_new=batch.max_new)
        return mixed

    def forward(self, x, batch, cache: CacheView):
        mixed = self.mix(x, batch, cache)
        with self.ctx.section("mixer.o_proj"):
            return self.o_proj(mixed, out_dtype=torch.float32)


register_part("gated_recurrence", GatedRecurrence, replace=True)
