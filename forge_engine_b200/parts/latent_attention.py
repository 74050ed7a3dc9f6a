"""Causal attention over one cached latent per token.

Queries pass through a normalised latent of their own: c_q = rmsnorm(W_dq x), q = W_uq c_q,
every head [head_dim elements that are not rotated | rot_dim that are].  Keys and values are
expanded from a second latent: W_dkv x gives kv_rank + rot_dim numbers; the first kv_rank,
RMS-normalised, are the latent c, the last rot_dim, rotated, are a key part that all heads
share.  Head h's key is [W_uk,h c | shared part], its value W_uv,h c.  Only c and the shared
part are kept in the cache: one vector of kv_rank + rot_dim per token for all heads.

The expansion is never carried out for cached tokens.  Since q_h . (W_uk,h c) =
(W_uk,h^T q_h) . c, the step's queries are taken through W_uk,h^T once (kv_rank numbers per
head), attention then runs with one shared "kv head" whose key is the cached vector itself
and whose value is its first kv_rank elements, and the weighted sum of latents is expanded by
W_uv,h afterwards.  A step's cost does not depend on how many heads read the cache.

A layer with ``kv_from`` has no W_dkv and reads the cache of the layer named there.

``window``: a query sees its own and the window - 1 tokens before it, and the pages the window
has passed go back to the pool.  ``sink``: a learned number per head whose exponential joins
the softmax's denominator once, as a weight on no key and no value.
"""

from __future__ import annotations

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..config.specs import local_name
from ..ops import native
from .base import BuildContext, CacheView, Mixer, WeightInfo, build_part, register_part
from .linear import Linear, fused_rows


class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.spec, self.ctx = spec, ctx
        self.h, self.d, self.r, self.dv = spec.num_heads, spec.head_dim, spec.rot_dim, spec.v_head_dim
        self.q_rank, self.kv_rank = spec.q_rank, spec.kv_rank
        self.own = spec.kv_from is None
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        # one projection for both latents of a layer that has both
        if self.own:
            down = fused_rows(weights, [name("dq"), name("dkv")], [self.q_rank, self.kv_rank + self.r])
        else:
            down = weights[name("dq")]
        self.down = Linear(down, status=ctx.status)
        self.q_norm = weights[name("dq.norm")].float().contiguous()
        self.kv_norm = weights[name("dkv.norm")].float().contiguous() if self.own else None
        self.up_q = Linear(weights[name("uq")], status=ctx.status)
        uk = weights[name("uk")]
        # [head, kv_rank, head_dim]: the transpose of every head's key expansion
        self.uk_t = uk.view(self.h, self.d, self.kv_rank).transpose(1, 2).contiguous()
        del uk
        self.uv = weights[name("uv")].contiguous().view(self.h, self.dv, self.kv_rank)
        self.o_proj = Linear(weights[name("o")], status=ctx.status)
        self.position = build_part(spec.position, {}, ctx)
        self.rot_dims = self.position.rotary()[1]
        self.window = getattr(spec, "window", None) or None
        self.sinks = None
        if getattr(spec, "sink", False):
            self.sinks = weights[name("sink")].to(device=ctx.device, dtype=torch.float32).contiguous()
        self.plan_key = ("latent_attention", self.h, self.kv_rank, self.r, self.window)

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        """The host's decision for a step of ``entries`` ((slot, cached, new) each): how many
        blocks share the keys of one tile of query rows (layers of one geometry share it)."""
        if self.plan_key not in plans:
            splits = 1
            if native.general_mma_takes(self.ctx.dtype, self.kv_rank + self.r, self.kv_rank):
                splits = native.general_splits(entries, self.h, 1, self.window)
            plans[self.plan_key] = splits

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        h, w = spec.num_heads, spec.hidden_size
        shapes = {
            name("dq"): WeightInfo((spec.q_rank, w)),
            name("dq.norm"): WeightInfo((spec.q_rank,), "norm"),
            name("uq"): WeightInfo((h * (spec.head_dim + spec.rot_dim), spec.q_rank)),
        }
        if spec.kv_from is None:
            shapes[name("dkv")] = WeightInfo((spec.kv_rank + spec.rot_dim, w))
            shapes[name("dkv.norm")] = WeightInfo((spec.kv_rank,), "norm")
        shapes[name("uk")] = WeightInfo((h * spec.head_dim, spec.kv_rank))
        shapes[name("uv")] = WeightInfo((h * spec.v_head_dim, spec.kv_rank))
        shapes[name("o")] = WeightInfo((w, h * spec.v_head_dim))
        if getattr(spec, "sink", False):
            shapes[name("sink")] = WeightInfo((h,), "bias")
        return shapes

    def cache_needs(self) -> CacheNeeds:
        return CacheNeeds(kv=PagedKVSpec(1, self.kv_rank + self.r, self.window, 0))

    def forward(self, x, batch, cache: CacheView):
        out = self.attend(x, batch, cache)
        with self.ctx.section("mixer.o_proj"):
            return self.o_proj(out)

    def _per_head(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
        """out[n, h] = x[n, h] @ w[h].T for x [N, heads, k], w [heads, o, k], out [N, heads, o]
        (x and out may be strided).  The 32-bit engine uses the plain FFMA kernel; bfloat16
        the library's batched product, as the large projections do."""
        if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[0] > native.TC5_MAX_ROWS:
            out.copy_(torch.bmm(x.transpose(0, 1), w.transpose(1, 2)).transpose(0, 1))
        else:
            native.gemm_simt_batched(x, w, out)

    def attend(self, x, batch, cache: CacheView):
        n, h, d, r, dv, rank = x.shape[0], self.h, self.d, self.r, self.dv, self.kv_rank
        latent_cache = cache.kv[0]
        table = batch.group_tables[cache.group]
        dtype = latent_cache.dtype
        with self.ctx.section("mixer.qkv_rope_cache"):
            down = self.down(x, out_dtype=torch.float32)
            angles = self.position.table(batch)
            c_q = torch.empty((n, self.q_rank), dtype=dtype, device=x.device)
            writes = self.own and cache.owns
            # the query latent is normalised; the key/value latent is normalised, its last
            # rot_dim elements are rotated instead, and the vector goes to its page
            native.qkv_prepare(
                q=down[:, : self.q_rank], q_heads=1, q_dim=self.q_rank,
                q_norm=(native.PREP_NORM_HEAD, self.q_rank, self.q_norm), q_rot_off=-1,
                q_out=c_q, q_out_strides=(self.q_rank, self.q_rank),
                k=down[:, self.q_rank:] if writes else None, k_heads=1, k_dim=rank + r,
                k_norm=(native.PREP_NORM_HEAD if writes else native.PREP_NORM_NONE, rank, self.kv_norm), k_rot_off=rank,
                eps=self.spec.norm_eps, table=angles, rot_dims=self.rot_dims, interleaved=self.position.interleaved,
                k_cache=latent_cache, block_table=table, positions=batch.positions, token_entry=batch.token_entry,
                status=self.ctx.status,
            )
            q = self.up_q(c_q)                                     # [N, heads * (d + r)]
            q_eff = torch.empty((n, h, rank + r), dtype=dtype, device=x.device)
            # rotated parts of the queries straight to where attention reads them
            native.qkv_prepare(
                q=q[:, d:], q_heads=h, q_dim=r, q_head_stride=d + r, q_rot_off=0,
                q_out=q_eff, q_out_strides=(h * (rank + r), rank + r), q_out_offset=rank,
                table=angles, rot_dims=self.rot_dims, interleaved=self.position.interleaved,
                positions=batch.positions, token_entry=batch.token_entry, status=self.ctx.status,
            )
            # the other parts through the transposed key expansion
            self._per_head(q.view(n, h, d + r)[:, :, :d], self.uk_t, q_eff[:, :, :rank])
        mixed = torch.empty((n, h, rank), dtype=dtype, device=x.device)
        if self.plan_key not in batch.plans:
            self.plan_step(batch.entries, latent_cache.shape[2], batch.plans)
        with self.ctx.section("mixer.attention"):
            native.attention_general(q_eff, (h * (rank + r), rank + r), latent_cache, rank + r, latent_cache, rank,
                                     mixed, (h * rank, rank), table, batch.positions, batch.token_entry, h, None, self.window,
                                     self.spec.scale, self.ctx.status,
                                     entries=(batch.cu_tokens, batch.starts, batch.n_entries, batch.max_new),
                                     splits=batch.plans[self.plan_key], sinks=self.sinks)
        heads = torch.empty((n, h, dv), dtype=dtype, device=x.device)
        with self.ctx.section("mixer.expand"):
            self._per_head(mixed, self.uv, heads)
        return heads.view(n, h * dv)


register_part("latent_attention", LatentAttention, replace=True)
