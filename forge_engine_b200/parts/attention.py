"""Causal grouped-query attention over the paged cache.

Formulas: src/forge_engine/qwen3.py:108-207.  One fused projection gives q, k, v; one
kernel normalises q and k per head, rotates them and stores k, v into their pages; the
attention kernel then reads everything it needs from the pages, so a step's new tokens
and the earlier ones are treated alike.  The mixer keeps PagedKVSpec(kv heads,
head_dim, window) between steps.
"""

from __future__ import annotations

import functools
import math
import os

import torch

from ..cache.manager import CacheNeeds, PagedKVSpec
from ..config.specs import local_name
from ..errors import ConfigError, UnsupportedShapeError
from ..ops import native
from .base import BuildContext, CacheView, Mixer, WeightInfo, build_part, register_part
from .linear import Linear, fused_rows


# Blocks of a decode kernel the GPU holds at once when nothing says otherwise (two per SM on
# the 148 SMs of a B200); a mixer asks the kernel library for the figure of its device.
DEFAULT_DECODE_SLOTS = 296
MAX_SPLITS = 64   # what the merge takes
SHORT_ENTRY_ROWS = 16   # general layers: entries with more rows (new tokens x heads per kv head) may take the tcgen05 prefill kernel
# With more tokens a block of the projection finishes so many that the separate kernel is
# faster (measured: 2.35 -> 2.27 ms per step at 1 token, no change at 8, 6.2 -> 6.7 ms at 64).
FUSED_PROJECTION_ROWS = 16
CLUSTER_SPLITS = 8            # this many blocks combine their results inside a cluster
CLUSTER_WORTH_TILES = 96      # from here on (6,144 keys) more than one cluster per pair pays

# Costs in units of one 64-key tile of one block (about 1.4 us), from measurements of the
# split decode kernel on a B200: combining the splits inside a cluster, through global
# memory, and what every round of blocks over the machine's slots costs beside its tiles.
MERGE_IN_CLUSTER, MERGE_THROUGH_MEMORY, ROUND_OVERHEAD = 2, 9, 3
SPLIT_TILE_US = 1.45
BALANCED_BASE_US, BALANCED_TILE_US, BALANCED_PAIR_US, BALANCED_PIECE_US = 15.0, 0.0049, 0.003, 0.27
BALANCED_MAX_ENTRIES = 256    # what the balanced kernel keeps in shared memory


def choose_splits(tile_counts, kv_heads: int, balanced: bool = False, slots: int = DEFAULT_DECODE_SLOTS) -> int:
    """How many blocks share one (request, kv head)'s keys; ``tile_counts`` are the 64-key
    tiles of the step's requests.  Every request gets the same number of splits.  With
    ``balanced`` the answer may be 0: the kernel that spreads all tiles evenly over the
    machine's blocks is expected to be faster than any split.  ``slots``: blocks of the
    decode kernels the GPU holds at once."""
    return _choose_splits(tuple(sorted(max(1, int(t)) for t in tile_counts)), int(kv_heads), bool(balanced),
                          max(1, int(slots)))


def _even_splits(pairs: int, tiles: int, DECODE_SLOTS: int) -> int:
    """Requests of about the same length (measured on a B200, 8 kv heads, head size 128).
    Few pairs: fill the machine's slots once, every block getting at least four tiles; up to 8
    blocks combine inside a cluster, and going beyond (clusters of 8 whose results pass through
    memory) pays from about 6,000 keys on (one request: 8,192 keys 22.9 us with 8 splits,
    17.3 us with 32; 2,048 keys 7.7 against 10.8 us with 16).  With more pairs than half the
    slots the machine is full anyway: one split up to 4,096 keys (512 pairs of 2,048 keys:
    100 us against 116 us with two), two beyond.  Clusters of 3, 5, 6 or 7 blocks measured
    badly (12 requests: 38.8 us with 3 splits, 28.3 us with 2), so counts are powers of two."""
    most = max(1, min(MAX_SPLITS, tiles // 4))
    if pairs * 2 > DECODE_SLOTS:
        return 1 if tiles <= 64 else min(most, 2)
    splits = max(1, min(most, DECODE_SLOTS // pairs))
    if splits > CLUSTER_SPLITS:
        return CLUSTER_SPLITS if tiles < CLUSTER_WORTH_TILES else splits - splits % CLUSTER_SPLITS
    return 1 << (splits.bit_length() - 1)


def _split_cost(tile_counts: tuple, kv_heads: int, splits: int, DECODE_SLOTS: int) -> int:
    """Estimate for ``splits`` blocks per pair, in tiles of one block: the longest request
    decides how long its blocks run, while all blocks together pass through the machine's
    slots, in rounds if they are more: max(longest / s, all tiles / slots, rounds x the median
    block) + the cost of combining + an overhead per round."""
    pairs = len(tile_counts) * kv_heads
    longest, median = tile_counts[-1], tile_counts[len(tile_counts) // 2]
    total = sum(tile_counts) * kv_heads
    rounds = -(-pairs * splits // DECODE_SLOTS)
    merge = 0 if splits == 1 else (MERGE_IN_CLUSTER if splits <= CLUSTER_SPLITS else MERGE_THROUGH_MEMORY)
    tiles = max(-(-longest // splits), -(-total // DECODE_SLOTS), rounds * -(-median // splits))
    return tiles + merge + ROUND_OVERHEAD * rounds


@functools.lru_cache(maxsize=4096)
def _choose_splits(tile_counts: tuple, kv_heads: int, balanced: bool, DECODE_SLOTS: int) -> int:
    pairs = len(tile_counts) * kv_heads
    longest = tile_counts[-1]
    median = tile_counts[len(tile_counts) // 2]
    if longest < 2 * median:
        best = _even_splits(pairs, longest, DECODE_SLOTS)
    else:
        # One request much longer than most.  Measured: one request of 32,768 keys beside seven
        # of 2,048: 176 us with the 4 splits of even requests, 94-102 us with 16-32; one of
        # 16,384 beside 31 of 1,024: 329 us with 1, 108 us with 8; one of 8,192 beside 63 of
        # 2,048: 219 us with 1, 171 us with 2, 147 us with 4.
        best, best_cost = 1, None
        for splits in (1, 2, 4, 8, 16, 24, 32, 40, 48, 56, 64):
            if splits > 1 and (longest // splits < 2 or splits > MAX_SPLITS):
                break
            cost = _split_cost(tile_counts, kv_heads, splits, DECODE_SLOTS)
            if best_cost is None or cost < best_cost:
                best, best_cost = splits, cost
    if balanced and len(tile_counts) <= BALANCED_MAX_ENTRIES:
        # The balanced kernel (and the kernel that combines the pairs it cut) measured
        # 15 us + 4.9 ns per tile + 3 ns per pair, whatever the lengths are (8 requests of 2,048
        # keys 26 us, 64 of them 97 us, 200 of 300 keys 61 us); a tile of the split kernel's
        # estimate is 1.45 us (32 requests of 2,048 keys: 35 tiles, 50 us measured).  The
        # balanced kernel wins where blocks would run in two uneven rounds (40 requests of
        # 3,000 keys: 134 -> 90 us) and wherever lengths differ much (one request of 32,768
        # keys beside seven of 2,048: 96 -> 49 us; 64 requests of 16 to 4,096 keys: 140 -> 95 us).
        # Combining costs by the pieces of the longest pair (one request of 8,192 keys is cut
        # into 37 pieces per kv head: 31 us, against 17 us with 32 splits).
        total = sum(tile_counts) * kv_heads
        pieces = min(DECODE_SLOTS, longest * DECODE_SLOTS // total + 1)
        balanced_us = (BALANCED_BASE_US + BALANCED_TILE_US * total + BALANCED_PAIR_US * pairs
                       + BALANCED_PIECE_US * pieces)
        if balanced_us < SPLIT_TILE_US * _split_cost(tile_counts, kv_heads, best, DECODE_SLOTS):
            return 0
    return best


class GQAttention(Mixer):
    @property
    def graph_safe(self) -> bool:
        """The kernels here are; a position encoding that rewrites q and k itself decides."""
        return bool(getattr(self.position, "graph_safe", False))

    @staticmethod
    def _is_general(spec) -> bool:
        """Whether the layer needs what only the general kernels do: values of another size
        than keys, q and k normalised over the whole projection, a bias on the distance, kept
        first tokens, capped scores, a query temperature, a gate per head, two maps per head, q and
        k normalised without a weight or after the rotation."""
        return (getattr(spec, "v_head_dim", None) not in (None, spec.head_dim)
                or (spec.qk_norm and getattr(spec, "qk_norm_scope", "head") == "whole")
                or getattr(spec, "distance_bias_base", None) is not None
                or getattr(spec, "distance_bias_table", None) is not None or not getattr(spec, "kv_projection", True)
                or bool(getattr(spec, "keep_first", 0)) or getattr(spec, "softcap", None) is not None
                or getattr(spec, "query_temperature", None) is not None or bool(getattr(spec, "head_gate", False))
                or getattr(spec, "differential", None) is not None
                or (spec.qk_norm and (not getattr(spec, "qk_norm_weight", True) or getattr(spec, "qk_norm_after_rotation", False))))

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        self.general = self._is_general(spec)
        if not self.general and (spec.head_dim % 16 or spec.head_dim > 256):
            raise UnsupportedShapeError(
                f"head_dim={spec.head_dim}: the attention kernels take multiples of 16 up to 256"
            )
        if spec.num_heads % spec.num_kv_heads:
            raise UnsupportedShapeError("num_heads must be a multiple of num_kv_heads")
        if getattr(spec, "qk_norm_scope", "head") not in ("head", "whole"):
            raise ConfigError(f"qk_norm_scope={spec.qk_norm_scope!r}; known: head, whole")
        self.spec = spec
        self.ctx = ctx
        self.nq, self.nkv, self.d = spec.num_heads, spec.num_kv_heads, spec.head_dim
        self.dv = getattr(spec, "v_head_dim", None) or self.d
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        # a differential layer has ``parts`` = 2 queries and keys of ``head_dim`` per head, side by side
        self.differential = getattr(spec, "differential", None)
        self.parts = 1 if self.differential is None else 2
        self.head_gate = bool(getattr(spec, "head_gate", False))
        self.keep_first = int(getattr(spec, "keep_first", 0) or 0) if spec.window else 0
        self.softcap = getattr(spec, "softcap", None)
        self.query_temperature = getattr(spec, "query_temperature", None)
        if self.parts > 1 and (spec.qk_norm or spec.bias or getattr(spec.position, "kind", "none") != "none"):
            raise ConfigError("a differential layer takes no q/k norm, no bias and no rotation")
        bias = None
        rows = [self.nq * self.parts * self.d, self.nkv * self.parts * self.d, self.nkv * self.dv]
        names = [name("q_proj.weight"), name("k_proj.weight"), name("v_proj.weight")]
        # a layer without keys and values of its own projects queries only and reads another run's cache
        self.kv_projection = bool(getattr(spec, "kv_projection", True))
        if not self.kv_projection:
            if spec.bias or self.head_gate:
                raise ConfigError("a layer without key and value projections takes no biases and no gates")
            rows, names = rows[:1], names[:1]
        if self.head_gate:
            # the gates' logits are further columns of the same product
            rows.append(self.nq)
            names.append(name("gate_proj.weight"))
        if spec.bias:
            if self.head_gate:
                raise ConfigError("a gate per head together with biases is not implemented")
            bias = fused_rows(weights, [name("q_proj.bias"), name("k_proj.bias"), name("v_proj.bias")], rows)
        # q, k and v are looked up one at a time and copied into the fused tensor
        self.qkv_proj = Linear(fused_rows(weights, names, rows), bias, status=ctx.status)
        self.diff_lambda = None
        if self.differential is not None:
            vectors = [weights[name(n)].float() for n in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2")]
            first, second = (vectors[0] * vectors[1]).sum(), (vectors[2] * vectors[3]).sum()
            self.diff_lambda = float((torch.exp(first) - torch.exp(second)).item() + float(self.differential.offset))
        self.o_proj = Linear(weights[name("o_proj.weight")], weights[name("o_proj.bias")] if self._o_bias(spec) else None,
                             status=ctx.status)
        self.q_norm = self.k_norm = None
        whole = getattr(spec, "qk_norm_scope", "head") == "whole"
        if spec.qk_norm and whole and (not getattr(spec, "qk_norm_weight", True) or getattr(spec, "qk_norm_after_rotation", False)):
            raise ConfigError("a norm over the whole projection has a weight and comes before the rotation")
        if spec.qk_norm and getattr(spec, "qk_norm_weight", True):
            self.q_norm = weights[name("q_norm.weight")].float().contiguous()
            self.k_norm = weights[name("k_norm.weight")].float().contiguous()
        self.position = build_part(spec.position, {}, ctx)
        self.slopes = None
        base = getattr(spec, "distance_bias_base", None)
        if base is not None:
            heads = torch.arange(1, self.nq + 1, dtype=torch.float64)
            self.slopes = (float(base) ** (-heads / self.nq)).float().to(ctx.device).contiguous()
        self.distance_bias = None
        table = getattr(spec, "distance_bias_table", None)
        if table is not None:
            self.distance_bias = self.expand_distance_bias(weights[name("rel")], float(table[1])).to(ctx.device)
        # the tcgen05 prefill kernel adds the bias to the unscaled score
        self.distance_bias_unscaled = None
        if self.distance_bias is not None and spec.scale > 0:
            self.distance_bias_unscaled = (self.distance_bias.double() / float(spec.scale)).float().contiguous()
        self._slots = None
        self.plan_key = ("gqa_attention", self.nq, self.nkv, self.d, spec.window) + (
            ("general", self.dv, self.parts, self.keep_first) if self.general else ())
        self.last_splits = None   # what the last step's decode entries ran with (0: balanced kernel)

    @staticmethod
    def _o_bias(spec) -> bool:
        """Whether the output projection has a bias: as q, k and v unless the spec says otherwise."""
        wish = getattr(spec, "o_bias", None)
        return bool(spec.bias) if wish is None else bool(wish)

    @staticmethod
    def expand_distance_bias(stored: torch.Tensor, far: float) -> torch.Tensor:
        """The learned bias by distance, one entry per distance: 32-bit [heads, L].  ``stored``
        [rows, heads]: distance n reads row n below h = rows // 2, and beyond that row
        min(rows - 1, h + floor(ln(n / h) / ln(far / h) * (rows - h))), which widens
        logarithmically and reaches the last row at distance ``far``; the kernels clamp the
        distance to L - 1, the first one that reads the last row."""
        rows = int(stored.shape[0])
        half = rows // 2
        if half < 1 or far <= half:
            raise ConfigError(f"a distance bias of {rows} rows needs at least 2 rows and its far distance ({far}) above {half}")
        reach = int(math.ceil(far)) + 1
        if reach > (1 << 22):
            raise UnsupportedShapeError(f"a distance bias that widens up to distance {far} is not implemented")
        n = torch.arange(reach, dtype=torch.float64)
        wide = half + torch.floor(torch.log(n.clamp(min=1) / half) / math.log(far / half) * (rows - half))
        bucket = torch.where(n < half, n, wide.clamp(max=rows - 1)).long()
        last = int((bucket == rows - 1).nonzero()[0]) if bool((bucket == rows - 1).any()) else reach - 1
        return stored.detach().float().cpu()[bucket[: last + 1]].t().contiguous()

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        dv = getattr(spec, "v_head_dim", None) or spec.head_dim
        parts = 1 if getattr(spec, "differential", None) is None else 2
        q, kv, h = spec.num_heads * parts * spec.head_dim, spec.num_kv_heads * parts * spec.head_dim, spec.hidden_size
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        shapes = {
            name("q_proj.weight"): WeightInfo((q, h)),
            name("k_proj.weight"): WeightInfo((kv, h)),
            name("v_proj.weight"): WeightInfo((spec.num_kv_heads * dv, h)),
            name("o_proj.weight"): WeightInfo((h, spec.num_heads * dv)),
        }
        if not getattr(spec, "kv_projection", True):
            del shapes[name("k_proj.weight")], shapes[name("v_proj.weight")]
        if getattr(spec, "distance_bias_table", None) is not None:
            # rows None: the stored tensor says how many rows the table has
            shapes[name("rel")] = WeightInfo((spec.distance_bias_table[0], spec.num_heads), "bias")
        if getattr(spec, "head_gate", False):
            shapes[name("gate_proj.weight")] = WeightInfo((spec.num_heads, h))
        if parts > 1:
            for vector in ("lambda_q1", "lambda_k1", "lambda_q2", "lambda_k2"):
                shapes[name(vector)] = WeightInfo((spec.head_dim,), "bias")
        if spec.qk_norm and getattr(spec, "qk_norm_weight", True):
            whole = getattr(spec, "qk_norm_scope", "head") == "whole"
            shapes[name("q_norm.weight")] = WeightInfo((q if whole else spec.head_dim,), "norm")
            shapes[name("k_norm.weight")] = WeightInfo((kv if whole else spec.head_dim,), "norm")
        if spec.bias:
            shapes[name("q_proj.bias")] = WeightInfo((q,), "bias")
            shapes[name("k_proj.bias")] = WeightInfo((kv,), "bias")
            shapes[name("v_proj.bias")] = WeightInfo((spec.num_kv_heads * dv,), "bias")
        if cls._o_bias(spec):
            shapes[name("o_proj.bias")] = WeightInfo((h,), "bias")
        return shapes

    def cache_needs(self) -> CacheNeeds:
        key = self.parts * self.d          # a differential layer caches both keys of a head in one row
        return CacheNeeds(kv=PagedKVSpec(self.nkv, key, self.spec.window, None if self.dv == key else self.dv,
                                         self.keep_first))

    def decode_slots(self) -> int:
        """Blocks of the decode kernels this device holds at once: what the balanced kernel
        of this head size is launched with (the library asks the occupancy of its own
        kernel), else two per SM."""
        if self._slots is None:
            blocks = native.attention_balanced_blocks(self.d) if self.d % 64 == 0 else 0
            if blocks <= 0:
                blocks = 2 * torch.cuda.get_device_properties(self.ctx.device).multi_processor_count
            self._slots = blocks
        return self._slots

    def forward(self, x, batch, cache: CacheView):
        out = self.attend(x, batch, cache)
        with self.ctx.section("mixer.o_proj"):
            return self.o_proj(out)

    def forward_add(self, x, batch, cache: CacheView, residual) -> bool:
        """``forward`` with the update added into the 32-bit ``residual`` by the output
        projection itself.  False (and nothing done) where that projection cannot."""
        if not self.o_proj.adds_into(x, residual) or self.ctx.timer is not None:
            return False
        return self.o_proj.add_into(self.attend(x, batch, cache), residual)

    def attend(self, x, batch, cache: CacheView):
        """Everything but the output projection: the heads' outputs [N, heads * head_dim]
        (a block that fuses ``o_proj`` with what follows takes them from here)."""
        if self.general:
            return self._attend_general(x, batch, cache)
        with self.ctx.section("mixer.qkv_rope_cache"):
            qkv = self._project(x, batch, cache)
        k_cache, v_cache = cache.kv
        table = batch.group_tables[cache.group]
        out = torch.empty((x.shape[0], self.nq * self.d), dtype=qkv.dtype, device=x.device)
        groups = self.nq // self.nkv
        with self.ctx.section("mixer.attention"):
            if qkv.dtype == torch.bfloat16 and groups <= native.ATTN_DECODE_ROWS:
                self._tensor_core_attention(qkv, k_cache, v_cache, table, batch, out, groups)
            else:
                native.attention_simt(
                    qkv, qkv.shape[1], k_cache, v_cache, table, batch.positions, batch.token_entry,
                    self.spec.window, self.spec.scale, out, self.nq, self.ctx.status,
                )
        return out

    def _attend_general(self, x, batch, cache: CacheView):
        """The layer in its general form.  The projection's 32-bit sums go to one kernel that
        normalises q and k (per head, or over the whole projection), rotates them if the
        position encoding is a rotation, and stores k and v in their pages; the attention
        kernel takes the distance bias and any key and value size."""
        n = x.shape[0]
        nq, nkv, dv = self.nq, self.nkv, self.dv
        d = self.d * self.parts              # what a head's query and key rows hold
        k_cache, v_cache = cache.kv
        table = batch.group_tables[cache.group]
        with self.ctx.section("mixer.qkv_rope_cache"):
            qkv = self.qkv_proj(x, out_dtype=torch.float32)
            rotary = self.position.rotary()
            angles, rot_dims = None, 0
            if rotary is None:
                self.position.apply(qkv, nq, nkv, d, batch)
            else:
                angles, rot_dims = self.position.table(batch), rotary[1]
            mode = native.PREP_NORM_NONE
            if self.spec.qk_norm:
                mode = native.PREP_NORM_WHOLE if self.spec.qk_norm_scope == "whole" else native.PREP_NORM_HEAD
                if getattr(self.spec, "qk_norm_after_rotation", False):
                    mode = native.PREP_NORM_HEAD_AFTER
            q = torch.empty((n, nq * d), dtype=k_cache.dtype, device=x.device)
            q_end, k_end = nq * d, (nq + nkv) * d
            if not self.kv_projection and cache.owns:
                raise ConfigError("a layer without key and value projections must read another run's cache")
            native.qkv_prepare(
                q=qkv[:, :q_end], q_heads=nq, q_dim=d, q_norm=(mode, d, self.q_norm), q_out=q, q_out_strides=(nq * d, d),
                k=qkv[:, q_end:k_end] if cache.owns else None, k_heads=nkv, k_dim=d, k_norm=(mode, d, self.k_norm),
                v=qkv[:, k_end : k_end + nkv * dv] if cache.owns else None, v_dim=dv, eps=self.spec.qk_norm_eps,
                table=angles, rot_dims=rot_dims, interleaved=getattr(self.position, "interleaved", False),
                k_cache=k_cache, v_cache=v_cache, block_table=table, positions=batch.positions,
                token_entry=batch.token_entry, status=self.ctx.status,
            )
        parts = self.parts
        # a differential layer's maps are kept in 32-bit side by side until they are combined
        out = torch.empty((n, nq * parts * dv), dtype=k_cache.dtype if parts == 1 else torch.float32, device=x.device)
        if self.plan_key not in batch.plans:
            self.plan_step(batch.entries, k_cache.shape[2], batch.plans)
        splits, long_entries, short_entries = batch.plans[self.plan_key]
        gate = qkv[:, k_end + nkv * dv :] if self.head_gate else None
        with self.ctx.section("mixer.attention"):
            if long_entries:
                # prompt portions of a plain softmax layer with heads of 64 or 128: the tcgen05 kernel
                native.attention_prefill_tc5(q, k_cache, v_cache, out, table, batch.cu_tokens, batch.starts, batch.n_entries,
                                             batch.max_new, nq, self.spec.window, self.keep_first, self.spec.scale, gate,
                                             SHORT_ENTRY_ROWS, self.ctx.status, distance_bias=self.distance_bias_unscaled,
                                             softcap=self.softcap)
            if short_entries:
                native.attention_general(q, (nq * d, d), k_cache, self.d, v_cache, dv, out, (nq * parts * dv, parts * dv), table,
                                         batch.positions, batch.token_entry, nq, self.slopes, self.spec.window,
                                         self.spec.scale, self.ctx.status,
                                         entries=(batch.cu_tokens, batch.starts, batch.n_entries, batch.max_new),
                                         splits=splits, keep_first=self.keep_first,
                                         softcap=self.softcap, query_temperature=self.query_temperature, parts=parts,
                                         part_strides=(self.d, self.d, dv) if parts > 1 else (0, 0, 0),
                                         gate=gate, row_hi=SHORT_ENTRY_ROWS if long_entries else 0,
                                         distance_bias=self.distance_bias)
            if parts > 1:
                maps = out
                out = torch.empty((n, nq * dv), dtype=k_cache.dtype, device=x.device)
                native.differential_combine(maps, out, dv, self.diff_lambda, self.differential.eps,
                                            1.0 - float(self.differential.offset))
        return out

    def _project(self, x, batch, cache: CacheView):
        """q, k, v of the step's tokens: projected, normalised per head, rotated; k and v
        stored in their pages.  Returns qkv with the finished queries."""
        k_cache, v_cache = cache.kv
        table = batch.group_tables[cache.group]
        rotary = self.position.rotary()
        if self._summed_projection(x, rotary, k_cache):
            # few tokens: the projection's k-splits add into a zeroed 32-bit buffer (no cluster,
            # more blocks), and the norm-and-rotate kernel reads the sums and leaves zeros behind
            width = self.qkv_proj.out_features
            # everything the second kernel needs is at hand before the first is launched: the
            # buffer is only zero again when both have run
            angles = self.position.table(batch) if hasattr(self.position, "table") else None
            qkv = torch.empty((x.shape[0], width), dtype=x.dtype, device=x.device)
            sums = native.projection_sums(x.device, x.shape[0] * width)[: x.shape[0] * width].view(x.shape[0], width)
            native.gemm_tc5(x, self.qkv_proj.weight, sums, native.TC5_ADD_F32, self.ctx.status, bias=self.qkv_proj.bias,
                            ksplit=native.tc5_ksplit_sums(width, self.qkv_proj.in_features, x.shape[0]))
            native.qk_rope_cache_sums(
                sums, qkv, self.q_norm, self.k_norm, self.spec.qk_norm_eps, rotary[0],
                batch.positions, batch.token_entry, k_cache, v_cache, table, self.nq, cache.owns, self.ctx.status,
                table=angles,
            )
        elif self._fused_projection(x, rotary, k_cache):
            # few tokens, heads of 128: norm, rotation and the page write happen in the
            # projection's own epilogue
            qkv = torch.empty((x.shape[0], self.qkv_proj.out_features), dtype=x.dtype, device=x.device)
            native.gemm_tc5_qkv_rope(
                x, self.qkv_proj.weight, self.qkv_proj.bias, qkv, self.q_norm, self.k_norm,
                self.spec.qk_norm_eps, self.position.table(batch), batch.positions, batch.token_entry, k_cache, v_cache, table,
                self.nq, cache.owns, self.ctx.status,
                ksplit=native.tc5_ksplit(self.qkv_proj.out_features, self.qkv_proj.in_features),
            )
        else:
            qkv = self.qkv_proj(x)
            angles = None
            if rotary is None:
                self.position.apply(qkv, self.nq, self.nkv, self.d, batch)
                inv_freq, rotary_dim = None, 0
            else:
                inv_freq, rotary_dim = rotary
                if hasattr(self.position, "table"):
                    angles = self.position.table(batch)
            native.qk_rope_cache(
                qkv, self.q_norm, self.k_norm, self.spec.qk_norm_eps, inv_freq, rotary_dim,
                batch.positions, batch.token_entry, k_cache, v_cache, table, self.nq,
                cache.owns, self.ctx.status, table=angles,
            )
        return qkv

    def _prefill_tc5(self, page_size: int) -> bool:
        """Whether prompt portions of this (general) layer run on the tcgen05 prefill kernel:
        a plain softmax over one map per head (a window, kept first tokens, a gate per head and
        either a bias by distance or capped scores it has), keys and values of 64 or 128."""
        return (self.parts == 1 and self.slopes is None and (self.softcap is None or self.distance_bias is None)
                and self.query_temperature is None
                and self.spec.scale > 0 and native.prefill_tc5_takes(self.ctx.dtype, self.d, self.dv, self.nq // self.nkv, page_size)
                and native.general_mma_takes(self.ctx.dtype, self.d, self.dv))

    def _summed_projection(self, x, rotary, k_cache) -> bool:
        """Whether the q/k/v projection adds its k-splits into a 32-bit buffer that a separate
        norm-and-rotate kernel reads: few tokens, the tcgen05 kernel takes the call, and the
        position encoding rotates whole heads.  Up to FORGE_ENGINE_SUMMED_QKV tokens (64; 0 turns
        it off).  Measured at the 4B shape against the projection that sums its k-splits inside
        a cluster and norms and rotates in its own epilogue: 2.473 against 2.509 ms a decode
        step at batch 8, 2.940 against 3.017 at 16, 3.866 against 3.921 at 32, 5.82 against 5.85
        at 64, no difference at batch 1 and 2."""
        limit = int(os.environ.get("FORGE_ENGINE_SUMMED_QKV", "64"))
        return (x.shape[0] <= limit and self.d in (64, 128, 256) and rotary is not None and rotary[1] == self.d
                and k_cache.dtype == torch.bfloat16 and self.qkv_proj._tc5_ok(x))

    def _fused_projection(self, x, rotary, k_cache) -> bool:
        """Whether the q/k/v projection's epilogue can do the per-head norms, the rotation
        and the page write: the tcgen05 kernel takes the call, a head is one 128-feature
        tile, and the whole head is rotated."""
        return (self.d == 128 and rotary is not None and rotary[1] == 128 and hasattr(self.position, "table")
                and k_cache.dtype == torch.bfloat16
                and x.shape[0] <= FUSED_PROJECTION_ROWS and self.qkv_proj._tc5_ok(x)
                and os.environ.get("FORGE_ENGINE_FUSED_QKV", "1") != "0")

    def plan_step(self, entries: list, page_size: int, plans: dict) -> None:
        """The host's decision for a step of ``entries`` ((slot, cached, new) each): entries
        with few rows (new tokens x heads per kv head <= 16) take the split decode kernel, the
        rest the prefill kernel; both may run in one step.  (run prefill, run decode, splits
        of the decode kernel - 0: the kernel that spreads all tiles evenly) under this
        mixer's key; layers with the same geometry share it."""
        if self.general:
            # the general kernels: (how many blocks share a row tile's keys, whether entries go
            # to the tcgen05 prefill kernel, whether entries go to the general kernel)
            if self.plan_key not in plans:
                groups = self.nq // self.nkv
                short = list(entries)
                if self._prefill_tc5(page_size):
                    short = [e for e in entries if e[2] * groups <= SHORT_ENTRY_ROWS]
                splits = 1
                if short and native.general_mma_takes(self.ctx.dtype, self.d, self.dv):
                    splits = native.general_splits(short, groups, self.nkv * self.parts, self.spec.window,
                                                   keep_first=self.keep_first)
                plans[self.plan_key] = (splits, len(short) < len(entries), bool(short))
            return
        if self.ctx.dtype != torch.bfloat16 or self.plan_key in plans:
            return
        groups = self.nq // self.nkv
        limit = native.ATTN_DECODE_ROWS
        small = [(start, count) for _, start, count in entries if count * groups <= limit]
        run_decode = bool(small)
        run_prefill = len(small) < len(entries)
        splits = 1
        if run_decode:
            contexts = [start + count for start, count in small]
            if self.spec.window:
                contexts = [min(c, self.spec.window + limit) for c in contexts]
            # FORGE_ENGINE_DECODE_BALANCED: 0 never uses the balanced kernel, "always" uses it
            # wherever it can run, anything else lets the estimate decide
            wish = os.environ.get("FORGE_ENGINE_DECODE_BALANCED", "1")
            balanced = (self.d % 64 == 0 and page_size <= 64 and 64 % page_size == 0
                        and len(entries) <= BALANCED_MAX_ENTRIES and wish != "0")
            splits = 0 if balanced and wish == "always" else choose_splits(
                [-(-c // 64) for c in contexts], self.nkv, balanced, self.decode_slots())
        plans[self.plan_key] = (run_prefill, run_decode, splits)

    def _tensor_core_attention(self, qkv, k_cache, v_cache, table, batch, out, groups) -> None:
        if self.plan_key not in batch.plans:
            self.plan_step(batch.entries, k_cache.shape[2], batch.plans)
        run_prefill, run_decode, splits = batch.plans[self.plan_key]
        if run_decode:
            self.last_splits = splits
        native.attention_mma(
            qkv, qkv.shape[1], k_cache, v_cache, table, batch.cu_tokens, batch.starts,
            batch.n_entries, batch.max_new, self.spec.window, self.spec.scale, out, self.nq,
            self.ctx.status, run_prefill, run_decode, splits,
        )


register_part("gqa_attention", GQAttention, replace=True)
