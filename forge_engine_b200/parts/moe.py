"""A routed feed-forward: per token the ``top`` of ``experts`` units (gated, or a plain
down(act(up(x))) without a gate) with the largest router scores, and optionally a shared unit
that every token uses.

The router's logits are a true 32-bit product.  Everything after them stays on the device:
the (token, choice) pairs are laid out by expert, two grouped products run over them (gate
and up with the gated unit in the epilogue; down), and one kernel sums a token's rows and
adds the shared unit's output times its sigmoid gate.  Nothing is decided on the host, so a
step replays from a CUDA graph.
"""

from __future__ import annotations

import os

import torch

from ..config.specs import local_name
from ..errors import ConfigError
from ..ops import native
from .base import BuildContext, FeedForward, WeightInfo, build_part, part_class, register_part
from .ffn import ACTIVATIONS, UNARY

MAX_TOP = 32
INTERLEAVE = 16       # gate and up features alternate in sixteens in the fused matrix


def _shared_spec(spec):
    """The shared unit's spec with its tensors under ``shared.``."""
    import dataclasses

    renamed = tuple((canonical, "shared." + local_name(spec.shared, canonical))
                    for canonical in ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
    return dataclasses.replace(spec.shared, rename=renamed)


class RoutedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.score not in ("sigmoid", "softmax"):
            raise ConfigError(f"router score {spec.score!r}; known: sigmoid, softmax")
        if spec.weight_on not in ("input", "output"):
            raise ConfigError(f"weight_on={spec.weight_on!r}; known: input, output")
        self.identity = int(getattr(spec, "identity", 0) or 0)
        if not 1 <= spec.top <= min(spec.experts + self.identity, MAX_TOP):
            raise ConfigError(f"top={spec.top} of {spec.experts + self.identity} experts; at most {MAX_TOP}")
        if self.identity and spec.weight_on != "output":
            raise ConfigError("identity experts take the weight on the output")
        unit = spec.expert
        # a unit without a gate: down(act(up(x))), act an activation of one argument, no biases
        self.gated = getattr(unit, "kind", "gated_mlp") != "dense_mlp"
        if (unit.activation not in ACTIVATIONS) if self.gated else (unit.activation not in UNARY or unit.bias):
            raise ConfigError(f"an expert with activation {unit.activation!r}" + ("" if self.gated else " (no gate)")
                              + " is not implemented")
        if getattr(spec, "group_score", "max") not in ("max", "top2"):
            raise ConfigError(f"group_score={spec.group_score!r}; known: max, top2")
        self.ctx = ctx
        self.experts, self.top, self.width, self.inter = spec.experts, spec.top, spec.hidden_size, unit.intermediate_size
        self.softmax, self.renormalise = spec.score == "softmax", bool(spec.renormalise)
        self.weight_on_input = spec.weight_on == "input"
        if self.gated:
            self.activation = ACTIVATIONS[unit.activation]
            self.limit, self.slope = float(unit.limit or 0.0), float(unit.slope)
        else:
            self.activation, self.limit, self.slope = UNARY[unit.activation], 0.0, 1.0
        self.groups = getattr(spec, "groups", None)
        self.group_top2 = getattr(spec, "group_score", "max") == "top2"
        self.renorm_floor = float(getattr(spec, "renorm_floor", 0.0))
        self.weight_scale = float(getattr(spec, "weight_scale", 1.0))
        self.correction = None
        if getattr(spec, "correction", False):
            self.correction = weights["correction"].to(device=ctx.device, dtype=torch.float32).contiguous()
        # the router's rows (identity units' last), and under them the shared unit's gate row: one 32-bit product
        rows = [weights["router"]]
        self.shared = None
        self.shared_gate = False
        if spec.shared is not None:
            self.shared_gate = bool(spec.shared_gate)
            if self.shared_gate:
                rows.append(weights["shared.sg"].reshape(1, -1))
        self.router = torch.cat([r.float() for r in rows], dim=0).contiguous()
        del rows
        names = [local_name(unit, n) for n in self._unit_names(unit)]
        # bfloat16 with sizes in sixteens: the products run on the tcgen05 kernel in its grouped
        # form, gate and up as one matrix per expert whose rows alternate 16 gate and 16 up features
        self.fused = (ctx.dtype == torch.bfloat16 and self.width % 8 == 0 and self.inter % (INTERLEAVE if self.gated else 8) == 0
                      and os.environ.get("FORGE_ENGINE_MOE_TC5", "1") != "0")
        stacks = []
        shapes = ((self.inter, self.width), (self.inter, self.width), (self.width, self.inter))
        for name, shape in zip(names, shapes if self.gated else shapes[1:]):
            stack = None
            for e in range(self.experts):
                tensor = weights[f"e{e}.{name}"]
                if stack is None:
                    stack = torch.empty((self.experts, *shape), dtype=tensor.dtype, device=tensor.device)
                stack[e].copy_(tensor)
                del tensor
            stacks.append(stack)
        if not self.gated:
            stacks.insert(0, None)
        self.gate, self.up, self.down_stack = stacks
        self.gate_up_stack = None
        if not self.gated:
            self.fused = self.fused and all(t.dtype == torch.bfloat16 for t in stacks[1:])
        elif self.fused and all(t.dtype == torch.bfloat16 for t in stacks):
            blocks = self.inter // INTERLEAVE
            self.gate_up_stack = torch.empty((self.experts, 2 * self.inter, self.width), dtype=torch.bfloat16, device=self.gate.device)
            view = self.gate_up_stack.view(self.experts, blocks, 2, INTERLEAVE, self.width)
            view[:, :, 0].copy_(self.gate.view(self.experts, blocks, INTERLEAVE, self.width))
            view[:, :, 1].copy_(self.up.view(self.experts, blocks, INTERLEAVE, self.width))
            self.gate = self.up = None
        else:
            self.fused = False
        if spec.shared is not None:
            self.shared = build_part(_shared_spec(spec), weights, ctx)
        # rows per expert, counted by the route kernel; the plan kernel reads them and leaves
        # zeros behind, so no launch is spent on clearing them
        self.counts = torch.zeros(self.experts + 1, dtype=torch.int32, device=ctx.device)

    @staticmethod
    def _unit_names(unit) -> tuple:
        """Canonical tensor names of one expert: a unit without a gate has none for it."""
        if getattr(unit, "kind", "gated_mlp") == "dense_mlp":
            return ("up_proj.weight", "down_proj.weight")
        return ("gate_proj.weight", "up_proj.weight", "down_proj.weight")

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        h, unit = spec.hidden_size, spec.expert
        outputs = spec.experts + int(getattr(spec, "identity", 0) or 0)
        shapes = {"router": WeightInfo((outputs, h))}
        if getattr(spec, "correction", False):
            shapes["correction"] = WeightInfo((outputs,), "bias")
        names = [local_name(unit, n) for n in cls._unit_names(unit)]
        for e in range(spec.experts):
            for name in names[:-1]:
                shapes[f"e{e}.{name}"] = WeightInfo((unit.intermediate_size, h))
            shapes[f"e{e}.{names[-1]}"] = WeightInfo((h, unit.intermediate_size))
        if spec.shared is not None:
            shared = _shared_spec(spec)
            shapes.update(part_class(shared).weight_shapes(shared))
            if spec.shared_gate:
                shapes["shared.sg"] = WeightInfo((1, h))
        return shapes

    def tile_rows(self, slots: int) -> int:
        """Rows of a row tile of the tcgen05 products: few rows per expert (decoding) take
        the narrow tiles, whose rings are deepest."""
        wish = int(os.environ.get("FORGE_ENGINE_MOE_TILE", "0"))
        if wish in (16, 32, 64, 128):
            return wish
        per_expert = slots / self.experts
        return 16 if per_expert <= 16 else 32 if per_expert <= 32 else 64 if per_expert <= 96 else 128

    def forward(self, x):
        n = x.shape[0]
        slots = n * self.top
        device = x.device
        section = self.ctx.section
        with section("ffn.router"):
            logits = torch.empty((n, self.router.shape[0]), dtype=torch.float32, device=device)
            if self.width <= 48 * 1024:
                native.moe_logits(x, self.router, logits)
            else:
                native.gemm_simt(x, self.router, logits)
        tile_rows = self.tile_rows(slots) if self.fused else 0
        max_tiles = native.moe_max_tiles(slots, self.experts, tile_rows)
        with section("ffn.route"):
            ints = torch.empty(4 * slots + self.experts + 2 + 2 * max_tiles, dtype=torch.int32, device=device)
            weight = torch.empty(slots, dtype=torch.float32, device=device)
            plan = native.moe_route(logits, self.experts, self.top, self.softmax, self.renormalise, self.counts, ints,
                                    weight, max_tiles, tile_rows, identity=self.identity, correction=self.correction,
                                    groups=self.groups, renorm_floor=self.renorm_floor, weight_scale=self.weight_scale,
                                    group_top2=self.group_top2)
        hidden = torch.empty((slots, self.inter), dtype=x.dtype, device=device)
        rows = torch.empty((slots, self.width), dtype=torch.float32, device=device)
        with section("ffn.experts"):
            if self.fused:
                sorted_x = torch.empty((slots, self.width), dtype=x.dtype, device=device)
                native.moe_gather(x, plan, self.top, weight if self.weight_on_input else None, sorted_x)
                if self.gated:
                    native.gemm_tc5_grouped(sorted_x, self.gate_up_stack, hidden, native.TC5_GATED[self.activation], plan,
                                            tile_rows, max_tiles, self.ctx.status, self.limit, self.slope)
                else:
                    native.gemm_tc5_grouped(sorted_x, self.up, hidden, native.TC5_UNARY[self.activation], plan,
                                            tile_rows, max_tiles, self.ctx.status)
                native.gemm_tc5_grouped(hidden, self.down_stack, rows, native.TC5_STORE_F32, plan, tile_rows, max_tiles,
                                        self.ctx.status)
            else:
                if self.gated:
                    native.moe_grouped(x, self.gate, self.up, hidden, plan, self.top, max_tiles, gather=True,
                                       slot_weight=weight if self.weight_on_input else None, act=self.activation,
                                       limit=self.limit, slope=self.slope)
                else:
                    native.moe_grouped(x, self.up, None, hidden, plan, self.top, max_tiles, gather=True,
                                       slot_weight=weight if self.weight_on_input else None,
                                       act=native.MOE_UNARY[self.activation])
                native.moe_grouped(hidden, self.down_stack, None, rows, plan, self.top, max_tiles, gather=False)
        with section("ffn.shared"):
            shared = None if self.shared is None else self.shared.forward(x)
        with section("ffn.combine"):
            out = torch.empty((n, self.width), dtype=torch.float32, device=device)
            native.moe_combine(rows, plan, self.top, out, slot_weight=None if self.weight_on_input else weight,
                               shared=shared,
                               shared_logit=logits[:, self.experts + self.identity] if self.shared_gate else None,
                               identity_input=x if self.identity else None, experts=self.experts)
        return out


register_part("routed_mlp", RoutedMLP, replace=True)
