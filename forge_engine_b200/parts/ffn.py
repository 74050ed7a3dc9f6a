"""Gated feed-forward: down(act(gate(x)) * up(x)) with act = SiLU
(src/forge_engine/qwen3.py:210-227) or the tanh form of GELU, or the clamped unit
down(g' sigmoid(slope g') (u' + 1)) with g' = min(gate(x), limit), u' = clamp(up(x), +-limit).
gate and up are one fused projection; the activation product is one kernel."""

from __future__ import annotations

import os

import torch

from ..config.specs import local_name
from ..errors import ConfigError
from ..ops import native
from .base import BuildContext, FeedForward, WeightInfo, register_part
from .linear import Linear, fused_rows, interleaved_rows

GATE_UP_BLOCK = 16
ACTIVATIONS = {"silu": native.ACT_SILU, "gelu_tanh": native.ACT_GELU_TANH, "clamped_swish": native.ACT_CLAMPED_SWISH}


class GatedMLP(FeedForward):
    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.activation not in ACTIVATIONS:
            raise ConfigError(f"activation {spec.activation!r} is not implemented; known: {', '.join(ACTIVATIONS)}")
        self.activation = ACTIVATIONS[spec.activation]
        self.limit = float(getattr(spec, "limit", None) or 0.0)
        self.slope = float(getattr(spec, "slope", 1.0))
        if self.activation == native.ACT_CLAMPED_SWISH and self.limit <= 0.0:
            raise ConfigError("the clamped unit needs a positive limit")
        self.inter = spec.intermediate_size
        gate, up, down = (local_name(spec, n) for n in ("gate_proj.weight", "up_proj.weight", "down_proj.weight"))
        # Rows of the fused weight alternate 16 gate and 16 up features where the size allows:
        # the tensor-core kernel then finishes act(gate) * up in its epilogue.
        self.block = GATE_UP_BLOCK if self.inter % GATE_UP_BLOCK == 0 else 0
        # the sources are looked up one at a time and copied into the fused tensor
        if self.block:
            fused = interleaved_rows(weights, gate, up, self.inter, self.block)
        else:
            fused = fused_rows(weights, [gate, up], [self.inter, self.inter])
        self.gate_up = Linear(fused, status=ctx.status)
        self.down = Linear(weights[down], status=ctx.status)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        h, i = spec.hidden_size, spec.intermediate_size
        return {
            local_name(spec, "gate_proj.weight"): WeightInfo((i, h)),
            local_name(spec, "up_proj.weight"): WeightInfo((i, h)),
            local_name(spec, "down_proj.weight"): WeightInfo((h, i)),
        }

    def forward_add(self, x, residual) -> bool:
        """``forward`` with the update added into the 32-bit ``residual`` by the down projection
        itself.  False (and nothing done) where that projection cannot."""
        if not (self.block == 16 and self.activation in (native.ACT_SILU, native.ACT_CLAMPED_SWISH)
                and self.down.adds_into(x, residual) and self.gate_up._tc5_ok(x)
                and self.gate_up.out_features % 32 == 0 and self.gate_up.bias is None):
            return False
        return self.down.add_into(self.gate_up.silu_mul(x, self.block, self.activation, self.limit, self.slope), residual)

    def forward(self, x):
        act = self.gate_up.silu_mul(x, self.block, self.activation, self.limit, self.slope) if self.block else None
        if act is None:
            act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
            if self.activation == native.ACT_SILU:
                native.silu_mul(self.gate_up(x), act, self.block)
            else:
                # the activation is taken of the 32-bit sums of the projection, not of their rounding
                native.act_mul(self.gate_up(x, out_dtype=torch.float32), act, self.activation, self.block,
                               self.limit, self.slope)
        return self.down(act)


UNARY = {"gelu_tanh": native.UNARY_GELU_TANH, "relu2": native.UNARY_RELU2}


class DenseMLP(FeedForward):
    """down(act(up(x) + b_up)) + b_down without a gate (biases optional).  The activation is
    taken of the projection's 32-bit sums plus the bias, in 32-bit, and rounded once.

    "xielu": act(z) = a_pos z^2 + z / 2 for z > 0 and a_neg (exp(z) - 1 - z) + z / 2 otherwise,
    with a_pos = softplus(p) and a_neg = 1/2 + softplus(q) from the two learned numbers
    ``act`` = (p, q), worked out once when the layer is built.  "gelu_tanh" (the tanh form of
    GELU) and "relu2" (the square of relu) have no tensors; for steps of few tokens they are
    the epilogue of the up projection's tcgen05 product."""

    graph_safe = True

    def __init__(self, spec, weights: dict, ctx: BuildContext) -> None:
        if spec.activation != "xielu" and spec.activation not in UNARY:
            raise ConfigError(f"activation {spec.activation!r} is not implemented; known: xielu, {', '.join(UNARY)}")
        self.ctx = ctx
        self.inter = spec.intermediate_size
        self.unary = UNARY.get(spec.activation)
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        self.up = Linear(weights[name("up_proj.weight")], status=ctx.status)
        self.up_bias = weights[name("up_proj.bias")].to(device=ctx.device, dtype=torch.float32).contiguous() if spec.bias else None
        self.down = Linear(weights[name("down_proj.weight")], weights[name("down_proj.bias")] if spec.bias else None,
                           status=ctx.status)
        self.a_pos = self.a_neg = 0.0
        if self.unary is None:
            p, q = (float(v) for v in weights[name("act")].double().cpu())
            softplus = lambda z: float(torch.nn.functional.softplus(torch.tensor(z, dtype=torch.float64), threshold=1e9))  # noqa: E731
            self.a_pos, self.a_neg = softplus(p), 0.5 + softplus(q)

    @classmethod
    def weight_shapes(cls, spec) -> dict:
        h, i = spec.hidden_size, spec.intermediate_size
        name = lambda canonical: local_name(spec, canonical)  # noqa: E731
        shapes = {name("up_proj.weight"): WeightInfo((i, h)), name("down_proj.weight"): WeightInfo((h, i))}
        if spec.activation == "xielu":
            shapes[name("act")] = WeightInfo((2,), "small")
        if spec.bias:
            shapes[name("up_proj.bias")] = WeightInfo((i,), "bias")
            shapes[name("down_proj.bias")] = WeightInfo((h,), "bias")
        return shapes

    def forward(self, x):
        act = torch.empty((x.shape[0], self.inter), dtype=x.dtype, device=x.device)
        if self.unary is not None and self.up._tc5_ok(x) and os.environ.get("FORGE_ENGINE_UNARY_EPILOGUE", "1") != "0":
            # few tokens: the activation is the product's own epilogue (32-bit sums + bias, one rounding)
            native.gemm_tc5(x, self.up.weight, act, native.TC5_UNARY[self.unary], self.ctx.status, bias=self.up_bias,
                            ksplit=native.tc5_ksplit(self.up.out_features, self.up.in_features))
            return self.down(act, out_dtype=torch.float32)
        sums = self.up(x, out_dtype=torch.float32)
        if self.unary is None:
            native.bias_xielu(sums, self.up_bias, act, self.a_pos, self.a_neg)
        else:
            native.bias_act(sums, self.up_bias, act, self.unary)
        return self.down(act, out_dtype=torch.float32)


register_part("gated_mlp", GatedMLP, replace=True)
register_part("dense_mlp", DenseMLP, replace=True)
