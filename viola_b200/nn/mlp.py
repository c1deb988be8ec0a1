"""Gated MLP ``down(act(gate(x)) * up(x))`` with the gating fused into the GEMM epilogues.

Same module surface as the reference (viola/nn/mlp.py:76-113): ``gate_up`` is one
``Linear(in, 2 * hidden)`` whose first ``hidden`` output rows are the gate branch, ``down`` is
``Linear(hidden, out)``; activations ``silu`` / ``gelu`` (tanh) / ``relu``; Linear's storage, format,
scaling and caching options pass through.  Here the whole block is a single autograd function over
the shared functional Linear core: the forward gate/up GEMM shares its A tile between both
branches and applies ``act(g) * u`` straight out of tensor memory; the backward dgrad of ``down``
applies the gated derivative in its epilogue and writes ``[dG | dU]`` directly.
"""

from __future__ import annotations

import torch
from torch import nn

from .linear import Linear, linear_backward, linear_forward


class _GatedMLPFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w_up, b_up, w_down, b_down, module, need_backward):
        gate_up, down = module.gate_up, module.down
        shape = x.shape
        x2 = x.reshape(-1, gate_up.in_features).contiguous()
        needs = ctx.needs_input_grad
        need_x = need_backward and needs[0]
        need_w_up = need_backward and needs[1]
        need_b_up = need_backward and b_up is not None and needs[2]
        need_w_down = need_backward and needs[3]
        need_up = need_x or need_w_up or need_b_up          # does anything upstream of h need a gradient?
        h, saved_up, aux = linear_forward(gate_up, x2, w_up, b_up, need_input_grad=need_x,
                                          need_weight_grad=need_w_up, gated=module.activation)
        if not need_up:
            aux = None
        y, saved_down, _ = linear_forward(down, h, w_down, b_down, need_input_grad=need_up,
                                          need_weight_grad=need_w_down)
        del h
        if need_backward:
            ctx.module, ctx.shape = module, shape
            ctx.saved_up, ctx.saved_down, ctx.aux = saved_up, saved_down, aux
            ctx.need_up = need_up
            ctx.bias_dtypes = tuple((getattr(b, "grad_dtype", None) or b.dtype) if b is not None else None
                                    for b in (b_up, b_down))
        return y.reshape(*shape[:-1], down.out_features)

    @staticmethod
    def backward(ctx, dy):
        module = ctx.module
        gate_up, down = module.gate_up, module.down
        needs = ctx.needs_input_grad
        dy2 = dy.reshape(-1, down.out_features).contiguous()
        dx = dw_up = db_up = dw_down = db_down = None
        if ctx.saved_down is not None:
            dz, dw_down, db_down = linear_backward(down, ctx.saved_down, dy2, need_input_grad=ctx.need_up,
                                                   need_weight_grad=needs[3], need_bias_grad=needs[4],
                                                   gated=module.activation, aux=ctx.aux)
        else:
            dz = None
            if needs[4]:
                db_down = dy2.sum(dim=0, dtype=ctx.bias_dtypes[1])
        ctx.aux = ctx.saved_down = None
        if dz is not None and ctx.saved_up is not None:
            dx, dw_up, db_up = linear_backward(gate_up, ctx.saved_up, dz, need_input_grad=needs[0],
                                               need_weight_grad=needs[1], need_bias_grad=needs[2])
        elif dz is not None and needs[2]:
            db_up = dz.sum(dim=0, dtype=ctx.bias_dtypes[0])
        ctx.saved_up = None
        if dx is not None:
            dx = dx.reshape(*ctx.shape[:-1], gate_up.in_features)
        return dx, dw_up, db_up, dw_down, db_down, None, None


class MLP(nn.Module):
    """``hidden_features`` is the width of each of the two branches."""

    def __init__(self, in_features, hidden_features, out_features=None, *, activation="silu", autotune=False,
                 **linear_options):
        super().__init__()
        if activation not in ("silu", "gelu", "relu"):
            raise ValueError("activation must be silu, gelu or relu")
        self.in_features = in_features
        self.hidden_features = hidden_features
        self.out_features = in_features if out_features is None else out_features
        self.activation, self.autotune = activation, autotune
        self.gate_up = Linear(in_features, 2 * hidden_features, autotune=autotune, **linear_options)
        self.down = Linear(hidden_features, self.out_features, autotune=autotune, **linear_options)

    def forward(self, x):
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        need_backward = torch.is_grad_enabled() and (x.requires_grad or any(p.requires_grad for p in self.parameters()))
        return _GatedMLPFunction.apply(x, self.gate_up.weight, self.gate_up.bias, self.down.weight, self.down.bias,
                                       self, need_backward)

    def extra_repr(self):
        return (f"in_features={self.in_features}, hidden_features={self.hidden_features}, "
                f"out_features={self.out_features}, activation={self.activation!r}")
