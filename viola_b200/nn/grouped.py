"""Expert (batched, ragged-M) FP8 linear: ``out[t] = x[t] @ W[expert(t)].T`` for tokens sorted by expert.

The reference has no expert GEMM (its "grouped" kernels are group-*scaled* GEMMs); the equivalent
there is a Python loop over per-expert ``viola.nn.Linear`` layers.  This module is that capability
as one persistent tcgen05 kernel launch per GEMM: a device-side tile -> (row range, expert) map lets
every CTA pick the right weight panel, so ragged token counts cost no host synchronisation.

Forward, dgrad and wgrad all run in FP8 with either per-tensor scales (``scaling='current'``) or
fp32 scales per (1 x 128) activation group and (128 x 128) weight block (``scaling='grouped'``).
"""

from __future__ import annotations

import math

import torch
from torch import nn

from .. import ops
from ..precision import settings

E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


class _ExpertLinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, offsets, layer):
        grouped = layer.scaling == "grouped"
        experts, n, k = weight.shape
        x2 = x.contiguous()
        qw, sw = layer.weight_codes()                   # cached until the weight changes
        if grouped:
            qx, sx = ops.group_quantize(x2, E4M3, (1, 128), kmajor=True)
            y = ops.expert_gemm(qx, qw, offsets, sx, sw, out_dtype=x.dtype, group=((1, 128), (128, 128)), sa_kmajor=True)
        else:
            sx = ops.tensor_scale(x2)
            qx, _ = ops.quantize(x2, sx)
            y = ops.expert_gemm(qx, qw, offsets, sx, sw, out_dtype=x.dtype)
        ctx.save_for_backward(x2, weight, offsets)
        ctx.layer = layer
        ctx.weight_grad_dtype = layer.weight.grad_dtype or torch.float32
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, offsets = ctx.saved_tensors
        layer = ctx.layer
        grouped = layer.scaling == "grouped"
        experts, n, k = weight.shape
        dy = dy.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[0]:
            # dX[t] = dY[t] @ W[e]: an expert GEMM against the per-expert transposed codes [E, K, N] (a byte
            # transpose of the cached codes; the scales of a transposed 128 x 128 block are the same numbers)
            qwt, swt = layer.weight_codes(transposed=True)
            if grouped:
                qg, sg = ops.group_quantize(dy, E5M2, (1, 128), kmajor=True)
                dx = ops.expert_gemm(qg, qwt, offsets, sg, swt, out_dtype=x.dtype, group=((1, 128), (128, 128)),
                                     sa_kmajor=True)
            else:
                sg = ops.tensor_scale(dy, fp8_dtype=E5M2)
                qg, _ = ops.quantize(dy, sg, fp8_dtype=E5M2)
                dx = ops.expert_gemm(qg, qwt, offsets, sg, swt, out_dtype=x.dtype)
        if ctx.needs_input_grad[1]:
            # dW[e] = dY[rows e]^T @ X[rows e]: K = the expert's token count, one GEMM per expert
            dw = torch.zeros(weight.shape, device=weight.device, dtype=ctx.weight_grad_dtype)
            bounds = offsets.tolist()
            for e in range(experts):
                lo, hi = bounds[e], bounds[e + 1]
                if hi <= lo:
                    continue
                if grouped:
                    gt, sgt = ops.group_quantize(dy[lo:hi], E5M2, (1, 128), transposed=True, kmajor=True)
                    xt, sxt = ops.group_quantize(x[lo:hi], E4M3, (1, 128), transposed=True, kmajor=True)
                    ops.group_gemm(gt, xt, sgt, sxt, (1, 128), (1, 128), out_dtype=dw.dtype, sa_kmajor=True,
                                   sb_kmajor=True, out=dw[e])
                else:
                    sg, sx = ops.tensor_scale(dy[lo:hi], fp8_dtype=E5M2), ops.tensor_scale(x[lo:hi])
                    _, gt = ops.quantize(dy[lo:hi], sg, rowwise=False, transpose=True, fp8_dtype=E5M2)
                    _, xt = ops.quantize(x[lo:hi], sx, rowwise=False, transpose=True)
                    ops.gemm(gt, xt, sg, sx, out_dtype=dw.dtype, out=dw[e])
        return dx, dw, None, None


class GroupedLinear(nn.Module):
    """``num_experts`` independent ``in_features -> out_features`` projections applied to sorted tokens.

    ``forward(x, offsets)``: ``x`` is ``[tokens, in_features]`` with the rows of expert ``e`` at
    ``offsets[e]:offsets[e + 1]`` (``offsets``: int32 ``[num_experts + 1]`` on the same device).
    """

    def __init__(self, num_experts, in_features, out_features, *, scaling="grouped", device=None, dtype=None):
        super().__init__()
        if scaling not in ("current", "grouped"):
            raise ValueError("scaling must be 'current' or 'grouped'")
        if scaling == "grouped" and (out_features % 128 or in_features % 128):
            raise ValueError("grouped scaling needs feature sizes that are multiples of 128")
        self.num_experts, self.in_features, self.out_features = num_experts, in_features, out_features
        self.scaling = scaling
        dtype = dtype or torch.get_default_dtype()
        self.weight = nn.Parameter(torch.empty((num_experts, out_features, in_features), device=device, dtype=dtype))
        self.weight.grad_dtype = settings()["gradient_dtype"] or torch.float32
        self._codes, self._codes_key = {}, None
        self.reset_parameters()

    @torch.no_grad()
    def reset_parameters(self):
        for expert in self.weight:
            nn.init.kaiming_uniform_(expert, a=math.sqrt(5))

    @torch.no_grad()
    def weight_codes(self, transposed=False):
        """FP8 codes and scales of the expert weights ([E, N, K], or [E, K, N] when ``transposed``), quantised once
        per weight version: every forward and backward until the next in-place update reuses them."""
        weight = self.weight
        key = (weight._version, weight.data_ptr(), weight.dtype, weight.device)
        if key != self._codes_key:
            self._codes, self._codes_key = {}, key
        experts, n, k = weight.shape
        if "rowwise" not in self._codes:
            flat = weight.detach().reshape(experts * n, k)
            if self.scaling == "grouped":
                q, s = ops.group_quantize(flat, E4M3, (128, 128))
            else:
                s = ops.tensor_scale(flat)
                q, _ = ops.quantize(flat, s)
            self._codes["rowwise"] = (q.view(experts, n, k), s)
        if not transposed:
            return self._codes["rowwise"]
        if "transposed" not in self._codes:
            q, s = self._codes["rowwise"]
            qt = q.view(torch.uint8).transpose(1, 2).contiguous().view(q.dtype)
            if self.scaling == "grouped":
                s = s.view(experts, n // 128, k // 128).transpose(1, 2).contiguous().view(experts * (k // 128), n // 128)
            self._codes["transposed"] = (qt, s)
        return self._codes["transposed"]

    def forward(self, x, offsets):
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        return _ExpertLinearFunction.apply(x, self.weight, offsets.to(torch.int32), self)

    def extra_repr(self):
        return (f"num_experts={self.num_experts}, in_features={self.in_features}, "
                f"out_features={self.out_features}, scaling={self.scaling!r}")
