"""Producer-fused FP8 linears for transformer blocks.

``norm_modulate_linear(x, shift, scale, layer)`` computes ``layer(LN(x) * (1 + scale) + shift)`` and
``activation_linear(z, layer, activation)`` computes ``layer(act(z))`` without ever writing the
normalised / activated tensor: the FP8 quantiser of the linear recomputes it from ``x`` / ``z`` in
the two passes a per-tensor scale needs anyway (row statistics + amax, then encode row-wise and
transposed), and LayerNorm + modulate have a single fused backward kernel.  The reference runs
these as separate PyTorch kernels in front of ``viola.nn.Linear`` (experiments/dit.py:33-39).

``gated_residual(x, gate, y)`` is the other half of an adaLN block, ``x + gate[:, None] * y``, as one
kernel forward and one backward (branch gradient and per-sample gate gradient from a single read).

The residual stream ``x`` may be fp32 (what autocast leaves it as, experiments/dit.py:60-75) or bf16; it is
read as stored, so no cast pass runs in front of the LayerNorm.  Everything falls back to the unfused
composition when the fast path does not apply (CPU tensors, other dtypes, group-scaled or rotated layers,
non-FP8 saved inputs, very wide rows).
"""

from __future__ import annotations

from types import SimpleNamespace

import torch
from torch.nn import functional as F

from .. import ops
from .linear import Linear, linear_backward, linear_forward


_STREAM_DTYPES = (torch.float32, torch.bfloat16)


def _eligible(layer, x, max_width=None, dtypes=(torch.bfloat16,)):
    return (isinstance(layer, Linear) and x.is_cuda and x.dtype in dtypes and not layer._grouped_scaling
            and not layer.rotation_size and layer.saved_input_dtype == "fp8" and x.shape[-1] % 16 == 0
            and (max_width is None or x.shape[-1] <= max_width))


def _stream_grad(dstream, x2):
    """The gradient that arrived for the carried stream, as the 2-D tensor the LayerNorm backward adds in."""
    if dstream is None:
        return None
    return dstream.reshape(x2.shape).to(x2.dtype).contiguous()


def _common(dtypes):
    """bf16 when every consumer of the per-sample sums wants bf16 (the kernel then rounds them itself), else fp32."""
    return torch.bfloat16 if all(d == torch.bfloat16 for d in dtypes) else torch.float32


def _needs(ctx, positions):
    return [ctx.needs_input_grad[p] for p in positions]


class _NormModulateLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, shift, scale, weight, bias, layer, eps):
        batch, tokens, width = x.shape
        x2 = x.reshape(-1, width).contiguous()
        need_w, need_b = ctx.needs_input_grad[3], bias is not None and ctx.needs_input_grad[4]
        quantizer = layer.input_quantizer
        limit = layer._quantization_limit(max(x2.shape), layer.fp8_dtype)
        q, qt, qscale, mean, rstd = ops.ln_modulate_quantize(
            x2, shift, scale, tokens, eps=eps, history=quantizer.history, index=quantizer.index,
            delayed=quantizer.scaling == "delayed", fp8_dtype=layer.fp8_dtype, quantization_limit=limit,
            transpose=need_w and not layer.in_place_operands)
        quantizer.index += 1
        encoded = SimpleNamespace(q=q, s=qscale, qt=qt, st=qscale)
        y, saved, _ = linear_forward(layer, x2, weight, bias, need_input_grad=True, need_weight_grad=need_w,
                                     encoded=encoded, out_dtype=torch.bfloat16)
        ctx.save_for_backward(x2, scale, mean, rstd)
        ctx.layer, ctx.saved, ctx.shape, ctx.need_b = layer, saved, x.shape, need_b
        ctx.mod_dtypes = (shift.dtype, scale.dtype)
        ctx.set_materialize_grads(False)
        # second output: the stream itself, for the residual connection that follows (see ``carry``)
        return y.reshape(batch, tokens, -1), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dstream):
        x2, scale, mean, rstd = ctx.saved_tensors
        layer = ctx.layer
        if dy is None:
            return (dstream, None, None, None, None, None, None)
        dy2 = dy.reshape(-1, layer.out_features).contiguous()
        dh, dw, db = linear_backward(layer, ctx.saved, dy2, need_input_grad=True, need_weight_grad=ctx.needs_input_grad[3],
                                     need_bias_grad=ctx.need_b)
        dx, dshift, dscale = ops.ln_modulate_backward(dh, x2, mean, rstd, scale, ctx.shape[1], _stream_grad(dstream, x2),
                                                      sums_dtype=_common(ctx.mod_dtypes))
        return (dx.view(ctx.shape), dshift.to(ctx.mod_dtypes[0]), dscale.to(ctx.mod_dtypes[1]), dw, db, None, None)


class _ActivationLinear(torch.autograd.Function):
    @staticmethod
    def forward(ctx, z, weight, bias, layer, activation):
        shape = z.shape
        z2 = z.reshape(-1, shape[-1]).contiguous()
        need_w, need_b = ctx.needs_input_grad[1], bias is not None and ctx.needs_input_grad[2]
        quantizer = layer.input_quantizer
        limit = layer._quantization_limit(max(z2.shape), layer.fp8_dtype)
        q, qt, qscale = ops.activation_quantize(z2, activation, history=quantizer.history, index=quantizer.index,
                                                delayed=quantizer.scaling == "delayed", fp8_dtype=layer.fp8_dtype,
                                                quantization_limit=limit, transpose=need_w and not layer.in_place_operands)
        quantizer.index += 1
        encoded = SimpleNamespace(q=q, s=qscale, qt=qt, st=qscale)
        y, saved, _ = linear_forward(layer, z2, weight, bias, need_input_grad=True, need_weight_grad=need_w,
                                     encoded=encoded)
        ctx.save_for_backward(z2)
        ctx.layer, ctx.saved, ctx.shape, ctx.need_b, ctx.activation = layer, saved, shape, need_b, activation
        return y.reshape(*shape[:-1], layer.out_features)

    @staticmethod
    def backward(ctx, dy):
        z2, = ctx.saved_tensors
        layer = ctx.layer
        dy2 = dy.reshape(-1, layer.out_features).contiguous()
        da, dw, db = linear_backward(layer, ctx.saved, dy2, need_input_grad=True, need_weight_grad=ctx.needs_input_grad[1],
                                     need_bias_grad=ctx.need_b)
        if ctx.activation == "gelu":
            dz = torch.ops.aten.gelu_backward(da, z2, approximate="tanh")
        else:
            dz = torch.ops.aten.silu_backward(da, z2)
        return dz.view(ctx.shape), dw, db, None, None


class _NormModulateMLP(torch.autograd.Function):
    """fc2(act(fc1(LN(x) * (1 + scale) + shift))) as one autograd node.

    Forward: statistics + amax, encode, GEMM, activation amax, encode, GEMM (the normalised and the activated
    tensors are never written; the second encode also emits act'(z), which replaces z as the saved tensor).
    Backward: dY is encoded once (bias gradient from the same pass); the fc2 dgrad epilogue multiplies by the
    saved slope and gathers the amax of dZ, so dZ is written once and read once (encode + bias gradient); then
    both wgrads, the fc1 dgrad and the fused LayerNorm backward."""

    @staticmethod
    def forward(ctx, x, shift, scale, w1, b1, w2, b2, fc1, fc2, activation, eps):
        batch, tokens, width = x.shape
        x2 = x.reshape(-1, width).contiguous()
        need = ctx.needs_input_grad
        q1, limit1 = fc1.input_quantizer, fc1._quantization_limit(max(x2.shape), fc1.fp8_dtype)
        q, _, qscale, mean, rstd = ops.ln_modulate_quantize(
            x2, shift, scale, tokens, eps=eps, history=q1.history, index=q1.index, delayed=q1.scaling == "delayed",
            fp8_dtype=fc1.fp8_dtype, quantization_limit=limit1)
        q1.index += 1
        z, saved1, _ = linear_forward(fc1, x2, w1, b1, need_input_grad=True, need_weight_grad=need[3],
                                      encoded=SimpleNamespace(q=q, s=qscale, qt=None, st=qscale),
                                      out_dtype=torch.bfloat16)
        q2, limit2 = fc2.input_quantizer, fc2._quantization_limit(max(z.shape), fc2.fp8_dtype)
        qa, _, ascale, slope = ops.activation_quantize(z, activation, history=q2.history, index=q2.index,
                                                       delayed=q2.scaling == "delayed", fp8_dtype=fc2.fp8_dtype,
                                                       quantization_limit=limit2, slope=True)
        q2.index += 1
        y, saved2, _ = linear_forward(fc2, z, w2, b2, need_input_grad=True, need_weight_grad=need[5],
                                      encoded=SimpleNamespace(q=qa, s=ascale, qt=None, st=ascale))
        ctx.save_for_backward(x2, scale, mean, rstd, slope)       # act'(z) stands in for z in the backward
        ctx.layers, ctx.saved, ctx.shape = (fc1, fc2), (saved1, saved2), x.shape
        ctx.need_bias = (b1 is not None and need[4], b2 is not None and need[6])
        ctx.mod_dtypes = (shift.dtype, scale.dtype)
        ctx.set_materialize_grads(False)
        return y.reshape(batch, tokens, -1), x.view_as(x)

    @staticmethod
    def backward(ctx, dy, dstream):
        if dy is None:
            return (dstream,) + (None,) * 10
        x2, scale, mean, rstd, slope = ctx.saved_tensors
        fc1, fc2 = ctx.layers
        saved1, saved2 = ctx.saved
        need = ctx.needs_input_grad
        dy2 = dy.reshape(-1, fc2.out_features).contiguous()
        amax = ops.amax_word(dy2.device)
        dz, dw2, db2 = linear_backward(fc2, saved2, dy2, need_input_grad=True, need_weight_grad=need[5],
                                       need_bias_grad=ctx.need_bias[1], act=(slope, amax))
        dh, dw1, db1 = linear_backward(fc1, saved1, dz, need_input_grad=True, need_weight_grad=need[3],
                                       need_bias_grad=ctx.need_bias[0], grad_amax=amax)
        del dz
        dx, dshift, dscale = ops.ln_modulate_backward(dh, x2, mean, rstd, scale, ctx.shape[1], _stream_grad(dstream, x2),
                                                      sums_dtype=_common(ctx.mod_dtypes))
        return (dx.view(ctx.shape), dshift.to(ctx.mod_dtypes[0]), dscale.to(ctx.mod_dtypes[1]), dw1, db1, dw2, db2,
                None, None, None, None)


def norm_modulate_mlp(x, shift, scale, fc1, fc2, activation="gelu", *, eps=1e-6, carry=False):
    """``fc2(act(fc1(LayerNorm(x) * (1 + scale[:, None]) + shift[:, None])))`` for ``x`` [batch, tokens, width].

    ``carry=True`` returns ``(result, x)``: use the returned ``x`` for the residual connection that follows.  Its
    gradient then reaches the LayerNorm backward kernel, which adds it to its own input gradient in the same pass
    (instead of autograd summing the two branches with a separate kernel)."""
    if (x.is_cuda and torch.is_autocast_enabled("cuda") and torch.get_autocast_dtype("cuda") == torch.bfloat16
            and x.dim() == 3 and torch.is_grad_enabled() and x.requires_grad
            and _eligible(fc1, x, 2048, _STREAM_DTYPES) and fc1.in_place_operands
            and isinstance(fc2, Linear) and fc2.in_place_operands and not fc2.rotation_size
            and fc2.saved_input_dtype == "fp8"):
        shift, scale = shift.to(torch.bfloat16), scale.to(torch.bfloat16)
        if _rows_of(shift, x) and _rows_of(scale, x) and shift.stride(0) == scale.stride(0):
            result, stream = _NormModulateMLP.apply(x, shift, scale, fc1.weight, fc1.bias, fc2.weight, fc2.bias, fc1,
                                                    fc2, activation, eps)
            return (result, stream) if carry else result
    result = activation_linear(norm_modulate_linear(x, shift, scale, fc1, eps=eps), fc2, activation)
    return (result, x) if carry else result


def _rows_of(vector, x):
    """Is ``vector`` a bf16 [batch, width] per-sample row set the kernels can read in place (rows may be strided)?"""
    return (vector.dim() == 2 and vector.dtype == torch.bfloat16 and vector.shape == (x.shape[0], x.shape[-1])
            and vector.stride(1) == 1 and vector.stride(0) % 8 == 0 and vector.data_ptr() % 16 == 0)


def norm_modulate_linear(x, shift, scale, layer, *, eps=1e-6, carry=False):
    """``layer(LayerNorm(x) * (1 + scale[:, None]) + shift[:, None])`` for ``x`` [batch, tokens, width].
    ``carry=True`` returns ``(result, x)`` as in :func:`norm_modulate_mlp`."""
    stream = x
    fused = False
    if x.is_cuda and torch.is_autocast_enabled("cuda"):
        dtype = torch.get_autocast_dtype("cuda")
        shift, scale = shift.to(dtype), scale.to(dtype)
        fused = (dtype == torch.bfloat16 and _eligible(layer, x, 2048, _STREAM_DTYPES) and x.dim() == 3
                 and _rows_of(shift, x) and _rows_of(scale, x) and shift.stride(0) == scale.stride(0)
                 and torch.is_grad_enabled() and x.requires_grad)
        if not fused:
            x = x.to(dtype)
    else:
        fused = (_eligible(layer, x, 2048) and x.dim() == 3 and _rows_of(shift, x) and _rows_of(scale, x)
                 and shift.stride(0) == scale.stride(0) and torch.is_grad_enabled() and x.requires_grad)
    if fused:
        result, stream = _NormModulateLinear.apply(x, shift, scale, layer.weight, layer.bias, layer, eps)
    else:
        normed = F.layer_norm(x, (x.shape[-1],), eps=eps)
        result = layer(torch.addcmul(shift[:, None], normed, (1 + scale)[:, None]))
    return (result, stream) if carry else result


def activation_linear(z, layer, activation="gelu"):
    """``layer(act(z))`` with ``act`` = tanh-GELU or SiLU."""
    if z.is_cuda and torch.is_autocast_enabled("cuda"):
        z = z.to(torch.get_autocast_dtype("cuda"))
    if _eligible(layer, z) and torch.is_grad_enabled() and z.requires_grad and z.shape[-1] % 16 == 0:
        return _ActivationLinear.apply(z, layer.weight, layer.bias, layer, activation)
    return layer(F.gelu(z, approximate="tanh") if activation == "gelu" else F.silu(z))


class _GatedResidual(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gate, y):
        batch, tokens, width = x.shape
        y2 = y.reshape(-1, width).contiguous()
        out = ops.gate_residual(x.reshape(-1, width).contiguous(), gate, y2, tokens)
        ctx.save_for_backward(gate, y2)
        ctx.shape = x.shape
        return out.view(x.shape)

    @staticmethod
    def backward(ctx, dout):
        gate, y2 = ctx.saved_tensors
        batch, tokens, width = ctx.shape
        dy, dgate = ops.gate_residual_backward(dout.reshape(-1, width).contiguous(), gate, y2, tokens,
                                               sums_dtype=gate.dtype)
        return dout, dgate.to(gate.dtype), dy.view(ctx.shape)


def gated_residual(x, gate, y):
    """``x + gate[:, None] * y`` for ``x`` / ``y`` [batch, tokens, width] and a per-sample ``gate`` [batch, width]."""
    if (x.is_cuda and x.dim() == 3 and x.dtype in _STREAM_DTYPES and y.dtype == torch.bfloat16 and y.shape == x.shape
            and _rows_of(gate, x) and x.shape[-1] <= 2048 and x.shape[-1] % 8 == 0 and torch.is_grad_enabled()
            and (x.requires_grad or y.requires_grad or gate.requires_grad)):
        return _GatedResidual.apply(x, gate, y)
    return torch.addcmul(x, gate[:, None], y)
