"""FP8 Linear layer: FP8 / BF16 / FP16 weight storage, FP8 tensor-core forward, dgrad and wgrad.

Public surface and semantics follow the reference layer (viola/nn/linear.py:150-412, grouped
recipe viola/nn/_grouped_linear.py:10-102): constructor options, parameter / buffer names
(``weight``, ``bias``, ``weight_scale``, the three quantizers' ``history`` + extra state), the
``refresh_weight`` / ``dequantize_weight`` / ``from_float`` / ``rebuild_weight_cache`` methods and
the memory / fast modes.  The implementation is different: one functional core
(:func:`linear_forward` / :func:`linear_backward`) drives the sm_100a kernels in
:mod:`viola_b200.ops` (tcgen05 GEMMs with TMEM accumulators, fused amax->scale, one-read
rowwise+transposed quantisers) and is shared with the fused gated MLP.

Scaling recipes: ``current`` / ``delayed`` = one fp32 scale per tensor; ``grouped`` = one fp32 scale
per (rows x cols) group, K-groups of 128 and wider run the two-level-accumulation tcgen05 kernel,
other shapes decode to bf16 first; ``mxfp8`` = power-of-two (UE8M0) scales per 32 K elements, chosen by the
encode kernel and applied by the tensor core (``tcgen05.mma.kind::mxf8f6f4.block_scale``).
The accumulator is always fp32 in tensor memory; ``accum_dtype='fp16'`` only keeps its documented
effect on the quantisation range (``_quantization_limit``).
"""

from __future__ import annotations

import math
from types import SimpleNamespace

import torch
from torch import nn

from .. import ops
from ..precision import settings

_FORMATS = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}
_STORAGE = {"bf16": torch.bfloat16, "fp16": torch.float16}
_SAVED = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32}


class _Quantizer(nn.Module):
    """Amax history ring for delayed scaling plus the running call index (checkpointed)."""

    def __init__(self, scaling, history_len, device):
        super().__init__()
        self.scaling = scaling
        self.index = 0
        self.register_buffer("history", torch.zeros(history_len, device=device, dtype=torch.float32))

    def scale(self, x, fp8_dtype=torch.float8_e4m3fn, quantization_limit=None, out=None):
        result = ops.tensor_scale(x, history=self.history, index=self.index, delayed=self.scaling == "delayed",
                                  fp8_dtype=fp8_dtype, quantization_limit=quantization_limit, out=out)
        self.index += 1
        return result

    def scale_gathered(self, amax_bits, fp8_dtype=torch.float8_e4m3fn, quantization_limit=None):
        """Same bookkeeping as :meth:`scale` for an amax that a producer kernel already gathered (float bits)."""
        result = ops.scale_from_amax(amax_bits, history=self.history, index=self.index,
                                     delayed=self.scaling == "delayed", fp8_dtype=fp8_dtype,
                                     quantization_limit=quantization_limit)
        self.index += 1
        return result

    def get_extra_state(self):
        return {"index": self.index, "scaling": self.scaling}

    def set_extra_state(self, state):
        self.index, self.scaling = state["index"], state["scaling"]


def transpose_group(group):
    """Group shape seen from the transposed matrix: 2-D blocks flip, 1-D row groups stay 1-D."""
    return tuple(group[::-1]) if group[0] >= 32 else tuple(group)


# ------------------------------------------------------------------------------------------------
# quantisation helpers (activation side)
# ------------------------------------------------------------------------------------------------
def _quantize_activation(layer, x, fmt, group, quantizer, limit, *, row, transposed, scale=None, colsum=None):
    """Returns SimpleNamespace(q, s, qt, st).  Per-tensor recipes share one scale for both layouts; ``colsum``
    (per-tensor only) receives the fp32 column sums of ``x`` from the same pass."""
    result = SimpleNamespace(q=None, s=None, qt=None, st=None)
    if layer._grouped_scaling:
        pow2 = layer._native_scaling          # MXFP8: every scale a power of two, chosen inside the encode kernel
        if row and transposed:
            result.q, result.s, result.qt, result.st = ops.group_quantize_pair(x, fmt, group, group, limit=limit,
                                                                               kmajor=True, pow2=pow2)
        elif row:
            result.q, result.s = ops.group_quantize(x, fmt, group, limit=limit, kmajor=True, pow2=pow2)
        elif transposed:
            result.qt, result.st = ops.group_quantize(x, fmt, group, limit=limit, transposed=True, kmajor=True,
                                                      pow2=pow2)
        return result
    if layer.rotation_size:
        x = ops.hadamard64(x)
    if scale is None:
        scale = quantizer.scale(x, fmt, limit)
    q, qt = ops.quantize(x, scale, rowwise=row, transpose=transposed, fp8_dtype=fmt, quantization_limit=limit,
                         colsum=colsum)
    result.q = q if row else None
    result.qt = qt if transposed else None
    result.s = result.st = scale
    return result


def _weight_operands(layer, weight, *, need_transpose):
    """FP8 codes + scales of W (and W^T when asked) for this call, from whatever storage W uses."""
    fmt = layer.fp8_dtype
    out = SimpleNamespace(q=None, s=None, qt=None, st=None)
    if layer._grouped_scaling:
        gw = layer.weight_group_shape
        limit = layer._group_limit(gw, fmt, weight=True)
        if layer.weight_dtype == "fp8":
            out.q, out.s = weight, layer._scale_float()
            if need_transpose and layer.weight_transpose.numel():
                out.qt, out.st = layer.weight_transpose, layer.weight_transpose_scale
        else:
            out.q, out.s = layer._encode_weight(weight, gw, limit)
            if need_transpose:
                out.qt, out.st = layer._encode_weight(weight, transpose_group(gw), limit, transposed=True)
        return out
    limit = layer._quantization_limit(max(weight.shape), fmt)
    if layer.weight_dtype == "fp8":
        out.q, out.s = weight, layer.weight_scale
        if need_transpose and layer.weight_transpose.numel():
            out.qt = layer.weight_transpose
    else:
        source = ops.hadamard64(weight) if layer.rotation_size else weight
        out.s = layer.weight_quantizer.scale(source, fmt, limit)
        out.q, qt = ops.quantize(source, out.s, transpose=need_transpose, fp8_dtype=fmt, quantization_limit=limit)
        out.qt = qt if need_transpose else None
    out.st = out.s
    return out


# ------------------------------------------------------------------------------------------------
# functional core, shared by Linear and the fused MLP
# ------------------------------------------------------------------------------------------------
def linear_forward(layer, x, weight, bias, *, need_input_grad, need_weight_grad, gated=None, encoded=None,
                   out_dtype=None):
    """y = x W^T + b on 2-D ``x``.  Returns (y, saved, aux) where ``saved`` feeds :func:`linear_backward`.

    ``gated`` = activation name turns the GEMM into the fused gate/up epilogue (``aux`` = [g | u]);
    ``encoded`` = already quantised input (q, s, qt, st) produced by a fused producer; ``out_dtype`` = dtype
    of y and of the input gradient when it differs from ``x.dtype`` (a fused producer reading an fp32 stream).
    """
    out_dtype = out_dtype or x.dtype
    fmt = layer.fp8_dtype
    need_backward = need_input_grad or need_weight_grad
    save_fp8 = need_weight_grad and layer.saved_input_dtype == "fp8"
    gx, gw = layer.input_group_shape, layer.weight_group_shape
    if layer._grouped_scaling:
        limit = layer._group_limit(gx, fmt)
    else:
        limit = layer._quantization_limit(max(x.shape), fmt)
    # per-tensor recipes hand the GEMM the row-wise codes for every product (the tensor core reads a
    # transposed operand MN-major in place), so no transposed copy of X, dY or W is ever written
    in_place = layer.in_place_operands
    qx = encoded if encoded is not None else _quantize_activation(
        layer, x, fmt, gx, layer.input_quantizer, limit, row=True, transposed=save_fp8 and not in_place)
    w = _weight_operands(layer, weight,
                         need_transpose=need_input_grad and layer.cache_weight_transpose and not in_place)
    aux = None
    if gated is not None:
        group = (gx, gw) if layer._grouped_scaling else None
        y, aux = ops.gated_gemm_forward(qx.q, w.q, qx.s, w.s, activation=gated, out_dtype=out_dtype, bias=bias,
                                        save=need_backward, group=group, sa_kmajor=True)
    elif layer._grouped_scaling:
        y = ops.group_gemm(qx.q, w.q, qx.s, w.s, gx, gw, out_dtype=out_dtype, bias=bias, sa_kmajor=True,
                           mx=layer._native_scaling)
    else:
        y = ops.gemm(qx.q, w.q, qx.s, w.s, out_dtype=out_dtype, bias=bias)
    saved = None
    if need_backward:
        saved = SimpleNamespace(x=None, x_scale=None, x_is_fp8=save_fp8, input_scale=qx.s, weight=weight,
                                weight_scale=w.s, wt=w.qt, wt_scale=w.st, limit=limit, x_dtype=out_dtype,
                                in_place=in_place, wq=None,
                                weight_grad_dtype=getattr(weight, "grad_dtype", None) or torch.float32,
                                bias_grad_dtype=(getattr(bias, "grad_dtype", None) or bias.dtype) if bias is not None else None,
                                # an engine may offer a place to write each gradient straight into (its landing
                                # buffer for the gradient reduction); asked for again at backward time
                                weight_slot=getattr(weight, "_viola_grad_slot", None),
                                bias_slot=getattr(bias, "_viola_grad_slot", None) if bias is not None else None)
        if in_place and need_input_grad and layer.weight_dtype != "fp8" and layer.cache_weight_transpose:
            saved.wq = w.q                              # fast mode: keep this call's codes for dgrad
        if save_fp8:
            saved.x, saved.x_scale = (qx.q, qx.s) if in_place else (qx.qt, qx.st)
        elif need_weight_grad:
            saved.x = x.to(_SAVED[layer.saved_input_dtype])
    return y, saved, aux


def _adds_up(slot):
    """Does this landing slot hold the running sum of the step's microbatches (the producer then adds into it)?"""
    return slot is not None and getattr(slot, "_viola_accumulate", False)


def _hand_back(slot):
    """Tell the engine that this landing slot will not be written by the producer after all."""
    release = getattr(slot, "_viola_release", None)
    if release is not None:
        release()
    return None


def _gradient_slot(offer, shape, dtype, device):
    """The engine's landing slot for a gradient about to be computed, when it offers one that fits."""
    if offer is None:
        return None
    slot = offer()
    if slot is None:
        return None
    if tuple(slot.shape) != tuple(shape) or slot.dtype != dtype or slot.device != device or not slot.is_contiguous():
        return _hand_back(slot)
    return slot


def linear_backward(layer, saved, dy, *, need_input_grad, need_weight_grad, need_bias_grad, gated=None, aux=None,
                    act=None, grad_amax=None):
    """Returns (dx, dw, db).  ``gated``: dx becomes [dG | dU] through the fused derivative epilogue.

    Layers with :attr:`Linear.in_place_operands` additionally take ``act=(slope, amax_bits)``: the layer's input
    was ``activation(z)`` with ``slope = activation'(z)``, and dx becomes the gradient of ``z`` straight from the
    dgrad epilogue, its amax gathered into ``amax_bits``; and ``grad_amax`` = such a gathered amax of ``dy``
    itself (skips the amax pass).
    """
    fmt, bfmt = layer.fp8_dtype, layer.backward_fp8_dtype
    gg, gx, gw = layer.grad_group_shape, layer.input_group_shape, layer.weight_group_shape
    grouped = layer._grouped_scaling
    if grouped:
        limit = layer._group_limit(gg, bfmt)
    else:
        limit = layer._quantization_limit(max(dy.shape), bfmt)
    dx = dw = db = None
    if saved.in_place:
        return _backward_in_place(layer, saved, dy, limit, need_input_grad, need_weight_grad, need_bias_grad, gated, aux,
                                  act, grad_amax)
    assert act is None and grad_amax is None, "fused activation backward needs in-place operands"
    # memory mode keeps one FP8 copy of dY alive at a time; fast mode encodes both layouts in one read
    both = need_input_grad and need_weight_grad and layer.mode == "fast"
    qg = _quantize_activation(layer_no_rotation(layer), dy, bfmt, gg, layer.grad_quantizer, limit,
                              row=need_input_grad, transposed=both or (need_weight_grad and not need_input_grad))
    if need_input_grad:
        wt, wt_scale = saved.wt, saved.wt_scale
        if wt is None or not wt.numel():
            wt, wt_scale = layer._transposed_weight(saved.weight, saved.weight_scale)
        if gated is not None and not layer.rotation_size:
            group = (gg, transpose_group(gw)) if grouped else None
            dx = ops.gated_gemm_backward(qg.q, wt, qg.s, wt_scale, aux, activation=gated, out_dtype=saved.x_dtype,
                                         group=group, sg_kmajor=True)
        else:
            if grouped:
                dx = ops.group_gemm(qg.q, wt, qg.s, wt_scale, gg, transpose_group(gw), out_dtype=saved.x_dtype,
                                    sa_kmajor=True, mx=layer._native_scaling)
            else:
                dx = ops.gemm(qg.q, wt, qg.s, wt_scale, out_dtype=saved.x_dtype)
            if layer.rotation_size:
                ops.hadamard64(dx, out=dx)
            if gated is not None:
                dx = ops.gated_backward(aux, dx, gated)
        del wt
    if need_weight_grad:
        if qg.qt is None:
            qg.q = None
            late = _quantize_activation(layer_no_rotation(layer), dy, bfmt, gg, layer.grad_quantizer, limit, row=False,
                                        transposed=True, scale=None if grouped else qg.s)
            qg.qt, qg.st = late.qt, late.st
        if saved.x_is_fp8:
            xt, xt_scale = saved.x, saved.x_scale
        else:
            enc = _quantize_activation(layer, saved.x, fmt, gx, layer.input_quantizer, saved.limit, row=False,
                                       transposed=True, scale=None if grouped else saved.input_scale)
            xt, xt_scale = enc.qt, enc.st
        if grouped:
            dw = ops.group_gemm(qg.qt, xt, qg.st, xt_scale, gg, gx, out_dtype=saved.weight_grad_dtype, sa_kmajor=True,
                                sb_kmajor=True, mx=layer._native_scaling)
        else:
            slot = _gradient_slot(getattr(saved, "weight_slot", None), (qg.qt.shape[0], xt.shape[0]),
                                  saved.weight_grad_dtype, dy.device)
            if _adds_up(slot) and layer.rotation_size:
                slot = _hand_back(slot)         # the rotation below works in place on this microbatch's gradient only
            dw = ops.gemm(qg.qt, xt, qg.st, xt_scale, out_dtype=saved.weight_grad_dtype, out=slot,
                          accumulate=_adds_up(slot))
        if layer.rotation_size:
            ops.hadamard64(dw, out=dw)
    if need_bias_grad:
        db = dy.sum(dim=0, dtype=saved.bias_grad_dtype)
    return dx, dw, db


def _backward_in_place(layer, saved, dy, limit, need_input_grad, need_weight_grad, need_bias_grad, gated, aux,
                       act=None, grad_amax=None):
    """Per-tensor backward from row-wise codes only: dX = dY W reads W as an MN-major B operand, dW = dY^T X
    reads both dY and X MN-major."""
    fmt, bfmt = layer.fp8_dtype, layer.backward_fp8_dtype
    dx = dw = db = None
    # the bias gradient (column sums of dY) comes out of the pass that encodes dY
    db_sum = None
    if need_bias_grad:
        slot = _gradient_slot(getattr(saved, "bias_slot", None), (dy.shape[1],), torch.float32, dy.device) \
            if saved.bias_grad_dtype == torch.float32 else None
        if slot is None:
            db_sum = torch.zeros(dy.shape[1], device=dy.device, dtype=torch.float32)
        else:                             # the engine clears all one-dimensional slots in one launch per microbatch,
            # or keeps the running sum of the step in them
            db_sum = slot if (getattr(slot, "_viola_zeroed", False) or _adds_up(slot)) else slot.zero_()
    grad_scale = layer.grad_quantizer.scale_gathered(grad_amax, bfmt, limit) if grad_amax is not None else None
    qg = _quantize_activation(layer_no_rotation(layer), dy, bfmt, None, layer.grad_quantizer, limit, row=True,
                              transposed=False, colsum=db_sum, scale=grad_scale)
    if need_input_grad:
        wq = saved.wq
        if wq is None and layer.weight_dtype == "fp8":
            wq = saved.weight
        elif wq is None:
            source = ops.hadamard64(saved.weight) if layer.rotation_size else saved.weight
            wq, _ = ops.quantize(source, saved.weight_scale, fp8_dtype=fmt,
                                 quantization_limit=layer._quantization_limit(max(source.shape), fmt))
        if act is not None:
            assert not layer.rotation_size and gated is None
            dx = ops.activation_backward_gemm(qg.q, wq, qg.s, saved.weight_scale, act[0], w_mn=True, amax_out=act[1])
        elif gated is not None and not layer.rotation_size:
            dx = ops.gated_gemm_backward(qg.q, wq, qg.s, saved.weight_scale, aux, activation=gated,
                                         out_dtype=saved.x_dtype, wt_mn=True)
        else:
            dx = ops.gemm(qg.q, wq, qg.s, saved.weight_scale, out_dtype=saved.x_dtype, b_mn=True)
            if layer.rotation_size:
                ops.hadamard64(dx, out=dx)
            if gated is not None:
                dx = ops.gated_backward(aux, dx, gated)
        del wq
    if need_weight_grad:
        if saved.x_is_fp8:
            xq, x_scale = saved.x, saved.x_scale
        else:
            enc = _quantize_activation(layer, saved.x, fmt, None, layer.input_quantizer, saved.limit, row=True,
                                       transposed=False, scale=saved.input_scale)
            xq, x_scale = enc.q, enc.s
        slot = _gradient_slot(getattr(saved, "weight_slot", None), (qg.q.shape[1], xq.shape[1]), saved.weight_grad_dtype,
                              dy.device)
        if _adds_up(slot) and layer.rotation_size:
            slot = _hand_back(slot)
        dw = ops.gemm(qg.q, xq, qg.s, x_scale, out_dtype=saved.weight_grad_dtype, a_mn=True, b_mn=True, out=slot,
                      accumulate=_adds_up(slot))
        if layer.rotation_size:
            ops.hadamard64(dw, out=dw)
    if need_bias_grad:
        db = db_sum.to(saved.bias_grad_dtype)
    return dx, dw, db


class _NoRotation:
    """View of a layer whose rotation is disabled (output gradients are never rotated)."""

    def __init__(self, layer):
        self._layer = layer

    rotation_size = 0

    def __getattr__(self, name):
        return getattr(self._layer, name)


def layer_no_rotation(layer):
    return _NoRotation(layer) if layer.rotation_size else layer


class _LinearFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, layer, need_backward):
        shape = x.shape
        x2 = x.reshape(-1, layer.in_features).contiguous()
        need_x = need_backward and ctx.needs_input_grad[0]
        need_w = need_backward and ctx.needs_input_grad[1]
        y, saved, _ = linear_forward(layer, x2, weight, bias, need_input_grad=need_x, need_weight_grad=need_w)
        if need_backward:
            ctx.layer, ctx.saved, ctx.shape = layer, saved, shape
            if saved is None:
                ctx.saved = SimpleNamespace(bias_grad_dtype=(getattr(bias, "grad_dtype", None) or bias.dtype)
                                            if bias is not None else None)
        return y.reshape(*shape[:-1], layer.out_features)

    @staticmethod
    def backward(ctx, dy):
        layer = ctx.layer
        dy2 = dy.reshape(-1, layer.out_features).contiguous()
        need_x, need_w, need_b = ctx.needs_input_grad[:3]
        if not (need_x or need_w):
            db = dy2.sum(dim=0, dtype=ctx.saved.bias_grad_dtype) if need_b else None
            return None, None, db, None, None
        dx, dw, db = linear_backward(layer, ctx.saved, dy2, need_input_grad=need_x, need_weight_grad=need_w,
                                     need_bias_grad=need_b)
        if dx is not None:
            dx = dx.reshape(*ctx.shape[:-1], layer.in_features)
        return dx, dw, db, None, None


class Linear(nn.Module):
    """FP8-compute linear layer with selectable weight storage.

    Build and move the model first, then construct the optimizer and call
    ``viola_b200.optim.bind_optimizer(model, optimizer)`` (or hand both to ``violaEngine``).  Inputs and
    outputs are ordinary 16/32-bit tensors.
    """

    def __init__(self, in_features, out_features, bias=True, *, mode="memory", weight_dtype="fp8",
                 forward_dtype="e4m3", backward_dtype="e5m2", cache_weight_transpose=None, saved_input_dtype="fp8",
                 scaling="current", history_len=16, autotune=False, accum_dtype="fp32", accum_block_size=0,
                 accum_reduce_dtype="fp32", quantization_limit=None, rotation_size=0, weight_group_shape=(32, 32),
                 input_group_shape=(1, 32), grad_group_shape=(1, 32), device=None, dtype=None):
        super().__init__()
        if mode not in ("memory", "fast"):
            raise ValueError("mode must be 'memory' or 'fast'")
        if weight_dtype not in ("fp8", "bf16", "fp16"):
            raise ValueError("weight_dtype must be fp8, bf16 or fp16")
        if saved_input_dtype not in ("fp8", "bf16", "fp16", "fp32"):
            raise ValueError("saved_input_dtype must be fp8, bf16, fp16 or fp32")
        if scaling not in ("current", "delayed", "grouped", "mxfp8") or history_len <= 0:
            raise ValueError("scaling must be current, delayed, grouped or mxfp8 and history_len positive")
        if accum_dtype not in ("fp32", "fp16") or accum_reduce_dtype not in ("fp32", "bf16"):
            raise ValueError("unsupported accumulation dtype")
        if accum_block_size < 0 or accum_block_size % 32:
            raise ValueError("accum_block_size must be a non-negative multiple of 32")
        if rotation_size not in (0, 64) or (rotation_size and in_features % rotation_size):
            raise ValueError("rotation_size must be 0 or 64 and divide in_features")
        self.in_features, self.out_features = in_features, out_features
        self.mode, self.weight_dtype, self.saved_input_dtype = mode, weight_dtype, saved_input_dtype
        self.forward_dtype, self.backward_dtype = forward_dtype, backward_dtype
        self.fp8_dtype, self.backward_fp8_dtype = _FORMATS[forward_dtype], _FORMATS[backward_dtype]
        self._grouped_scaling = scaling in ("grouped", "mxfp8")
        self._native_scaling = scaling == "mxfp8"
        self.weight_group_shape = tuple(weight_group_shape)
        self.input_group_shape = tuple(input_group_shape)
        self.grad_group_shape = tuple(grad_group_shape)
        if self._grouped_scaling:
            if rotation_size:
                raise ValueError("grouped scaling does not combine with rotation_size")
            for gr, gc in (self.weight_group_shape, self.input_group_shape, self.grad_group_shape):
                if gr <= 0 or gr & (gr - 1) or gc < 32 or gc & (gc - 1):
                    raise ValueError("group shapes must be powers of two with at least 32 columns")
            if self._native_scaling and (accum_dtype != "fp32" or accum_block_size or accum_reduce_dtype != "fp32"):
                raise ValueError("mxfp8 accumulates in fp32")
        self.autotune = autotune
        if autotune:
            from .. import tuning
            tuning.enable()          # first-use tile search for every GEMM signature, cached on disk
        self.accum_dtype, self.accum_block_size, self.accum_reduce_dtype = accum_dtype, accum_block_size, accum_reduce_dtype
        self.quantization_limit = quantization_limit
        self.rotation_size = rotation_size
        self.cache_weight_transpose = (mode == "fast") if cache_weight_transpose is None else cache_weight_transpose
        policy = settings()
        master_dtype = policy["master_weight_dtype"] or torch.float32
        gradient_dtype = policy["gradient_dtype"] or torch.float32
        dtype = dtype or torch.get_default_dtype()
        fp8_storage = weight_dtype == "fp8"
        # With FP8 storage the initial real-valued weight is kept aside and handed to the optimizer
        # as its master copy; 16-bit storage is initialised in place.
        self._initial_weight = (torch.empty((out_features, in_features), device=device, dtype=master_dtype)
                                if fp8_storage else None)
        self._master_ref = None
        storage = self.fp8_dtype if fp8_storage else _STORAGE[weight_dtype]
        self.weight = nn.Parameter(torch.empty((out_features, in_features), device=device, dtype=storage))
        self.weight.grad_dtype = gradient_dtype
        self.bias = nn.Parameter(torch.empty(out_features, device=device, dtype=dtype)) if bias else None
        if self.bias is not None:
            self.bias.grad_dtype = gradient_dtype
        if self._grouped_scaling:
            shape = ops.scale_shape((out_features, in_features), self.weight_group_shape) if fp8_storage else (0, 0)
        else:
            shape = (1,) if fp8_storage else (0,)
        scale_dtype = torch.uint8 if self._native_scaling else torch.float32
        self.register_buffer("weight_scale", torch.full(shape, 127 if self._native_scaling else 1, device=device,
                                                        dtype=scale_dtype), persistent=fp8_storage)
        self.register_buffer("weight_transpose", torch.empty(0, 0, device=device, dtype=self.fp8_dtype),
                             persistent=False)
        if self._grouped_scaling:
            self.register_buffer("weight_transpose_scale", torch.empty(0, 0, device=device, dtype=torch.float32),
                                 persistent=False)
        self.weight_quantizer = _Quantizer(scaling, history_len, device)
        self.input_quantizer = _Quantizer(scaling, history_len, device)
        self.grad_quantizer = _Quantizer(scaling, history_len, device)
        self.reset_parameters()

    # ------------------------------------------------------------------ quantisation range policy
    def _quantization_limit(self, reduction, fp8_dtype):
        maximum = torch.finfo(fp8_dtype).max
        if self.quantization_limit is not None:
            return min(self.quantization_limit, maximum)
        if self.accum_dtype == "fp32":
            return None
        if self.accum_block_size:
            reduction = self.accum_block_size
        return min(2.0 ** math.floor(math.log2(math.sqrt(32768.0 / reduction))), maximum)

    def _group_limit(self, shape, dtype, weight=False):
        maximum = torch.finfo(dtype).max
        if self.quantization_limit is not None:
            return min(self.quantization_limit, maximum)
        if self.accum_dtype == "fp32":
            return None
        reduction = max(shape) if weight else shape[1]
        if self.accum_block_size:
            reduction = math.gcd(reduction, self.accum_block_size)
        return min(2.0 ** math.floor(math.log2(math.sqrt(32768.0 / reduction))), maximum)

    # ------------------------------------------------------------------ weight (re)quantisation
    def _scale_float(self, scale=None):
        scale = self.weight_scale if scale is None else scale
        return torch.exp2(scale.float() - 127) if scale.dtype == torch.uint8 else scale

    def _encode_weight(self, master, group, limit, *, transposed=False):
        return ops.group_quantize(master, self.fp8_dtype, group, limit=limit, transposed=transposed,
                                  pow2=self._native_scaling)

    @property
    def in_place_operands(self):
        """True when every product of this layer runs from row-wise FP8 codes (per-tensor scaling with
        16-byte aligned rows): the backward GEMMs then read W, X and dY MN-major in place and the layer keeps
        no transposed weight cache."""
        return not self._grouped_scaling and self.in_features % 16 == 0 and self.out_features % 16 == 0

    @property
    def _caches_transpose(self):
        return self.cache_weight_transpose and not self.in_place_operands

    def _transposed_weight(self, weight, scale):
        """W^T codes and scales for dgrad, built from the stored weight without touching its scale state."""
        if self._grouped_scaling:
            gw = self.weight_group_shape
            limit = self._group_limit(gw, self.fp8_dtype, weight=True)
            if self.weight_dtype != "fp8":
                return self._encode_weight(weight, transpose_group(gw), limit, transposed=True)
            scale = self._scale_float(scale)
            if gw[0] >= 32:
                return ops.transpose(weight), scale.t().contiguous()
            decoded = ops.group_dequantize(weight, scale, gw)
            return self._encode_weight(decoded, gw, limit, transposed=True)
        if self.weight_dtype != "fp8":
            source = ops.hadamard64(weight) if self.rotation_size else weight
            _, wt = ops.quantize(source, scale, rowwise=False, transpose=True, fp8_dtype=self.fp8_dtype,
                                 quantization_limit=self._quantization_limit(max(weight.shape), self.fp8_dtype))
            return wt, scale
        return ops.transpose(weight), scale

    @torch.no_grad()
    def reset_parameters(self):
        if self._master_ref is not None and self._master_ref() is not None:
            master = self._master_ref()
        else:
            master = self.weight if self.weight_dtype != "fp8" else self._initial_weight
        nn.init.kaiming_uniform_(master, a=math.sqrt(5))
        if self.bias is not None:
            bound = 1 / math.sqrt(self.in_features)
            nn.init.uniform_(self.bias, -bound, bound)
        self.refresh_weight(master)

    @torch.no_grad()
    def quantize_master(self, master, *, out=None, out_t=None):
        """FP8 codes of ``master`` under this layer's recipe; updates ``weight_scale`` and quantizer state.

        ``out`` / ``out_t`` receive the codes and (per-tensor recipes only) their transpose; with
        ``out=None`` a new tensor is returned and ``self.weight`` is left untouched, which is what an
        owner rank uses before shipping codes to the other ranks.
        """
        if self._grouped_scaling:
            gw = self.weight_group_shape
            limit = self._group_limit(gw, self.fp8_dtype, weight=True)
            q, s = self._encode_weight(master, gw, limit)
            self.weight_scale.copy_(torch.log2(s) + 127 if self._native_scaling else s)
            return q if out is None else out.copy_(q)
        limit = self._quantization_limit(max(self.in_features, self.out_features), self.fp8_dtype)
        source = ops.hadamard64(master) if self.rotation_size else master
        scale = self.weight_quantizer.scale(source, self.fp8_dtype, limit, out=self.weight_scale)
        q, _ = ops.quantize(source, scale, transpose=out_t is not None, fp8_dtype=self.fp8_dtype, out=out, out_t=out_t,
                            quantization_limit=limit)
        return q

    @torch.no_grad()
    def refresh_weight(self, master):
        """Re-derive the compute weight from an updated master (called after every optimizer step)."""
        if self.weight_dtype != "fp8":
            if master is not self.weight:
                self.weight.copy_(master)
            return
        if self._grouped_scaling:
            self.quantize_master(master, out=self.weight.data)
            if self.cache_weight_transpose:
                self.weight_transpose, self.weight_transpose_scale = self._transposed_weight(self.weight,
                                                                                             self.weight_scale)
            return
        if self._caches_transpose and self.weight_transpose.numel() == 0:
            self.weight_transpose = torch.empty((self.in_features, self.out_features), device=master.device,
                                                dtype=self.fp8_dtype)
        self.quantize_master(master, out=self.weight.data,
                             out_t=self.weight_transpose if self._caches_transpose else None)

    def dequantize_weight(self):
        """The real-valued weight in the original (unrotated) coordinates, as fp32."""
        if self.weight_dtype != "fp8":
            return self.weight.float()
        if self._grouped_scaling:
            return ops.group_dequantize(self.weight, self._scale_float(), self.weight_group_shape)
        weight = self.weight.float() * self.weight_scale
        return ops.hadamard64(weight) if self.rotation_size else weight

    @classmethod
    @torch.no_grad()
    def from_float(cls, linear, **kwargs):
        layer = cls(linear.in_features, linear.out_features, linear.bias is not None, device=linear.weight.device,
                    dtype=linear.weight.dtype, **kwargs)
        master = layer.weight if layer.weight_dtype != "fp8" else layer._initial_weight
        master.copy_(linear.weight)
        layer.weight_quantizer.history.zero_()      # the throw-away initialiser must not leak its amax
        layer.weight_quantizer.index = 0
        layer.refresh_weight(master)
        if linear.bias is not None:
            layer.bias.copy_(linear.bias)
            layer.bias.requires_grad_(linear.bias.requires_grad)
        layer.weight.requires_grad_(linear.weight.requires_grad)
        return layer

    @torch.no_grad()
    def rebuild_weight_cache(self):
        """Recompute the cached W^T from the current codes / scales; W itself is left alone."""
        if self._caches_transpose and self.weight_dtype == "fp8":
            if self._grouped_scaling:
                self.weight_transpose, self.weight_transpose_scale = self._transposed_weight(self.weight,
                                                                                             self.weight_scale)
            else:
                self.weight_transpose = ops.transpose(self.weight)

    def clear_weight_cache(self):
        if self.weight_transpose.numel() == 0 and (not hasattr(self, "weight_transpose_scale")
                                                  or self.weight_transpose_scale.numel() == 0):
            return                      # nothing cached (the usual case on the write-back path)
        self.weight_transpose = self.weight_transpose.new_empty((0, 0))
        if hasattr(self, "weight_transpose_scale"):
            self.weight_transpose_scale = self.weight_transpose_scale.new_empty((0, 0))

    # ------------------------------------------------------------------ forward
    def _needs_backward(self, x):
        return torch.is_grad_enabled() and (x.requires_grad or self.weight.requires_grad
                                            or (self.bias is not None and self.bias.requires_grad))

    def forward(self, x):
        if x.is_cuda and torch.is_autocast_enabled("cuda"):
            x = x.to(torch.get_autocast_dtype("cuda"))
        elif not x.is_cuda and torch.is_autocast_enabled("cpu"):
            x = x.to(torch.get_autocast_dtype("cpu"))
        return _LinearFunction.apply(x, self.weight, self.bias, self, self._needs_backward(x))

    # ------------------------------------------------------------------ device moves / checkpoints
    def __deepcopy__(self, memo):
        # Parameter.grad_dtype is not carried by copy.deepcopy; an FP8 parameter would then ask
        # autograd for FP8 gradients.
        import copy
        clone = self.__class__.__new__(self.__class__)
        memo[id(self)] = clone
        for key, value in self.__dict__.items():
            clone.__dict__[key] = copy.deepcopy(value, memo)
        for name in ("weight", "bias"):
            source, target = self._parameters.get(name), clone._parameters.get(name)
            if source is not None and target is not None:
                target.grad_dtype = source.grad_dtype
        return clone

    def _apply(self, fn, recurse=True):
        # Only the device of the FP8 codes, scales and histories may change; dtype casts such as
        # .half() must leave them alone.
        weight = self._parameters["weight"]
        self._parameters["weight"] = None
        grad_dtype = getattr(weight, "grad_dtype", None)
        names = ["weight_scale", "weight_transpose"] + (["weight_transpose_scale"] if self._grouped_scaling else [])
        held = [(self, name, self._buffers.pop(name)) for name in names]
        for quantizer in (self.weight_quantizer, self.input_quantizer, self.grad_quantizer):
            held.append((quantizer, "history", quantizer._buffers.pop("history")))
        super()._apply(fn, recurse)

        def move(tensor):
            return tensor.to(device=fn(torch.empty(0, device=tensor.device, dtype=torch.float32)).device)

        weight.data = move(weight.data)
        if weight.grad is not None:
            weight.grad = move(weight.grad)
        if grad_dtype is not None:
            weight.grad_dtype = grad_dtype
            if self.bias is not None:
                self.bias.grad_dtype = grad_dtype
        self._parameters["weight"] = weight
        for module, name, tensor in held:
            module._buffers[name] = move(tensor)
        if self._initial_weight is not None:
            self._initial_weight = move(self._initial_weight)
        return self

    def _load_from_state_dict(self, state_dict, prefix, *args, **kwargs):
        expected = self.fp8_dtype if self.weight_dtype == "fp8" else _STORAGE[self.weight_dtype]
        key = prefix + "weight"
        if key in state_dict and state_dict[key].dtype != expected:
            raise RuntimeError("checkpoint weight storage / FP8 format differs from this layer's configuration")
        super()._load_from_state_dict(state_dict, prefix, *args, **kwargs)
        self._initial_weight = None
        self.rebuild_weight_cache()

    def extra_repr(self):
        groups = (f", weight_group_shape={self.weight_group_shape}, input_group_shape={self.input_group_shape}, "
                  f"grad_group_shape={self.grad_group_shape}") if self._grouped_scaling else ""
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, "
                f"mode={self.mode!r}, weight_dtype={self.weight_dtype!r}, forward_dtype={self.forward_dtype!r}, "
                f"backward_dtype={self.backward_dtype!r}, cache_weight_transpose={self.cache_weight_transpose}, "
                f"saved_input_dtype={self.saved_input_dtype!r}, scaling={self.weight_quantizer.scaling!r}, "
                f"accum_dtype={self.accum_dtype!r}, rotation_size={self.rotation_size}{groups}")
