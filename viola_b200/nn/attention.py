"""Self-attention on a packed ``[batch, tokens, 3, heads, head_dim]`` projection.

The reference leaves attention to PyTorch SDPA (experiments/dit.py:36).  Here the packed projection is consumed as
the qkv GEMM wrote it and the result comes back as ``[batch, tokens, heads * head_dim]`` without a transpose or a
stacking copy.  Forward, for 256-token sequences (the DiT shapes): this package's tcgen05 kernel, one CTA per
(sample, head) with the whole score matrix in tensor memory (``csrc/attention_sm100.cu``).  Backward, and the
forward of every other shape: the flash-attention library's packed entry points.  Falls back to SDPA on CPU, for
dtypes flash-attention does not take, or when the package is unavailable.
"""

from __future__ import annotations

import torch
from torch.nn import functional as F

from .. import ops

try:
    from flash_attn import flash_attn_qkvpacked_func as _packed
    from flash_attn.flash_attn_interface import _wrapped_flash_attn_backward as _library_backward
except Exception:  # pragma: no cover - optional dependency
    _packed = _library_backward = None

_state = {"flash": _packed is not None, "native": True}


class _NativeForward(torch.autograd.Function):
    """Forward on this package's kernel; backward through the library kernel, which needs q, k, v, out and the
    log-sum-exp of every row, exactly what the forward kernel returns."""

    @staticmethod
    def forward(ctx, qkv):
        scale = qkv.shape[-1] ** -0.5
        out, lse = ops.attention_forward(qkv, scale)
        ctx.save_for_backward(qkv, out, lse)
        ctx.scale = scale
        return out

    @staticmethod
    def backward(ctx, dout):
        qkv, out, lse = ctx.saved_tensors
        dqkv = torch.empty_like(qkv)
        _library_backward(dout.contiguous(), qkv[:, :, 0], qkv[:, :, 1], qkv[:, :, 2], out, lse, dqkv[:, :, 0], dqkv[:, :, 1],
                          dqkv[:, :, 2], 0.0, ctx.scale, False, -1, -1, 0.0, None, False, rng_state=None)
        return dqkv


def packed_attention(qkv):
    """``qkv``: [batch, tokens, 3, heads, head_dim] -> [batch, tokens, heads * head_dim]."""
    batch, tokens, _, heads, head_dim = qkv.shape
    if _state["native"] and _library_backward is not None and ops.attention_eligible(qkv):
        return _NativeForward.apply(qkv).reshape(batch, tokens, heads * head_dim)
    if (_state["flash"] and qkv.is_cuda and qkv.dtype in (torch.bfloat16, torch.float16) and head_dim % 8 == 0
            and head_dim <= 256):
        try:
            return _packed(qkv).reshape(batch, tokens, heads * head_dim)
        except RuntimeError:
            _state["flash"] = False          # e.g. a build without kernels for this GPU: use SDPA from now on
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    return F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(batch, tokens, heads * head_dim)
