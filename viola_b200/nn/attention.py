"""Self-attention on a packed ``[batch, tokens, 3, heads, head_dim]`` projection.

Attention itself is library code here as it is in the reference (PyTorch SDPA in
experiments/dit.py:36).  What this wrapper adds is layout discipline: the packed-QKV flash-attention
entry consumes the qkv GEMM output as it is and returns ``[batch, tokens, heads * head_dim]`` as a view,
and its backward writes one packed gradient, so the two full-size copies of the SDPA formulation
(output transpose -> reshape, and stacking dq / dk / dv) disappear.  Falls back to SDPA on CPU, for
dtypes flash-attention does not take, or when the package is unavailable.
"""

from __future__ import annotations

import torch
from torch.nn import functional as F

try:
    from flash_attn import flash_attn_qkvpacked_func as _packed
except Exception:  # pragma: no cover - optional dependency
    _packed = None

_state = {"flash": _packed is not None}


def packed_attention(qkv):
    """``qkv``: [batch, tokens, 3, heads, head_dim] -> [batch, tokens, heads * head_dim]."""
    batch, tokens, _, heads, head_dim = qkv.shape
    if (_state["flash"] and qkv.is_cuda and qkv.dtype in (torch.bfloat16, torch.float16) and head_dim % 8 == 0
            and head_dim <= 256):
        try:
            return _packed(qkv).reshape(batch, tokens, heads * head_dim)
        except RuntimeError:
            _state["flash"] = False          # e.g. a build without kernels for this GPU: use SDPA from now on
    q, k, v = qkv.permute(2, 0, 3, 1, 4).unbind(0)
    return F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(batch, tokens, heads * head_dim)
