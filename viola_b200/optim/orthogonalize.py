"""Quintic Newton-Schulz orthogonalisation on the tcgen05 GEMM kernel.

Two recurrences with the reference's coefficients and rounding points
(viola/optim/_orthogonalize.py:10-54; kernel epilogues viola/optim/_orthogonalize_kernels.py:16-50):

* ``standard`` (bf16): ``X <- 3.4445 X + (-4.775 G + 2.0315 G G) X`` with ``G = X X^T``;
* ``gram`` (fp16): the polynomial is composed on the small Gram matrix and applied to ``X`` once per
  segment (two iterations, then the rest), falling back to the standard recurrence for square inputs.

Every product is one launch of the warp-specialised tcgen05 kernel with the polynomial fused into
its epilogue (``alpha * round(acc) + beta * R``).  Gram-side products are symmetric, so only the
upper-triangular tiles are computed and mirrored.  The iterate is kept in its stored orientation and
never transposed: the tensor core reads it K-major or MN-major as the product needs (wide ``X``:
``G = X X^T`` K-major, ``P X`` with ``X`` as the MN-major B operand; tall ``X``: ``G = X^T X`` with
both operands MN-major, ``X P`` K-major since ``P`` is symmetric).
"""

from __future__ import annotations

import torch

from .. import ops

_A, _B, _C = 3.4445, -4.7750, 2.0315


def _prescale(matrix, dtype):
    """matrix / (||matrix||_F + 1e-7) rounded to ``dtype``, in the input's orientation."""
    rows, cols = matrix.shape[-2:]
    accum = torch.zeros(max(1, matrix.numel() // (rows * cols)), device=matrix.device, dtype=torch.float32)
    source = matrix.contiguous()
    ops.sumsq(source, dtype, accum)
    scaled = torch.empty(matrix.shape, device=matrix.device, dtype=dtype)
    ops.ns_prescale(source, accum, out=scaled)
    return scaled


def _mn_readable(x, k):
    """Can ``x`` ([.., k, mn]) be read in place as an MN-major operand?  Rows must be 16-byte aligned, and a
    stack needs whole K blocks per matrix (a partial block would read the next matrix's rows)."""
    return (x.shape[-1] * x.element_size()) % 16 == 0 and (x.ndim == 2 or k % 64 == 0)


def _gram_matrix(x, tall):
    """The small Gram matrix: X X^T for a wide iterate, X^T X for a tall one."""
    if not tall:
        return ops.ns_gemm(x, x, symmetric=True)
    if _mn_readable(x, x.shape[-2]):
        return ops.ns_gemm(x, x, symmetric=True, a_mn=True, b_mn=True)
    flipped = x.mT.contiguous()
    return ops.ns_gemm(flipped, flipped, symmetric=True)


def _apply(p, x, tall, *, beta=0.0, resid=None, out=None):
    """round(P X) (wide) or round(X P) (tall) for a symmetric P, plus ``beta * resid``."""
    if tall:
        return ops.ns_gemm(x, p, alpha=1.0, beta=beta, resid=resid, out=out)
    if _mn_readable(x, x.shape[-2]):
        return ops.ns_gemm(p, x, alpha=1.0, beta=beta, resid=resid, out=out, b_mn=True)
    return ops.ns_gemm(p, x.mT.contiguous(), alpha=1.0, beta=beta, resid=resid, out=out)


def _poly(r):
    """-4.775 R + 2.0315 R R for a symmetric R."""
    return ops.ns_gemm(r, r, alpha=_C, beta=_B, resid=r, symmetric=True)


def _standard_2d(matrix, steps, dtype, out=None):
    x = _prescale(matrix, dtype)
    tall = matrix.shape[-2] > matrix.shape[-1]
    for step in range(steps):
        poly = _poly(_gram_matrix(x, tall))
        x = _apply(poly, x, tall, beta=_A, resid=x, out=out if step == steps - 1 else None)
    return x


def _gram_2d(matrix, steps, out=None):
    dtype = torch.float16
    if matrix.shape[-2] == matrix.shape[-1]:
        return _standard_2d(matrix, steps, dtype, out)
    x = _prescale(matrix, dtype)
    tall = matrix.shape[-2] > matrix.shape[-1]
    segments = [length for length in (min(steps, 2), max(steps - 2, 0)) if length]
    for index, length in enumerate(segments):
        r = _gram_matrix(x, tall)
        q = None
        for i in range(length):
            z = _poly(r)
            if i == 0:
                q = z.clone()
                q.diagonal(dim1=-2, dim2=-1).add_(_A)
            else:
                q = ops.ns_gemm(z, q, alpha=1.0, beta=_A, resid=q, symmetric=True)
            if i + 1 < length:
                rz = ops.ns_gemm(z, r, alpha=1.0, beta=_A, resid=r, symmetric=True)
                r = ops.ns_gemm(z, rz, alpha=1.0, beta=_A, resid=rz, symmetric=True)
        x = _apply(q, x, tall, out=out if index == len(segments) - 1 else None)
    return x


def _batched(fn, matrix, *args):
    """2-D inputs run as is; stacks of matrices run as ONE batched launch per GEMM of the recurrence."""
    if matrix.ndim == 2:
        return fn(matrix, *args)
    flat = matrix.reshape(-1, *matrix.shape[-2:])
    return fn(flat, *args).reshape(matrix.shape)


def standard(matrix, steps=5, out=None):
    """bf16 Newton-Schulz; returns the orthogonalised matrix in bf16 with the input's shape.

    ``out`` (CUDA only): a bf16 tensor of the input's shape (at most one leading batch dimension) that
    receives the result, so callers can keep a stable address across steps."""
    if not matrix.is_cuda:
        return ops.reference.ns_standard(matrix, steps)
    if out is not None and matrix.ndim <= 3:
        return _standard_2d(matrix, steps, torch.bfloat16, out)
    return _batched(_standard_2d, matrix, steps, torch.bfloat16)


def gram(matrix, steps=5, out=None):
    """fp16 Gram-matrix Newton-Schulz; returns fp16 (``out``: optional fp16 result buffer, CUDA only)."""
    if not matrix.is_cuda:
        return ops.reference.ns_gram(matrix, steps)
    if out is not None and matrix.ndim <= 3:
        return _gram_2d(matrix, steps, out)
    return _batched(_gram_2d, matrix, steps)

OUTPUT_DTYPE = {"standard": torch.bfloat16, "gram": torch.float16}


def orthogonalize(matrix, *, method="standard", steps=5, autotune=True):
    """Entry point with the keyword surface of the reference's kernel-backed path
    (viola/optim/_orthogonalize_kernels.py:200-202).  ``autotune``: search the tile width of this shape's GEMMs on
    first use and remember it on disk (:mod:`viola_b200.tuning`), as the reference's per-shape planner does."""
    if autotune and matrix.is_cuda:
        from .. import tuning
        previous = tuning.enabled()
        tuning.enable()
        try:
            return METHODS[method](matrix, steps=steps)
        finally:
            tuning.enable(previous)
    return METHODS[method](matrix, steps=steps)


METHODS = {"standard": standard, "gram": gram}
