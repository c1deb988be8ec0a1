"""Operator layer: CUDA tensors run the hand-written sm_100a kernels in ``viola_b200/_C.so``
(``torch.ops.viola_b200.*``); CPU tensors run the PyTorch restatements in ``reference.py``.

There is no silent fallback on a GPU: if a CUDA tensor reaches an op and the extension cannot be
loaded, the call raises.  Function names and argument conventions mirror the reference's kernel
wrappers (viola/nn/_linear_kernels.py:231-291, viola/nn/_grouped_kernels.py:127-171,310-328,
viola/optim/_kernels.py:61-83,296-337, viola/distributed/_fp8_kernels.py:84-93) so the module layer
reads the same.
"""

from __future__ import annotations

import math
import os
import threading
from pathlib import Path

import torch

from . import reference
from .. import tuning
from .reference import packet_bytes, packet_views, scale_shape, state_sizes  # noqa: F401

_LIB_PATH = Path(__file__).resolve().parent.parent / "_C.so"
_lock = threading.Lock()
_loaded = False
_load_error = None

FP8_DTYPES = (torch.float8_e4m3fn, torch.float8_e5m2)
_FMT = {torch.float8_e4m3fn: 0, torch.float8_e5m2: 1}
_ACT = {"silu": 0, "gelu": 1, "relu": 2}
EPI_LINEAR, EPI_AXPBY, EPI_GATED_FWD, EPI_GATED_BWD, EPI_ACT_BWD = 0, 1, 2, 3, 4
_NO_GROUP = (0, 0, 0, 0, 0, 0, 0)

launch_count = 0  # number of library kernels launched through this layer (bench bookkeeping)


def load(build_if_missing: bool = True):
    """Load ``_C.so`` (building it in-tree when absent).  Raises if that is impossible."""
    global _loaded, _load_error
    if _loaded:
        return True
    with _lock:
        if _loaded:
            return True
        try:
            if not _LIB_PATH.exists() and build_if_missing:
                from ..build import build
                build()
            torch.ops.load_library(str(_LIB_PATH))
            _loaded = True
        except Exception as error:  # pragma: no cover - exercised only on broken installs
            _load_error = error
            raise RuntimeError(f"viola_b200: cannot load the sm_100a kernel library {_LIB_PATH}: {error}") from error
    return True


def _ops():
    load()
    return torch.ops.viola_b200


def _count(n=1):
    global launch_count
    launch_count += n


# ------------------------------------------------------------------------------ workspaces
_scratch = {}
_status = {}


def _amax_scratch(device):
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buffer = _scratch.get(key)
    if buffer is None:
        buffer = _scratch[key] = torch.zeros(2, device=device, dtype=torch.int32)
    return buffer


_amax_words = {}


def amax_word(device):
    """Per-(device, stream) uint32[1] that producer epilogues gather an amax into (float bits); the consumer
    (:func:`scale_from_amax`) re-zeroes it, so one word serves every producer / consumer pair on a stream."""
    key = (torch.device(device), torch.cuda.current_stream(device).cuda_stream if torch.device(device).type == "cuda" else 0)
    word = _amax_words.get(key)
    if word is None:
        word = _amax_words[key] = torch.zeros(1, device=device, dtype=torch.int32)
    return word


_colsum_space = {}


def _colsum_workspace(device, rows, cols):
    """Per-(device, stream) fp32 scratch of the reproducible column-sum reduction (tickets + per-panel sums)."""
    strips = (cols + 127) // 128
    need = 1024 + ((rows + 255) // 256) * strips * 128
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buffer = _colsum_space.get(key)
    if buffer is None or buffer.numel() < need:
        buffer = _colsum_space[key] = torch.zeros(max(need, 1 << 20), device=device, dtype=torch.float32)
    return buffer


_sum_space = {}


def _sample_sum_workspace(device, rows, tokens, width):
    """(workspace, tickets) of the reproducible per-sample column sums, per (device, stream)."""
    need = _ops().row_block_count(int(rows), int(tokens)) * width
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    entry = _sum_space.get(key)
    if entry is None or entry[0].numel() < need or entry[1].numel() < rows // tokens:
        entry = _sum_space[key] = (torch.empty(max(need, 1 << 22), device=device, dtype=torch.float32),
                                   torch.zeros(max(rows // tokens, 4096), device=device, dtype=torch.int32))
    return entry


def status_word(device):
    """Per-device int32[8] error word written by bounded waits inside the kernels."""
    device = torch.device(device)
    word = _status.get(device)
    if word is None:
        word = _status[device] = torch.zeros(8, device=device, dtype=torch.int32)
    return word


_STATUS_NAMES = {1: "wait for TMA data timed out", 2: "wait for a free smem stage timed out",
                 3: "wait for the MMA commit timed out", 4: "wait for TMEM drain timed out",
                 5: "wait on a peer flag timed out", 6: "wait on a gathered panel timed out", 7: "bad argument"}


def check_status(device=None):
    """Synchronising check of the kernel status words; raises with the recorded location."""
    for dev, word in list(_status.items()):
        if device is not None and torch.device(device) != dev:
            continue
        values = word.tolist()
        if values[0]:
            word.zero_()
            raise RuntimeError(f"viola_b200 kernel reported: {_STATUS_NAMES.get(values[0], values[0])} "
                               f"(block {values[1]}, warp {values[2]}, detail {values[3]}) on {dev}")


def status_message(values, device="?"):
    """Text for a non-zero status word ``[code, block, warp, detail, ...]``."""
    return (f"viola_b200 kernel reported: {_STATUS_NAMES.get(int(values[0]), int(values[0]))} "
            f"(block {int(values[1])}, warp {int(values[2])}, detail {int(values[3])}) on {device}")


class StatusMonitor:
    """Reads a device's kernel status word without stalling the training loop.

    ``snapshot()`` enqueues a copy of the word into pinned host memory behind the work issued so far;
    ``poll()`` looks at the latest snapshot that has completed (it never waits) and raises when a kernel
    recorded a failure.  A loop that calls ``poll()`` then ``snapshot()`` once per step therefore learns of
    a timed-out wait one step late but pays no synchronisation; ``check()`` is the synchronising form for
    places that write something durable (checkpoints) or shut down.  ``pending`` lets a test or a host-side
    fault model put a code in without any GPU work.
    """

    def __init__(self, device):
        self.device = torch.device(device)
        self.pending = 0                  # host-injected code, reported by the next poll()/check()
        self._host = self._event = None
        if self.device.type == "cuda":
            self._host = torch.zeros(8, dtype=torch.int32).pin_memory()
            self._event = torch.cuda.Event()
            self._armed = False

    def local_code(self):
        """The code this rank would report right now without waiting for the GPU."""
        if self.pending:
            return int(self.pending)
        if self._host is not None and self._armed and self._event.query():
            return int(self._host[0])
        return 0

    def snapshot(self):
        if self._host is None:
            return
        self._host.copy_(status_word(self.device), non_blocking=True)
        self._event.record(torch.cuda.current_stream(self.device))
        self._armed = True

    def poll(self):
        code = self.local_code()
        if code:
            self.raise_for(code)

    def check(self):
        if self.pending:
            self.raise_for(self.pending)
        if self._host is not None:
            check_status(self.device)

    def raise_for(self, code, rank=None):
        values = [code, 0, 0, 0]
        if self._host is not None and int(self._host[0]) == code:
            values = self._host.tolist()
        self.pending = 0
        where = f"{self.device}" if rank is None else f"rank {rank}"
        raise RuntimeError(status_message(values, where))


def _limit(dtype, limit):
    return reference.fp8_limit(dtype, limit)


# ------------------------------------------------------------------------------ per-tensor scaling
def tensor_scale(x, *, history=None, index=0, delayed=False, fp8_dtype=torch.float8_e4m3fn, quantization_limit=None,
                 out=None):
    """scale = max(amax, 1e-30) / limit as an fp32[1] tensor (written into ``out`` when given)."""
    if not x.is_cuda:
        result = reference.tensor_scale(x, history=history, index=index, delayed=delayed, fp8_dtype=fp8_dtype,
                                        quantization_limit=quantization_limit)
        return result if out is None else out.copy_(result)
    scale = out if out is not None else torch.empty(1, device=x.device, dtype=torch.float32)
    _ops().amax_scale(x.detach().contiguous().view(-1), history, int(index), bool(delayed),
                      _limit(fp8_dtype, quantization_limit), scale, _amax_scratch(x.device))
    _count()
    return scale


def quantize(x, scale, *, rowwise=True, transpose=False, fp8_dtype=torch.float8_e4m3fn, out=None, out_t=None,
             quantization_limit=None, colsum=None):
    """FP8 codes of ``x / scale`` row-wise and / or transposed.  ``colsum`` (fp32 [cols], zero-initialised by the
    caller) additionally receives the column sums of ``x``: on CUDA they come out of the same read when only
    row-wise codes are asked for (the bias gradient of a linear layer's output gradient)."""
    if not x.is_cuda:
        if colsum is not None:
            colsum.add_(x.detach().float().sum(dim=0))
        return reference.quantize(x, scale, rowwise=rowwise, transpose=transpose, fp8_dtype=fp8_dtype, out=out,
                                  out_t=out_t, quantization_limit=quantization_limit)
    x = x.detach().contiguous()
    if colsum is not None and (transpose or out_t is not None or x.shape[1] % 16 or x.data_ptr() % 16):
        colsum.add_(x.float().sum(dim=0))
        colsum = None
    empty = None
    q = out if out is not None else (torch.empty(x.shape, device=x.device, dtype=fp8_dtype) if rowwise else None)
    qt = out_t if out_t is not None else (
        torch.empty(x.shape[::-1], device=x.device, dtype=fp8_dtype) if transpose else None)
    if q is not None or qt is not None:
        workspace = _colsum_workspace(x.device, *x.shape) if colsum is not None else None
        _ops().quantize(x, scale, _limit(fp8_dtype, quantization_limit), q, qt, _FMT[fp8_dtype], colsum, workspace)
        _count()
    if q is None or qt is None:
        empty = torch.empty((0, 0), device=x.device, dtype=fp8_dtype)
    return (q if q is not None else empty), (qt if qt is not None else empty)


def transpose(q, out=None):
    if not q.is_cuda:
        return reference.transpose(q, out)
    if out is None:
        out = torch.empty(q.shape[::-1], device=q.device, dtype=q.dtype)
    _ops().transpose_u8(q.contiguous(), out)
    _count()
    return out


def _pad_k(t, multiple):
    k = t.shape[1]
    if k % multiple == 0 and t.stride(1) == 1 and (t.stride(0) * t.element_size()) % 16 == 0 \
            and t.data_ptr() % 16 == 0:
        return t
    padded = torch.zeros((t.shape[0], (k + multiple - 1) // multiple * multiple), device=t.device, dtype=torch.uint8
                         if t.element_size() == 1 else t.dtype)
    if t.element_size() == 1:
        padded[:, :k] = t.view(torch.uint8)
        return padded.view(t.dtype)
    padded[:, :k] = t
    return padded


def _check_mn(t):
    # an MN-major operand ([K, MN], MN contiguous) is read in place: TMA needs 16-byte aligned rows
    if t.stride(1) != 1 or (t.stride(0) * t.element_size()) % 16 or t.data_ptr() % 16:
        raise ValueError("an MN-major GEMM operand needs unit column stride and 16-byte aligned rows")
    return t


def _gemm(a, b, out, epilogue, n_logical, *, sa=None, sb=None, layout=_NO_GROUP, bias=None, alpha=1.0, beta=0.0,
          resid=None, out_t=None, symmetric=False, activation=0, aux=None, expert_offsets=None, tile_map=None,
          force_bn=0, batch=1, a_mn=False, b_mn=False, amax_out=None, force_split=0, accumulate=False):
    multiple = 16 if a.element_size() == 1 else 8
    a = _check_mn(a) if a_mn else _pad_k(a, multiple)
    b = _check_mn(b) if b_mn else _pad_k(b, multiple)
    status = status_word(a.device)

    def launch(tile):
        _ops().gemm(a, b, out, epilogue, n_logical, sa, sb, list(layout), bias, float(alpha), float(beta), resid, out_t,
                    bool(symmetric), int(activation), aux, expert_offsets, tile_map, status,
                    int(tile) | (int(force_split) << 16), int(batch),
                    bool(a_mn), bool(b_mn), amax_out, bool(accumulate))

    if not force_bn and not accumulate and (tuning._enabled or tuning._choices):
        # the output-tile width of this shape: recorded choice, or (tuning on) measured now on these operands
        in_place = resid is not None and resid.data_ptr() == out.data_ptr()
        tunable = (epilogue in (EPI_LINEAR, EPI_AXPBY, EPI_ACT_BWD) and not layout[0] and not symmetric
                   and expert_offsets is None and not in_place and n_logical > 128)
        signature = (int(epilogue), tuple(a.shape), tuple(b.shape), str(a.dtype), str(b.dtype), str(out.dtype), bool(a_mn),
                     bool(b_mn), int(batch), bias is not None, int(activation), out_t is not None)
        pairs = epilogue == EPI_LINEAR and batch == 1 and out.shape[0] >= 256 and n_logical >= 256
        force_bn = tuning.choose(signature, launch, lambda: out, tunable=tunable,
                                 candidates=(128, 256, 512) if pairs else (128, 256))
    launch(force_bn)
    _count(2 if expert_offsets is not None else 1)
    return out


def gemm(a, b, sa, sb, *, out_dtype, bias=None, out=None, force_bn=0, a_mn=False, b_mn=False, force_split=0,
         accumulate=False):
    """(a * sa) @ (b * sb).T (+ bias): FP8 or 16-bit operands with per-tensor fp32 scales.

    ``a_mn`` / ``b_mn``: the tensor passed holds the operand transposed (``a`` is [K, M] / ``b`` is [K, N]);
    the tensor core reads it MN-major in place, so no transposed copy is needed.
    ``force_split``: work units per output tile along K for fp32 results (0 = chosen from the wave count, 1 = none).
    ``accumulate``: ``out += product`` (``out`` required); fp32 outputs with 16-byte rows add inside the GEMM's
    epilogue (TMA reduce), everything else computes the product and adds it.
    """
    if not a.is_cuda:
        result = reference.gemm(a.t() if a_mn else a, b.t() if b_mn else b, sa, sb, out_dtype=out_dtype, bias=bias)
        if accumulate:
            return out.add_(result)
        return result if out is None else out.copy_(result)
    m = a.shape[1] if a_mn else a.shape[0]
    n = b.shape[1] if b_mn else b.shape[0]
    if accumulate and not (out.dtype == torch.float32 and bias is None and out.data_ptr() % 16 == 0
                           and out.stride(-2) % 4 == 0 and out.stride(-1) == 1):
        product = torch.empty((m, n), device=a.device, dtype=out_dtype)
        _gemm(a, b, product, EPI_LINEAR, n, sa=sa, sb=sb, bias=bias, force_bn=force_bn, a_mn=a_mn, b_mn=b_mn,
              force_split=force_split)
        return out.add_(product)
    if out is None:
        out = torch.empty((m, n), device=a.device, dtype=out_dtype)
    return _gemm(a, b, out, EPI_LINEAR, n, sa=sa, sb=sb, bias=bias, force_bn=force_bn, a_mn=a_mn, b_mn=b_mn,
                 force_split=force_split, accumulate=accumulate)


# ------------------------------------------------------------------------------ group scaling
def _log2(v):
    assert v > 0 and v & (v - 1) == 0, f"{v} is not a power of two"
    return v.bit_length() - 1


def group_quantize(x, dtype, group, *, limit=None, transposed=False, out=None, scale_out=None, kmajor=False,
                   pow2=False):
    """Encode ``x`` (or ``x.T`` when ``transposed``) with one fp32 scale per ``group`` block.

    Scales come back as ``[ceil(R/gr), ceil(C/gc)]`` or, with ``kmajor``, as its transpose
    (one contiguous row of scales per K-block: the layout the GEMM promotion loop reads).
    """
    if not x.is_cuda:
        q, s = reference.group_quantize(x, dtype, group, limit=limit, transposed=transposed, out=out, pow2=pow2)
        if kmajor:
            s = s.t().contiguous()
        if scale_out is not None:
            s = scale_out.copy_(s)
        return q, s
    x = x.detach().contiguous()
    shape = tuple(x.shape[::-1]) if transposed else tuple(x.shape)
    nr, nc = scale_shape(shape, group)
    q = out if out is not None else torch.empty(shape, device=x.device, dtype=dtype)
    s = scale_out if scale_out is not None else torch.empty((nc, nr) if kmajor else (nr, nc), device=x.device,
                                                            dtype=torch.float32)
    s_row, s_col = (1, nr) if kmajor else (nc, 1)
    gr, gc = group
    if transposed:
        _ops().group_encode(x, _FMT[dtype], _limit(dtype, limit), None, None, 1, 32, 0, 0, q, s, gr, gc, s_row, s_col,
                            bool(pow2))
    else:
        _ops().group_encode(x, _FMT[dtype], _limit(dtype, limit), q, s, gr, gc, s_row, s_col, None, None, 1, 32, 0, 0,
                            bool(pow2))
    _count()
    return q, s


def group_quantize_pair(x, dtype, group, group_t, *, limit=None, kmajor=False, pow2=False):
    """Rowwise and transposed encodings from one read of ``x``: returns (q, s, qt, st)."""
    if not x.is_cuda or max(*group, *group_t) > 128:
        q, s = group_quantize(x, dtype, group, limit=limit, kmajor=kmajor, pow2=pow2)
        qt, st = group_quantize(x, dtype, group_t, limit=limit, transposed=True, kmajor=kmajor, pow2=pow2)
        return q, s, qt, st
    x = x.detach().contiguous()
    rows, cols = x.shape
    nr, nc = scale_shape((rows, cols), group)
    tnr, tnc = scale_shape((cols, rows), group_t)
    q = torch.empty((rows, cols), device=x.device, dtype=dtype)
    qt = torch.empty((cols, rows), device=x.device, dtype=dtype)
    s = torch.empty((nc, nr) if kmajor else (nr, nc), device=x.device, dtype=torch.float32)
    st = torch.empty((tnc, tnr) if kmajor else (tnr, tnc), device=x.device, dtype=torch.float32)
    s_row, s_col = (1, nr) if kmajor else (nc, 1)
    st_row, st_col = (1, tnr) if kmajor else (tnc, 1)
    # the 1x128 fast path only exists for the single-output call; the pair always uses the tile kernel
    _ops().group_encode(x, _FMT[dtype], _limit(dtype, limit), q, s, group[0], group[1], s_row, s_col, qt, st,
                        group_t[0], group_t[1], st_row, st_col, bool(pow2))
    _count()
    return q, s, qt, st


def group_dequantize(q, scale, group, *, kmajor=False):
    if not q.is_cuda:
        return reference.group_dequantize(q, scale.t() if kmajor else scale, group)
    out = torch.empty(q.shape, device=q.device, dtype=torch.float32)
    nr, nc = scale_shape(tuple(q.shape), group)
    s_row, s_col = (1, nr) if kmajor else (nc, 1)
    _ops().group_decode(q.contiguous(), scale.contiguous(), group[0], group[1], s_row, s_col, out)
    _count()
    return out


def _group_layout(a, b_rows, k, ga, gb, sa_kmajor, sb_kmajor):
    """scale_layout for the kernel, or None when the group shapes need the dequantise fallback."""
    if ga[0] != 1 or ga[1] != gb[1] or ga[1] < 128:
        return None
    gk = ga[1]
    nk = (k + gk - 1) // gk
    m = a.shape[0]
    nb = (b_rows + gb[0] - 1) // gb[0]
    sa_row, sa_k = (1, m) if sa_kmajor else (nk, 1)
    sb_row, sb_k = (1, nb) if sb_kmajor else (nk, 1)
    return (1, sa_row, sa_k, sb_row, sb_k, _log2(gb[0]), _log2(gk // 128))


def mx_pack_scales(scales, rows, k, *, group_rows=1, kmajor=False):
    """UE8M0 scale bytes of an MXFP8 operand [rows, k] in the tiled layout the block-scaled tensor-core GEMM reads.

    ``scales``: fp32 powers of two or uint8 exponents, one per (``group_rows`` rows, 32 K elements), stored
    [rows / group_rows, k / 32] or, with ``kmajor``, [k / 32, rows / group_rows]."""
    scales = scales.contiguous()
    row_groups, k_groups = (rows + group_rows - 1) // group_rows, (k + 31) // 32
    row_stride, group_stride = (1, row_groups) if kmajor else (k_groups, 1)
    return _ops().mx_pack_scales(scales, row_stride, group_stride, int(rows), int(k), _log2(group_rows))


def mx_gemm(a, b, sfa, sfb, *, out_dtype, bias=None, out=None):
    """MXFP8 GEMM on the hardware block-scaled path: ``sfa`` / ``sfb`` come from :func:`mx_pack_scales`."""
    if out is None:
        out = torch.empty((a.shape[0], b.shape[0]), device=a.device, dtype=out_dtype)
    _ops().mx_gemm(a.view(torch.uint8) if a.dtype != torch.uint8 else a, _FMT.get(a.dtype, 0),
                   b.view(torch.uint8) if b.dtype != torch.uint8 else b, _FMT.get(b.dtype, 0), sfa, sfb, out, bias,
                   status_word(a.device))
    _count()
    return out


def attention_eligible(qkv):
    """Can :func:`attention_forward` take this packed projection ([B, 256, 3, H, D], 16-bit, D % 8 == 0, D <= 128)?"""
    return (qkv.is_cuda and qkv.dim() == 5 and qkv.shape[1] == 256 and qkv.shape[2] == 3
            and qkv.dtype in (torch.bfloat16, torch.float16) and qkv.shape[4] % 8 == 0 and 16 <= qkv.shape[4] <= 128
            and qkv.is_contiguous())


def attention_forward(qkv, scale=None):
    """softmax(Q K^T * scale) V for a packed ``qkv`` [B, 256, 3, H, D]: returns (out [B, 256, H, D], lse [B, H, 256] fp32).

    One tcgen05 kernel, one CTA per (sample, head): both 128 x 256 score tiles stay in tensor memory, the
    probabilities go back to the tensor core through shared memory.  ``lse`` = log(sum(exp(score * scale)))."""
    scale = qkv.shape[-1] ** -0.5 if scale is None else float(scale)
    if not qkv.is_cuda:
        return reference.attention_forward(qkv, scale)
    batch, tokens, _, heads, head_dim = qkv.shape
    out = torch.empty((batch, tokens, heads, head_dim), device=qkv.device, dtype=qkv.dtype)
    lse = torch.empty((batch, heads, tokens), device=qkv.device, dtype=torch.float32)
    _ops().attention_forward(qkv, out, lse, scale, status_word(qkv.device))
    _count()
    return out, lse


def _mx_eligible(a, b, ga, gb):
    return (tuple(ga) == (1, 32) and gb[1] == 32 and gb[0] & (gb[0] - 1) == 0 and a.shape[1] % 16 == 0
            and a.dtype in FP8_DTYPES and b.dtype in FP8_DTYPES and a.is_contiguous() and b.is_contiguous())


def group_gemm(a, b, sa, sb, ga, gb, *, out_dtype, bias=None, sa_kmajor=False, sb_kmajor=False, out=None, mx=False):
    """Group-scaled FP8 GEMM: sum over K-groups of (A_g . B_g^T) * sa[row, g] * sb[col-block, g].

    ``mx=True`` states that every scale is a power of two with groups of 32 along K (the MXFP8 recipe); the
    product then runs on the hardware block-scaled tensor-core path (``tcgen05.mma.kind::mxf8f6f4.block_scale``)."""
    if not a.is_cuda:
        result = reference.group_gemm(a, b, sa.t() if sa_kmajor else sa, sb.t() if sb_kmajor else sb, ga, gb,
                                      out_dtype=out_dtype, bias=bias)
        return result if out is None else out.copy_(result)
    if out is None:
        out = torch.empty((a.shape[0], b.shape[0]), device=a.device, dtype=out_dtype)
    if mx and _mx_eligible(a, b, ga, gb) and out.dtype in _DT and out.stride(-1) == 1:
        rows_a, rows_b, k = a.shape[0], b.shape[0], a.shape[1]
        sfa = mx_pack_scales(sa, rows_a, k, kmajor=sa_kmajor)
        sfb = mx_pack_scales(sb, rows_b, k, group_rows=gb[0], kmajor=sb_kmajor)
        _count(2)
        return mx_gemm(a, b, sfa, sfb, out_dtype=out.dtype, bias=bias, out=out)
    layout = _group_layout(a, b.shape[0], a.shape[1], ga, gb, sa_kmajor, sb_kmajor)
    if layout is None:
        # Group shapes the tcgen05 promotion loop does not cover (K-groups below 128 or multi-row
        # activation groups): decode to bf16 and run the 16-bit tensor-core GEMM.
        da = group_dequantize(a, sa, ga, kmajor=sa_kmajor).to(torch.bfloat16)
        db = group_dequantize(b, sb, gb, kmajor=sb_kmajor).to(torch.bfloat16)
        return _gemm(da, db, out, EPI_LINEAR, b.shape[0], bias=bias)
    return _gemm(a, b, out, EPI_LINEAR, b.shape[0], sa=sa, sb=sb, layout=layout, bias=bias)


# ------------------------------------------------------------------------------ fused gated MLP GEMMs
def gated_gemm_forward(a, w, sa, sw, *, activation, out_dtype, bias=None, save=True, group=None, sa_kmajor=False,
                       sw_kmajor=False):
    """h = act(A.Wg^T) * (A.Wu^T) with W = [Wg; Wu] ([2H, K]); returns (h, aux=[g|u] or None)."""
    hidden = w.shape[0] // 2
    if not a.is_cuda:
        if group is None:
            z = reference.gemm(a, w, sa, sw, out_dtype=out_dtype, bias=bias)
        else:
            z = reference.group_gemm(a, w, sa.t() if sa_kmajor else sa, sw.t() if sw_kmajor else sw, group[0],
                                     group[1], out_dtype=out_dtype, bias=bias)
        return reference.gated_forward(z, activation), (z if save else None)
    h = torch.empty((a.shape[0], hidden), device=a.device, dtype=out_dtype)
    aux = torch.empty((a.shape[0], 2 * hidden), device=a.device, dtype=out_dtype) if save else None
    layout = _NO_GROUP
    if group is not None:
        layout = _group_layout(a, w.shape[0], a.shape[1], group[0], group[1], sa_kmajor, sw_kmajor)
        if layout is None or (layout[5] > 0 and hidden % (1 << layout[5])):
            z = group_gemm(a, w, sa, sw, group[0], group[1], out_dtype=out_dtype, bias=bias, sa_kmajor=sa_kmajor,
                           sb_kmajor=sw_kmajor)
            return gated_forward(z, activation), (z if save else None)
    _gemm(a, w, h, EPI_GATED_FWD, hidden, sa=sa, sb=sw, layout=layout, bias=bias, activation=_ACT[activation], aux=aux)
    return h, aux


def gated_gemm_backward(dy, wt, sg, st, aux, *, activation, out_dtype, group=None, sg_kmajor=False, st_kmajor=False,
                        wt_mn=False):
    """[dG | dU] from d = dY.Wdown (wt = Wdown^T, [H, out]) and the saved aux = [g | u].

    ``wt_mn`` (per-tensor scaling only): ``wt`` is Wdown itself ([out, H]), read MN-major in place."""
    hidden = wt.shape[1] if wt_mn else wt.shape[0]
    if not dy.is_cuda:
        if group is None:
            d = reference.gemm(dy, wt.t() if wt_mn else wt, sg, st, out_dtype=out_dtype)
        else:
            d = reference.group_gemm(dy, wt, sg.t() if sg_kmajor else sg, st.t() if st_kmajor else st, group[0],
                                     group[1], out_dtype=out_dtype)
        return reference.gated_backward(aux, d, activation)
    out = torch.empty((dy.shape[0], 2 * hidden), device=dy.device, dtype=out_dtype)
    layout = _NO_GROUP
    if group is not None:
        layout = _group_layout(dy, hidden, dy.shape[1], group[0], group[1], sg_kmajor, st_kmajor)
        if layout is None:
            d = group_gemm(dy, wt, sg, st, group[0], group[1], out_dtype=out_dtype, sa_kmajor=sg_kmajor,
                           sb_kmajor=st_kmajor)
            return gated_backward(aux, d, activation)
    _gemm(dy, wt, out, EPI_GATED_BWD, hidden, sa=sg, sb=st, layout=layout, activation=_ACT[activation], aux=aux,
          b_mn=wt_mn)
    return out


def activation_backward_gemm(dy, w, sg, sw, slope, *, w_mn=False, amax_out=None):
    """``dz = round(dy @ W) * slope`` in ``slope``'s dtype: the input gradient of ``act(z) @ W^T`` through the
    activation, from the dgrad GEMM's epilogue (per-tensor scales); ``slope`` = ``act'(z)`` saved by the forward
    (:func:`activation_quantize`).  ``w`` is W^T ([in, out], K-major) or, with ``w_mn``, W itself ([out, in]).
    ``amax_out`` (int32 [1], zero-initialised) gathers ``max |dz|`` as float bits; :func:`scale_from_amax` turns
    it into an FP8 scale without another pass over ``dz``."""
    if not dy.is_cuda:
        d = reference.gemm(dy, w.t() if w_mn else w, sg, sw, out_dtype=slope.dtype).float()
        dz = (d * slope.float()).to(slope.dtype)
        if amax_out is not None:
            amax_out.copy_(torch.maximum(amax_out.view(torch.float32), dz.float().abs().max().reshape(1)).view(amax_out.dtype))
        return dz
    n = w.shape[1] if w_mn else w.shape[0]
    out = torch.empty((dy.shape[0], n), device=dy.device, dtype=slope.dtype)
    return _gemm(dy, w, out, EPI_ACT_BWD, n, sa=sg, sb=sw, aux=slope, b_mn=w_mn, amax_out=amax_out)


def scale_from_amax(amax_bits, *, history=None, index=0, delayed=False, fp8_dtype=torch.float8_e4m3fn,
                    quantization_limit=None, out=None):
    """FP8 scale from an amax gathered as float bits by a producer kernel; the gather word is re-zeroed."""
    limit = _limit(fp8_dtype, quantization_limit)
    if not amax_bits.is_cuda:
        amax = amax_bits.view(torch.float32).clone()
        amax_bits.zero_()
        chosen = amax
        if history is not None:
            if delayed and index != 0:
                chosen = history.max().reshape(1)
            history[index % history.numel()] = amax[0]
        result = torch.clamp(chosen, min=1e-30) / limit
        return result if out is None else out.copy_(result)
    scale = out if out is not None else torch.empty(1, device=amax_bits.device, dtype=torch.float32)
    _ops().scale_from_amax(amax_bits, history, int(index), bool(delayed), limit, scale)
    _count()
    return scale


def gated_forward(gu, activation):
    if not gu.is_cuda:
        return reference.gated_forward(gu, activation)
    gu = gu.contiguous()
    out = torch.empty((*gu.shape[:-1], gu.shape[-1] // 2), device=gu.device, dtype=gu.dtype)
    _ops().gated_forward(gu.view(-1, gu.shape[-1]), _ACT[activation], out)
    _count()
    return out


def gated_backward(gu, dh, activation):
    if not gu.is_cuda:
        return reference.gated_backward(gu, dh, activation)
    gu, dh = gu.contiguous(), dh.contiguous()
    out = torch.empty_like(gu)
    _ops().gated_backward(gu.view(-1, gu.shape[-1]), dh.view(-1, dh.shape[-1]), _ACT[activation], out)
    _count()
    return out


# ------------------------------------------------------------------------------ expert (ragged-M) GEMM
def expert_gemm(a, w, offsets, sa, sw, *, out_dtype, group=None, sa_kmajor=False, sw_kmajor=False, out=None):
    """out[rows of expert e] = A[rows of e] . W[e]^T.  ``w`` is [E, N, K]; ``offsets`` int32 [E+1] on device."""
    experts, n, k = w.shape
    if not a.is_cuda:
        result = torch.empty((a.shape[0], n), dtype=out_dtype)
        bounds = offsets.tolist()
        for e in range(experts):
            lo, hi = bounds[e], bounds[e + 1]
            if group is None:
                result[lo:hi] = reference.gemm(a[lo:hi], w[e], sa, sw[e] if sw is not None and sw.numel() > 1 else sw,
                                               out_dtype=out_dtype)
            else:
                sa_e = (sa.t() if sa_kmajor else sa)[lo:hi]
                sw_all = sw.t() if sw_kmajor else sw                  # [E * N / block, K / block]
                sw_e = sw_all.reshape(experts, -1, sw_all.shape[-1])[e]
                result[lo:hi] = reference.group_gemm(a[lo:hi], w[e], sa_e, sw_e, group[0], group[1],
                                                     out_dtype=out_dtype)
        return result if out is None else out.copy_(result)
    if out is None:
        out = torch.empty((a.shape[0], n), device=a.device, dtype=out_dtype)
    tile_map = torch.empty(3 * ((a.shape[0] + 127) // 128 + experts), device=a.device, dtype=torch.int32)
    w2 = w.reshape(experts * n, k)
    layout = _NO_GROUP
    if group is not None:
        layout = _group_layout(a, experts * n, k, group[0], group[1], sa_kmajor, sw_kmajor)
        assert layout is not None and n % group[1][0] == 0, "expert GEMM needs 1xK activation groups and N % block == 0"
        sw = sw.reshape(-1, sw.shape[-1]) if not sw_kmajor else sw
    return _gemm(a, w2, out, EPI_LINEAR, n, sa=sa, sb=sw, layout=layout, expert_offsets=offsets, tile_map=tile_map)


# ------------------------------------------------------------------------------ Newton-Schulz GEMM
def ns_gemm(a, b, *, out=None, alpha=1.0, beta=0.0, resid=None, out_t=None, symmetric=False, force_bn=0,
            a_mn=False, b_mn=False):
    """out = alpha * round(a @ b^T) + beta * resid in the operands' 16-bit dtype.

    ``a`` [.., m, k] and ``b`` [.., n, k] may carry one leading batch dimension (contiguous stacks):
    the whole stack is one persistent-kernel launch.  With ``a_mn`` / ``b_mn`` the tensor holds the operand
    transposed ([.., k, m] / [.., k, n]) and is read MN-major in place.
    """
    if not a.is_cuda:
        acc = ((a.mT if a_mn else a).float() @ (b if b_mn else b.mT).float()).to(a.dtype).float()
        result = (alpha * acc + (beta * resid.float() if resid is not None else 0.0)).to(a.dtype)
        if out_t is not None:
            out_t.copy_(result.mT)
        return result if out is None else out.copy_(result)
    batch = a.shape[0] if a.ndim == 3 else 1
    m, n = a.shape[-1 if a_mn else -2], b.shape[-1 if b_mn else -2]
    if out is None:
        out = torch.empty((*a.shape[:-2], m, n), device=a.device, dtype=a.dtype)
    a2 = a.reshape(batch * a.shape[-2], a.shape[-1]) if a.ndim == 3 else a
    b2 = b.reshape(batch * b.shape[-2], b.shape[-1]) if b.ndim == 3 else b
    _gemm(a2, b2, out, EPI_AXPBY, n, alpha=alpha, beta=beta, resid=resid, out_t=out_t, symmetric=symmetric,
          force_bn=force_bn, batch=batch, a_mn=a_mn, b_mn=b_mn)
    return out


def sumsq(x, round_dtype, accum):
    """accum[b] += sum of squares of x[b] (rounded to ``round_dtype`` first); accum has one entry per matrix."""
    code = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}[round_dtype]
    _ops().sumsq(x.contiguous(), code, accum)
    _count()


def ns_prescale(x, sumsq_t, *, out=None, out_t=None, eps=1e-7):
    _ops().ns_prescale(x.contiguous(), sumsq_t, eps, out, out_t)
    _count()


# ------------------------------------------------------------------------------ optimizer kernels
def momentum_dequantize(q, scales, shape, **quant):
    return reference.momentum_dequantize(q, scales, shape, **quant)


def momentum_update(grad, q, scales, next_q, next_scales, out, *, beta, tile_size=256, nesterov=True, loss_scale=1.0,
                    granularity="tile", block_shape=(16, 16), matrix_shape=None, rounding="nearest", rounding_step=0,
                    rounding_key=0):
    if not grad.is_cuda:
        return reference.momentum_update(grad, q, scales, next_q, next_scales, out, beta=beta, tile_size=tile_size,
                                         nesterov=nesterov, loss_scale=loss_scale, granularity=granularity,
                                         block_shape=block_shape, matrix_shape=matrix_shape, rounding=rounding,
                                         rounding_step=rounding_step, rounding_key=rounding_key)
    flat = grad.detach().reshape(-1)
    if not flat.is_contiguous():
        flat = flat.contiguous()
    key = int(rounding_key) & ((1 << 63) - 1)
    if granularity == "tile":
        _ops().momentum_1d(flat, q, scales, next_q, next_scales, out, int(tile_size), float(beta),
                           1.0 / float(loss_scale), bool(nesterov), rounding == "stochastic", int(rounding_step), key)
    else:
        rows, cols = matrix_shape[-2:]
        _ops().momentum_2d(flat, math.prod(matrix_shape[:-2]), rows, cols, q, scales, next_q, next_scales, out,
                           int(block_shape[0]), int(block_shape[1]), float(beta), 1.0 / float(loss_scale),
                           bool(nesterov), rounding == "stochastic", int(rounding_step), key)
    _count()


def weight_update(weight, update, lr, weight_decay, *, update_scale=1.0, rounding="nearest", step=0, key=0, offset=0):
    if not weight.is_cuda:
        return reference.weight_update(weight, update, lr, weight_decay, update_scale=update_scale, rounding=rounding,
                                       step=step, key=key, offset=offset)
    _ops().weight_update(weight.detach().view(-1), update.detach().reshape(-1).contiguous(), float(lr),
                         float(weight_decay), float(update_scale), rounding == "stochastic", int(step),
                         int(key) & ((1 << 63) - 1), int(offset))
    _count()


def adam_update(weight, grad, first, second, *, lr, weight_decay, betas, eps, step, rounding="nearest", key=0,
                offset=0, adamw=True, maximize=False, bias_correction=True):
    if not weight.is_cuda:
        return reference.adam_update(weight, grad, first, second, lr=lr, weight_decay=weight_decay, betas=betas,
                                     eps=eps, step=step, rounding=rounding, key=key, offset=offset, adamw=adamw,
                                     maximize=maximize, bias_correction=bias_correction)
    b1, b2 = betas
    inv_c1 = 1.0 / (1.0 - b1 ** step) if bias_correction else 1.0
    inv_c2 = 1.0 / (1.0 - b2 ** step) if bias_correction else 1.0
    _ops().adam_update(weight.detach().view(-1), grad.detach().reshape(-1).contiguous(), first.view(-1),
                       second.view(-1), float(lr), float(weight_decay), float(b1), float(b2), inv_c1, inv_c2,
                       float(eps), bool(adamw), bool(maximize), rounding == "stochastic", int(step - 1),
                       int(key) & ((1 << 63) - 1), int(offset))
    _count()


def copy_scaled(update, partition, src, dst, count, scale):
    if not update.is_cuda:
        return reference.copy_scaled(update, partition, src, dst, count, scale)
    _ops().copy_scaled(update.contiguous().view(-1), partition.view(-1), int(src), int(dst), int(count), float(scale))
    _count()


def momentum16(grad, momentum, out, beta, nesterov=True):
    if not grad.is_cuda:
        return reference.momentum16(grad, momentum, out, beta, nesterov)
    _ops().momentum16(grad.detach().reshape(-1).contiguous(), momentum.view(-1), out, float(beta), bool(nesterov))
    _count()


def ema_lerp(ema, master, decay):
    if not ema.is_cuda:
        return reference.ema_lerp(ema, master, decay)
    _ops().ema_lerp(ema.view(-1), master.detach().reshape(-1).contiguous(), float(decay))
    _count()


def philox(element, step, key, count=1, device=None):
    """``count`` consecutive Philox words starting at ``element`` (device kernel on CUDA, NumPy on CPU)."""
    if device is None or torch.device(device).type != "cuda":
        import numpy as np
        return torch.from_numpy(reference.philox(np.arange(element, element + count, dtype=np.uint64), step, key)
                                .astype("int64"))
    out = torch.empty(count, device=device, dtype=torch.int32)
    _ops().philox_kat(int(element), int(step), int(key), out)
    _count()
    return out.to(torch.int64) & 0xFFFFFFFF


def hadamard64(x, out=None):
    if not x.is_cuda:
        result = reference.hadamard64(x)
        return result if out is None else out.copy_(result)
    x = x.contiguous()
    out = torch.empty_like(x) if out is None else out
    _ops().hadamard64(x, out)
    _count()
    return out


# ------------------------------------------------------------------------------ wire codec
def wire_pack(source, packet, tile_size, fp8_dtype):
    if not source.is_cuda:
        return reference.wire_pack(source, packet, tile_size, fp8_dtype)
    rows = packet.shape[0]
    groups = packet.shape[1] // (tile_size + 4)
    _ops().wire_pack(source.contiguous().view(-1), rows, groups, int(tile_size), _FMT[fp8_dtype], packet,
                     packet.stride(0))
    _count()


def wire_unpack(packet, out, tile_size, fp8_dtype, *, reduce=False, accumulate=False):
    if not out.is_cuda:
        return reference.wire_unpack(packet, out, tile_size, fp8_dtype, reduce=reduce, accumulate=accumulate)
    rows = packet.shape[0]
    groups = packet.shape[1] // (tile_size + 4)
    _ops().wire_unpack(packet, packet.stride(0), rows, groups, int(tile_size), _FMT[fp8_dtype], bool(reduce),
                       out.view(-1), bool(accumulate))
    _count()


# ------------------------------------------------------------------------------ producer-fused quantisers
_MODES = {"ln_modulate": 1, "gelu": 2, "silu": 3}


def ln_modulate_quantize(x, shift, scale, tokens, *, eps=1e-6, history=None, index=0, delayed=False,
                         fp8_dtype=torch.float8_e4m3fn, quantization_limit=None, transpose=False):
    """FP8 codes of ``LN(x) * (1 + scale[b]) + shift[b]`` without materialising it (CUDA only).

    ``x`` [rows, cols] in fp32 or bf16 (the residual stream is read as stored), ``shift`` / ``scale`` bf16
    [rows // tokens, cols] (row-strided views are fine).  Returns (q, qt or None, qscale, mean, rstd).
    """
    rows, cols = x.shape
    limit = _limit(fp8_dtype, quantization_limit)
    mean = torch.empty(rows, device=x.device, dtype=torch.float32)
    rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
    qscale = torch.empty(1, device=x.device, dtype=torch.float32)
    _ops().ln_stats_amax(x, float(eps), shift, scale, int(tokens), mean, rstd, history, int(index), bool(delayed), limit,
                         qscale, _amax_scratch(x.device))
    q = torch.empty((rows, cols), device=x.device, dtype=fp8_dtype)
    qt = torch.empty((cols, rows), device=x.device, dtype=fp8_dtype) if transpose else None
    _ops().fused_quantize(x, 1, mean, rstd, shift, scale, int(tokens), qscale, limit, _FMT[fp8_dtype], q, qt, None)
    _count(2)
    return q, qt, qscale, mean, rstd


def activation_quantize(z, activation, *, history=None, index=0, delayed=False, fp8_dtype=torch.float8_e4m3fn,
                        quantization_limit=None, transpose=False, slope=False):
    """FP8 codes of ``act(z)`` (gelu / silu) without materialising it.  Returns (q, qt or None, qscale), plus
    ``act'(z)`` in bf16 when ``slope`` is set (row-wise codes only): the backward pass then needs neither ``z``
    nor another transcendental."""
    rows, cols = z.shape
    limit = _limit(fp8_dtype, quantization_limit)
    qscale = torch.empty(1, device=z.device, dtype=torch.float32)
    mode = _MODES[activation]
    _ops().act_amax(z, mode, history, int(index), bool(delayed), limit, qscale, _amax_scratch(z.device))
    q = torch.empty((rows, cols), device=z.device, dtype=fp8_dtype)
    qt = torch.empty((cols, rows), device=z.device, dtype=fp8_dtype) if transpose else None
    slope_out = torch.empty_like(z) if slope else None
    _ops().fused_quantize(z, mode, None, None, None, None, 1, qscale, limit, _FMT[fp8_dtype], q, qt, slope_out)
    _count(2)
    return (q, qt, qscale, slope_out) if slope else (q, qt, qscale)


def ln_modulate_backward(dh, x, mean, rstd, scale, tokens, grad_in=None, sums_dtype=torch.float32):
    """Gradients of LN + modulate: returns (dx [rows, cols] in x's dtype, dshift, dscale [samples, cols]).
    ``grad_in`` (x's shape and dtype) is added to dx: the gradient that reaches x along the residual path.
    ``sums_dtype``: fp32, or bf16 to get the per-sample sums (accumulated in fp32) rounded by the kernel."""
    rows, cols = x.shape
    dx = torch.empty_like(x)
    sums_dtype = sums_dtype if sums_dtype == torch.bfloat16 else torch.float32
    dshift = torch.empty((rows // tokens, cols), device=x.device, dtype=sums_dtype)
    dscale = torch.empty_like(dshift)
    workspace, tickets = _sample_sum_workspace(x.device, rows, tokens, 2 * cols)
    _ops().ln_modulate_backward(dh, x, mean, rstd, scale, int(tokens), grad_in, dx, dshift, dscale, workspace, tickets)
    _count()
    return dx, dshift, dscale


def gate_residual(x, gate, y, tokens):
    """``x + gate[row // tokens] * y`` for a 2-D residual stream ``x`` (fp32 or bf16) and bf16 ``y`` / ``gate``."""
    if not x.is_cuda:
        return reference.gate_residual(x, gate, y, tokens)
    out = torch.empty_like(x)
    _ops().gate_residual(x, gate, y, int(tokens), out)
    _count()
    return out


def gate_residual_backward(dout, gate, y, tokens, sums_dtype=torch.float32):
    """Branch gradients of the gated residual: (dy bf16 [rows, cols], dgate [samples, cols] in ``sums_dtype``:
    fp32, or bf16 rounded by the kernel from its fp32 sums)."""
    if not dout.is_cuda:
        dy, dgate = reference.gate_residual_backward(dout, gate, y, tokens)
        return dy, dgate.to(sums_dtype)
    rows, cols = dout.shape
    dy = torch.empty((rows, cols), device=dout.device, dtype=torch.bfloat16)
    sums_dtype = sums_dtype if sums_dtype == torch.bfloat16 else torch.float32
    dgate = torch.empty((rows // tokens, cols), device=dout.device, dtype=sums_dtype)
    workspace, tickets = _sample_sum_workspace(dout.device, rows, tokens, cols)
    _ops().gate_residual_backward(dout, gate, y, int(tokens), dy, dgate, workspace, tickets)
    _count()
    return dy, dgate


# ------------------------------------------------------------------------------ multi-tensor optimizer ops
_DT = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}
_CHUNK = 4096


class TensorTable:
    """Device-resident descriptor table for the multi-tensor kernels (built once per parameter set).

    ``rows``: one tuple per tensor ``(p0, p1, p2, p3, n, i0, f0, f1, d0, d1)`` with tensors (or None / ints)
    in the pointer slots.  Keeps the referenced tensors alive.
    """

    def __init__(self, rows, device):
        import struct
        self.keep = [t for row in rows for t in row[:4] if isinstance(t, torch.Tensor)]
        packed, prefix = [], [0]
        for p0, p1, p2, p3, n, i0, f0, f1, d0, d1 in rows:
            pointers = [t.data_ptr() if isinstance(t, torch.Tensor) else int(t or 0) for t in (p0, p1, p2, p3)]
            floats = struct.unpack("<q", struct.pack("<ff", float(f0), float(f1)))[0]
            codes = struct.unpack("<q", struct.pack("<ii", int(d0), int(d1)))[0]
            signed = int(i0) & ((1 << 63) - 1)
            packed.append([*(p if p < (1 << 63) else p - (1 << 64) for p in pointers), int(n), signed, floats, codes])
            prefix.append(prefix[-1] + (int(n) + _CHUNK - 1) // _CHUNK)
        # pinned staging + asynchronous upload: building a table must not synchronise the stream
        host_table = torch.tensor(packed, dtype=torch.int64).pin_memory()
        host_prefix = torch.tensor(prefix, dtype=torch.int32).pin_memory()
        self.table = host_table.to(device, non_blocking=True)
        self.prefix = host_prefix.to(device, non_blocking=True)
        self.keep.extend((host_table, host_prefix))
        self.blocks = prefix[-1]
        self.pointers = tuple(tuple(row[:4]) for row in packed)

    def matches(self, rows):
        """True when ``rows`` still name the same storage (pointers can change after a re-allocation)."""
        if len(rows) != len(self.pointers):
            return False
        for row, known in zip(rows, self.pointers):
            current = tuple((t.data_ptr() if isinstance(t, torch.Tensor) else int(t or 0)) for t in row[:4])
            if tuple(p if p < (1 << 63) else p - (1 << 64) for p in current) != known:
                return False
        return True


def multi_ema(table, decay):
    _ops().multi_ema(table.table, table.prefix, table.blocks, float(decay))
    _count()


def multi_adam(table, *, lr, weight_decay, betas, eps, step, rounding="nearest", adamw=True, maximize=False):
    b1, b2 = betas
    _ops().multi_adam(table.table, table.prefix, table.blocks, float(lr), float(weight_decay), float(b1), float(b2),
                      1.0 / (1.0 - b1 ** step), 1.0 / (1.0 - b2 ** step), float(eps), bool(adamw), bool(maximize),
                      rounding == "stochastic", int(step - 1))
    _count()


def multi_weight_update(table, lr, weight_decay, *, rounding="nearest", step=0):
    _ops().multi_weight_update(table.table, table.prefix, table.blocks, float(lr), float(weight_decay),
                               rounding == "stochastic", int(step))
    _count()


def multi_momentum(table, *, tile_size, beta, nesterov=True, loss_scale=1.0, rounding="nearest", step=0):
    _ops().multi_momentum(table.table, table.prefix, table.blocks, int(tile_size), float(beta), 1.0 / float(loss_scale),
                          bool(nesterov), rounding == "stochastic", int(step))
    _count()


class WritebackTable:
    """Device-resident table for :func:`multi_writeback` (16 int64 words per owned parameter).

    ``rows``: dicts with ``master`` (tensor), ``ema`` (tensor or None), ``n``, ``slab_elems``, ``dst_offset``,
    ``header_offset`` (-1 for none), ``base_index``, ``limit``, ``history_len``, ``mode`` (0 e4m3, 1 e5m2, 2 cast)
    and ``out_dtype`` (torch dtype, cast rows only).  One uint32 amax slot per row is allocated here.
    """

    def __init__(self, rows, device):
        import struct
        self.rows = len(rows)
        self.amax = torch.zeros(max(1, len(rows)), device=device, dtype=torch.int32)
        self.keep = [row["master"] for row in rows] + [row["ema"] for row in rows if row.get("ema") is not None]
        base = self.amax.data_ptr()
        packed, prefix = [], [0]

        def pair(a, b, first_float=False):
            return struct.unpack("<q", struct.pack("<fi" if first_float else "<ii", a, b))[0]

        def signed(value):
            return value if value < (1 << 63) else value - (1 << 64)

        for position, row in enumerate(rows):
            master, ema = row["master"], row.get("ema")
            packed.append([signed(master.data_ptr()), signed(ema.data_ptr()) if ema is not None else 0,
                           signed(base + 4 * position), int(row["n"]), int(row["slab_elems"]),
                           signed(int(row["dst_offset"])), signed(int(row["header_offset"])) if row["header_offset"] >= 0 else -1,
                           int(row["base_index"]),
                           pair(float(row.get("limit", 448.0)), int(row.get("history_len", 0)), first_float=True),
                           pair(_DT[master.dtype], _DT[ema.dtype] if ema is not None else 0),
                           pair(int(row["mode"]), _DT.get(row.get("out_dtype"), 0)), 0, 0, 0, 0, 0])
            prefix.append(prefix[-1] + (int(row["n"]) + _CHUNK - 1) // _CHUNK)
        host_table = torch.tensor(packed, dtype=torch.int64).reshape(-1).pin_memory() if packed else torch.zeros(0, dtype=torch.int64)
        host_prefix = torch.tensor(prefix, dtype=torch.int32).pin_memory()
        self.table = host_table.to(device, non_blocking=True)
        self.prefix = host_prefix.to(device, non_blocking=True)
        self.keep.extend((host_table, host_prefix))
        self.blocks = prefix[-1]
        self.pointers = tuple((row[0], row[1]) for row in packed)

    def matches(self, rows):
        if len(rows) != len(self.pointers):
            return False
        for row, (master, ema) in zip(rows, self.pointers):
            if (row["master"].data_ptr() & ((1 << 64) - 1)) != (master & ((1 << 64) - 1)):
                return False
            current = row["ema"].data_ptr() if row.get("ema") is not None else 0
            if (current & ((1 << 64) - 1)) != (ema & ((1 << 64) - 1)):
                return False
        return True


def multi_writeback(table, *, heaps, rank, calls, decay=0.0, with_ema=False):
    """Owner write-back of every row of ``table`` in two launches (amax + EMA, then encode + peer stores).

    ``heaps``: every rank's symmetric-heap base address (``[0]`` with absolute offsets for a single process).
    ``calls``: write-backs since the table was built (selects the amax-history slot)."""
    if not table.rows:
        return
    table.amax.zero_()
    _ops().multi_writeback(table.table, table.prefix, table.blocks, float(decay), bool(with_ema), list(heaps), int(rank),
                           int(calls))
    _count(2)
