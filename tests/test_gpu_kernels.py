"""Numerics of every sm_100a kernel against the plain PyTorch fp32 restatement of the same op.

Tolerances follow the reference's acceptance bounds: group-scaled / fp32-output GEMM < 2e-5
relative L2 (checks/check_grouped_linear.py:42), bf16-output Linear < 0.3 % (checks/linear.py:38),
fused gated MLP < 2.5 % (checks/mlp.py:44), wire codec reduce < 2e-6 (checks/fp8_communication.py:75).
"""
import math

import numpy as np
import pytest
import torch

from conftest import rel_l2
from viola_b200 import ops
from viola_b200.ops import reference as ref

pytestmark = pytest.mark.gpu
E4M3, E5M2 = torch.float8_e4m3fn, torch.float8_e5m2


@pytest.fixture(autouse=True)
def _status():
    yield
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        ops.check_status()


def dev():
    return torch.device("cuda", 0)


@pytest.mark.parametrize("shape", [(64, 64), (257, 130), (1000, 777), (4096, 1152)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_tensor_scale_and_quantize(shape, dtype):
    torch.manual_seed(0)
    x = (torch.randn(shape, device=dev()) * 3).to(dtype)
    history = torch.zeros(16, device=dev())
    scale = ops.tensor_scale(x, history=history, index=0, delayed=True)
    expected = x.float().abs().max() / 448
    torch.testing.assert_close(scale[0], expected, rtol=1e-6, atol=0)
    assert history[0].item() == x.float().abs().max().item()
    scale2 = ops.tensor_scale(x * 2, history=history, index=1, delayed=True)   # delayed: uses history max
    torch.testing.assert_close(scale2[0], expected, rtol=1e-6, atol=0)
    for fmt in (E4M3, E5M2):
        q, qt = ops.quantize(x, scale, transpose=True, fp8_dtype=fmt)
        rq, rqt = ref.quantize(x.cpu(), scale.cpu(), transpose=True, fp8_dtype=fmt)
        assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
        assert torch.equal(qt.cpu().view(torch.uint8), rqt.view(torch.uint8))
        assert torch.equal(ops.transpose(q).cpu().view(torch.uint8), rqt.view(torch.uint8))


@pytest.mark.parametrize("shape", [(300, 256), (4096, 1152), (1000, 4608), (33, 16)])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_quantize_rows_with_column_sums(shape, dtype):
    """Row-wise-only path (16-byte vectors, reciprocal + exact correction instead of a division) gives the same
    codes as the division oracle, and the fused column sums equal the plain reduction."""
    torch.manual_seed(7)
    x = (torch.randn(shape, device=dev()) * 5).to(dtype)
    x[1, 3], x[2, 5] = float("inf"), float("nan")
    for fmt, limit in ((E4M3, None), (E5M2, None), (E4M3, 240.0)):
        scale = ops.tensor_scale(torch.nan_to_num(x, posinf=0.0), fp8_dtype=fmt, quantization_limit=limit)
        colsum = torch.zeros(shape[1], device=dev())
        q, _ = ops.quantize(x, scale, fp8_dtype=fmt, quantization_limit=limit, colsum=colsum)
        rq, _ = ref.quantize(x.cpu(), scale.cpu(), fp8_dtype=fmt, quantization_limit=limit)
        assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
        expected = torch.nan_to_num(x.float(), nan=0.0, posinf=0.0).sum(dim=0)
        got = colsum.clone()
        got[3] = got[5] = expected[3] = expected[5] = 0          # the inf / nan columns
        assert rel_l2(got, expected) < 1e-5
        assert torch.isinf(colsum[3]) and torch.isnan(colsum[5])


def test_quantize_preserves_nan():
    x = torch.randn(64, 64, device=dev())
    x[3, 5] = float("nan")
    scale = torch.tensor([0.01], device=dev())
    q, _ = ops.quantize(x, scale)
    assert torch.isnan(q.float()[3, 5]) and torch.isnan(q.float()).sum() == 1


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 256, 512), (1000, 520, 1152), (4096, 1152, 4608),
                                    (77, 3456, 1152)])
@pytest.mark.parametrize("formats", [(E4M3, E4M3), (E5M2, E4M3)])
def test_fp8_gemm_per_tensor(m, n, k, formats):
    torch.manual_seed(1)
    a = torch.randn(m, k, device=dev()).to(formats[0])
    b = torch.randn(n, k, device=dev()).to(formats[1])
    sa, sb = torch.tensor([0.37], device=dev()), torch.tensor([1.9], device=dev())
    bias = torch.randn(n, device=dev(), dtype=torch.bfloat16)
    expected = (a.float() @ b.float().t()) * 0.37 * 1.9
    out32 = ops.gemm(a, b, sa, sb, out_dtype=torch.float32)
    assert rel_l2(out32, expected) < 2e-5
    out = ops.gemm(a, b, sa, sb, out_dtype=torch.bfloat16, bias=bias)
    assert rel_l2(out, expected + bias.float()) < 3e-3
    for bn in (128, 256):
        forced = ops.gemm(a, b, sa, sb, out_dtype=torch.float32, force_bn=bn)
        assert rel_l2(forced, expected) < 2e-5


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (384, 256, 1152), (1000, 640, 2048), (4096, 1152, 4608)])
@pytest.mark.parametrize("weight_group", [(128, 128), (1, 128)])
def test_fp8_gemm_group_scaled(m, n, k, weight_group):
    torch.manual_seed(2)
    x = torch.randn(m, k, device=dev(), dtype=torch.bfloat16) * torch.rand(m, 1, device=dev()).mul(4).exp()
    w = torch.randn(n, k, device=dev(), dtype=torch.bfloat16) * 0.05
    for kmajor in (False, True):
        qx, sx = ops.group_quantize(x, E4M3, (1, 128), kmajor=kmajor)
        qw, sw = ops.group_quantize(w, E4M3, weight_group)
        rqx, rsx = ref.group_quantize(x.cpu(), E4M3, (1, 128))
        assert torch.equal(qx.cpu().view(torch.uint8), rqx.view(torch.uint8))
        torch.testing.assert_close((sx.t() if kmajor else sx).cpu(), rsx, rtol=1e-6, atol=0)
        rqw, rsw = ref.group_quantize(w.cpu(), E4M3, weight_group)
        assert torch.equal(qw.cpu().view(torch.uint8), rqw.view(torch.uint8))
        expected = ref.group_dequantize(rqx, rsx, (1, 128)).to(dev()) @ ref.group_dequantize(rqw, rsw, weight_group).to(dev()).t()
        out = ops.group_gemm(qx, qw, sx, sw, (1, 128), weight_group, out_dtype=torch.float32, sa_kmajor=kmajor)
        assert rel_l2(out, expected) < 2e-5


def test_group_quantize_pair_and_transposed():
    torch.manual_seed(3)
    x = torch.randn(300, 520, device=dev(), dtype=torch.bfloat16)
    q, s, qt, st = ops.group_quantize_pair(x, E5M2, (1, 128), (1, 128), kmajor=True)
    rq, rs = ref.group_quantize(x.cpu(), E5M2, (1, 128))
    rqt, rst = ref.group_quantize(x.cpu(), E5M2, (1, 128), transposed=True)
    assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    assert torch.equal(qt.cpu().view(torch.uint8), rqt.view(torch.uint8))
    torch.testing.assert_close(s.t().cpu(), rs, rtol=1e-6, atol=0)
    torch.testing.assert_close(st.t().cpu(), rst, rtol=1e-6, atol=0)
    for group in ((32, 32), (1, 32), (128, 128), (1, 256), (256, 256)):
        q, s = ops.group_quantize(x, E4M3, group)
        rq, rs = ref.group_quantize(x.cpu(), E4M3, group)
        assert torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8)), group
        torch.testing.assert_close(s.cpu(), rs, rtol=1e-6, atol=0)
        torch.testing.assert_close(ops.group_dequantize(q, s, group).cpu(), ref.group_dequantize(rq, rs, group))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("m,k", [(128, 256), (1152, 1152), (640, 4608), (200, 1000)])
def test_ns_gemm(dtype, m, k):
    torch.manual_seed(4)
    x = (torch.randn(m, k, device=dev()) / math.sqrt(k)).to(dtype)
    gram_expected = (x.float() @ x.float().t()).to(dtype)
    gram = ops.ns_gemm(x, x)
    assert rel_l2(gram, gram_expected) < 2e-3
    gram_sym = ops.ns_gemm(x, x, symmetric=True)
    assert rel_l2(gram_sym, gram_expected) < 2e-3
    assert torch.equal(gram_sym, gram_sym.t())
    poly_expected = (-4.775 * gram.float() + 2.0315 * (gram.float() @ gram.float()).to(dtype).float()).to(dtype)
    poly = ops.ns_gemm(gram, gram, alpha=2.0315, beta=-4.775, resid=gram, symmetric=True)
    assert rel_l2(poly, poly_expected) < 4e-3
    xt = x.t().contiguous()
    new_t = torch.empty(k, m, device=dev(), dtype=dtype)
    new = ops.ns_gemm(poly, xt, alpha=1.0, beta=3.4445, resid=x, out_t=new_t)
    new_expected = (3.4445 * x.float() + (poly.float() @ x.float()).to(dtype).float()).to(dtype)
    assert rel_l2(new, new_expected) < 4e-3
    assert torch.equal(new_t, new.t())


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (640, 384, 1152), (1008, 528, 2000), (1152, 4608, 4096), (256, 512, 300)])
def test_gemm_mn_major_operands(a_mn, b_mn, m, n, k):
    """Operands handed over transposed ([K, M] / [K, N]) are read MN-major in place and give the K-major result."""
    torch.manual_seed(11)
    a8 = torch.randn(m, k, device=dev()).to(E4M3)
    b8 = torch.randn(n, k, device=dev()).to(E5M2 if not (a_mn and b_mn) else E4M3)
    sa, sb = torch.tensor([0.5], device=dev()), torch.tensor([1.25], device=dev())
    base = ops.gemm(a8, b8, sa, sb, out_dtype=torch.float32)
    assert rel_l2(base, (a8.float() @ b8.float().t()) * 0.625) < 2e-5
    a_arg = a8.view(torch.uint8).t().contiguous().view(a8.dtype) if a_mn else a8
    b_arg = b8.view(torch.uint8).t().contiguous().view(b8.dtype) if b_mn else b8
    for bn in (0, 128, 256):
        out = ops.gemm(a_arg, b_arg, sa, sb, out_dtype=torch.float32, a_mn=a_mn, b_mn=b_mn, force_bn=bn)
        assert torch.equal(out, base), (bn, rel_l2(out, base))
    for dtype in (torch.bfloat16, torch.float16):
        a16 = (torch.randn(m, k, device=dev()) / math.sqrt(k)).to(dtype)
        b16 = torch.randn(n, k, device=dev()).to(dtype)
        resid = torch.randn(m, n, device=dev()).to(dtype)
        base16 = ops.ns_gemm(a16, b16, alpha=0.75, beta=-1.5, resid=resid)
        out16 = ops.ns_gemm(a16.t().contiguous() if a_mn else a16, b16.t().contiguous() if b_mn else b16, alpha=0.75,
                            beta=-1.5, resid=resid, a_mn=a_mn, b_mn=b_mn)
        assert torch.equal(out16, base16), rel_l2(out16, base16)
    ops.check_status()


@pytest.mark.parametrize("a_mn,b_mn", [(True, False), (False, True), (True, True)])
def test_batched_ns_gemm_mn_major(a_mn, b_mn):
    torch.manual_seed(12)
    batch, m, n, k = 5, 384, 640, 1152
    a = (torch.randn(batch, m, k, device=dev()) / math.sqrt(k)).bfloat16()
    b = torch.randn(batch, n, k, device=dev()).bfloat16()
    base = ops.ns_gemm(a, b)
    assert rel_l2(base, a.float() @ b.float().mT) < 4e-3
    out = ops.ns_gemm(a.mT.contiguous() if a_mn else a, b.mT.contiguous() if b_mn else b, a_mn=a_mn, b_mn=b_mn)
    assert torch.equal(out, base)
    ops.check_status()


@pytest.mark.parametrize("activation", ["silu", "gelu", "relu"])
@pytest.mark.parametrize("grouped", [False, True])
def test_gated_gemm(activation, grouped):
    torch.manual_seed(5)
    m, k, hidden = 520, 1152, 1280
    x = torch.randn(m, k, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(2 * hidden, k, device=dev(), dtype=torch.bfloat16) * 0.03
    bias = torch.randn(2 * hidden, device=dev(), dtype=torch.bfloat16) * 0.1
    if grouped:
        qx, sx = ops.group_quantize(x, E4M3, (1, 128), kmajor=True)
        qw, sw = ops.group_quantize(w, E4M3, (128, 128))
        z = ops.group_gemm(qx, qw, sx, sw, (1, 128), (128, 128), out_dtype=torch.bfloat16, bias=bias, sa_kmajor=True)
        h, aux = ops.gated_gemm_forward(qx, qw, sx, sw, activation=activation, out_dtype=torch.bfloat16, bias=bias,
                                        group=((1, 128), (128, 128)), sa_kmajor=True)
    else:
        sx, sw = ops.tensor_scale(x), ops.tensor_scale(w)
        qx, _ = ops.quantize(x, sx)
        qw, _ = ops.quantize(w, sw)
        z = ops.gemm(qx, qw, sx, sw, out_dtype=torch.bfloat16, bias=bias)
        h, aux = ops.gated_gemm_forward(qx, qw, sx, sw, activation=activation, out_dtype=torch.bfloat16, bias=bias)
    assert rel_l2(aux, z) < 1e-3
    assert rel_l2(h, ref.gated_forward(z, activation)) < 5e-3
    assert rel_l2(ops.gated_forward(z, activation), ref.gated_forward(z, activation)) < 5e-3
    # backward: d = dY . Wdown ; [dG|dU]
    out_features = 640
    dy = torch.randn(m, out_features, device=dev(), dtype=torch.bfloat16)
    wdown_t = torch.randn(hidden, out_features, device=dev(), dtype=torch.bfloat16) * 0.03   # = Wdown^T
    if grouped:
        qg, sg = ops.group_quantize(dy, E5M2, (1, 128), kmajor=True)
        qt, st = ops.group_quantize(wdown_t, E4M3, (128, 128))
        d = ops.group_gemm(qg, qt, sg, st, (1, 128), (128, 128), out_dtype=torch.bfloat16, sa_kmajor=True)
        dz = ops.gated_gemm_backward(qg, qt, sg, st, aux, activation=activation, out_dtype=torch.bfloat16,
                                     group=((1, 128), (128, 128)), sg_kmajor=True)
    else:
        sg, st = ops.tensor_scale(dy, fp8_dtype=E5M2), ops.tensor_scale(wdown_t)
        qg, _ = ops.quantize(dy, sg, fp8_dtype=E5M2)
        qt, _ = ops.quantize(wdown_t, st)
        d = ops.gemm(qg, qt, sg, st, out_dtype=torch.bfloat16)
        dz = ops.gated_gemm_backward(qg, qt, sg, st, aux, activation=activation, out_dtype=torch.bfloat16)
    expected = ref.gated_backward(aux, d, activation)
    assert rel_l2(dz, expected) < 1e-2
    assert rel_l2(ops.gated_backward(aux, d, activation), expected) < 1e-2


@pytest.mark.parametrize("hidden", [1000, 1004, 96])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("save", [True, False])
def test_gated_gemm_ragged_widths(hidden, dtype, save):
    """Widths that end inside a 32-column chunk (1000), that cannot use 16-byte rows (1004: per-thread stores) and
    below one tile (96), rows that end inside a tile, both 16-bit types, with and without the saved halves: nothing
    may land outside the valid region and the values must match the unfused pair of kernels."""
    torch.manual_seed(11)
    m, k, out_features = 333, 256, 384
    x = torch.randn(m, k, device=dev(), dtype=dtype)
    w = torch.randn(2 * hidden, k, device=dev(), dtype=dtype) * 0.05
    sx, sw = ops.tensor_scale(x), ops.tensor_scale(w)
    qx, _ = ops.quantize(x, sx)
    qw, _ = ops.quantize(w, sw)
    z = ops.gemm(qx, qw, sx, sw, out_dtype=dtype)
    h, aux = ops.gated_gemm_forward(qx, qw, sx, sw, activation="silu", out_dtype=dtype, save=save)
    assert (aux is None) == (not save)
    if save:
        assert rel_l2(aux, z) < 1e-3
    expected = ref.gated_forward(z, "silu")
    assert rel_l2(h, expected) < 5e-3
    assert (h.float() - expected.float()).abs().max() < 0.05 * expected.float().abs().max()
    dy = torch.randn(m, out_features, device=dev(), dtype=dtype)
    wdown_t = torch.randn(hidden, out_features, device=dev(), dtype=dtype) * 0.05
    sg, st = ops.tensor_scale(dy, fp8_dtype=E5M2), ops.tensor_scale(wdown_t)
    qg, _ = ops.quantize(dy, sg, fp8_dtype=E5M2)
    qt, _ = ops.quantize(wdown_t, st)
    d = ops.gemm(qg, qt, sg, st, out_dtype=dtype)
    dz = ops.gated_gemm_backward(qg, qt, sg, st, z, activation="silu", out_dtype=dtype)
    want = ref.gated_backward(z, d, "silu")
    assert rel_l2(dz, want) < 1e-2
    assert (dz.float() - want.float()).abs().max() < 0.05 * want.float().abs().max()
    ops.check_status()


@pytest.mark.parametrize("grouped", [False, True])
def test_expert_gemm(grouped):
    torch.manual_seed(6)
    experts, n, k = 4, 512, 1024
    counts = [300, 0, 129, 515]
    offsets = torch.tensor([0, *np.cumsum(counts)], device=dev(), dtype=torch.int32)
    tokens = sum(counts)
    x = torch.randn(tokens, k, device=dev(), dtype=torch.bfloat16)
    w = torch.randn(experts, n, k, device=dev(), dtype=torch.bfloat16) * 0.05
    if grouped:
        qx, sx = ops.group_quantize(x, E4M3, (1, 128), kmajor=True)
        qw, sw = ops.group_quantize(w.view(-1, k), E4M3, (128, 128))
        out = ops.expert_gemm(qx, qw.view(experts, n, k), offsets, sx, sw, out_dtype=torch.float32,
                              group=((1, 128), (128, 128)), sa_kmajor=True)
        dx = ops.group_dequantize(qx, sx, (1, 128), kmajor=True)
        dw = ops.group_dequantize(qw, sw, (128, 128)).view(experts, n, k)
    else:
        sx, sw = ops.tensor_scale(x), ops.tensor_scale(w)
        qx, _ = ops.quantize(x, sx)
        qw, _ = ops.quantize(w.view(-1, k), sw)
        out = ops.expert_gemm(qx, qw.view(experts, n, k), offsets, sx, sw, out_dtype=torch.float32)
        dx, dw = qx.float() * sx, (qw.float() * sw).view(experts, n, k)
    bounds = offsets.tolist()
    for e in range(experts):
        lo, hi = bounds[e], bounds[e + 1]
        if hi > lo:
            assert rel_l2(out[lo:hi], dx[lo:hi] @ dw[e].t()) < 2e-5, e


def test_philox_known_answers():
    answers = [int(ops.philox(e, s, k, 1, dev())[0]) for e, s, k in
               [(0, 0, 0), (-1, -1, -1), (0x85a308d3243f6a88 - (1 << 64), 0x0370734413198a2e, 0x299f31d0a4093822)]]
    assert answers == [0x6627e8d5, 0x408f276d, 0xd16cfe09]


@pytest.mark.parametrize("quant", [dict(granularity="tile", tile_size=t) for t in (64, 128, 256, 512, 1024)]
                         + [dict(granularity="block", block_shape=b) for b in ((8, 8), (16, 16), (16, 32), (64, 64))])
@pytest.mark.parametrize("shape", [(17, 31), (2, 33, 67), (256, 1152)])
@pytest.mark.parametrize("rounding", ["nearest", "stochastic"])
def test_momentum_update(quant, shape, rounding):
    torch.manual_seed(7)
    n = math.prod(shape)
    qn, sn = ops.state_sizes(shape, **quant)
    q = torch.zeros(qn + 1, dtype=torch.uint8, device=dev())[1:]        # deliberately unaligned
    scale = torch.ones(sn + 1, device=dev())[1:]
    u = torch.empty(n + 1, dtype=torch.bfloat16, device=dev())[1:]
    rq, rscale, ru = torch.zeros(qn, dtype=torch.uint8), torch.ones(sn), torch.empty(n, dtype=torch.bfloat16)
    for step in range(4):
        g = torch.randn(n + 1, device=dev())[1:] * (1e-8 if step < 1 else 1.0)
        rq.copy_(q.cpu()), rscale.copy_(scale.cpu())      # follow the device state so errors do not compound
        old = ref.momentum_dequantize(rq, rscale, shape, **quant)
        fresh = 0.95 * old + (1 - 0.95) * g.cpu()
        ops.momentum_update(g, q, scale, q, scale, u, beta=0.95, matrix_shape=shape, rounding=rounding,
                            rounding_step=step, rounding_key=123, **quant)
        ref.momentum_update(g.cpu(), rq, rscale, rq, rscale, ru, beta=0.95, matrix_shape=shape, rounding=rounding,
                            rounding_step=step, rounding_key=123, **quant)
        torch.testing.assert_close(scale.cpu(), rscale, rtol=2e-6, atol=1e-30)
        torch.testing.assert_close(u.float().cpu(), ru.float(), rtol=0.01, atol=2e-7)
        current = ref.momentum_dequantize(q.cpu(), scale.cpu(), shape, **quant)
        assert rel_l2(current, fresh) < 0.06
        mismatch = (q.cpu()[:n] != rq[:n]).float().mean().item()
        assert mismatch < 5e-3, mismatch      # fp32 contraction differences may flip a rare rounding tie


def test_stochastic_rounding_probability():
    n = 1 << 18
    tile = 256
    value = 448.0 * (1 + 0.27 / 8)      # 27 % of the way between two E4M3 codes at the top binade / 8 grid... scaled below
    g = torch.full((n,), 20.0 * (1 + 0.27 * 0.125) / 0.05, device=dev())
    g[::tile] = 20.0 * 28.0 / 0.05        # one large element per tile pins the scale: amax -> 448
    q = torch.zeros(n, dtype=torch.uint8, device=dev())
    scale = torch.ones(n // tile, device=dev())
    u = torch.empty(n, dtype=torch.bfloat16, device=dev())
    ops.momentum_update(g, q, scale, q, scale, u, beta=0.95, tile_size=tile, rounding="stochastic", rounding_step=5,
                        rounding_key=99)
    codes = q.view(torch.float8_e4m3fn).float().view(-1, tile)[:, 1:]
    low = codes.min().item()
    ups = (codes > low).float().mean().item()
    assert abs(ups - 0.27) < 0.005, ups
    del value


@pytest.mark.parametrize("wdt", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("gdt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rounding", ["nearest", "stochastic"])
def test_weight_and_adam_update(wdt, gdt, rounding):
    torch.manual_seed(8)
    n = 5000
    w = torch.randn(n, device=dev()).to(wdt)
    upd = torch.randn(n, device=dev()).to(gdt)
    rw = w.cpu().clone()
    ops.weight_update(w, upd, 1e-2, 0.1, update_scale=3.0, rounding=rounding, step=3, key=11, offset=7)
    ref.weight_update(rw, upd.cpu(), 1e-2, 0.1, update_scale=3.0, rounding=rounding, step=3, key=11, offset=7)
    ulp = {torch.float32: 2e-6, torch.bfloat16: 8e-3, torch.float16: 1e-3}[wdt]
    torch.testing.assert_close(w.cpu().float(), rw.float(), rtol=ulp, atol=ulp * 1e-2)
    for sdt in (torch.float32, torch.bfloat16):
        w = torch.randn(n, device=dev()).to(wdt)
        g = torch.randn(n, device=dev()).to(gdt)
        m1, m2 = torch.zeros(n, device=dev(), dtype=sdt), torch.zeros(n, device=dev(), dtype=sdt)
        rw, rm1, rm2 = w.cpu().clone(), m1.cpu().clone(), m2.cpu().clone()
        for step in (1, 2):
            ops.adam_update(w, g, m1, m2, lr=1e-2, weight_decay=0.01, betas=(0.9, 0.95), eps=1e-8, step=step,
                            rounding=rounding, key=5)
            ref.adam_update(rw, g.cpu(), rm1, rm2, lr=1e-2, weight_decay=0.01, betas=(0.9, 0.95), eps=1e-8, step=step,
                            rounding=rounding, key=5)
        torch.testing.assert_close(w.cpu().float(), rw.float(), rtol=ulp * 2, atol=ulp * 2e-2)
        torch.testing.assert_close(m1.cpu().float(), rm1.float(), rtol=1e-2, atol=1e-6)


@pytest.mark.parametrize("tile", [32, 128, 256])
@pytest.mark.parametrize("fmt", [E4M3, E5M2])
def test_wire_codec(tile, fmt):
    torch.manual_seed(9)
    world, n = 4, 100_003
    groups = math.ceil(n / (world * tile))
    stride = ops.packet_bytes(groups, tile)
    x = torch.randn(n, device=dev()) * 1e-3
    x[::997] *= 100
    packet = torch.zeros(world, stride, device=dev(), dtype=torch.uint8)
    ops.wire_pack(x, packet, tile, fmt)
    rpacket = torch.zeros(world, stride, dtype=torch.uint8)
    ref.wire_pack(x.cpu(), rpacket, tile, fmt)
    codes, scales = ops.packet_views(packet.cpu(), tile, fmt)
    rcodes, rscales = ops.packet_views(rpacket, tile, fmt)
    torch.testing.assert_close(scales, rscales, rtol=1e-6, atol=0)
    assert (codes.view(torch.uint8) != rcodes.view(torch.uint8)).float().mean() < 1e-3
    out = torch.empty(n, device=dev())
    ops.wire_unpack(packet, out, tile, fmt)
    rout = torch.empty(n)
    ref.wire_unpack(packet.cpu(), rout, tile, fmt)
    assert rel_l2(out.cpu(), rout) < 2e-6
    width = groups * tile
    partial = torch.empty(width, device=dev())
    ops.wire_unpack(packet, partial, tile, fmt, reduce=True)
    rpartial = torch.empty(width)
    ref.wire_unpack(packet.cpu(), rpartial, tile, fmt, reduce=True)
    assert rel_l2(partial.cpu(), rpartial) < 2e-6
    x[5] = float("nan")
    ops.wire_pack(x, packet, tile, fmt)
    ops.wire_unpack(packet, out, tile, fmt)
    assert torch.isnan(out[:tile]).all() and torch.isfinite(out[tile:]).all()


def test_hadamard64_and_misc():
    torch.manual_seed(10)
    x = torch.randn(37, 256, device=dev(), dtype=torch.bfloat16)
    y = ops.hadamard64(x)
    assert rel_l2(y, ref.hadamard64(x.cpu()).to(dev())) < 5e-3
    assert rel_l2(ops.hadamard64(y), x) < 1e-2
    ema = torch.randn(1000, device=dev())
    master = torch.randn(1000, device=dev())
    expected = ema * 0.999 + master * (1 - 0.999)
    ops.ema_lerp(ema, master, 0.999)
    torch.testing.assert_close(ema, expected, rtol=1e-6, atol=1e-7)


# ------------------------------------------------------------------------------------------------ MXFP8 (hardware block scaling)
@pytest.mark.parametrize("shape", [(128, 128, 128), (256, 384, 512), (200, 136, 160), (1024, 1152, 4608)])
@pytest.mark.parametrize("formats", [(torch.float8_e4m3fn, torch.float8_e4m3fn), (torch.float8_e5m2, torch.float8_e4m3fn)])
def test_mx_gemm_matches_dequantised_product(shape, formats):
    """tcgen05 block-scaled MMA with UE8M0 scales in tensor memory against the fp32 product of the decoded operands
    (bound of checks/check_grouped_linear.py:42 for fp32 accumulation and output)."""
    m, n, k = shape
    torch.manual_seed(m + n + k)
    a = (torch.randn(m, k, device="cuda") * 2).to(formats[0])
    b = (torch.randn(n, k, device="cuda") * 2).to(formats[1])
    groups = (k + 31) // 32
    sa = torch.randint(118, 134, (m, groups), device="cuda", dtype=torch.uint8)        # 2^-9 .. 2^6
    sb = torch.randint(118, 134, (n, groups), device="cuda", dtype=torch.uint8)
    bias = torch.randn(n, device="cuda")
    out = ops.mx_gemm(a, b, ops.mx_pack_scales(sa, m, k), ops.mx_pack_scales(sb, n, k), out_dtype=torch.float32, bias=bias)
    torch.cuda.synchronize()
    ops.check_status()
    expected = ref.mx_gemm(a, b, sa, sb, out_dtype=torch.float32, bias=bias)
    assert rel_l2(out, expected) < 2e-5
    half = ops.mx_gemm(a, b, ops.mx_pack_scales(sa, m, k), ops.mx_pack_scales(sb, n, k), out_dtype=torch.bfloat16)
    assert rel_l2(half, ref.mx_gemm(a, b, sa, sb, out_dtype=torch.float32)) < 4e-3


def test_mx_scales_from_fp32_powers_of_two_and_weight_blocks():
    """Packing accepts fp32 powers of two in either storage order and 32 x 32 weight blocks (one scale per 32 rows)."""
    m, n, k = 256, 192, 256
    torch.manual_seed(5)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    ea = torch.randint(120, 131, (m, k // 32), device="cuda", dtype=torch.uint8)
    eb = torch.randint(120, 131, (n // 32, k // 32), device="cuda", dtype=torch.uint8)
    fa, fb = torch.exp2(ea.float() - 127), torch.exp2(eb.float() - 127)
    sfa = ops.mx_pack_scales(fa.t().contiguous(), m, k, kmajor=True)                    # K-block-major fp32
    sfb = ops.mx_pack_scales(fb, n, k, group_rows=32)
    assert torch.equal(sfa, ops.mx_pack_scales(ea, m, k))
    out = ops.mx_gemm(a, b, sfa, sfb, out_dtype=torch.float32)
    expected = ref.mx_gemm(a, b, ea, eb.repeat_interleave(32, 0), out_dtype=torch.float32)
    assert rel_l2(out, expected) < 2e-5


@pytest.mark.parametrize("transposed", [False, True])
def test_power_of_two_group_encode_matches_oracle(transposed):
    x = torch.randn(300, 416, device="cuda", dtype=torch.bfloat16) * 3
    x[7, 40:72] = 0                                                    # an all-zero group
    x[9, :32] = torch.tensor(2.0 ** 5)                                 # amax / limit exactly representable
    q, s = ops.group_quantize(x, torch.float8_e4m3fn, (1, 32), transposed=transposed, pow2=True)
    rq, rs = ref.group_quantize(x.cpu(), torch.float8_e4m3fn, (1, 32), transposed=transposed, pow2=True)
    assert torch.equal(s.cpu(), rs) and torch.equal(q.cpu().view(torch.uint8), rq.view(torch.uint8))
    exponent = (s.view(torch.int32) >> 23) & 0xff
    assert torch.equal(torch.exp2(exponent.float() - 127), s)          # every scale is a power of two


def test_mxfp8_linear_runs_on_the_block_scaled_path_and_matches_cpu():
    from viola_b200.nn import Linear
    torch.manual_seed(11)
    layer = Linear(256, 384, scaling="mxfp8", device="cuda", dtype=torch.bfloat16)
    x = torch.randn(512, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    before = ops.launch_count
    y = layer(x)
    y.float().square().mean().backward()
    torch.cuda.synchronize()
    ops.check_status()
    assert ops.launch_count > before
    clone = Linear(256, 384, scaling="mxfp8", device="cpu", dtype=torch.bfloat16)
    clone.load_state_dict({k: v.cpu() if isinstance(v, torch.Tensor) else v for k, v in layer.state_dict().items()})
    xc = x.detach().cpu().requires_grad_(True)
    yc = clone(xc)
    yc.float().square().mean().backward()
    assert rel_l2(y.detach().cpu(), yc.detach()) < 1e-2
    assert rel_l2(x.grad.cpu(), xc.grad) < 2e-2
    assert rel_l2(layer.weight.grad.cpu(), clone.weight.grad) < 2e-2


@pytest.mark.parametrize("head_dim", [72, 64, 128, 40])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_attention_forward_matches_the_fp32_softmax(head_dim, dtype):
    """The 256-token attention kernel against softmax(Q K^T / sqrt(D)) V in fp32, including the log-sum-exp rows that
    the backward consumes; scores are scaled up so the softmax is far from uniform."""
    torch.manual_seed(head_dim)
    batch, heads = 3, 5
    qkv = (torch.randn(batch, 256, 3, heads, head_dim, device=dev()) * 1.5).to(dtype)
    out, lse = ops.attention_forward(qkv)
    want, want_lse = ref.attention_forward(qkv, head_dim ** -0.5)
    ops.check_status()
    assert out.shape == (batch, 256, heads, head_dim) and lse.shape == (batch, heads, 256)
    assert rel_l2(out, want) < (8e-3 if dtype == torch.bfloat16 else 2e-3)
    assert (lse - want_lse).abs().max() < 2e-3
    again, _ = ops.attention_forward(qkv)
    assert torch.equal(out, again)


def test_packed_attention_gradients_match_the_library_path():
    from viola_b200.nn import attention
    torch.manual_seed(3)
    qkv = torch.randn(2, 256, 3, 4, 72, device=dev(), dtype=torch.bfloat16, requires_grad=True)
    weight = torch.randn(2, 256, 4 * 72, device=dev(), dtype=torch.bfloat16)
    (attention.packed_attention(qkv) * weight).sum().backward()
    native = qkv.grad.clone()
    qkv.grad = None
    attention._state["native"] = False
    try:
        (attention.packed_attention(qkv) * weight).sum().backward()
    finally:
        attention._state["native"] = True
    assert rel_l2(native, qkv.grad) < 1e-2


# ------------------------------------------------------------------------------------------------ memory-safety substitutes
def _guarded(shape, dtype, pad=4096):
    """A tensor of ``shape`` carved out of a larger buffer whose bytes before and after it are a known pattern."""
    count = int(np.prod(shape))
    itemsize = torch.empty((), dtype=dtype).element_size()
    raw = torch.full((2 * pad + count * itemsize,), 0xA5, device="cuda", dtype=torch.uint8)
    view = raw[pad:pad + count * itemsize].view(dtype).view(shape)

    def intact():
        return bool((raw[:pad] == 0xA5).all() and (raw[pad + count * itemsize:] == 0xA5).all())

    return view, intact


@pytest.mark.parametrize("shape", [(200, 136, 160), (384, 520, 1152), (130, 264, 96)])
def test_gemm_outputs_stay_inside_their_buffers_and_repeat_bit_for_bit(shape):
    """No sanitizer on this pool: outputs are carved out of canary-padded buffers (ragged shapes, so edge tiles are
    exercised), and every kernel is run twice and must reproduce its result exactly."""
    m, n, k = shape
    torch.manual_seed(m * n + k)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").to(torch.float8_e4m3fn)
    one = torch.ones(1, device="cuda")
    for dtype in (torch.bfloat16, torch.float32):
        out, intact = _guarded((m, n), dtype)
        ops.gemm(a, b, one, one, out_dtype=dtype, out=out)
        first = out.clone()
        ops.gemm(a, b, one, one, out_dtype=dtype, out=out)
        torch.cuda.synchronize()
        assert intact() and torch.equal(first, out)
        assert rel_l2(out, a.float() @ b.float().t()) < 1e-2
    # hardware block-scaled path
    sa = torch.randint(120, 132, (m, (k + 31) // 32), device="cuda", dtype=torch.uint8)
    sb = torch.randint(120, 132, (n, (k + 31) // 32), device="cuda", dtype=torch.uint8)
    out, intact = _guarded((m, n), torch.float32)
    sfa, sfb = ops.mx_pack_scales(sa, m, k), ops.mx_pack_scales(sb, n, k)
    ops.mx_gemm(a, b, sfa, sfb, out_dtype=torch.float32, out=out)
    first = out.clone()
    ops.mx_gemm(a, b, sfa, sfb, out_dtype=torch.float32, out=out)
    torch.cuda.synchronize()
    assert intact() and torch.equal(first, out)
    ops.check_status()


@pytest.mark.parametrize("shape", [(1152, 1152, 4096), (200, 520, 2064), (1152, 4608, 8192)])
@pytest.mark.parametrize("layout", ["k-major", "mn-major"])
def test_split_k_matches_the_unsplit_product_and_repeats(shape, layout):
    """fp32 results computed by several work units per tile (TMA reduce-add in a fixed order) against the same
    product from one unit per tile, with and without a bias, into a guarded buffer, twice."""
    m, n, k = shape
    torch.manual_seed(k + n)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").to(torch.float8_e5m2)
    sa, sb = torch.full((1,), 0.5, device="cuda"), torch.full((1,), 0.25, device="cuda")
    bias = torch.randn(n, device="cuda")
    mn = layout == "mn-major"
    if mn and (m % 16 or n % 16):
        pytest.skip("MN-major operands need 16-byte rows")
    left, right = (a.t().contiguous(), b.t().contiguous()) if mn else (a, b)
    expected = (a.float() @ b.float().t()) * 0.125
    for use_bias in (False, True):
        base = ops.gemm(left, right, sa, sb, out_dtype=torch.float32, bias=bias if use_bias else None, a_mn=mn, b_mn=mn,
                        force_split=1)
        for split in (2, 3, 5, 0):
            out, intact = _guarded((m, n), torch.float32)
            ops.gemm(left, right, sa, sb, out_dtype=torch.float32, bias=bias if use_bias else None, a_mn=mn, b_mn=mn,
                     out=out, force_split=split)
            first = out.clone()
            ops.gemm(left, right, sa, sb, out_dtype=torch.float32, bias=bias if use_bias else None, a_mn=mn, b_mn=mn,
                     out=out, force_split=split)
            torch.cuda.synchronize()
            assert intact() and torch.equal(first, out)
            assert rel_l2(out, base) < 1e-5
        assert rel_l2(base, expected + (bias if use_bias else 0.0)) < 1e-5
    ops.check_status()


@pytest.mark.parametrize("shape", [(512, 512, 256), (1000, 712, 1152), (130, 264, 96), (4096, 3456, 1152)])
@pytest.mark.parametrize("layout", ["k-major", "b-mn", "mn-major"])
def test_cta_pair_gemm_matches_the_single_cta_kernel(shape, layout):
    """256 x 256 tiles computed by CTA pairs (tcgen05 cta_group::2, each CTA loading half of B) against the
    single-CTA kernel on the same operands: identical accumulation order per output element, so bit-identical."""
    m, n, k = shape
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").to(torch.float8_e5m2)
    sa, sb = torch.full((1,), 0.5, device="cuda"), torch.full((1,), 0.25, device="cuda")
    bias = torch.randn(n, device="cuda").bfloat16()
    a_mn, b_mn = layout == "mn-major", layout in ("b-mn", "mn-major")
    if (a_mn and m % 16) or (b_mn and n % 16):
        pytest.skip("MN-major operands need 16-byte rows")
    left = a.t().contiguous() if a_mn else a
    right = b.t().contiguous() if b_mn else b
    for dtype in (torch.bfloat16, torch.float32):
        for use_bias in (False, True):
            kwargs = dict(out_dtype=dtype, bias=bias if use_bias else None, a_mn=a_mn, b_mn=b_mn)
            base = ops.gemm(left, right, sa, sb, force_bn=256, force_split=1, **kwargs)
            out, intact = _guarded((m, n), dtype)
            ops.gemm(left, right, sa, sb, force_bn=512, out=out, **kwargs)
            torch.cuda.synchronize()
            ops.check_status()
            assert intact()
            assert torch.equal(out, base)
    assert rel_l2(base, (a.float() @ b.float().t()) * 0.125 + bias.float()) < 1e-2


@pytest.mark.parametrize("shape", [(1152, 1152, 4096), (200, 520, 2064), (264, 130, 96)])
def test_gemm_adds_into_its_output(shape):
    """``accumulate=True``: out += A.B^T through the TMA reduce epilogue (with and without split-K), and through the
    compute-then-add fallback for outputs the reduce path cannot take (bf16)."""
    m, n, k = shape
    torch.manual_seed(m + k)
    a = torch.randn(m, k, device="cuda").to(torch.float8_e4m3fn)
    b = torch.randn(n, k, device="cuda").to(torch.float8_e5m2)
    one = torch.ones(1, device="cuda")
    product = ops.gemm(a, b, one, one, out_dtype=torch.float32, force_split=1)
    before = torch.randn(m, n, device="cuda")
    for split in (1, 0, 3):
        out, intact = _guarded((m, n), torch.float32)
        out.copy_(before)
        ops.gemm(a, b, one, one, out_dtype=torch.float32, out=out, accumulate=True, force_split=split)
        torch.cuda.synchronize()
        assert intact()
        assert rel_l2(out - before, product) < 1e-5
    half = before.bfloat16()
    ops.gemm(a, b, one, one, out_dtype=torch.bfloat16, out=half, accumulate=True)
    assert rel_l2(half.float(), before.bfloat16().float() + product) < 1e-2
    ops.check_status()


def test_quantiser_outputs_stay_inside_their_buffers_and_repeat_bit_for_bit():
    rows, cols = 333, 416
    x = torch.randn(rows, cols, device="cuda", dtype=torch.bfloat16)
    scale = ops.tensor_scale(x)
    q, q_ok = _guarded((rows, cols), torch.float8_e4m3fn)
    qt, qt_ok = _guarded((cols, rows), torch.float8_e4m3fn)
    ops.quantize(x, scale, transpose=True, out=q, out_t=qt)
    first, first_t = q.clone().view(torch.uint8), qt.clone().view(torch.uint8)
    ops.quantize(x, scale, transpose=True, out=q, out_t=qt)
    torch.cuda.synchronize()
    assert q_ok() and qt_ok()
    assert torch.equal(first, q.view(torch.uint8)) and torch.equal(first_t, qt.view(torch.uint8))
    assert torch.equal(qt.view(torch.uint8), q.view(torch.uint8).t())
    for group, transposed in (((1, 128), False), ((1, 32), True), ((128, 128), False)):
        shape = (cols, rows) if transposed else (rows, cols)
        g, g_ok = _guarded(shape, torch.float8_e4m3fn)
        _, s1 = ops.group_quantize(x, torch.float8_e4m3fn, group, transposed=transposed, out=g)
        keep = g.clone().view(torch.uint8)
        _, s2 = ops.group_quantize(x, torch.float8_e4m3fn, group, transposed=transposed, out=g)
        torch.cuda.synchronize()
        assert g_ok() and torch.equal(keep, g.view(torch.uint8)) and torch.equal(s1, s2)
    ops.check_status()
