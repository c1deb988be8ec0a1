"""CPU oracles: known-answer and self-consistency tests of the PyTorch/NumPy restatements."""
import math

import numpy as np
import torch

from viola_b200.ops import reference as ref
from viola_b200 import ops

E4M3 = torch.float8_e4m3fn


def test_philox_known_answers():
    # Random123 kat_vectors for philox4x32-10 (first output word).
    cases = [(0, 0, 0), (0xffffffffffffffff,) * 3, (0x85a308d3243f6a88, 0x0370734413198a2e, 0x299f31d0a4093822)]
    answers = [int(ref.philox(np.array([e], dtype=np.uint64), s, k)[0]) for e, s, k in cases]
    assert answers == [0x6627e8d5, 0x408f276d, 0xd16cfe09]


def test_stochastic_rounding_adjacent_and_probability():
    table = torch.arange(127, dtype=torch.uint8).view(E4M3).float()
    values = torch.full((200000,), 16.54)
    rounded = ref.stochastic_e4m3(values, np.arange(values.numel(), dtype=np.uint64), 3, 77)
    assert set(rounded.unique().tolist()) == {16.0, 18.0}
    assert abs((rounded == 18.0).float().mean().item() - 0.27) < 0.005
    assert all(v in table.tolist() for v in rounded.unique().tolist())
    again = ref.stochastic_e4m3(values, np.arange(values.numel(), dtype=np.uint64), 3, 77)
    assert torch.equal(rounded, again)
    other = ref.stochastic_e4m3(values, np.arange(values.numel(), dtype=np.uint64), 4, 77)
    assert not torch.equal(rounded, other)
    quarter = torch.full((200000,), 1.0 + 2.0 ** -9)        # a quarter bf16 ulp above 1.0
    kept = ref.stochastic_bf16(quarter, np.arange(quarter.numel(), dtype=np.uint64), 0, 1)
    assert abs((kept > 1.0).float().mean().item() - 0.25) < 0.005


def test_group_quantize_roundtrip_and_shapes():
    torch.manual_seed(0)
    x = torch.randn(70, 200)
    for group in ((1, 32), (32, 32), (1, 128), (128, 128)):
        q, s = ref.group_quantize(x, E4M3, group)
        assert s.shape == ref.scale_shape(x.shape, group)
        back = ref.group_dequantize(q, s, group)
        assert ((back - x).norm() / x.norm()).item() < 0.05
        qt, st = ref.group_quantize(x, E4M3, group, transposed=True)
        assert qt.shape == (200, 70)
    q, s = ops.group_quantize(x, E4M3, (1, 128), kmajor=True)
    assert s.shape == (2, 70)


def test_momentum_tile_and_block_geometry():
    torch.manual_seed(1)
    for quant in (dict(granularity="tile", tile_size=64), dict(granularity="block", block_shape=(8, 32))):
        for shape in ((17, 31), (2, 33, 67)):
            n = math.prod(shape)
            qn, sn = ref.state_sizes(shape, **quant)
            q, s = torch.zeros(qn, dtype=torch.uint8), torch.ones(sn)
            u = torch.empty(n, dtype=torch.bfloat16)
            g = torch.randn(n)
            ref.momentum_update(g, q, s, q, s, u, beta=0.95, matrix_shape=shape, **quant)
            current = ref.momentum_dequantize(q, s, shape, **quant)
            fresh = 0.05 * g
            assert ((current - fresh).norm() / fresh.norm()).item() < 0.06
            torch.testing.assert_close(u.float(), ((0.05 + 0.95 * 0.05) * g).bfloat16().float(), rtol=0.01, atol=1e-7)


def test_newton_schulz_orthogonalises():
    torch.manual_seed(2)
    for shape in ((64, 64), (48, 160), (160, 48)):
        x = torch.randn(shape)
        for result in (ref.ns_standard(x, 5).float(), ref.ns_gram(x, 5).float()):
            singular = torch.linalg.svdvals(result)
            assert singular.max() < 1.3 and singular.min() > 0.5


def test_wire_codec_roundtrip_and_nan():
    torch.manual_seed(3)
    tile, world, n = 128, 2, 1000
    groups = math.ceil(n / (world * tile))
    packet = torch.zeros(world, ref.packet_bytes(groups, tile), dtype=torch.uint8)
    x = torch.randn(n)
    ref.wire_pack(x, packet, tile, E4M3)
    out = torch.empty(n)
    ref.wire_unpack(packet, out, tile, E4M3)
    assert ((out - x).norm() / x.norm()).item() < 0.05
    x[3] = float("nan")
    ref.wire_pack(x, packet, tile, E4M3)
    ref.wire_unpack(packet, out, tile, E4M3)
    assert torch.isnan(out[:tile]).all() and torch.isfinite(out[tile:]).all()


def test_hadamard_is_orthogonal_and_self_inverse():
    h = ref.hadamard64_matrix()
    torch.testing.assert_close(h @ h, torch.eye(64), atol=1e-6, rtol=0)
    torch.testing.assert_close(h, h.t())


def test_block_fusion_ops_on_cpu():
    """CPU paths of the transformer-block ops: gated residual, activation-slope GEMM, gathered amax, column sums."""
    from viola_b200 import ops
    from torch.nn import functional as F
    torch.manual_seed(4)
    rows, cols, tokens = 24, 32, 6
    x = torch.randn(rows, cols, requires_grad=True)
    y = torch.randn(rows, cols).bfloat16().requires_grad_(True)
    gate = torch.randn(rows // tokens, cols).bfloat16().requires_grad_(True)
    out = ops.gate_residual(x.detach(), gate.detach(), y.detach(), tokens)
    expected = x + gate.float().repeat_interleave(tokens, dim=0) * y.float()
    torch.testing.assert_close(out, expected.detach())
    dout = torch.randn(rows, cols)
    expected.backward(dout)
    dy, dgate = ops.gate_residual_backward(dout, gate.detach(), y.detach(), tokens)
    torch.testing.assert_close(dy.float(), y.grad.float(), rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(dgate, gate.grad.float(), rtol=2e-2, atol=2e-2)

    z = torch.randn(rows, cols).bfloat16()
    zf = z.float().requires_grad_(True)
    slope, = torch.autograd.grad(F.gelu(zf, approximate="tanh").sum(), zf)
    slope = slope.bfloat16()
    dyq = torch.randn(rows, 16).to(torch.float8_e5m2)
    w = (torch.randn(16, cols) * 0.1).to(E4M3)
    one = torch.ones(1)
    amax = torch.zeros(1, dtype=torch.int32)
    dz = ops.activation_backward_gemm(dyq, w, one, one, slope, w_mn=True, amax_out=amax)
    reference = ((dyq.float() @ w.float()).bfloat16().float() * slope.float()).bfloat16()
    torch.testing.assert_close(dz.float(), reference.float())
    assert amax.view(torch.float32).item() == dz.float().abs().max().item()
    history = torch.zeros(4)
    scale = ops.scale_from_amax(amax, history=history, index=1, fp8_dtype=torch.float8_e5m2)
    assert amax.item() == 0 and history[1].item() == dz.float().abs().max().item()
    torch.testing.assert_close(scale, dz.float().abs().max().reshape(1) / 57344)

    colsum = torch.zeros(cols)
    q, _ = ops.quantize(x.detach(), torch.tensor([0.05]), colsum=colsum)
    torch.testing.assert_close(colsum, x.detach().sum(dim=0))
    assert q.shape == x.shape


def test_power_of_two_scale_rule_is_exact():
    """MXFP8 scales are the smallest power of two >= amax / limit, with no logarithm rounding at the boundaries."""
    from viola_b200.ops import reference
    values = torch.tensor([1.0, 1.0 + 2 ** -23, 0.75, 0.5, 0.5 - 2 ** -25, 3e-30, 2.0 ** -126, 448.0])
    expected = torch.tensor([1.0, 2.0, 1.0, 0.5, 0.5, 2.0 ** -98, 2.0 ** -126, 512.0])
    assert torch.equal(reference.ceil_pow2(values), expected)
    x = torch.randn(64, 96) * 5
    q, s = reference.group_quantize(x, torch.float8_e4m3fn, (1, 32), pow2=True)
    assert torch.equal(torch.exp2(torch.round(torch.log2(s))), s)
    plain = reference.group_quantize(x, torch.float8_e4m3fn, (1, 32))[1]
    assert ((s >= plain) & (s < 2 * plain)).all()
    decoded = reference.group_dequantize(q, s, (1, 32))
    assert ((decoded - x).abs() <= 0.0625 * x.abs() + 1e-6 + s.repeat_interleave(32, 1) * 2 ** -9).all()
