"""GPU parity tests of the FP8 / NVFP4 activation quantizers: bit-exact against the CPU
oracle and, where it has been built, against the reference's own kernels on the same GPU."""
import ctypes

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from layerstormgemmkernels_b200 import ops as _ops
    return _ops


def bits_of(t):
    return t.view(torch.int16).cpu().numpy().view(np.uint16)


def _p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("M,K", [(1, 128), (7, 384), (32, 1024), (5, 200), (3, 100), (64, 7168), (2, 8)])
@pytest.mark.parametrize("m_major", [False, True])
def test_dynamic_fp8_quant_bit_exact(ops, M, K, m_major):
    g = torch.Generator().manual_seed(M * K)
    x = torch.randn(M, K, generator=g) * 3
    if K >= 256:
        x[0, 128:256] = 0            # all-zero block: scale 1.0
    x[-1, 0] = 3e4                   # outlier
    xb = x.to(torch.bfloat16).cuda()
    out, sc = ops.dynamic_fp8_quant(xb, m_major)
    ref_out, ref_sc = oracle.dynamic_fp8_quant(bits_of(xb), m_major)
    np.testing.assert_array_equal(out.view(torch.uint8).cpu().numpy(), ref_out)
    np.testing.assert_array_equal(sc.cpu().numpy(), ref_sc)
    assert out.dtype == torch.float8_e4m3fn and tuple(sc.shape) == ref_sc.shape
    lib = oracle.ref_lib()
    if lib is not None:              # the reference's own kernel
        want = torch.zeros((M, K), dtype=torch.uint8, device="cuda")
        wsc = torch.zeros_like(sc)
        assert lib.ref_dynamic_fp8_quant(_p(xb), _p(want), _p(wsc), M, K, int(m_major), _stream()) == 0
        torch.cuda.synchronize()
        assert torch.equal(out.view(torch.uint8), want) and torch.equal(sc, wsc)


def test_dynamic_fp8_quant_full_size_roundtrip(ops):
    """4096 x 4096 (the NVFP4 config's tensor): dequantized values within half an e4m3 ulp."""
    x = torch.randn(4096, 4096, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).cuda()
    out, sc = ops.dynamic_fp8_quant(x)
    deq = out.float().view(4096, 32, 128) * sc.view(4096, 32, 1)
    xf = x.float().view(4096, 32, 128)
    amax = xf.abs().amax(-1, keepdim=True)
    # (torch divides by a scalar through its reciprocal, hence not bit-equal to amax / 448)
    torch.testing.assert_close(sc.view(4096, 32, 1), amax / 448.0, rtol=3e-7, atol=0)
    assert ((deq - xf).abs() <= xf.abs() * 2.0 ** -4 + amax * (2.0 ** -10 / 448.0) * 1.01 + 1e-9).all()


CASES = [
    (256, [0, 3, 3, 131, 148]),          # ragged, one empty expert (reference test)
    (64, [0, 1]),
    (4096, [0, 5, 9, 9, 40]),
    (768, [0, 0, 200, 200, 513]),        # > 128 rows: several scale atoms per expert
    (14336, [0, 2, 3]),
]


@pytest.mark.parametrize("K,offs", CASES)
@pytest.mark.parametrize("with_is", [False, True])
def test_bf16_to_nvfp4_grouped_bit_exact(ops, K, offs, with_is):
    T, E = offs[-1], len(offs) - 1
    g = torch.Generator().manual_seed(K + T)
    x = torch.randn(T, K, generator=g) * 0.5
    x[0, :16] = 0                          # zero group -> scale floor 2^-9
    x[T - 1, 16:32] *= 1e-4                # tiny group
    xb = x.to(torch.bfloat16).cuda()
    offs_t = torch.tensor(offs, dtype=torch.int32, device="cuda")
    isc = (torch.rand(E, generator=g) * 1e-3 + 1e-4).cuda() if with_is else None
    if with_is:
        isc[0] = 0.0                       # non-positive entry behaves as 1.0
    packed, scales, sf = ops.bf16_to_nvfp4_grouped(xb, offs_t, isc)
    rp, rs, rsf = oracle.bf16_to_nvfp4_grouped(bits_of(xb), offs, isc.cpu().numpy() if with_is else None)
    np.testing.assert_array_equal(sf.cpu().numpy(), rsf)
    np.testing.assert_array_equal(packed.cpu().numpy(), rp)
    np.testing.assert_array_equal(scales.cpu().numpy(), rs)
    lib = oracle.ref_lib()
    if lib is not None:
        wp = torch.zeros_like(packed)
        wsc = torch.zeros_like(scales)
        assert lib.ref_bf16_to_nvfp4_grouped(_p(xb), _p(wp), _p(wsc), _p(offs_t), _p(sf), T, E, K,
                                             _p(isc), _stream()) == 0
        torch.cuda.synchronize()
        assert torch.equal(packed, wp) and torch.equal(scales, wsc)


def test_offsets_on_cpu_are_accepted(ops):
    x = torch.randn(8, 64).to(torch.bfloat16).cuda()
    a = ops.bf16_to_nvfp4_grouped(x, torch.tensor([0, 3, 8], dtype=torch.int32))
    b = ops.bf16_to_nvfp4_grouped(x, torch.tensor([0, 3, 8], dtype=torch.int32, device="cuda"))
    for u, v in zip(a, b):
        assert torch.equal(u, v)
    with pytest.raises(RuntimeError, match="divisible by 64"):
        ops.bf16_to_nvfp4_grouped(x[:, :32].contiguous(), torch.tensor([0, 8], dtype=torch.int32))
    with pytest.raises(RuntimeError, match="end at total_tokens"):
        ops.bf16_to_nvfp4_grouped(x, torch.tensor([0, 7], dtype=torch.int32))


@pytest.mark.parametrize("K,offs", CASES[:4])
@pytest.mark.parametrize("with_is", [False, True])
def test_silu_mul_fused_equals_unfused_bytes(ops, K, offs, with_is):
    """tests/test_kernels.py:667-731: the fused SwiGLU quantizer must produce the bytes of
    SwiGLU (rounded to bf16) followed by the plain quantizer.  The unfused activation is
    formed here with torch on the GPU from the same expression."""
    T, E = offs[-1], len(offs) - 1
    g = torch.Generator().manual_seed(K * 3 + T)
    gate = (torch.randn(T, K, generator=g) * 1.5).to(torch.bfloat16).cuda()
    up = (torch.randn(T, K, generator=g)).to(torch.bfloat16).cuda()
    offs_t = torch.tensor(offs, dtype=torch.int32, device="cuda")
    isc = (torch.rand(E, generator=g) * 1e-2 + 1e-3).cuda() if with_is else None
    fp, fs, fsf = ops.silu_mul_to_nvfp4_grouped(gate, up, offs_t, isc)
    lib = oracle.ref_lib()
    if lib is not None:
        # bit-exact against the reference's fused kernel
        wp = torch.zeros_like(fp)
        wsc = torch.zeros_like(fs)
        assert lib.ref_silu_mul_to_nvfp4_grouped(_p(gate), _p(up), _p(wp), _p(wsc), _p(offs_t), _p(fsf),
                                                 T, E, K, _p(isc), _stream()) == 0
        torch.cuda.synchronize()
        assert torch.equal(fp, wp) and torch.equal(fs, wsc)
    # against torch's SwiGLU: tanh implementations may differ in the last bit, which can
    # move a value across a bf16 or e2m1 boundary in rare cases
    gf, uf = gate.float(), up.float()
    act = ((gf * (0.5 * torch.tanh(0.5 * gf) + 0.5)) * uf).to(torch.bfloat16)
    up_, us_, _ = ops.bf16_to_nvfp4_grouped(act, offs_t, isc)
    assert (fp != up_).float().mean().item() < 2e-3
    assert (fs != us_).float().mean().item() < 2e-3
