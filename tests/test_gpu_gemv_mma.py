"""The tensor-core decode GEMV (arithmetic variant 4: mma.sync integer products on 15-bit
block-floating-point activations) against the numpy oracle and against the exact SIMT
variants, over ragged shapes, every batch size, both code widths and every fused option.

Tolerances: the activations are rounded at 2^-15 of their group maximum, so fp32 outputs are
compared at 5e-4 (measured values are printed by -s); bf16 outputs are those rounded once."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import rel_l2, seeded
from llmquant_b200.core import QuantizationArgs, QuantizationScheme
from oracle import llama_ops

pytestmark = pytest.mark.gpu

TOL_F32 = 5e-4


def _module(w, bits, bias=None):
    from llmquant_b200.quantizers import KernelQuantLinear

    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128), input_activations=None)
    linear = torch.nn.Linear(w.shape[1], w.shape[0], bias=bias is not None)
    linear.weight.data = w
    if bias is not None:
        linear.bias.data = bias
    return KernelQuantLinear.from_linear(linear.cuda(), scheme)


def _want(w, x, bits):
    q, scale = oracle.quantize_weight(w.float().numpy(), bits, 128)
    return oracle.real_linear(x.float().numpy(), q, scale, bits, 128)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("n,k", [(16, 128), (40, 256), (96, 1000), (512, 2048), (1030, 4096), (300, 14336)])
@pytest.mark.parametrize("M", [1, 2, 4])
def test_matches_the_oracle(bits, n, k, M):
    from llmquant_b200 import native

    w = seeded((n, k), 10 + n, 0.02, torch.bfloat16)
    x = seeded((M, k), 20 + k).bfloat16()
    module = _module(w, bits)
    if not module.tensor_core_gemv_ok(M):
        assert k > 8192 and (bits == 8 or M > 1)  # rows too long for the ring, or planes too large
        with pytest.raises(RuntimeError, match="tensor-core GEMV"):
            module.gemv(x.cuda(), variant=4)
        return
    want = _want(w, x, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, variant=4)
    assert native.library().lq_gemv_device_error() == 0
    err = rel_l2(got.cpu().numpy(), want)
    print(f"bits={bits} n={n} k={k} M={M} rel_l2={err:.2e}")
    assert err <= TOL_F32
    exact = module.gemv(x.cuda(), out_dtype=torch.float32, variant=3)
    assert rel_l2(got.cpu().numpy(), exact.cpu().numpy()) <= TOL_F32
    got16 = module.gemv(x.cuda(), variant=4)
    assert got16.dtype == torch.bfloat16 and torch.equal(got16, got.bfloat16())  # one rounding at the end


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [3, 5, 6, 7, 8])
def test_every_batch_size(bits, M):
    n, k = 272, 1024
    w = seeded((n, k), 31, 0.02, torch.bfloat16)
    x = seeded((M, k), 32).bfloat16()
    module = _module(w, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, variant=4)
    assert rel_l2(got.cpu().numpy(), _want(w, x, bits)) <= TOL_F32
    # a row's result does not depend on which other rows share the call
    alone = torch.cat([module.gemv(x[i:i + 1].cuda(), out_dtype=torch.float32, variant=4) for i in range(M)])
    assert torch.equal(got, alone)


@pytest.mark.parametrize("bits", [4, 8])
def test_outliers_and_zero_rows(bits):
    """Activation groups with one dominant channel, an all-zero row, and values at the top of a
    binade (the case where the block exponent has to be bumped)."""
    n, k = 128, 512
    w = seeded((n, k), 41, 0.02, torch.bfloat16)
    x = seeded((4, k), 42).bfloat16()
    x[0, 7] = 300.0
    x[1] = 0
    x[2, :128] = torch.tensor(1.9921875).bfloat16()  # (2 - 2^-7): the largest bf16 below 2
    x[3, 130] = -255.0
    module = _module(w, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, variant=4)
    want = _want(w, x, bits)
    assert np.all(got[1].cpu().numpy() == 0)
    for row in (0, 2, 3):
        assert rel_l2(got[row].cpu().numpy(), want[row]) <= TOL_F32, row
    # scaling the activations by a power of two scales the result exactly
    twice = module.gemv((x * 2).cuda(), out_dtype=torch.float32, variant=4)
    assert torch.equal(twice, got * 2)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [1, 4, 8])
@pytest.mark.parametrize("k", [2048, 4096])
def test_rmsnorm_prologue(bits, M, k):
    w = seeded((528, k), 1, 0.02, torch.bfloat16)
    x = (seeded((M, k), 2) * 3).bfloat16()
    gamma = (seeded((k,), 3) * 0.1 + 1).bfloat16()
    module = _module(w, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, norm_weight=gamma.cuda(), norm_eps=1e-5, pdl=True,
                      variant=4)
    normed = llama_ops.rmsnorm(x.float().numpy(), gamma.float().numpy(), 1e-5)
    want = _want(w, torch.from_numpy(normed), bits)
    assert rel_l2(got.cpu().numpy(), want) <= 1e-3
    simt = module.gemv(x.cuda(), out_dtype=torch.float32, norm_weight=gamma.cuda(), norm_eps=1e-5, variant=3)
    assert rel_l2(got.cpu().numpy(), simt.cpu().numpy()) <= TOL_F32


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [1, 3, 6])
def test_silu_mul_epilogue_bias_and_residual(bits, M):
    from llmquant_b200.runtime.decoder import _fuse_rows

    k, inter = 2048, 1000
    gate_w = seeded((inter, k), 4, 0.02, torch.bfloat16)
    up_w = seeded((inter, k), 5, 0.02, torch.bfloat16)
    x = seeded((M, k), 6).bfloat16()
    gate, up = _module(gate_w, bits), _module(up_w, bits)
    fused = _fuse_rows([gate, up], interleave=True)
    got = fused.gemv(x.cuda(), epilogue=1, variant=4)
    assert got.shape == (M, inter)
    g = gate.gemv(x.cuda(), variant=4).float().cpu().numpy()
    u = up.gemv(x.cuda(), variant=4).float().cpu().numpy()
    assert rel_l2(got.float().cpu().numpy(), llama_ops.silu_mul(g, u)) <= 2e-3
    res = seeded((M, inter), 7).bfloat16().cuda()
    with_res = gate.gemv(x.cuda(), residual=res, variant=4)
    want_res = (gate.gemv(x.cuda(), variant=4).float() + res.float()).bfloat16()
    assert torch.equal(with_res, want_res)
    res32 = seeded((M, inter), 8).cuda()
    with_res32 = gate.gemv(x.cuda(), residual=res32, out_dtype=torch.float32, variant=4)
    plain32 = gate.gemv(x.cuda(), out_dtype=torch.float32, variant=4)
    assert torch.equal(with_res32, plain32 + res32)
    bias = seeded((inter,), 9, 0.1, torch.bfloat16)
    biased = _module(gate_w, bits, bias=bias)
    got_b = biased.gemv(x.cuda(), out_dtype=torch.float32, variant=4)
    assert torch.allclose(got_b, plain32 + bias.float().cuda(), rtol=0, atol=1e-6)


def test_rejects_groups_it_is_not_built_for():
    """Per-head groups of 64 stored codes stay on the SIMT kernel."""
    from llmquant_b200.quantizers import KernelQuantLinear

    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=8, strategy="group", group_size=128, head_dim=64), input_activations=None)
    linear = torch.nn.Linear(256, 64, bias=False)
    module = KernelQuantLinear.from_linear(linear.cuda(), scheme)
    x = seeded((1, 256), 61).bfloat16().cuda()
    with pytest.raises(RuntimeError, match="tensor-core GEMV"):
        module.gemv(x, variant=4)
    module.gemv(x)  # the default still serves it


@pytest.mark.parametrize("bits,m", [(4, 2), (8, 4), (4, 8)])
@pytest.mark.parametrize("epilogue", [0, 1])
def test_output_row_stride(bits, m, epilogue):
    """`ldo`: a launch can write (and read its residual from) a block of columns of a wider
    matrix. Both GEMV kernels (2 rows: SIMT; 4 and 8 rows: tensor-core), bias, residual, SiLU."""
    import ctypes

    from llmquant_b200 import native

    n, k, wide, col0 = 256, 1024, 700, 136
    w = seeded((n, k), 71, 0.02, torch.bfloat16)
    bias = None if epilogue == 1 else seeded((n,), 72, 0.1, torch.bfloat16)
    module = _module(w, bits, bias=bias)
    x = seeded((m, k), 73).bfloat16().cuda()
    n_out = n // 2 if epilogue == 1 else n
    residual = None if epilogue == 1 else seeded((m, wide), 74).bfloat16().cuda()
    variant = 4 if m > 2 else 2
    plain = module.gemv(x, residual=None if residual is None else residual[:, col0:col0 + n_out].contiguous(),
                        epilogue=epilogue, variant=variant)
    out = torch.full((m, wide), 7.0, dtype=torch.bfloat16, device="cuda")
    bias16 = None if bias is None else bias.cuda()
    args = native.GemvArgs(
        x=x.data_ptr(), ldx=k, norm_weight=None, norm_eps=1e-5, codes=module.codes.data_ptr(),
        scale_tiles=module.scale_tiles.data_ptr(), bias=native.ptr(bias16),
        residual=None if residual is None else residual.data_ptr() + col0 * 2, out=out.data_ptr() + col0 * 2,
        out_dtype=native.LQ_BF16, M=m, N=n, K=k, Kd=k, span=128, bits=bits, epilogue=epilogue, variant=variant, pdl=0,
        tp=None, ldo=wide)
    native.call("lq_wq_gemv_fused", ctypes.byref(args), native.stream_ptr())
    torch.cuda.synchronize()
    assert torch.equal(out[:, col0:col0 + n_out], plain)
    assert bool((out[:, :col0] == 7).all()) and bool((out[:, col0 + n_out:] == 7).all())
    args.ldo = n_out - 1
    assert native.library().lq_wq_gemv_fused(ctypes.byref(args), native.stream_ptr()) != 0
    assert "ldo" in native.last_error()
