"""The tensor-core decode GEMM (variant 5 of lq_wq_gemv_fused: tcgen05 kind::i8 products of
the weight codes with 15-bit block-floating-point activation planes, up to 64 rows per pass
over the weight) against the numpy oracle and against the GEMV variants, over ragged shapes,
every padded row count, both code widths and every fused option.

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


def _module(w, bits, bias=None, group=128):
    from llmquant_b200.quantizers import KernelQuantLinear

    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=group), input_activations=None)
    linear = torch.nn.Linear(w.shape[1], w.shape[0], bias=bias is not None)
    linear.weight.data = w
    if bias is not None:
        linear.bias.data = bias
    return KernelQuantLinear.from_linear(linear.cuda(), scheme)


def _want(w, x, bits):
    q, scale = oracle.quantize_weight(w.float().numpy(), bits, 128)
    return oracle.real_linear(x.float().numpy(), q, scale, bits, 128)


def _no_device_error():
    from llmquant_b200 import native

    assert native.library().lq_decode_gemm_device_error() == 0


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("n,k", [(16, 128), (136, 256), (96, 1000), (600, 2048), (1030, 4096), (300, 14336)])
@pytest.mark.parametrize("M", [1, 9, 32])
def test_matches_the_oracle(bits, n, k, M):
    """Ragged row counts (tiles of 128 weight rows), a reduction axis that is not a multiple of
    the group (K = 1000), one scale group only, and the long axis of down_proj."""
    w = seeded((n, k), 10 + n, 0.02, torch.bfloat16)
    x = seeded((M, k), 20 + k).bfloat16()
    module = _module(w, bits)
    want = _want(w, x, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, variant=5)
    _no_device_error()
    err = rel_l2(got.cpu().numpy(), want)
    print(f"bits={bits} n={n} k={k} M={M} rel_l2={err:.2e}")
    assert err <= TOL_F32
    got16 = module.gemv(x.cuda(), variant=5)
    assert got16.dtype == torch.bfloat16 and torch.equal(got16, got.bfloat16())  # one rounding at the end


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [3, 24, 64])
def test_long_runs_of_groups_per_cta(bits, M):
    """Enough row tiles to fill the GPU, so a CTA walks all 40 scale groups of its rows by itself
    and every ring of the kernel wraps several times."""
    n, k = 19072, 5120
    w = seeded((n, k), 81, 0.02, torch.bfloat16)
    x = seeded((M, k), 82).bfloat16()
    module = _module(w, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, variant=5)
    _no_device_error()
    assert rel_l2(got.cpu().numpy(), _want(w, x, bits)) <= TOL_F32


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [12, 24, 64])
def test_weights_not_in_cache(bits, M):
    """The same product with the weights evicted from L2 before every call (256 MB written in
    between). Then the weight side sets the pace, the activation planes wait in their ring, and
    a slot is handed back to the copy thread the moment its group has been drained: the regime
    in which a drain warp once read the units of a later group. The tokens here have groups
    whose unit differs from their neighbours', which is what makes a stale unit visible."""
    n, k = 19072, 5120
    w = seeded((n, k), 81, 0.02, torch.bfloat16)
    x = seeded((M, k), 82).bfloat16()
    module = _module(w, bits)
    want = _want(w, x, bits)
    evict = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    xc = x.cuda()
    for round_ in range(6):
        evict.fill_(round_)
        got = module.gemv(xc, out_dtype=torch.float32, variant=5)
        _no_device_error()
        assert rel_l2(got.cpu().numpy(), want) <= TOL_F32, round_


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [2, 8, 12, 16, 17, 31, 33, 50, 64, 70, 130])
def test_every_padded_row_count(bits, M):
    """8, 16, 32 and 64 padded rows, and more rows than a call takes (64 per call)."""
    n, k = 272, 1024
    w = seeded((n, k), 31, 0.02, torch.bfloat16)
    x = seeded((M, k), 32).bfloat16()
    module = _module(w, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32, variant=5)
    _no_device_error()
    assert got.shape == (M, n)
    assert rel_l2(got.cpu().numpy(), _want(w, x, bits)) <= TOL_F32
    # a row's result does not depend on which other rows share the call
    alone = torch.cat([module.gemv(x[i:i + 1].cuda(), out_dtype=torch.float32, variant=5) for i in (0, M - 1)])
    assert torch.equal(got[[0, M - 1]], alone)
    # and more than 8 rows take this path by default
    if M > 8:
        assert torch.equal(module.gemv(x.cuda(), out_dtype=torch.float32), got)


@pytest.mark.parametrize("bits", [4, 8])
def test_agrees_with_the_gemv_variants(bits):
    """Same activations, same block floating point as the tensor-core GEMV (variant 4): the two
    differ only in the order of the fp32 sum over the groups."""
    n, k = 1024, 4096
    w = seeded((n, k), 51, 0.02, torch.bfloat16)
    x = seeded((8, k), 52).bfloat16().cuda()
    module = _module(w, bits)
    a = module.gemv(x, out_dtype=torch.float32, variant=5)
    b = module.gemv(x, out_dtype=torch.float32, variant=4)
    c = module.gemv(x, out_dtype=torch.float32, variant=3)
    assert rel_l2(a.cpu().numpy(), b.cpu().numpy()) <= 1e-5
    assert rel_l2(a.cpu().numpy(), c.cpu().numpy()) <= TOL_F32


@pytest.mark.parametrize("bits", [4, 8])
def test_outliers_and_zero_rows(bits):
    n, k = 128, 512
    w = seeded((n, k), 41, 0.02, torch.bfloat16)
    x = seeded((12, k), 42).bfloat16()
    x[0, 7] = 300.0
    x[1] = 0
    x[2, :128] = torch.tensor(1.9921875).bfloat16()  # (2 - 2^-7): the largest bf16 below 2
    x[3, 130] = -255.0
    module = _module(w, bits)
    got = module.gemv(x.cuda(), out_dtype=torch.float32)
    want = _want(w, x, bits)
    assert np.all(got[1].cpu().numpy() == 0)
    for row in (0, 2, 3, 11):
        assert rel_l2(got[row].cpu().numpy(), want[row]) <= TOL_F32, row
    # scaling the activations by a power of two scales the result exactly
    twice = module.gemv((x * 2).cuda(), out_dtype=torch.float32)
    assert torch.equal(twice, got * 2)
    _no_device_error()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [9, 32, 64])
def test_fused_options(bits, M):
    """RMSNorm prologue, bias, residual (bf16 and fp32) and the silu(gate) * up epilogue against
    the numpy restatement of the bf16 modules, dependent launches on."""
    k, n = 2048, 528
    w = seeded((n, k), 1, 0.02, torch.bfloat16)
    bias = seeded((n,), 5, 0.1, torch.bfloat16)
    x = (seeded((M, k), 2) * 3).bfloat16()
    gamma = (seeded((k,), 3) * 0.1 + 1).bfloat16()
    normed = llama_ops.rmsnorm(x.float().numpy(), gamma.float().numpy(), 1e-5)
    module = _module(w, bits, bias=bias)
    want = _want(w, torch.from_numpy(normed), bits) + bias.float().numpy()
    got = module.gemv(x.cuda(), out_dtype=torch.float32, norm_weight=gamma.cuda(), norm_eps=1e-5, pdl=True)
    assert rel_l2(got.cpu().numpy(), want) <= TOL_F32
    res = seeded((M, n), 7).bfloat16().cuda()
    with_res = module.gemv(x.cuda(), norm_weight=gamma.cuda(), norm_eps=1e-5, residual=res, pdl=True)
    assert torch.equal(with_res, (got.bfloat16().float() + res.float()).bfloat16())  # round, add, round
    res32 = seeded((M, n), 8).cuda()
    assert torch.equal(module.gemv(x.cuda(), out_dtype=torch.float32, norm_weight=gamma.cuda(), norm_eps=1e-5,
                                   residual=res32), got + res32)
    # gate | up interleaved
    plain = _module(w, bits)
    g_u = plain.gemv(x.cuda(), out_dtype=torch.float32, norm_weight=gamma.cuda(), norm_eps=1e-5)
    act = plain.gemv(x.cuda(), norm_weight=gamma.cuda(), norm_eps=1e-5, epilogue=1, pdl=True)
    want_act = llama_ops.silu_mul(g_u[:, 0::2].bfloat16().float().cpu().numpy(), g_u[:, 1::2].bfloat16().float().cpu().numpy())
    assert act.shape == (M, n // 2) and rel_l2(act.float().cpu().numpy(), want_act) <= 2e-3
    _no_device_error()


def test_other_group_sizes_fall_back_and_bad_workspaces_are_refused():
    w = seeded((256, 512), 61, 0.02, torch.bfloat16)
    x = seeded((12, 512), 62).bfloat16().cuda()
    module = _module(w, 8, group=64)  # 64-wide groups: row blocks through the GEMV
    q, scale = oracle.quantize_weight(w.float().numpy(), 8, 64)
    want = oracle.real_linear(x.float().cpu().numpy(), q, scale, 8, 64)
    assert rel_l2(module.gemv(x, out_dtype=torch.float32).cpu().numpy(), want) <= TOL_F32
    with pytest.raises(RuntimeError, match="scale groups of 128"):
        module.gemv(x, variant=5)
    module = _module(w, 8)
    with pytest.raises(ValueError, match="workspace"):
        module.gemv(x, workspace=torch.zeros(256, dtype=torch.uint8, device="cuda"))
    big = torch.zeros(module.decode_workspace_bytes(12) + 256, dtype=torch.uint8, device="cuda")
    a = module.gemv(x, out_dtype=torch.float32, workspace=big)
    assert torch.equal(a, module.gemv(x, out_dtype=torch.float32))
