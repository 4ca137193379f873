"""The tcgen05/TMEM prefill GEMM against the reference's real mode: golden outputs for the
four weight layouts with bf16 activations (A16) and with dynamic int8 activations (A8), and
the numpy oracle at ragged larger shapes. Tolerance: rel-L2 <= 2e-3 (bf16 output vs fp32
reference), the bound stated for layer outputs."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import bf16_from_bits, index_of, rel_l2, seeded
from llmquant_b200 import native
from llmquant_b200.core import QuantizationArgs, QuantizationScheme

pytestmark = pytest.mark.gpu

LAYOUTS = ["plain8", "plain4", "oproj8", "oproj4", "qproj8", "tail4"]
TOL = 2e-3


def _module(w, bits, **kw):
    from llmquant_b200.quantizers import KernelQuantLinear

    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128, **kw),
        input_activations=None)
    linear = torch.nn.Linear(w.shape[1], w.shape[0], bias=False)
    linear.weight.data = w
    return KernelQuantLinear.from_linear(linear.cuda(), scheme)


@pytest.mark.parametrize("name", LAYOUTS)
@pytest.mark.parametrize("act", [16, 8])
def test_prefill_gemm_against_real_mode_golden(golden, name, act):
    blob = golden("linear")
    spec = next(c for c in index_of(blob) if c["name"] == name)
    w = bf16_from_bits(blob[f"{name}_w"], "cpu")
    module = _module(w, spec["bits"], head_dim=spec.get("head_dim"), out_group=spec.get("out_group"))
    for M in (1, 4):
        x = bf16_from_bits(blob[f"{name}_x{M}"])
        got = module.gemm(x, a8=(act == 8))
        want = blob[f"{name}_y{M}_a{act}_f32"]
        assert got.shape == want.shape and got.dtype == torch.bfloat16
        assert rel_l2(got.float().cpu().numpy(), want) <= TOL, (name, act, M)
    assert native.library().lq_gemm_device_error() == 0


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(200, 300, 512), (16, 4096, 4096), (129, 1024, 1152), (512, 2048, 2048)])
def test_prefill_gemm_against_oracle(bits, shape):
    m, n, k = shape
    w = seeded((n, k), 11, 0.02, torch.bfloat16)
    x = seeded((m, k), 12, 1.0, torch.bfloat16)
    module = _module(w, bits)
    q, scale = oracle.quantize_weight(w.float().numpy(), bits, 128)
    want16 = oracle.real_linear(x.float().numpy(), q, scale, bits, 128)
    want8 = oracle.real_linear(x.float().numpy(), q, scale, bits, 128, act_bits=8)
    got16 = module.gemm(x.cuda())
    got8 = module.gemm(x.cuda(), a8=True)
    assert rel_l2(got16.float().cpu().numpy(), want16) <= TOL
    assert rel_l2(got8.float().cpu().numpy(), want8) <= TOL
    # the unpipelined kernel (the one groups of 64 stored codes always take) on the same product
    for a8, want in ((True, want8), (False, want16)):
        serial = module.gemm(x.cuda(), a8=a8, serial=True)
        assert rel_l2(serial.float().cpu().numpy(), want) <= TOL, ("serial", a8)
    assert rel_l2(module.gemm(x.cuda(), fold_scales=True, serial=True).float().cpu().numpy(), want16) <= TOL
    # the prefill path and the decode GEMV agree on the same rows
    rows = module.gemv(x[:4].cuda())
    assert rel_l2(got16[:4].float().cpu().numpy(), rows.float().cpu().numpy()) <= TOL
    assert native.library().lq_gemm_device_error() == 0


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("shape", [(200, 300, 512), (48, 4096, 4096), (96, 4096, 4096), (129, 1024, 1152), (600, 2048, 2048)])
def test_folded_scale_gemm_is_the_reference_kernel_mode_product(bits, shape):
    """With the scales folded into the operand the kernel multiplies by bf16(code * scale): the
    tensor the reference's kernel mode dequantizes (quantizers/kernel.py:68-79) before its
    library GEMM. Compared with exactly that product in fp32, and with the real-mode oracle at
    the looser bound the weights' bf16 rounding (2^-9 per weight) implies."""
    m, n, k = shape
    w = seeded((n, k), 21, 0.02, torch.bfloat16)
    x = seeded((m, k), 22, 1.0, torch.bfloat16)
    module = _module(w, bits)
    got = module.gemm(x.cuda(), fold_scales=True).float().cpu().numpy()
    q, scale = oracle.quantize_weight(w.float().numpy(), bits, 128)
    groups = scale.shape[1]
    padded = np.zeros((n, groups * 128), dtype=np.float32)
    padded[:, :k] = q
    dense = (padded.reshape(n, groups, 128) * scale.reshape(n, groups, 1).astype(np.float32)).reshape(n, -1)
    dense = torch.from_numpy(dense).bfloat16().float()[:, :k]
    same = (x.float() @ dense.T).numpy()
    assert rel_l2(got, same) <= 2.5e-3            # only the bf16 rounding of the output and the sum order differ
    assert rel_l2(got, oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(same))) <= 4e-4
    want = oracle.real_linear(x.float().numpy(), q, scale, bits, 128)
    assert rel_l2(got, want) <= 4e-3
    # the module's forward takes this path above FORWARD_DECODE_GEMM_MAX_ROWS (up to which the decode GEMM
    # keeps the exact per-group arithmetic) and up to PREFILL_TENSOR_CORE_MAX_ROWS rows when the
    # output is wide enough to fill the GPU, and the same bf16 weights through the library GEMM
    # otherwise
    from llmquant_b200.quantizers import kernel as kq

    fwd = module(x.cuda())
    if kq.FORWARD_DECODE_GEMM_MAX_ROWS < m <= kq.PREFILL_TENSOR_CORE_MAX_ROWS and n >= kq.PREFILL_TENSOR_CORE_MIN_FEATURES:
        assert torch.equal(fwd, module.gemm(x.cuda(), fold_scales=True))
    elif m <= kq.FORWARD_DECODE_GEMM_MAX_ROWS:
        assert rel_l2(fwd.float().cpu().numpy(), want) <= 2e-3  # exact integer sums, bf16 output
    else:
        assert rel_l2(fwd.float().cpu().numpy(), got) <= 3e-3
    assert native.library().lq_gemm_device_error() == 0
