"""The REFERENCE's own modules running on this library.

`python oracle/make_ref.py` stages the reference package under oracle/_ref (git-ignored; it
travels with the working tree). Here its `llmquant.cuda.build.load_extension` -- the JIT build
of its three CUDA files -- is replaced by `llmquant_b200.cuda.load_extension`, which returns an
object with the same four callables, and the reference's `KernelQuantLinear`,
`fake_quantize_cuda` and cache factory then run unchanged on the sm_100a kernels. What the
reference's tests assert about them (tests/test_kernel_linear.py:49-59,
tests/test_cuda_kernel.py:28-43 of the reference) is asserted here against the reference's
`real` mode executed by the same imported package.

Skipped when the reference has not been staged."""

import sys

import pytest
import torch
import torch.nn as nn

from gpu_util import rel_l2
from oracle import make_ref

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not make_ref.available(), reason="the reference is not staged under oracle/_ref")]

K, N, HEAD_DIM = 2048, 512, 64


@pytest.fixture(scope="module")
def ref():
    """The staged reference with its extension loader pointed at this library."""
    make_ref.import_reference()
    import llmquant.cuda.build as ref_build
    import llmquant.cuda.ops as ref_ops
    import llmquant.quantizers.kernel as ref_kernel

    import llmquant_b200.cuda as ours

    saved = (ref_build.load_extension, ref_ops.load_extension, ref_kernel.load_extension)
    ref_build.load_extension = ref_ops.load_extension = ref_kernel.load_extension = ours.load_extension
    yield sys.modules["llmquant"]
    ref_build.load_extension, ref_ops.load_extension, ref_kernel.load_extension = saved


def _scheme(bits, **kw):
    from llmquant.core.scheme import GROUP_SIZE, QuantizationArgs, QuantizationScheme

    return QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=GROUP_SIZE, **kw),
        input_activations=None)


LAYOUTS = {"plain": (8, {}), "int4": (4, {}), "o_proj": (8, dict(head_dim=HEAD_DIM)),
           "q_proj": (8, dict(out_group=HEAD_DIM))}


@pytest.mark.parametrize("name", list(LAYOUTS))
@pytest.mark.parametrize("M", [1, 4])
def test_reference_kernel_linear_on_this_library_matches_its_real_mode(ref, name, M):
    from llmquant.quantizers import KernelQuantLinear, RealQuantLinear

    bits, kw = LAYOUTS[name]
    scheme = _scheme(bits, **kw)
    torch.manual_seed(0)
    linear = nn.Linear(K, N, bias=False).cuda().to(torch.bfloat16)
    x = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    module = KernelQuantLinear.from_linear(linear, scheme)
    assert module._gemv.__qualname__.startswith("_Kernels")  # this library's shim, not a JIT module
    got = module(x)
    want = RealQuantLinear.from_linear(linear, scheme)(x)
    assert got.shape == want.shape and got.dtype == want.dtype
    # same grouped integer arithmetic, fp32 partial sums added in another order: the bf16
    # results differ by at most one rounding step, almost everywhere not at all
    err = rel_l2(got.float().cpu().numpy(), want.float().cpu().numpy())
    assert err <= 2e-3, (name, err)
    assert (got == want).float().mean() > 0.9
    assert ((got.float() - want.float()).abs() <= 2 ** -7 * want.float().abs() + 1e-6).all()


def test_reference_fake_quantize_cuda_on_this_library_is_bit_exact(ref):
    from llmquant.core.quant_ops import fake_quantize
    from llmquant.core.scheme import QuantizationArgs
    from llmquant.cuda import fake_quantize_cuda

    for bits in (4, 8):
        for dtype in (torch.bfloat16, torch.float16, torch.float32):
            for shape in ((16, 128), (512, 2048), (2, 7, 2048)):
                torch.manual_seed(0)
                x = (torch.randn(*shape, device="cuda") * 3).to(dtype)
                args = QuantizationArgs(num_bits=bits, strategy="group", group_size=128)
                got, scale = fake_quantize_cuda(x, args, return_scale=True)
                assert torch.equal(got, fake_quantize(x, args)), (bits, dtype, shape)


def test_reference_prefill_branch_and_model_level_oneshot(ref):
    """Above its row threshold the reference dequantizes and calls the library GEMM (no
    extension involved); and its whole `oneshot(..., mode="kernel")` runs on this library:
    a tiny Llama quantized by the REFERENCE's modifier decodes like its real mode."""
    from llmquant.core import QuantConfig, oneshot
    from llmquant.quantizers import KernelQuantLinear, make_cache_factory

    from oracle.real_mode import greedy, tiny_llama

    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    kernel_model = oneshot(tiny_llama(seed=0, head_dim=64).cuda(), cfg.to_modifier(mode="kernel"))
    real_model = oneshot(tiny_llama(seed=0, head_dim=64).cuda(), cfg.to_modifier(mode="real"))
    assert isinstance(kernel_model.model.layers[0].self_attn.q_proj, KernelQuantLinear)
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, 512, (1, 24), generator=g).cuda()
    toks_k, logits_k = greedy(kernel_model, prompt, 8, cache=make_cache_factory(8)())
    toks_r, logits_r = greedy(real_model, prompt, 8, cache=make_cache_factory(8)())
    assert rel_l2(logits_k.cpu().numpy(), logits_r.cpu().numpy()) <= 2e-2
