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


class _StubTokenizer:
    vocab_size, eos_token_id = 512, 1


def test_reference_latency_harness_measures_this_librarys_graphed_int8_decode(ref):
    """The reference's `measure_latency` (llmquant/eval/evaluate.py:167-223) -- the body of its
    run.py latency report -- called as it is, on a model quantized by THIS library with THIS
    library's integer cache factory, its `llmquant.runtime` graph entry points replaced by
    this library's: `can_graph` admits the integer cache, so the harness times the fused
    graphed decoder; without graphs it drives transformers' generate with the integer cache."""
    import llmquant.runtime as ref_runtime
    from llmquant.eval.evaluate import measure_latency

    from llmquant_b200.core import QuantConfig, oneshot
    from llmquant_b200.quantizers import make_cache_factory
    from llmquant_b200.runtime import can_graph, graphed_generate
    from oracle.real_mode import tiny_llama

    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(tiny_llama(seed=0, head_dim=64).cuda(), cfg.to_modifier(mode="kernel"))
    saved = (ref_runtime.can_graph, ref_runtime.graphed_generate)
    ref_runtime.can_graph, ref_runtime.graphed_generate = can_graph, graphed_generate
    try:
        row = measure_latency(model, _StubTokenizer(), prompt_tokens=48, new_tokens=8, iters=1,
                              cache_factory=make_cache_factory(8), use_cuda_graph=True)
        assert row["cuda_graph"] is True and row["decode_tps"] > 0 and row["ttft_ms"] > 0
        assert model.__dict__["_graph_kv_cache_bits"] == 8
        eager = measure_latency(model, _StubTokenizer(), prompt_tokens=48, new_tokens=8, iters=1,
                                cache_factory=make_cache_factory(8), use_cuda_graph=False)
        assert eager["cuda_graph"] is False and eager["decode_tps"] > 0
    finally:
        ref_runtime.can_graph, ref_runtime.graphed_generate = saved


def _save_tokenizer(directory):
    """A word-level tokenizer with a chat template, made offline (no checkpoint on this machine)."""
    from tokenizers import Tokenizer, models, pre_tokenizers
    from transformers import PreTrainedTokenizerFast

    vocab = {"<unk>": 0, "<eos>": 1, "system": 2, "user": 3, "assistant": 4}
    vocab.update({f"w{i}": i for i in range(5, 512)})
    tok = Tokenizer(models.WordLevel(vocab, unk_token="<unk>"))
    tok.pre_tokenizer = pre_tokenizers.Whitespace()
    fast = PreTrainedTokenizerFast(tokenizer_object=tok, unk_token="<unk>", eos_token="<eos>", pad_token="<eos>")
    fast.chat_template = ("{% for m in messages %}{{ m['role'] }} {{ m['content'] }} {% endfor %}"
                          "{% if add_generation_prompt %}assistant {% endif %}")
    fast.save_pretrained(directory)


def test_chat_on_a_packed_file_with_the_reference_session_and_with_this_librarys(ref, tmp_path):
    """`examples/chat.py --load-packed` in two ways: the reference's `load_for_chat` +
    `ChatSession` (its own modules on this library's kernels) reading a file THIS library
    wrote, and this library's `load_for_chat` + `ChatSession` on the same file. Both carry the
    integer KV cache across turns."""
    from llmquant.runtime.chat import ChatSession as RefSession
    from llmquant.runtime.chat import load_for_chat as ref_load_for_chat

    from llmquant_b200.core import QuantConfig, oneshot
    from llmquant_b200.packing import save_packed_model
    from llmquant_b200.quantizers import KernelQuantCache
    from llmquant_b200.runtime import ChatSession, load_for_chat
    from oracle.real_mode import tiny_llama

    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(tiny_llama(seed=0, head_dim=64).cuda(), cfg.to_modifier(mode="kernel"))
    model_id = tmp_path / "tiny-llama"
    model.config.save_pretrained(model_id)
    _save_tokenizer(model_id)
    path = save_packed_model(model, tmp_path / "model.bin", str(model_id), kv_cache_bits=8)

    ours_model, ours_tok, ours_factory = load_for_chat(str(path))
    assert isinstance(ours_factory(), KernelQuantCache)
    session = ChatSession(ours_model, ours_tok, max_new_tokens=6, cache_factory=ours_factory)
    first = session.ask("w7 w8 w9")
    second = session.ask("w10 w11")
    assert len(session.history) == 4 and len(session.last_reply_ids) == 6 and session._cache is not None
    assert session._cache.get_seq_length() > 10  # the cache was carried across the turns

    ref_model, ref_tok, ref_factory = ref_load_for_chat(str(path))
    ref_session = RefSession(ref_model, ref_tok, max_new_tokens=6, cache_factory=ref_factory)
    ref_first, ref_second = ref_session.ask("w7 w8 w9"), ref_session.ask("w10 w11")
    # (both are greedy decodes of the same weights; on a random-init model a near-tie may send
    # them different ways, so only the shape of the conversation is compared)
    assert len(ref_session.last_reply_ids) == 6 and len(ref_session.history) == 4
    assert all(isinstance(r, str) and r for r in (first, second, ref_first, ref_second))
    # a context limit drops whole turns and the stale cache with them
    tight = ChatSession(ours_model, ours_tok, max_new_tokens=6, cache_factory=ours_factory,
                        max_context_tokens=24, system_prompt=None)
    for turn in range(4):
        tight.ask("w20 w21 w22")
    assert len(tight.history) < 8
