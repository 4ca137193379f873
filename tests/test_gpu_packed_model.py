"""Whole models through the file and the reference-named runtime entry points:

* a tiny Llama: `oneshot` -> `save_packed_model` -> `load_packed_model` (its config found
  through a local directory as `model_id`, as the reference's own tests do,
  tests/test_moe.py:142-147) -> bit-identical logits; `graphed_generate` with the integer KV
  cache and on the transformers StaticCache route (`GraphedDecoder`), `can_graph`;
* a tiny Mixtral: the modifier swaps the stacked expert block, the file carries an `experts`
  record, the model reloads bit-identically (reference: tests/test_moe.py:162-171);
* and, when the reference is staged under oracle/_ref, the REFERENCE's `load_packed_model`
  reads the file this library wrote and its `save_packed_model` writes it back: the bytes
  must be identical, for both models."""

import pathlib

import numpy as np
import pytest
import torch

from gpu_util import rel_l2
from llmquant_b200.core import QuantConfig, oneshot
from oracle import make_ref

pytestmark = pytest.mark.gpu


def _tiny_llama():
    from oracle.real_mode import tiny_llama

    return tiny_llama(seed=0, head_dim=64).cuda()


def _tiny_mixtral():
    from transformers import MixtralConfig, MixtralForCausalLM

    torch.manual_seed(0)
    cfg = MixtralConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=8,
                        num_key_value_heads=4, vocab_size=1000, num_local_experts=4, num_experts_per_tok=2,
                        max_position_embeddings=512)
    return MixtralForCausalLM(cfg).to(torch.bfloat16).cuda().eval()


def _reference_rewrites_the_same_bytes(path, workdir):
    """The staged reference, its extension loader pointed at this library, loads `path` and
    saves it again; returns the bytes it wrote (None when the reference is not staged)."""
    if not make_ref.available():
        return None
    make_ref.import_reference()
    import llmquant.cuda.build as ref_build
    import llmquant.cuda.ops as ref_ops
    import llmquant.quantizers.kernel as ref_kernel
    from llmquant.packing import load_packed_model as ref_load
    from llmquant.packing import read_header as ref_header
    from llmquant.packing import save_packed_model as ref_save

    import llmquant_b200.cuda as ours

    saved = (ref_build.load_extension, ref_ops.load_extension, ref_kernel.load_extension)
    ref_build.load_extension = ref_ops.load_extension = ref_kernel.load_extension = ours.load_extension
    try:
        meta = ref_header(path)["meta"]
        model = ref_load(path, device="cuda")
        again = pathlib.Path(workdir) / "rewritten.bin"
        ref_save(model, again, meta["model_id"], kv_cache_bits=meta.get("kv_cache_bits"))
        return again.read_bytes(), model
    finally:
        ref_build.load_extension, ref_ops.load_extension, ref_kernel.load_extension = saved


def test_llama_round_trip_and_graphed_generation(tmp_path):
    from llmquant_b200.packing import describe_packed, load_packed_model, packed_dtypes, save_packed_model
    from llmquant_b200.quantizers import KernelQuantLinear, make_cache_factory
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from llmquant_b200.runtime.graph_decode import GraphedDecoder, can_graph, graphed_generate

    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(_tiny_llama(), cfg.to_modifier(mode="kernel"))
    model_id = tmp_path / "tiny-llama"
    model.config.save_pretrained(model_id)
    path = save_packed_model(model, tmp_path / "model.bin", str(model_id), kv_cache_bits=8)
    assert packed_dtypes(path) == {"attn_weight": "int8", "mlp_weight": "int4", "head_weight": "int8",
                                   "kv_cache": "int8", "activation": "bf16"}
    assert describe_packed(path)["quantized_layers"] == 2 * 7 + 1

    loaded = load_packed_model(path, device="cuda")
    assert isinstance(loaded.model.layers[1].mlp.down_proj, KernelQuantLinear)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 512, (2, 24), generator=g).cuda()
    with torch.no_grad():
        assert torch.equal(model(ids).logits, loaded(ids).logits)
        assert torch.equal(model(ids[:, :1]).logits, loaded(ids[:, :1]).logits)  # the decode GEMV path

    # ---- the reference-named graph entry points
    assert can_graph(loaded) and can_graph(loaded, make_cache_factory(8))
    assert not can_graph(loaded.cpu() if False else torch.nn.Linear(2, 2))  # nothing on a GPU: refused
    new = 12
    tokens = graphed_generate(loaded, ids, new, kv_cache_bits=8)
    direct = FusedLlamaDecoder(model, 2, ids.shape[1] + new + 1, kv_bits=8).generate(ids, new)
    assert tokens.shape == (2, ids.shape[1] + new) and torch.equal(tokens, direct)

    # bf16 KV on transformers' StaticCache (the reference's own route): every graphed step
    # against the eager model fed the same tokens
    bf16_tokens = graphed_generate(loaded, ids[:1], new)
    assert bf16_tokens.shape == (1, ids.shape[1] + new)
    dec = GraphedDecoder(loaded, ids.shape[1], new, batch=1)
    nxt = dec.prefill(ids[:1])
    with torch.no_grad():
        eager = loaded(ids[:1], use_cache=True)
    assert torch.equal(nxt.reshape(-1), eager.logits[:, -1].argmax(-1))
    dec.token.copy_(nxt)
    dec.capture(ids.shape[1])
    cache = eager.past_key_values
    feed = nxt
    for i in range(1, 6):
        got = dec.step(feed, ids.shape[1] + i - 1)
        with torch.no_grad():
            out = loaded(feed.reshape(1, 1), past_key_values=cache, use_cache=True)
        err = rel_l2(dec.logits[:, -1].float().cpu().numpy(), out.logits[:, -1].float().cpu().numpy())
        assert err <= 1e-2, (i, err)
        feed = out.logits[:, -1:].argmax(-1)
        if torch.equal(got.reshape(-1), feed.reshape(-1)) is False:
            top2 = out.logits[0, -1].float().topk(2).values
            assert float(top2[0] - top2[1]) < 0.05  # only a near-tie may decide differently
    assert torch.equal(bf16_tokens[:, : ids.shape[1] + 1], torch.cat([ids[:1], nxt.reshape(1, 1)], 1))

    rewritten = _reference_rewrites_the_same_bytes(path, tmp_path)
    if rewritten is not None:
        assert rewritten[0] == pathlib.Path(path).read_bytes()


def test_mixture_of_experts_through_oneshot_file_and_reload(tmp_path):
    from llmquant_b200.packing import describe_packed, load_packed_model, read_header, save_packed_model
    from llmquant_b200.quantizers import KernelQuantExperts, KernelQuantLinear

    model = _tiny_mixtral()
    gate_before = model.model.layers[0].mlp.gate.weight.data.clone()
    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8")
    oneshot(model, cfg.to_modifier(mode="kernel"))
    block = model.model.layers[0].mlp.experts
    assert isinstance(block, KernelQuantExperts) and block.qgate_up.dtype == torch.int8
    assert isinstance(model.model.layers[0].self_attn.q_proj, KernelQuantLinear)
    assert torch.equal(model.model.layers[0].mlp.gate.weight.data, gate_before)  # the router stays as it is
    ids = torch.randint(0, 1000, (1, 8), device="cuda")
    with torch.no_grad():
        before = model(ids).logits.float()
        before_one = model(ids[:, :1]).logits.float()
    model_id = tmp_path / "tiny-mixtral"
    model.config.save_pretrained(model_id)
    path = save_packed_model(model, tmp_path / "moe.bin", str(model_id))
    meta = read_header(path)["meta"]
    assert sorted(meta["experts"]) == ["model.layers.0.mlp.experts", "model.layers.1.mlp.experts"]
    spec = meta["experts"]["model.layers.0.mlp.experts"]
    assert spec["num_experts"] == 4 and spec["gate_up_shape"] == [4, 1024, 2, 128]
    stored = set(read_header(path)["tensors"])
    assert {"model.layers.0.mlp.experts.qgate_up", "model.layers.0.mlp.experts.sdown"} <= stored
    assert not any(n.endswith(("_gemv", "gate_up_proj")) for n in stored)
    assert describe_packed(path)["expert_blocks"] == 2

    loaded = load_packed_model(path, device="cuda")
    assert isinstance(loaded.model.layers[1].mlp.experts, KernelQuantExperts)
    with torch.no_grad():
        assert torch.equal(before, loaded(ids).logits.float())
        assert torch.equal(before_one, loaded(ids[:, :1]).logits.float())

    rewritten = _reference_rewrites_the_same_bytes(path, tmp_path)
    if rewritten is not None:
        assert rewritten[0] == pathlib.Path(path).read_bytes()
        with torch.no_grad():
            ref_logits = rewritten[1](ids).logits.float()
        assert rel_l2(ref_logits.cpu().numpy(), before.cpu().numpy()) <= 2e-2
