"""The fused decoder on the random-init Llama-3.2-1B-shaped model (16 layers, 128256-word
vocabulary, 512-token prompt, 64 new tokens) against the reference's own real-mode run of the
same seeded model (tests/golden/llama_1b.npz, made by tests/golden/make_golden_1b.py).

Teacher-forced with the reference's tokens, every step's logits must agree within rel-L2
2e-2 (two bf16 pipelines that round at every layer boundary, summing in different orders) and
the argmax must agree wherever the reference's top-2 margin exceeds the numeric noise.
Free-running, the token stream must be the reference's up to the first step whose margin is
inside that noise; the index of the first difference is printed."""

import importlib.util
import pathlib

import numpy as np
import pytest
import torch

from gpu_util import rel_l2
from llmquant_b200.core import QuantConfig, oneshot

pytestmark = pytest.mark.gpu


def _generator_module():
    path = pathlib.Path(__file__).resolve().parent / "golden" / "make_golden_1b.py"
    spec = importlib.util.spec_from_file_location("make_golden_1b", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.timeout(1500)
def test_llama_1b_logits_and_greedy_stream_against_the_reference(golden):
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from oracle.real_mode import tiny_llama

    gen = _generator_module()
    blob = golden("llama_1b")
    tokens = torch.from_numpy(blob["tokens"].astype(np.int64)).cuda()
    n_prompt, new = gen.PROMPT, gen.NEW
    assert tokens.shape == (1, n_prompt + new)
    assert np.array_equal(blob["tokens"][:, :n_prompt], gen.prompt_ids().numpy())
    sub = torch.from_numpy(blob["subset_index"].astype(np.int64)).cuda()
    top_idx = torch.from_numpy(blob["top_index"].astype(np.int64)).cuda()

    model = tiny_llama(seed=0, **gen.LLAMA_1B).cuda()
    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    model = oneshot(model, cfg.to_modifier(mode="kernel"))
    dec = FusedLlamaDecoder(model, 1, n_prompt + new + 8, kv_bits=8)

    # ---- teacher-forced: the reference's token goes in at every step
    dec.prefill(tokens[:, :n_prompt])
    rows = [dec.logits[0].float().clone()]
    for i in range(1, new):
        dec.tokens.copy_(tokens[:, n_prompt + i - 1])
        dec.step()
        rows.append(dec.logits[0].float().clone())
    got = torch.stack(rows)  # [new, vocab]
    got_sub = got[:, sub].cpu().numpy()
    got_top = torch.gather(got, 1, top_idx).cpu().numpy()
    err = rel_l2(got_sub, blob["subset_logits"])
    norm_err = np.abs(got.norm(dim=-1).cpu().numpy() - blob["row_norm"]) / blob["row_norm"]
    assert err <= 2e-2, err
    assert norm_err.max() <= 2e-2
    noise = np.maximum(np.abs(got_sub - blob["subset_logits"]).max(-1), np.abs(got_top - blob["top_values"]).max(-1))
    margin = blob["top_values"][:, 0] - blob["top_values"][:, 1]
    decided = margin > 4 * noise
    same = got.argmax(-1).cpu().numpy() == blob["top_index"][:, 0]
    assert same[decided].all()
    first_undecided = int(np.argmin(decided)) if not decided.all() else new

    # ---- free-running greedy decode
    stream = dec.generate(tokens[:, :n_prompt], new).cpu().numpy()
    equal = stream[0, n_prompt:] == blob["tokens"][0, n_prompt:]
    first_difference = int(np.argmin(equal)) if not equal.all() else new
    print(f"LLAMA_1B teacher-forced rel-L2 {err:.3e}; decided steps {int(decided.sum())}/{new}; "
          f"first undecided step {first_undecided}; first free-running difference at token {first_difference} of {new}")
    assert first_difference >= first_undecided
