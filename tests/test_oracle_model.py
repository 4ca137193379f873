"""The torch restatement of real mode + fake-quant KV (oracle/real_mode.py) against the
reference's own run of the same seeded tiny Llama (tests/golden/tiny_llama.npz)."""

import numpy as np
import pytest
import torch

from oracle.real_mode import FakeQuantKV, apply_real_mode, greedy, tiny_llama


@pytest.mark.parametrize("tag,kw", [("hd64", dict(head_dim=64)),
                                    ("hd128", dict(head_dim=128, hidden=512, inter=1024))])
def test_real_mode_model_reproduces_the_reference(golden, tag, kw):
    blob = golden("tiny_llama")
    model = apply_real_mode(tiny_llama(seed=0, **kw), attn_bits=8, mlp_bits=4, head_bits=8)
    prompt = torch.from_numpy(blob[f"{tag}_prompt"])
    tokens, logits = greedy(model, prompt, 32, cache=FakeQuantKV(8))
    assert np.array_equal(tokens.numpy(), blob[f"{tag}_tokens"])
    assert np.array_equal(logits.numpy(), blob[f"{tag}_logits"])
