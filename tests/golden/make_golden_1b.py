"""Generate tests/golden/llama_1b.npz: the REFERENCE's `real`-mode greedy run of the random-init
Llama-3.2-1B-shaped decoder (16 layers, hidden 2048, 32 query / 8 KV heads of 64, FFN 8192,
vocabulary 128256, tied embedding, weights ~ N(0, 0.02) from a seed; attention int8, MLP int4,
lm_head int8 as an untied copy, FakeQuantCache(8)) on a 512-token uniform-random prompt, 64
new tokens, on CPU.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_1b.py /path/to/llm-quant

The full logits would be 33 MB, so the fixture keeps, per generated position: the logits at
1024 fixed vocabulary indices (chosen by a seed), the 16 largest logits with their indices,
and the norm of the full row -- enough for a relative error, the argmax and the top-2 margin.
The model is rebuilt from the same seed by the test (oracle.real_mode.tiny_llama).
"""

import pathlib
import sys
import time

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

LLAMA_1B = dict(hidden=2048, layers=16, heads=32, kv_heads=8, head_dim=64, inter=8192,
                vocab=128256, tie=True)
PROMPT, NEW, SUBSET, TOPK = 512, 64, 1024, 16


def prompt_ids():
    g = torch.Generator().manual_seed(1)
    return torch.randint(0, LLAMA_1B["vocab"], (1, PROMPT), generator=g)


def subset_indices():
    g = torch.Generator().manual_seed(2)
    return torch.randperm(LLAMA_1B["vocab"], generator=g)[:SUBSET].sort().values


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from llmquant.core import QuantConfig, oneshot
    from llmquant.quantizers import make_cache_factory

    from oracle.real_mode import greedy, tiny_llama

    t0 = time.time()
    model = tiny_llama(seed=0, **LLAMA_1B)
    cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    oneshot(model, cfg.to_modifier(mode="real"))
    print(f"model ready after {time.time() - t0:.0f} s", flush=True)
    tokens, logits = greedy(model, prompt_ids(), NEW, cache=make_cache_factory(8)())
    logits = logits[0]  # [NEW, vocab] fp32
    idx = subset_indices()
    top = logits.topk(TOPK, dim=-1)
    np.savez_compressed(
        HERE / "llama_1b.npz",
        tokens=tokens.numpy().astype(np.int32),
        subset_index=idx.numpy().astype(np.int32),
        subset_logits=logits[:, idx].numpy().astype(np.float32),
        top_values=top.values.numpy().astype(np.float32),
        top_index=top.indices.numpy().astype(np.int32),
        row_norm=logits.norm(dim=-1).numpy().astype(np.float32),
    )
    print(f"written {HERE / 'llama_1b.npz'} after {time.time() - t0:.0f} s")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path to an llm-quant checkout>" % sys.argv[0])
    main(sys.argv[1])
