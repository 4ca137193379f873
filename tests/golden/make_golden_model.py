"""Generate tests/golden/tiny_llama.npz: greedy tokens and logits of a random-init tiny
Llama quantized by the REFERENCE in `real` mode with its FakeQuantCache(8), on CPU.

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden_model.py /path/to/llm-quant

The model is built by oracle.real_mode.tiny_llama (seeded, no checkpoint involved).
"""

import pathlib
import sys

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))


def main(ref_root):
    sys.path.insert(0, ref_root)
    sys.dont_write_bytecode = True
    from llmquant.core import QuantConfig, oneshot
    from llmquant.quantizers import make_cache_factory

    from oracle.real_mode import greedy, tiny_llama

    out = {}
    for tag, kw in (("hd64", dict(head_dim=64)), ("hd128", dict(head_dim=128, hidden=512, inter=1024))):
        model = tiny_llama(seed=0, **kw)
        cfg = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
        oneshot(model, cfg.to_modifier(mode="real"))
        g = torch.Generator().manual_seed(1)
        prompt = torch.randint(0, model.config.vocab_size, (2, 24), generator=g)
        tokens, logits = greedy(model, prompt, 32, cache=make_cache_factory(8)())
        out[f"{tag}_prompt"] = prompt.numpy()
        out[f"{tag}_tokens"] = tokens.numpy()
        out[f"{tag}_logits"] = logits.numpy().astype(np.float32)
    np.savez_compressed(HERE / "tiny_llama.npz", **out)
    print("written", HERE / "tiny_llama.npz")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: python %s <path to an llm-quant checkout>" % sys.argv[0])
    main(sys.argv[1])
