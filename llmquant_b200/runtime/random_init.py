"""Random-init Llama models quantized layer by layer on the GPU.

The benchmark configurations are random-init decoders of the Llama-3.2-1B and Llama-3-8B
shapes (there are no checkpoints to load). The model is created on the meta device and each
Linear is materialised, quantized into a `KernelQuantLinear` and dropped in turn, so the bf16
form of the whole model never exists -- the same peak-memory property the packed loader has
(llmquant/packing/model_io.py:157-231 of the reference).
"""

import torch
import torch.nn as nn

from llmquant_b200.core.config import QuantConfig

SHAPES = {
    "llama-3.2-1b": dict(hidden_size=2048, num_hidden_layers=16, num_attention_heads=32,
                         num_key_value_heads=8, head_dim=64, intermediate_size=8192,
                         vocab_size=128256, tie_word_embeddings=True),
    "llama-3-8b": dict(hidden_size=4096, num_hidden_layers=32, num_attention_heads=32,
                       num_key_value_heads=8, head_dim=128, intermediate_size=14336,
                       vocab_size=128256, tie_word_embeddings=False),
}


def llama_config(name: str, **overrides):
    from transformers import LlamaConfig

    kw = dict(SHAPES[name], rms_norm_eps=1e-5, max_position_embeddings=8192,
              rope_parameters={"rope_type": "default", "rope_theta": 500000.0},
              attention_bias=False, mlp_bias=False)
    kw.update(overrides)
    return LlamaConfig(**kw)


@torch.no_grad()
def random_quantized_llama(config, quant: QuantConfig, device="cuda", seed=0, std=0.02,
                           shard=None):
    """LlamaForCausalLM with every >= 2-D parameter ~ N(0, std) and the linears the config
    names swapped for KernelQuantLinear. `shard(name, weight)` may cut a weight before it is
    quantized (tensor parallelism)."""
    from transformers import LlamaForCausalLM

    modifier = quant.to_modifier(mode="kernel")
    with torch.device("meta"):
        model = LlamaForCausalLM(config)
    modifier.resolve(model)
    gen = torch.Generator(device=device).manual_seed(seed)
    from llmquant_b200.quantizers import KernelQuantLinear

    for name, module in list(model.named_modules()):
        if not isinstance(module, nn.Linear):
            continue
        scheme = modifier.scheme_for(name)
        weight = (torch.randn(module.weight.shape, generator=gen, device=device) * std).to(torch.bfloat16)
        if shard is not None:
            weight = shard(name, weight)
        if scheme is None:
            real = nn.Linear(weight.shape[1], weight.shape[0], bias=False, device=device, dtype=torch.bfloat16)
            real.weight.copy_(weight)
            new = real
        else:
            holder = nn.Linear(weight.shape[1], weight.shape[0], bias=False, device="meta")
            holder.weight = nn.Parameter(weight, requires_grad=False)
            new = KernelQuantLinear.from_linear(holder, scheme)
        parent, _, child = name.rpartition(".")
        setattr(model.get_submodule(parent) if parent else model, child, new)
        del weight
    for name, param in list(model.named_parameters()):
        if not param.is_meta:
            continue
        if param.dim() >= 2:
            data = (torch.randn(param.shape, generator=gen, device=device) * std).to(torch.bfloat16)
        else:
            data = torch.ones(param.shape, dtype=torch.bfloat16, device=device)
        parent, _, child = name.rpartition(".")
        setattr(model.get_submodule(parent) if parent else model, child,
                nn.Parameter(data, requires_grad=False))
    # non-persistent buffers (rotary inv_freq) were created on meta: rebuild the module
    model.model.rotary_emb = type(model.model.rotary_emb)(config, device=device)
    return model.eval()
