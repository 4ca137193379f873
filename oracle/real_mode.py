"""Whole-model oracle: a transformers Llama with the reference's `real`-mode linears and its
fake-quantizing KV cache, restated with torch CPU ops. TEST INFRASTRUCTURE ONLY.

`RealLinear` follows llmquant/quantizers/real.py:50-103 (per-group fp32 matmul of
integer-valued operands, scaled and accumulated in group order); `FakeQuantKV` follows
llmquant/quantizers/fake.py:39-55; `apply_real_mode` follows the targeting rules of
llmquant/core/modifier.py:152-199 for a QuantConfig-style choice of bit widths. The
arithmetic inside goes through the numpy-pinned rules of oracle/quant_oracle.py, expressed
in torch so that a model forward stays fast enough.

Parity status: pinned by tests/golden/tiny_llama.npz, produced by the reference itself.
"""

import re

import torch
import torch.nn as nn
from transformers.cache_utils import DynamicCache


def _group_view(x, gs, head_dim=None):
    def pad(t):
        rem = t.shape[-1] % gs
        return t if not rem else nn.functional.pad(t, (0, gs - rem))

    if head_dim is None:
        p = pad(x)
        return p.reshape(*p.shape[:-1], p.shape[-1] // gs, gs)
    lead, k = x.shape[:-1], x.shape[-1]
    per_head = pad(x.reshape(*lead, k // head_dim, head_dim))
    return per_head.reshape(*lead, -1, gs)


def _ungroup(y, shape, gs, head_dim=None):
    lead, k = tuple(shape[:-1]), shape[-1]
    if head_dim is None:
        return y.reshape(*lead, -1)[..., :k]
    padded = -(-head_dim // gs) * gs
    return y.reshape(*lead, k // head_dim, padded)[..., :head_dim].reshape(*lead, k)


def _scale(x, bits, gs, head_dim=None, out_group=None):
    qmax = torch.tensor(float(2 ** (bits - 1) - 1), dtype=torch.float32)
    view = _group_view(x.float(), gs, head_dim)
    if out_group:
        n = view.shape[0]
        rem = n % out_group
        if rem:
            view = nn.functional.pad(view, [0, 0] * (view.dim() - 1) + [0, out_group - rem])
        amax = view.reshape(-1, out_group, *view.shape[1:]).abs().amax(dim=(1, -1), keepdim=True)
    else:
        amax = view.abs().amax(dim=-1, keepdim=True)
    return (amax / qmax).clamp(min=1e-8)


def _quantize(x, scale, bits):
    qmax = 2 ** (bits - 1) - 1
    return torch.clamp(torch.round(x.float() / scale), -qmax - 1, qmax)


def fake_quantize(x, bits, gs=128):
    scale = _scale(x, bits, gs)
    view = _group_view(x, gs)
    return _ungroup(_quantize(view, scale, bits) * scale, x.shape, gs).to(x.dtype)


class RealLinear(nn.Module):
    def __init__(self, linear, bits, gs=128, head_dim=None, out_group=None):
        super().__init__()
        w = linear.weight.detach()
        self.bits, self.gs, self.head_dim, self.out_group = bits, gs, head_dim, out_group
        scale = _scale(w, bits, gs, head_dim, out_group)
        grouped = _group_view(w, gs, head_dim)
        if out_group:
            n = grouped.shape[0]
            rem = n % out_group
            padded = nn.functional.pad(grouped, [0, 0] * (grouped.dim() - 1) + [0, out_group - rem]) if rem else grouped
            blocked = padded.reshape(-1, out_group, *grouped.shape[1:])
            q = _quantize(blocked, scale, bits).reshape(-1, *grouped.shape[1:])[:n]
        else:
            q = _quantize(grouped, scale, bits)
        self.register_buffer("qgroups", q.float().contiguous())  # [N, G, gs], integer-valued
        self.register_buffer("wscale", scale)
        self.bias = linear.bias
        self.out_features, self.in_features = w.shape

    def _group_scale(self, g):
        if self.out_group:
            return self.wscale[:, 0, g, 0].repeat_interleave(self.out_group)[: self.out_features]
        return self.wscale[:, g, 0]

    def forward(self, x):
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        xg = _group_view(flat.float(), self.gs, self.head_dim)
        out = torch.zeros(flat.shape[0], self.out_features, dtype=torch.float32)
        for g in range(self.qgroups.shape[1]):
            out += (xg[:, g] @ self.qgroups[:, g].T) * self._group_scale(g)
        if self.bias is not None:
            out = out + self.bias.float()
        return out.to(x.dtype).reshape(*shape[:-1], self.out_features)


class FakeQuantKV(DynamicCache):
    def __init__(self, bits, *args, **kwargs):
        super().__init__(*args, **kwargs)
        self.bits = bits

    def update(self, key_states, value_states, layer_idx, *args, **kwargs):
        return super().update(fake_quantize(key_states, self.bits),
                              fake_quantize(value_states, self.bits), layer_idx, *args, **kwargs)


def apply_real_mode(model, attn_bits=None, mlp_bits=None, head_bits=None, gs=128,
                    qkv_out_scale_per_head=True):
    cfg = model.config
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    swaps = []
    for name, module in model.named_modules():
        if type(module).__name__ != "Linear":
            continue
        if name == "lm_head":
            if head_bits:
                swaps.append((name, RealLinear(module, head_bits, gs)))
        elif re.match(r".*\.self_attn\..*_proj$", name) and attn_bits:
            if name.endswith("o_proj"):
                swaps.append((name, RealLinear(module, attn_bits, gs, head_dim=head_dim)))
            elif qkv_out_scale_per_head:
                swaps.append((name, RealLinear(module, attn_bits, gs, out_group=head_dim)))
            else:
                swaps.append((name, RealLinear(module, attn_bits, gs)))
        elif re.match(r".*\.mlp\..*_proj$", name) and mlp_bits:
            swaps.append((name, RealLinear(module, mlp_bits, gs)))
    for name, new in swaps:
        parent, _, child = name.rpartition(".")
        setattr(model.get_submodule(parent) if parent else model, child, new)
    return model


def tiny_llama(seed=0, hidden=256, layers=2, heads=4, kv_heads=2, head_dim=64, inter=512,
               vocab=512, tie=False):
    """A random-init Llama: every >= 2-D parameter ~ N(0, 0.02) from `seed`, norms at one."""
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(hidden_size=hidden, num_hidden_layers=layers, num_attention_heads=heads,
                      num_key_value_heads=kv_heads, head_dim=head_dim, intermediate_size=inter,
                      vocab_size=vocab, rms_norm_eps=1e-5, max_position_embeddings=2048,
                      rope_parameters={"rope_type": "default", "rope_theta": 500000.0},
                      tie_word_embeddings=tie, attention_bias=False, mlp_bias=False)
    with torch.device("meta"):
        model = LlamaForCausalLM(cfg)
    model = model.to_empty(device="cpu")
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for name, p in sorted(model.named_parameters()):
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g) * 0.02)
            else:
                p.fill_(1.0)
    # rotary buffers are non-persistent and were left uninitialised by to_empty()
    model.model.rotary_emb = type(model.model.rotary_emb)(cfg)
    if tie:
        model.tie_weights()
    return model.to(torch.bfloat16).eval()


@torch.no_grad()
def greedy(model, input_ids, new_tokens, cache=None):
    """Plain greedy loop; returns (tokens [B, prompt+new], last-position logits per step)."""
    out = model(input_ids, past_key_values=cache, use_cache=True)
    cache = out.past_key_values
    logits = [out.logits[:, -1].float()]
    tokens = [logits[-1].argmax(-1)]
    for _ in range(new_tokens - 1):
        out = model(tokens[-1][:, None], past_key_values=cache, use_cache=True)
        logits.append(out.logits[:, -1].float())
        tokens.append(logits[-1].argmax(-1))
    return torch.cat([input_ids, torch.stack(tokens, 1)], 1), torch.stack(logits, 1)
