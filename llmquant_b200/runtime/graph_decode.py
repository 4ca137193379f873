"""Graphed greedy decode with the reference's entry points.

`can_graph`, `GraphedDecoder` and `graphed_generate` keep the names and call shapes of
llmquant/runtime/graph_decode.py:40-157. Two things are lifted: a quantized KV cache can be
graphed (its write cursor lives in device memory), and so can a batch of sequences (up to
`decoder.MAX_BATCH`).
A kernel-mode Llama takes the fused decoder (`runtime/decoder.py`); anything else that sits
on a CUDA device takes the transformers `StaticCache` route the reference uses.
"""

import torch

from llmquant_b200.runtime import decoder as fused

__all__ = ["GraphedDecoder", "can_graph", "graphed_generate"]

WARMUP_CALLS = 3


def can_graph(model, cache_factory=None) -> bool:
    """Whether a graphed decode is possible for this model and cache choice."""
    if not torch.cuda.is_available():
        return False
    try:
        on_cuda = next(model.parameters()).device.type == "cuda"
    except StopIteration:
        return False
    if not on_cuda:
        return False
    # Callers written for the reference ask `can_graph(model, cache_factory)` and then call
    # `graphed_generate(model, ids, n)` without saying which cache they meant
    # (llmquant/eval/evaluate.py:186-199). The answer given here is therefore remembered on the
    # model: the next graphed_generate without an explicit `kv_cache_bits` uses that cache.
    bits = None
    if cache_factory is not None:
        if not fused.supports(model):
            return False  # the integer cache is graphed by the fused decoder only
        bits = getattr(cache_factory() if callable(cache_factory) else cache_factory, "num_bits", None)
        if bits is None:
            return False  # some other cache class: not one this library can capture
    model.__dict__["_graph_kv_cache_bits"] = bits
    return True


class GraphedDecoder:
    """One captured decode step on a transformers `StaticCache` (bf16 KV), replayed per token."""

    def __init__(self, model, prompt_tokens: int, new_tokens: int, batch: int = 1):
        from transformers import StaticCache

        self.model = model
        self.device = next(model.parameters()).device
        # a StaticLayer writes at its own cursor and advances it on every call, so the warm-up
        # and capture calls need slots too; _rewind hands them back
        self.max_len = prompt_tokens + new_tokens + WARMUP_CALLS + 1
        self.cache = StaticCache(config=model.config, max_batch_size=batch,
                                 max_cache_len=self.max_len, device=self.device,
                                 dtype=torch.bfloat16)
        self.token = torch.zeros(batch, 1, dtype=torch.long, device=self.device)
        self.position = torch.zeros(1, dtype=torch.long, device=self.device)
        self.graph = None
        self.logits = None

    def _step(self):
        return self.model(self.token, past_key_values=self.cache, use_cache=True,
                          cache_position=self.position)

    @torch.no_grad()
    def prefill(self, input_ids):
        out = self.model(input_ids, past_key_values=self.cache, use_cache=True,
                         cache_position=torch.arange(input_ids.shape[1], device=self.device))
        return out.logits[:, -1:].argmax(-1)

    def _rewind(self, to: int):
        for layer in self.cache.layers:
            cursor = getattr(layer, "cumulative_length", None)
            if cursor is not None:
                cursor.fill_(to)

    @torch.no_grad()
    def capture(self, position: int):
        self.position.fill_(position)
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for _ in range(WARMUP_CALLS):
                self._step()
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            out = self._step()
        self.logits = out.logits
        self._rewind(position)

    @torch.no_grad()
    def step(self, token, position: int):
        self.token.copy_(token.reshape(self.token.shape))
        self.position.fill_(position)
        self.graph.replay()
        return self.logits[:, -1:].argmax(-1)


@torch.no_grad()
def graphed_generate(model, input_ids, max_new_tokens: int, kv_cache_bits=None):
    """Greedy generation with the decode step replayed; None if it cannot be graphed.

    `kv_cache_bits` selects the integer KV cache (fused decoder); None means the cache the last
    `can_graph(model, cache_factory)` call was asked about, bf16 KV if there was none."""
    if kv_cache_bits is None:
        kv_cache_bits = model.__dict__.get("_graph_kv_cache_bits")  # what can_graph was asked about
    if kv_cache_bits:
        from llmquant_b200.quantizers.kv_cache import make_cache_factory

        ok = can_graph(model, make_cache_factory(kv_cache_bits))
    else:
        ok = can_graph(model)
    if not ok:
        return None
    prompt = input_ids.shape[1]
    if kv_cache_bits:
        dec = fused.FusedLlamaDecoder(model, input_ids.shape[0], prompt + max_new_tokens + 1,
                                      kv_bits=kv_cache_bits)
        return dec.generate(input_ids, max_new_tokens)
    dec = GraphedDecoder(model, prompt, max_new_tokens, batch=input_ids.shape[0])
    nxt = dec.prefill(input_ids)
    out = [nxt]
    if max_new_tokens > 1:
        dec.token.copy_(nxt)
        dec.capture(prompt)
        for i in range(1, max_new_tokens):
            nxt = dec.step(nxt, prompt + i - 1)
            out.append(nxt)
    return torch.cat([input_ids, *out], dim=1)
