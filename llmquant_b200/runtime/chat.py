"""Chat on a packed model: the loader and the session the reference's `examples/chat.py` drives
(llmquant/runtime/chat.py:37-174), on this library's loader, integer KV cache and kernels.

`load_for_chat(packed_path)` returns `(model, tokenizer, cache_factory)` exactly as the
reference does; the model's quantized linears are `KernelQuantLinear`s built straight from
the packed bytes, and the cache factory yields the integer cache when the file records
`kv_cache_bits`. `ChatSession` has the reference's fields and methods (history, a KV cache
carried across turns, whole turns dropped off the front when the context would overflow,
optional streaming); it only talks to `model.generate`, so it serves any causal LM.
"""

from dataclasses import dataclass, field
from typing import Optional

import torch

SYSTEM_PROMPT = "You are a helpful assistant."


@dataclass
class ChatSession:
    """A conversation and the KV cache that belongs to it."""

    model: object
    tokenizer: object
    max_new_tokens: int = 2048
    system_prompt: Optional[str] = SYSTEM_PROMPT
    stream: bool = False          # print tokens as they are decoded
    cache_factory: object = None  # zero-argument callable giving a fresh cache, or None
    max_context_tokens: Optional[int] = None  # None: the model's max_position_embeddings
    history: list = field(default_factory=list)
    last_reply_ids: list = field(default_factory=list)
    _cache: object = field(default=None, repr=False)

    def reset(self):
        self.history.clear()
        self.last_reply_ids = []
        self._cache = None
        return self

    def _messages(self):
        head = [{"role": "system", "content": self.system_prompt}] if self.system_prompt else []
        return head + self.history

    def _context_limit(self):
        if self.max_context_tokens is not None:
            return self.max_context_tokens
        return getattr(getattr(self.model, "config", None), "max_position_embeddings", None)

    def _encode(self):
        return self.tokenizer.apply_chat_template(
            self._messages(), add_generation_prompt=True, return_tensors="pt", return_dict=True)

    def _fit_to_context(self):
        """Encoded prompt that leaves room for the reply; oldest turns go first. The flag says
        whether anything was dropped (the carried cache is then stale)."""
        limit = self._context_limit()
        inputs = self._encode()
        dropped = False
        while limit is not None and inputs["input_ids"].shape[1] + self.max_new_tokens > limit:
            if len(self.history) <= 1:
                need = inputs["input_ids"].shape[1] + self.max_new_tokens
                raise ValueError(
                    f"this turn needs {need} tokens of context and the limit is {limit}. "
                    f"Shorten the message or lower max_new_tokens.")
            del self.history[0]
            dropped = True
            inputs = self._encode()
        return inputs, dropped

    @torch.no_grad()
    def ask(self, prompt: str) -> str:
        self.history.append({"role": "user", "content": prompt})
        device = next(self.model.parameters()).device
        inputs, dropped = self._fit_to_context()
        inputs = inputs.to(device)
        if dropped:
            self._cache = None
        if self._cache is None and self.cache_factory is not None:
            self._cache = self.cache_factory()
        extra = {}
        if self.stream:
            from transformers import TextStreamer

            extra["streamer"] = TextStreamer(self.tokenizer, skip_prompt=True, skip_special_tokens=True)
        if self._cache is not None:
            extra["past_key_values"] = self._cache
        generated = self.model.generate(**inputs, max_new_tokens=self.max_new_tokens, do_sample=False,
                                        pad_token_id=self.tokenizer.eos_token_id, **extra)
        new_ids = generated[0, inputs["input_ids"].shape[1]:]
        self.last_reply_ids = new_ids.tolist()
        reply = self.tokenizer.decode(new_ids, skip_special_tokens=True).strip()
        self.history.append({"role": "assistant", "content": reply})
        return reply


def load_for_chat(packed_path=None, config=None, device="cuda"):
    """(model, tokenizer, cache_factory) from a packed file, or from a run configuration
    (anything with `.model`, `.quantize`, `.quant` (a QuantConfig) and `.to_modifier()`) to
    quantize now."""
    from transformers import AutoModelForCausalLM, AutoTokenizer

    from llmquant_b200.quantizers import make_cache_factory

    if packed_path is not None:
        from llmquant_b200.packing import load_packed_model, read_header

        meta = read_header(packed_path)["meta"]
        model = load_packed_model(packed_path, device=device)
        tokenizer = AutoTokenizer.from_pretrained(meta["model_id"])
        kv_bits = meta.get("kv_cache_bits")
    elif config is not None:
        from llmquant_b200.core import oneshot

        model = AutoModelForCausalLM.from_pretrained(config.model, dtype=torch.bfloat16).to(device).eval()
        tokenizer = AutoTokenizer.from_pretrained(config.model)
        recipe = config.to_modifier()
        if recipe is not None:
            oneshot(model, recipe)
        kv_bits = config.quant.kv_cache_bits if config.quantize else None
    else:
        raise ValueError("chat needs either a packed file or a config")
    if kv_bits:
        from llmquant_b200.quantizers import enable_fused_kv_attention

        enable_fused_kv_attention(model)  # decode steps read the integer cache as it is
    return model, tokenizer, make_cache_factory(kv_bits, model=model)
