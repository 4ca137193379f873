"""Fused greedy decoder for Llama-class models whose linears are `KernelQuantLinear`.

The reference decodes by calling the transformers model once per token -- each projection a
separate `wq_gemv` launch with PyTorch ops in between (RMSNorm, RoPE, cache update, SiLU,
residual adds), optionally replayed from a CUDA graph (llmquant/runtime/graph_decode.py:52-131).
This decoder walks the same layer sequence with the library's kernels only:

    per layer   GEMV[RMSNorm -> q|k|v]  ->  [RoPE + int8 KV write + int8-KV attention + merge]
                -> GEMV[o_proj + residual]  ->  GEMV[RMSNorm -> gate|up -> silu*mul]
                -> GEMV[down_proj + residual]
    then        GEMV[final RMSNorm -> lm_head]  ->  argmax  ->  embedding row of the new token

q/k/v and gate/up are concatenated once at construction so each is one pass over one weight.
Every launch uses programmatic dependent launch, so a kernel's first weight loads overlap the
tail of the kernel before it. One step is captured into a CUDA graph and replayed per token;
the write cursor of the KV cache lives in device memory. Prefill runs through the
transformers modules (eagerly, as in the reference) into the same integer cache.

The arithmetic (bf16 roundings of RMSNorm, RoPE, SiLU*mul and the residual adds) follows
transformers' Llama modules, so greedy tokens match the module-by-module path.
"""

import torch

from llmquant_b200 import native
from llmquant_b200.core.scheme import QuantizationScheme
from llmquant_b200.quantizers.kernel import KernelQuantLinear
from llmquant_b200.quantizers.kv_cache import KernelQuantCache


MAX_BATCH = 64


def _fuse_rows(modules, interleave=False):
    """One KernelQuantLinear holding the rows of several (same geometry, same scheme)."""
    first = modules[0]
    args = first.scheme.weights
    for m in modules[1:]:
        a = m.scheme.weights
        same = (a.num_bits, a.group_size, a.head_dim, a.out_group) == (
            args.num_bits, args.group_size, args.head_dim, args.out_group)
        if not same or m.in_features != first.in_features or not m._stream:
            raise ValueError("projections to fuse must share one weight scheme and input width")
    if args.out_group and any(m.out_features % args.out_group for m in modules):
        raise ValueError("row groups would straddle the fused projections")
    codes = [m.qweight for m in modules]
    scales = [m.wscale for m in modules]
    if interleave:
        if len({m.out_features for m in modules}) != 1 or args.out_group:
            raise ValueError("interleaving needs equal row counts and per-row scales")
        qweight = torch.stack(codes, dim=1).reshape(-1, *codes[0].shape[1:])
        wscale = torch.stack(scales, dim=1).reshape(-1, scales[0].shape[1])
    else:
        qweight = torch.cat(codes, dim=0)
        wscale = torch.cat(scales, dim=0)
    bias = None
    if any(m.bias is not None for m in modules):
        if interleave:
            raise ValueError("the fused gate/up epilogue takes no bias")
        parts = [m.bias if m.bias is not None
                 else torch.zeros(m.out_features, dtype=torch.bfloat16, device=qweight.device)
                 for m in modules]
        bias = torch.cat([p.detach().to(torch.bfloat16) for p in parts])
    return KernelQuantLinear(qweight.contiguous(), wscale.contiguous(), bias, first.scheme,
                             first.in_features)


def _unwrap(module):
    """The KernelQuantLinear inside a tensor-parallel wrapper (or the module itself)."""
    return getattr(module, "inner", module)


def supports(model) -> bool:
    """Whether `model` is a Llama-layout decoder fully on kernel-mode linears."""
    try:
        layers = model.model.layers
        cfg = model.config
    except AttributeError:
        return False
    if not torch.cuda.is_available() or len(layers) == 0:
        return False
    names = ("q_proj", "k_proj", "v_proj", "o_proj")
    for layer in layers:
        attn, mlp = getattr(layer, "self_attn", None), getattr(layer, "mlp", None)
        if attn is None or mlp is None:
            return False
        mods = [_unwrap(getattr(attn, n, None)) for n in names]
        mods += [_unwrap(getattr(mlp, n, None)) for n in ("gate_proj", "up_proj", "down_proj")]
        if not all(isinstance(m, KernelQuantLinear) and m._stream for m in mods):
            return False
    head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
    groups = cfg.num_attention_heads // cfg.num_key_value_heads
    return head_dim in (64, 128) and groups in (1, 2, 4, 8) and cfg.hidden_act == "silu"


class FusedLlamaDecoder:
    """Greedy decode of a kernel-mode Llama: eager prefill, then one replayed graph per token."""

    def __init__(self, model, max_batch: int, max_len: int, kv_bits: int = 8, use_graph: bool = True,
                 pdl: bool = True, tp=None, attn_splits: int = 0, gather_logits: bool = False,
                 exchange=None, attn_impl: int = 0):
        if not supports(model):
            raise ValueError("FusedLlamaDecoder needs a Llama-layout model whose attention and MLP "
                             "linears are KernelQuantLinear (head_dim 64/128, silu MLP)")
        if max_batch > MAX_BATCH:
            raise ValueError(f"the fused decoder serves up to {MAX_BATCH} sequences (the decode GEMV takes 8 rows "
                             f"per launch; larger batches run as several launches per linear)")
        cfg = model.config
        self.model = model
        self.device = next(model.parameters()).device
        self.B, self.max_len, self.kv_bits = max_batch, max_len, kv_bits
        self.use_graph, self.pdl = use_graph, pdl
        self.hidden = cfg.hidden_size
        self.tp = tp if tp is not None and tp.world > 1 else None
        world = self.tp.world if self.tp else 1
        # under tensor parallelism every rank owns Hq/world query heads and Hkv/world KV heads
        self.Hq, self.Hkv = cfg.num_attention_heads // world, cfg.num_key_value_heads // world
        self.D = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        self.eps = cfg.rms_norm_eps
        self.scaling = self.D ** -0.5
        self.vocab = cfg.vocab_size
        dev, bf16 = self.device, torch.bfloat16

        self.layers = []
        for layer in model.model.layers:
            attn, mlp = layer.self_attn, layer.mlp
            self.layers.append({
                "qkv": _fuse_rows([attn.q_proj, attn.k_proj, attn.v_proj]),
                "o": _unwrap(attn.o_proj),
                "gate_up": _fuse_rows([mlp.gate_proj, mlp.up_proj], interleave=True),
                "down": _unwrap(mlp.down_proj),
                "ln1": layer.input_layernorm.weight.detach().to(bf16).contiguous(),
                "ln2": layer.post_attention_layernorm.weight.detach().to(bf16).contiguous(),
            })
        self.final_norm = model.model.norm.weight.detach().to(bf16).contiguous()
        self.lm_head = _unwrap(model.lm_head)
        self.embed = model.model.embed_tokens.weight

        # rotary tables from the model's own module, so scaling variants come along
        positions = torch.arange(max_len, device=dev)[None]
        probe = torch.zeros(1, 1, self.D, dtype=bf16, device=dev)
        with torch.no_grad():
            cos, sin = model.model.rotary_emb(probe, positions)
        self.cos = cos[0].to(bf16).contiguous()
        self.sin = sin[0].to(bf16).contiguous()

        B, H = self.B, self.hidden
        inter = self.layers[0]["down"].in_features
        self.h = [torch.zeros(B, H, dtype=bf16, device=dev) for _ in range(2)]
        self.qkv = torch.zeros(B, (self.Hq + 2 * self.Hkv) * self.D, dtype=bf16, device=dev)
        self.q_rot = torch.zeros(B, self.Hq * self.D, dtype=bf16, device=dev)
        self.attn = torch.zeros(B, self.Hq * self.D, dtype=bf16, device=dev)
        self.act = torch.zeros(B, inter, dtype=bf16, device=dev)
        self.logits = torch.zeros(B, self.vocab, dtype=bf16, device=dev)
        # the step's bookkeeping (embedding gather, argmax, cursor, history) in the library's two
        # small kernels when the tensors are what they expect, else with torch ops
        self._glue = (self.embed.dtype == bf16 and self.embed.is_contiguous() and self.embed.device == dev)
        self.peer = None       # separate one-shot all-reduce kernel over peer memory
        self.exchange = None   # all-reduce folded into the GEMVs (PeerExchange)
        self.gather_logits = gather_logits
        if self.tp and exchange is not None:
            self.exchange = exchange  # the caller set the buffers up (ranks sharing one GPU)
        elif self.tp:
            self._setup_tensor_parallel(B, H, dev)
        if self.tp:
            self.partial = torch.zeros(B, H, dtype=torch.float32, device=dev)
            self.local_logits = torch.zeros(B, self.vocab // world, dtype=bf16, device=dev)
        self.tokens = torch.zeros(B, dtype=torch.long, device=dev)
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)
        self.history = torch.zeros(B, max_len + 1, dtype=torch.long, device=dev)
        self.ticket = torch.zeros(1, dtype=torch.int32, device=dev)
        # slices of the cached context per KV head: about two CTAs per SM in all
        # (as many as fit the GPU at two CTAs per SM in one wave: a few CTAs over that run as a
        # second wave; measured at batch 8 and 32)
        want = attn_splits if attn_splits > 0 else max(1, 2 * 148 // (B * self.Hkv))
        self.splits = max(1, min(want, max_len // 64 or 1))
        self.attn_impl = attn_impl
        nbytes = native.library().lq_attn_fused_scratch_bytes(B, self.Hq, self.Hkv, self.D, self.splits)
        self.scratch = torch.zeros(-(-nbytes // 4), dtype=torch.float32, device=dev)
        self.cache = KernelQuantCache(kv_bits, max_cache_len=max_len)
        # scratch of the tensor-core decode GEMM that batches above 8 rows go through
        self.workspace = None
        from llmquant_b200.quantizers.kernel import DECODE_GEMM_MIN_ROWS
        self.decode_gemm = B >= DECODE_GEMM_MIN_ROWS and (self.tp is None or self.exchange is None)
        if self.decode_gemm:
            linears = [spec[k] for spec in self.layers for k in ("qkv", "o", "gate_up", "down")]
            if isinstance(self.lm_head, KernelQuantLinear):
                linears.append(self.lm_head)
            need = max(m.decode_workspace_bytes(B) for m in linears)
            self.workspace = torch.empty(need, dtype=torch.uint8, device=dev)
        self.graph = None
        separate_reduce = self.tp is not None and self.exchange is None
        per_linear = 3 if self.decode_gemm else 1  # the decode GEMM is planes, product, finish
        self.launches_per_step = (len(self.layers) * (4 * per_linear + 1 + (2 if separate_reduce else 0)) + per_linear
                                  + (2 if self._glue else 0))
        if not self.tp:
            self.allreduce = "none"
        elif self.exchange is not None:
            self.allreduce = "folded into the GEMVs (partials pushed to peer memory, summed in the consumer's prologue)"
        else:
            self.allreduce = "peer-memory one-shot kernel" if self.peer is not None else "nccl"

    def _setup_tensor_parallel(self, B, H, dev):
        """Choose the all-reduce route, the same on every rank. Order of preference: folded
        into the GEMVs (batch <= 2, the rows one GEMV pass takes), the separate one-shot kernel
        over peer memory, NCCL. Each attempt ends in a vote, so a rank on which symmetric memory
        cannot be set up takes all ranks to the next route instead of leaving them in kernels
        that wait for it."""
        from llmquant_b200.runtime.tp import PeerAllReduce, PeerExchange, all_ranks_agree

        self.peer_error = None
        want_peer = getattr(self.tp, "peer_allreduce", True) and (B * H) % 4 == 0
        want_fused = (want_peer and getattr(self.tp, "fused_allreduce", True) and B <= 2 and self._glue
                      and isinstance(self.lm_head, KernelQuantLinear) and self.lm_head._stream
                      and H % 4 == 0)
        for route in ("fused", "kernel"):
            wanted = want_fused if route == "fused" else want_peer
            if not all_ranks_agree(self.tp, wanted, dev):
                continue
            made = None
            try:
                if route == "fused":
                    made = PeerExchange.over_symmetric_memory(self.tp, B, H, dev)
                else:
                    made = PeerAllReduce(self.tp, B * H, dev)
            except Exception as exc:  # symmetric memory unavailable on this rank
                self.peer_error = repr(exc)
            if all_ranks_agree(self.tp, made is not None, dev):
                if route == "fused":
                    self.exchange = made
                else:
                    self.peer = made
                return

    # ------------------------------------------------------------------ one token
    def _attention(self, cache, pos_ptr, pdl, stream):
        native.call("lq_attn_decode_fused", self.qkv.data_ptr(), self.cos.data_ptr(),
                    self.sin.data_ptr(), cache.k_codes.data_ptr(), cache.v_codes.data_ptr(),
                    cache.k_scales.data_ptr(), cache.v_scales.data_ptr(), self.attn.data_ptr(),
                    self.scratch.data_ptr(), self.B, self.Hq, self.Hkv, self.D, cache.capacity,
                    self.cos.shape[0], pos_ptr, 0, self.kv_bits, self.scaling, self.splits,
                    self.attn_impl, pdl, stream)

    def _folded_launches(self):
        """The step under tensor parallelism with the all-reduce folded into the GEMVs: o_proj and
        down_proj push their fp32 partial rows into every rank's exchange buffer; gate|up, the
        next layer's q|k|v and lm_head first build their input -- bf16(bf16(sum of the partials)
        + residual) -- and go on as usual. Five launches per layer, as on one GPU. A generator
        that yields after every launch, so that several ranks living on one GPU can be advanced
        in lock step (each launch of all ranks before the next); the token exchange that ends
        the step is `_folded_token`."""
        ex, L = self.exchange, len(self.layers)
        stream = native.stream_ptr(self.device)
        pdl = 1 if self.pdl else 0
        h0, h1 = self.h
        native.call("lq_embed_gather", self.embed.data_ptr(), self.tokens.data_ptr(), h0.data_ptr(),
                    self.B, self.hidden, self.embed.shape[0], pdl, stream)
        yield
        pos_ptr = self.pos.data_ptr()
        for l, (spec, cache) in enumerate(zip(self.layers, self.cache.layers)):
            tp = None
            if l > 0:  # hidden = down_proj(l - 1) summed over the ranks + its residual
                tp = ex.sum_args(1, h1)
            spec["qkv"].gemv(h0, norm_weight=spec["ln1"], norm_eps=self.eps, pdl=self.pdl, workspace=self.workspace, out=self.qkv, tp=tp)
            yield
            self._attention(cache, pos_ptr, pdl, stream)
            yield
            spec["o"].gemv(self.attn, out_dtype=torch.float32, pdl=self.pdl, workspace=self.workspace, tp=ex.push_args(0))
            yield
            tp = ex.sum_args(0, h0)
            spec["gate_up"].gemv(h1, norm_weight=spec["ln2"], norm_eps=self.eps, epilogue=1,
                                 pdl=self.pdl, workspace=self.workspace, out=self.act, tp=tp)
            yield
            spec["down"].gemv(self.act, out_dtype=torch.float32, pdl=self.pdl, workspace=self.workspace, tp=ex.push_args(1))
            yield
        tp = ex.sum_args(1, h1)
        self.lm_head.gemv(h0, norm_weight=self.final_norm, norm_eps=self.eps, pdl=self.pdl, workspace=self.workspace,
                          out=self.local_logits, tp=tp)
        yield

    def _folded_token(self):
        """End of a folded step: every rank sends its local maximum to all ranks and picks the
        same token; cursor and step counter advance. With `gather_logits` the full logits are
        gathered as well (for inspection: the token does not need them)."""
        if self.gather_logits:
            self.tp.all_gather_last_dim(self.logits, self.local_logits)
        self.exchange.next_token(self.local_logits, self.tokens, self.pos, self.history, self.ticket, self.pdl)

    def _step_kernels(self):
        if self.exchange is not None:
            for _ in self._folded_launches():
                pass
            return self._folded_token()
        stream = native.stream_ptr(self.device)
        pdl = 1 if self.pdl else 0
        cur, nxt = self.h
        if self._glue:
            native.call("lq_embed_gather", self.embed.data_ptr(), self.tokens.data_ptr(), cur.data_ptr(),
                        self.B, self.hidden, self.embed.shape[0], pdl, stream)
        else:
            cur.copy_(self.embed.index_select(0, self.tokens))
        pos_ptr = self.pos.data_ptr()
        for spec, cache in zip(self.layers, self.cache.layers):
            spec["qkv"].gemv(cur, norm_weight=spec["ln1"], norm_eps=self.eps, pdl=self.pdl, workspace=self.workspace, out=self.qkv)
            self._attention(cache, pos_ptr, pdl, stream)
            self._row_parallel(spec["o"], self.attn, cur, nxt, 0)
            spec["gate_up"].gemv(nxt, norm_weight=spec["ln2"], norm_eps=self.eps, epilogue=1,
                                 pdl=self.pdl, workspace=self.workspace, out=self.act)
            self._row_parallel(spec["down"], self.act, nxt, cur, 1)
        if isinstance(self.lm_head, KernelQuantLinear) and self.lm_head._stream:
            head_out = self.local_logits if self.tp else self.logits
            self.lm_head.gemv(cur, norm_weight=self.final_norm, norm_eps=self.eps, pdl=self.pdl, workspace=self.workspace,
                              out=head_out)
            if self.tp:
                self.tp.all_gather_last_dim(self.logits, self.local_logits)
        else:
            with torch.no_grad():
                self.logits.copy_(self.lm_head(self.model.model.norm(cur)))
        if self._glue:
            native.call("lq_next_token", self.logits.data_ptr(), self.logits.shape[1], self.tokens.data_ptr(),
                        pos_ptr, self.history.data_ptr(), self.history.shape[1], self.ticket.data_ptr(),
                        self.B, pdl, stream)
        else:
            torch.argmax(self.logits, dim=-1, out=self.tokens)
            self.pos.add_(1)
            self.history.index_copy_(1, self.pos, self.tokens.unsqueeze(1))

    def gemv_launches(self):
        """Only the GEMV launches of one step, in order and with the step's own fusions and
        buffers (no attention, no all-reduce, no token bookkeeping): what a benchmark captures
        to time the dominant kernel by itself. Leaves the hidden-state buffers overwritten."""
        cur, nxt = self.h
        for spec in self.layers:
            spec["qkv"].gemv(cur, norm_weight=spec["ln1"], norm_eps=self.eps, pdl=self.pdl, workspace=self.workspace, out=self.qkv)
            spec["o"].gemv(self.attn, residual=cur, pdl=self.pdl, workspace=self.workspace, out=nxt)
            spec["gate_up"].gemv(nxt, norm_weight=spec["ln2"], norm_eps=self.eps, epilogue=1,
                                 pdl=self.pdl, workspace=self.workspace, out=self.act)
            spec["down"].gemv(self.act, residual=nxt, pdl=self.pdl, workspace=self.workspace, out=cur)
        if isinstance(self.lm_head, KernelQuantLinear) and self.lm_head._stream:
            self.lm_head.gemv(cur, norm_weight=self.final_norm, norm_eps=self.eps, pdl=self.pdl, workspace=self.workspace,
                              out=self.local_logits if self.tp else self.logits)

    def gemv_bytes(self):
        """Algorithmic HBM bytes of `gemv_launches`: codes + scales of every linear."""
        total = sum(spec[key].weight_bytes() for spec in self.layers for key in ("qkv", "o", "gate_up", "down"))
        if isinstance(self.lm_head, KernelQuantLinear):
            total += self.lm_head.weight_bytes()
        return total

    def _row_parallel(self, linear, x, residual, out, slot):
        """out = residual + linear(x). One GPU: fused in the GEMV epilogue. Tensor parallel:
        fp32 partial, summed over the ranks (one-shot kernel over peer memory, or NCCL),
        then the same rounding and residual add."""
        if not self.tp:
            linear.gemv(x, residual=residual, pdl=self.pdl, workspace=self.workspace, out=out)
            return
        if self.peer is not None:
            linear.gemv(x, out_dtype=torch.float32, pdl=self.pdl, workspace=self.workspace,
                        out=self.peer.slot(slot, out.shape[0], out.shape[1]))
            self.peer.reduce(slot, residual, out, self.pdl)
            return
        linear.gemv(x, out_dtype=torch.float32, pdl=self.pdl, workspace=self.workspace, out=self.partial)
        self.tp.all_reduce(self.partial)
        native.call("lq_residual_add", self.partial.data_ptr(), residual.data_ptr(), out.data_ptr(),
                    out.numel(), 1 if self.pdl else 0, native.stream_ptr(self.device))

    # ------------------------------------------------------------------ prefill / capture
    @torch.no_grad()
    def prefill(self, input_ids):
        """Eager pass over the prompt through the transformers modules into the int cache.
        Returns the first generated token per sequence, [B]."""
        if input_ids.shape[0] != self.B:
            raise ValueError(f"decoder was built for batch {self.B}, got {input_ids.shape[0]}")
        prompt = input_ids.shape[1]
        if prompt >= self.max_len:
            raise ValueError(f"prompt of {prompt} tokens does not fit a cache of {self.max_len}")
        for layer in self.cache.layers:
            layer.reset()
        out = self.model(input_ids, past_key_values=self.cache, use_cache=True, logits_to_keep=1)
        self.logits.copy_(out.logits[:, -1])  # the prompt's last position, for callers that inspect it
        first = out.logits[:, -1].argmax(-1)
        self._begin_sequence()
        self.tokens.copy_(first)
        self.pos.fill_(prompt)
        self.history.zero_()
        self.history[:, :prompt] = input_ids
        self.history[:, prompt] = first
        return first

    def _begin_sequence(self):
        """State the folded tensor-parallel step expects at its first launch: the second
        hidden-state buffer empty (its rows are rebuilt by the first summing GEMV and read by
        CTAs that wait for them to appear)."""
        if self.exchange is not None:
            self.exchange.mark_empty(self.h[1])

    @torch.no_grad()
    def start_empty(self, first_tokens):
        """Begin decoding from an empty cache with `first_tokens` ([B], e.g. the BOS id) as the
        token to feed: no prefill pass. The cache layers are allocated here."""
        dummy = torch.zeros(self.B, self.Hkv, 1, self.D, dtype=torch.bfloat16, device=self.device)
        while len(self.cache.layers) < len(self.layers):
            self.cache.layers.append(self.cache.layer_class_to_replicate())
        for layer in self.cache.layers:
            if not layer.is_initialized:
                layer.lazy_initialization(dummy, dummy)
            layer.reset()
        self._begin_sequence()
        self.tokens.copy_(first_tokens.to(self.device))
        self.pos.zero_()
        self.history.zero_()
        self.history[:, 0] = self.tokens

    @torch.no_grad()
    def capture(self):
        """Warm up on a side stream, then capture one step. The warm-up and the capture write
        real entries at the cursor; the cursor and token are restored afterwards and the
        entries are overwritten by the first replay."""
        saved_pos, saved_tok = self.pos.clone(), self.tokens.clone()
        saved_hist = self.history.clone()
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.pos.copy_(saved_pos)
                self.tokens.copy_(saved_tok)
                self._step_kernels()
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        self.pos.copy_(saved_pos)
        self.tokens.copy_(saved_tok)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step_kernels()
        self.pos.copy_(saved_pos)
        self.tokens.copy_(saved_tok)
        self.history.copy_(saved_hist)

    @torch.no_grad()
    def step(self):
        """Decode one token for every sequence (in place: tokens, pos, history advance)."""
        if self.use_graph:
            if self.graph is None:
                self.capture()
            self.graph.replay()
        else:
            self._step_kernels()

    def check_device_errors(self):
        """Raise if a bounded wait inside one of the step's kernels ever ran out (a pipeline
        stall, or under tensor parallelism a rank that never arrived): the tokens produced since
        the last check cannot be trusted. Reads device words, so it synchronizes."""
        lib = native.library()
        words = {"gemv": lib.lq_gemv_device_error(), "attention": lib.lq_attn_device_error()}
        if self.workspace is not None:
            words["decode gemm"] = lib.lq_decode_gemm_device_error()
        if self.tp:
            words["allreduce"] = lib.lq_allreduce_device_error()
            words["token exchange"] = lib.lq_glue_device_error()
        bad = {k: v for k, v in words.items() if v != 0}
        if bad:
            raise RuntimeError(f"a bounded device wait expired during decode: {bad}")

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens: int):
        """Greedy generation; returns prompt + new tokens, like `model.generate(do_sample=False)`."""
        prompt = input_ids.shape[1]
        if prompt + max_new_tokens > self.max_len:
            raise ValueError("prompt + new tokens exceed the decoder's cache")
        self.prefill(input_ids.to(self.device))
        for _ in range(max_new_tokens - 1):
            self.step()
        for layer in self.cache.layers:
            layer.length = prompt + max_new_tokens - 1
        out = self.history[:, : prompt + max_new_tokens].clone()
        self.check_device_errors()
        return out
