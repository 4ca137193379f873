"""Tensor-parallel decode over the GPUs of one node.

The reference is single-GPU. Sharding follows the usual column-then-row split of a Llama
layer, cut so that quantization is unaffected (scales are per output row and per 128-wide
group of the reduction axis, so any cut on row or group boundaries leaves every code and
scale exactly what the unsharded weight would get):

  column-parallel (rows):      q_proj, k_proj, v_proj by heads; gate_proj, up_proj; lm_head
  row-parallel (reduction K):  o_proj by heads, down_proj by groups of 128 -> all-reduce (sum)
                               of the [batch, hidden] partial outputs, two per layer

The KV cache and the attention are sharded by KV head with no exchange. One process per GPU;
`torch.distributed` (NCCL over NVLink) carries the all-reduce and the logits all-gather, both
of which are captured into the decode graph.
"""

import re
from dataclasses import dataclass

import torch
import torch.nn as nn

ROW_SPLIT = re.compile(r".*\.(self_attn\.(q|k|v)_proj|mlp\.(gate|up)_proj)$|^lm_head$")
K_SPLIT = re.compile(r".*\.(self_attn\.o_proj|mlp\.down_proj)$")


@dataclass
class TPContext:
    rank: int
    world: int
    group: object = None  # torch.distributed process group (None = the default group)
    peer_allreduce: bool = True  # use peer memory for the all-reduce before falling back to NCCL
    fused_allreduce: bool = True  # fold the all-reduce into the GEMVs where the batch allows

    def all_reduce(self, tensor):
        import torch.distributed as dist
        dist.all_reduce(tensor, group=self.group)
        return tensor

    def all_gather_last_dim(self, out, shard):
        """out [B, world * n] <- concatenation over ranks of shard [B, n]."""
        import torch.distributed as dist
        rows, n = shard.shape
        gathered = torch.empty(self.world * rows, n, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(gathered, shard.contiguous(), group=self.group)
        out.view(rows, self.world, n).copy_(gathered.view(self.world, rows, n).permute(1, 0, 2))
        return out


def check_divisible(config, world: int, group_size: int = 128):
    heads, kv = config.num_attention_heads, config.num_key_value_heads
    if heads % world or kv % world:
        raise ValueError(f"tensor parallel degree {world} must divide {heads} query and {kv} KV heads")
    if config.intermediate_size % (world * group_size):
        raise ValueError(f"intermediate_size {config.intermediate_size} must be a multiple of "
                         f"{world} x {group_size} so down_proj splits on group boundaries")
    if config.vocab_size % (4 * world):
        raise ValueError(f"vocab_size {config.vocab_size} must be a multiple of {4 * world}")
    head_dim = getattr(config, "head_dim", None) or config.hidden_size // heads
    if (heads // world) * head_dim % group_size and head_dim >= group_size:
        raise ValueError("o_proj's reduction slice must fall on group boundaries")


def shard_weight(name: str, weight: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """This rank's slice of a Linear weight [out, in]; replicated tensors come back whole."""
    if world == 1:
        return weight
    if ROW_SPLIT.match(name):
        n = weight.shape[0]
        if n % world:
            raise ValueError(f"{name}: {n} rows do not divide by {world}")
        step = n // world
        return weight[rank * step:(rank + 1) * step].contiguous()
    if K_SPLIT.match(name):
        k = weight.shape[1]
        if k % world:
            raise ValueError(f"{name}: reduction width {k} does not divide by {world}")
        step = k // world
        return weight[:, rank * step:(rank + 1) * step].contiguous()
    return weight


class RowParallelOutput(nn.Module):
    """Wraps a K-sharded linear for the module-by-module (prefill) path: the partial
    products are summed over the ranks in fp32 and rounded once."""

    def __init__(self, inner, ctx: TPContext):
        super().__init__()
        self.inner, self.ctx = inner, ctx

    def forward(self, x):
        if x.shape[:-1].numel() <= 8 and hasattr(self.inner, "gemv"):
            flat = x.reshape(-1, x.shape[-1])
            partial = self.inner.gemv(flat, out_dtype=torch.float32)
        else:
            partial = self.inner(x).float()
        self.ctx.all_reduce(partial)
        return partial.to(x.dtype).reshape(*x.shape[:-1], -1)


class GatheredOutput(nn.Module):
    """Wraps a row-sharded lm_head: every rank ends up with the full logits."""

    def __init__(self, inner, ctx: TPContext):
        super().__init__()
        self.inner, self.ctx = inner, ctx

    def forward(self, x):
        local = self.inner(x)
        flat = local.reshape(-1, local.shape[-1])
        out = torch.empty(flat.shape[0], flat.shape[1] * self.ctx.world, dtype=flat.dtype, device=flat.device)
        self.ctx.all_gather_last_dim(out, flat)
        return out.reshape(*local.shape[:-1], -1)


@torch.no_grad()
def shard_linears_(model, ctx: TPContext):
    """Slice every nn.Linear of a Llama in place (call BEFORE quantizing it)."""
    check_divisible(model.config, ctx.world)
    for name, module in model.named_modules():
        if isinstance(module, nn.Linear):
            cut = shard_weight(name, module.weight.data, ctx.rank, ctx.world)
            if cut.shape != module.weight.shape:
                module.weight = nn.Parameter(cut, requires_grad=False)
                module.out_features, module.in_features = cut.shape
                if module.bias is not None and ROW_SPLIT.match(name):
                    step = module.bias.shape[0] // ctx.world
                    module.bias = nn.Parameter(
                        module.bias.data[ctx.rank * step:(ctx.rank + 1) * step].contiguous(),
                        requires_grad=False)
                elif module.bias is not None and ctx.rank != 0:
                    module.bias = None  # a row-parallel bias is added once, by rank 0
    return model


def wrap_for_prefill_(model, ctx: TPContext):
    """After quantization: make the module-by-module forward (prefill) tensor-parallel by
    wrapping o_proj / down_proj with the all-reduce and lm_head with the all-gather."""
    if ctx.world == 1:
        return model
    for layer in model.model.layers:
        layer.self_attn.o_proj = RowParallelOutput(layer.self_attn.o_proj, ctx)
        layer.mlp.down_proj = RowParallelOutput(layer.mlp.down_proj, ctx)
    model.lm_head = GatheredOutput(model.lm_head, ctx)
    return model


class PeerAllReduce:
    """The fused all-reduce + residual add over NVLink peer memory (`lq_allreduce_residual`).

    Each rank allocates one symmetric buffer (two fp32 slots of `max_floats` plus the flag
    arrays), all ranks map each other's buffers, and the row-parallel GEMV writes its partial
    straight into the rank's own slot. Raises if symmetric memory cannot be set up; the caller
    then stays on the NCCL path."""

    def __init__(self, ctx: TPContext, max_floats: int, device):
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        from llmquant_b200 import native

        lib = native.library()
        self.ctx = ctx
        self.slot_floats = -(-max_floats // 4) * 4
        self.flag_off = -(-(2 * self.slot_floats * 4) // 16) * 16
        total = self.flag_off + 2 * lib.lq_allreduce_max_world() * 4
        self.buffer = symm.empty(total // 4, dtype=torch.float32, device=device)
        self.buffer.zero_()
        group = ctx.group if ctx.group is not None else dist.group.WORLD
        self.handle = symm.rendezvous(self.buffer, group)
        ptrs = [int(p) for p in self.handle.buffer_ptrs]
        if len(ptrs) != ctx.world:
            raise RuntimeError("symmetric memory rendezvous returned the wrong number of peers")
        self.peers = torch.tensor(ptrs, dtype=torch.int64, device=device)
        self.seq = torch.zeros(1, dtype=torch.int32, device=device)
        self.wait_cycles = 0  # 0 = the library's default bound (about two seconds)
        torch.cuda.synchronize(device)
        dist.barrier(group=ctx.group)  # every buffer is zeroed before anyone signals

    def slot(self, index: int, rows: int, width: int) -> torch.Tensor:
        """fp32 view [rows, width] of this rank's slot `index` (the GEMV's output buffer)."""
        if rows * width > self.slot_floats:
            raise ValueError("partial output larger than the all-reduce slot")
        start = index * self.slot_floats
        return self.buffer[start:start + rows * width].view(rows, width)

    def reduce(self, index: int, residual, out, pdl: bool = True):
        from llmquant_b200 import native

        native.call("lq_allreduce_residual", self.peers.data_ptr(), self.ctx.rank, self.ctx.world,
                    index, self.slot_floats, self.flag_off, self.seq.data_ptr(),
                    native.ptr(residual), out.data_ptr(), out.numel(), self.wait_cycles,
                    1 if pdl else 0, native.stream_ptr(out.device))


class PeerExchange:
    """Exchange buffers of the fused tensor-parallel decode step (`lq_gemv_tp`,
    `lq_next_token_tp`): the row-parallel GEMVs write their fp32 partial rows straight into
    every rank's buffer and the GEMV that consumes the sum adds them up in its prologue, so no
    separate all-reduce launch is left in the step.

    One buffer per rank, mapped by all ranks (symmetric memory over NVLink):

        float    part[2 slots][world][rows][width]    partial outputs, by source rank; a word
                                                      holds 0xFFFFFFFF while no value is there
        uint64   records[2 banks][16][max_batch]      (token index, logit, step tag) per rank

    plus, local to the rank, the step counter that tags the records. Slot 0 carries o_proj's
    output, slot 1 down_proj's. The hidden-state rows the consuming GEMVs rebuild follow the
    same convention (`empty_rows`): empty until written, emptied again by their last reader."""

    def __init__(self, rank: int, world: int, rows: int, width: int, device, buffer, peer_ptrs,
                 max_batch: int = 8):
        if rows * width % 4:
            raise ValueError("rows * width of the exchanged partials must be a multiple of 4")
        if world > 16 or rows > max_batch:
            raise ValueError("the exchange buffer holds at most 16 ranks and max_batch rows")
        self.rank, self.world, self.rows, self.width = rank, world, rows, width
        self.max_batch = max_batch
        self.buffer = buffer
        self.slot_bytes = world * rows * width * 4
        self.record_off = 2 * self.slot_bytes
        if buffer.numel() * buffer.element_size() < self.bytes_needed(world, rows, width, max_batch):
            raise ValueError("exchange buffer too small")
        if len(peer_ptrs) != world:
            raise RuntimeError("the exchange needs one mapped buffer per rank")
        self.peers = torch.tensor([int(p) for p in peer_ptrs], dtype=torch.int64, device=device)
        self.base = int(peer_ptrs[rank])
        self.step = torch.zeros(1, dtype=torch.int32, device=device)
        self.wait_cycles = 0  # 0 = the library's default bound (about two seconds)

    @staticmethod
    def bytes_needed(world, rows, width, max_batch=8):
        return 2 * world * rows * width * 4 + 2 * 16 * max_batch * 8

    @staticmethod
    def clear(buffer, world, rows, width):
        """The state before the first step: every partial word empty, every record zero."""
        words = buffer.view(torch.int32)
        n = 2 * world * rows * width
        words[:n] = -1
        words[n:] = 0

    @classmethod
    def over_symmetric_memory(cls, ctx: TPContext, rows: int, width: int, device, max_batch: int = 8):
        """Collective: every rank of `ctx` allocates its buffer and maps the others'."""
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        nbytes = cls.bytes_needed(ctx.world, rows, width, max_batch)
        buffer = symm.empty(-(-nbytes // 4), dtype=torch.float32, device=device)
        cls.clear(buffer, ctx.world, rows, width)
        group = ctx.group if ctx.group is not None else dist.group.WORLD
        handle = symm.rendezvous(buffer, group)
        ptrs = [int(p) for p in handle.buffer_ptrs]
        self = cls(ctx.rank, ctx.world, rows, width, device, buffer, ptrs, max_batch)
        self.handle = handle
        torch.cuda.synchronize(device)
        dist.barrier(group=ctx.group)  # every buffer is cleared before anyone writes into it
        return self

    @classmethod
    def on_one_device(cls, world: int, rows: int, width: int, device, max_batch: int = 8):
        """`world` exchanges whose buffers all live on one GPU: the ranks of a group run one
        after the other on one stream (all pushing launches before the launch that consumes
        them). For single-GPU tests of the multi-rank arithmetic."""
        nbytes = cls.bytes_needed(world, rows, width, max_batch)
        buffers = [torch.zeros(-(-nbytes // 4), dtype=torch.float32, device=device) for _ in range(world)]
        for b in buffers:
            cls.clear(b, world, rows, width)
        ptrs = [b.data_ptr() for b in buffers]
        return [cls(r, world, rows, width, device, buffers[r], ptrs, max_batch) for r in range(world)]

    # ---- per-launch argument blocks
    def push_args(self, slot: int):
        from llmquant_b200 import native

        return native.GemvTp(mode=native.TP_PUSH, world=self.world, rank=self.rank,
                             peers=self.peers.data_ptr(), data_offset=slot * self.slot_bytes)

    def sum_args(self, slot: int, residual):
        from llmquant_b200 import native

        return native.GemvTp(mode=native.TP_SUM, world=self.world, rank=self.rank,
                             parts=self.base + slot * self.slot_bytes, residual=residual.data_ptr(),
                             wait_cycles=self.wait_cycles)

    @staticmethod
    def empty_rows(rows: int, width: int, device):
        """A bf16 [rows, width] hidden-state buffer in the "nothing here yet" state."""
        return torch.full((rows, width), -1, dtype=torch.int16, device=device).view(torch.bfloat16)

    @staticmethod
    def mark_empty(tensor):
        tensor.view(torch.int16).fill_(-1)

    def next_token(self, local_logits, tokens, pos, history, ticket, pdl: bool = True):
        from llmquant_b200 import native

        native.call("lq_next_token_tp", local_logits.data_ptr(), local_logits.shape[1], self.rank,
                    self.world, self.peers.data_ptr(), self.record_off, self.max_batch,
                    tokens.data_ptr(), pos.data_ptr(), native.ptr(history),
                    history.shape[1] if history is not None else 0, ticket.data_ptr(),
                    self.step.data_ptr(), local_logits.shape[0], self.wait_cycles, 1 if pdl else 0,
                    native.stream_ptr(local_logits.device))


def all_ranks_agree(ctx: TPContext, ok: bool, device) -> bool:
    """True only if `ok` holds on every rank (a collective: every rank must call it)."""
    import torch.distributed as dist

    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=ctx.group)
    return bool(int(flag.item()))
