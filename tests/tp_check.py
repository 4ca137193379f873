"""Run under torchrun with 2+ ranks (see test_gpu_tp.py): tensor-parallel fused decode of a
seeded tiny Llama against the single-GPU fused decoder. Prints TP_CHECK_OK on rank 0."""

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))


def main():
    from gpu_util import rel_l2
    from llmquant_b200 import native
    from llmquant_b200.core import QuantConfig, oneshot
    from llmquant_b200.runtime import tp
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from oracle.real_mode import tiny_llama

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    device = torch.device("cuda", torch.cuda.current_device())
    dist.init_process_group("nccl", device_id=device)
    quant = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    kw = dict(head_dim=128, hidden=1024, inter=2048, heads=8, kv_heads=world if world > 2 else 2,
              vocab=512)
    g = torch.Generator().manual_seed(3)
    prompt = torch.randint(0, 512, (2, 20), generator=g).cuda()
    new = 12

    # single-GPU reference on rank 0, its tokens broadcast for teacher forcing
    ref_tokens = torch.zeros(2, new, dtype=torch.long, device=device)
    ref_logits = []
    if rank == 0:
        full = oneshot(tiny_llama(seed=0, **kw).cuda(), quant.to_modifier(mode="kernel"))
        ref = FusedLlamaDecoder(full, 2, 64, kv_bits=8, use_graph=False)
        ref.prefill(prompt)
        for i in range(new):
            ref_tokens[:, i] = ref.tokens
            ref.step()
            ref_logits.append(ref.logits.float().cpu().numpy().copy())
        del ref, full
    dist.broadcast(ref_tokens, src=0)

    ok = True
    for use_peer in (True, False):
        ctx = tp.TPContext(rank, world, peer_allreduce=use_peer)
        sharded = tp.shard_linears_(tiny_llama(seed=0, **kw), ctx).cuda()
        oneshot(sharded, quant.to_modifier(mode="kernel"))
        tp.wrap_for_prefill_(sharded, ctx)
        dec = FusedLlamaDecoder(sharded, 2, 64, kv_bits=8, tp=ctx)
        if use_peer and dec.peer is None:
            print(f"rank {rank}: peer all-reduce unavailable: {getattr(dec, 'peer_error', '?')}", flush=True)
        dec.prefill(prompt)
        produced = []
        for i in range(new):
            dec.tokens.copy_(ref_tokens[:, i])
            dec.step()
            produced.append(dec.tokens.clone())
            if rank == 0:
                err = rel_l2(dec.logits.float().cpu().numpy(), ref_logits[i])
                ok &= err <= 2e-2
        mine = torch.stack(produced)
        theirs = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(theirs, mine)
        ok &= all(torch.equal(theirs[0], t) for t in theirs)  # every rank decodes the same tokens
        ok &= native.library().lq_allreduce_device_error() == 0
        del dec, sharded
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_CHECK_OK" if int(flag) == 1 else "TP_CHECK_FAILED", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
