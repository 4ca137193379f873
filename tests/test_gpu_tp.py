"""Tensor-parallel decode on two GPUs (skipped on a single-GPU box): both ranks produce the
same tokens, and their logits agree with the single-GPU fused decoder on the same model."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, results):
    import torch.distributed as dist

    from gpu_util import rel_l2
    from llmquant_b200.core import QuantConfig, oneshot
    from llmquant_b200.runtime import tp
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from oracle.real_mode import tiny_llama

    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    try:
        quant = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
        kw = dict(head_dim=128, hidden=512, inter=1024, heads=4, kv_heads=2)
        g = torch.Generator().manual_seed(3)
        prompt = torch.randint(0, 512, (2, 20), generator=g).cuda()
        new = 12

        ctx = tp.TPContext(rank, world)
        sharded = tp.shard_linears_(tiny_llama(seed=0, **kw), ctx).cuda()
        oneshot(sharded, quant.to_modifier(mode="kernel"))
        tp.wrap_for_prefill_(sharded, ctx)
        dec = FusedLlamaDecoder(sharded, 2, 64, kv_bits=8, tp=ctx)
        dec.prefill(prompt)
        tp_logits = []
        for _ in range(new):
            dec.step()
            tp_logits.append(dec.logits.float().cpu().numpy().copy())
        tokens = dec.history[:, : prompt.shape[1] + new + 1].cpu()

        gathered = [torch.empty_like(tokens) for _ in range(world)]
        dist.all_gather_object(gathered, tokens)
        same_across_ranks = all(torch.equal(gathered[0], t) for t in gathered)

        ok_logits = True
        if rank == 0:
            full = oneshot(tiny_llama(seed=0, **kw).cuda(), quant.to_modifier(mode="kernel"))
            ref = FusedLlamaDecoder(full, 2, 64, kv_bits=8)
            ref.prefill(prompt)
            for i in range(new):
                # teacher-forced with the tensor-parallel run's tokens
                ref.tokens.copy_(tokens[:, prompt.shape[1] + i].cuda())
                ref.step()
                err = rel_l2(tp_logits[i], ref.logits.float().cpu().numpy())
                ok_logits &= err <= 2e-2
        results[rank] = (bool(same_across_ranks), bool(ok_logits))
    finally:
        dist.destroy_process_group()


def test_two_gpu_decode_matches_single_gpu():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import socket

    import torch.multiprocessing as mp

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, True), 1: (True, True)}
