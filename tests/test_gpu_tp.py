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

        # single-GPU reference first (rank 0), its tokens broadcast for teacher forcing
        ref_tokens = torch.zeros(2, new, dtype=torch.long, device="cuda")
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

        ctx = tp.TPContext(rank, world)
        sharded = tp.shard_linears_(tiny_llama(seed=0, **kw), ctx).cuda()
        oneshot(sharded, quant.to_modifier(mode="kernel"))
        tp.wrap_for_prefill_(sharded, ctx)
        dec = FusedLlamaDecoder(sharded, 2, 64, kv_bits=8, tp=ctx)
        first = dec.prefill(prompt)
        produced = [first.cpu().tolist()]
        ok_logits = True
        for i in range(new):
            dec.tokens.copy_(ref_tokens[:, i])
            dec.step()
            produced.append(dec.tokens.cpu().tolist())
            if rank == 0:
                ok_logits &= rel_l2(dec.logits.float().cpu().numpy(), ref_logits[i]) <= 2e-2
        torch.cuda.synchronize()
        dist.barrier()
        results[rank] = (produced, bool(ok_logits))
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
    out = dict(results)
    assert out[0][1] and out[1][1]
    assert out[0][0] == out[1][0]  # both ranks decode the same tokens
