"""Tensor-parallel sharding on CPU ranks (gloo, world size 2): cutting a weight on row /
group boundaries commutes with quantization, and the all-reduced partial products of the
row-parallel linears equal the unsharded product. No GPU involved: the arithmetic on each
rank is the numpy oracle."""

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle
from llmquant_b200.runtime import tp


def _worker(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(0)
        hidden, inter, heads, hd = 512, 1024, 4, 128
        w_up = (torch.randn(inter, hidden, generator=g) * 0.02).bfloat16().float()
        w_down = (torch.randn(hidden, inter, generator=g) * 0.02).bfloat16().float()
        w_o = (torch.randn(hidden, heads * hd, generator=g) * 0.02).bfloat16().float()
        x = torch.randn(2, hidden, generator=g).bfloat16().float()
        a = torch.randn(2, heads * hd, generator=g).bfloat16().float()

        # column-parallel: the shard's codes and scales are a slice of the unsharded ones
        q_full, s_full = oracle.quantize_weight(w_up.numpy(), 4, 128)
        mine = tp.shard_weight("model.layers.0.mlp.up_proj", w_up, rank, world)
        q_mine, s_mine = oracle.quantize_weight(mine.numpy(), 4, 128)
        step = inter // world
        ok = np.array_equal(q_mine, q_full[rank * step:(rank + 1) * step])
        ok &= np.array_equal(s_mine, s_full[rank * step:(rank + 1) * step])
        up_full = oracle.real_linear(x.numpy(), q_full, s_full, 4, 128)
        up_mine = oracle.real_linear(x.numpy(), q_mine, s_mine, 4, 128)
        ok &= oracle.rel_l2(up_mine, up_full[:, rank * step:(rank + 1) * step]) < 1e-6

        # row-parallel: K slices on group / head boundaries, partial sums all-reduced
        for name, w, inp, head_dim in (("model.layers.0.mlp.down_proj", w_down, torch.from_numpy(up_full), None),
                                       ("model.layers.0.self_attn.o_proj", w_o, a, hd)):
            qf, sf = oracle.quantize_weight(w.numpy(), 8, 128, head_dim=head_dim)
            want = oracle.real_linear(inp.numpy(), qf, sf, 8, 128, head_dim=head_dim)
            cut = tp.shard_weight(name, w, rank, world)
            k = w.shape[1] // world
            qm, sm = oracle.quantize_weight(cut.numpy(), 8, 128, head_dim=head_dim)
            ok &= np.array_equal(qm, qf[:, rank * k:(rank + 1) * k])
            part = torch.from_numpy(oracle.real_linear(inp[:, rank * k:(rank + 1) * k].numpy(), qm, sm, 8, 128,
                                                       head_dim=head_dim))
            dist.all_reduce(part)
            ok &= oracle.rel_l2(part.numpy(), want) < 1e-6

        # replicated tensors are left alone; the logits gather restores the vocabulary order
        ok &= tp.shard_weight("model.embed_tokens", w_up, rank, world) is w_up
        ctx = tp.TPContext(rank, world)
        shard = torch.full((2, 3), float(rank))
        out = torch.empty(2, 3 * world)
        ctx.all_gather_last_dim(out, shard)
        ok &= bool((out[:, :3] == 0).all() and (out[:, 3:] == 1).all())
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_sharding_commutes_with_quantization_and_sums_back():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: True, 1: True}


def test_divisibility_rules():
    from llmquant_b200.runtime.random_init import llama_config

    cfg = llama_config("llama-3-8b")
    for world in (1, 2, 4, 8):
        tp.check_divisible(cfg, world)
    with pytest.raises(ValueError, match="must divide"):
        tp.check_divisible(cfg, 3)
    with pytest.raises(ValueError, match="must divide"):
        tp.check_divisible(cfg, 16)
