"""Host side of the tensor-parallel decode on CPU: the exchange buffer's layout and the argument
blocks built from it, its refusals (a peer missing, a buffer too small), and the vote by which
all ranks take the same all-reduce route when one of them could not set a route up -- with the
failing rank made on the host (gloo, world size 2), never on a GPU."""

import ctypes

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from llmquant_b200 import native
from llmquant_b200.runtime import tp
from llmquant_b200.runtime.tp import PeerExchange


def _exchange(world=4, rows=2, width=1024, rank=1):
    nbytes = PeerExchange.bytes_needed(world, rows, width)
    buf = torch.zeros(-(-nbytes // 4), dtype=torch.float32)
    ptrs = [1 << 20, 2 << 20, 3 << 20, 4 << 20][:world]
    return PeerExchange(rank, world, rows, width, torch.device("cpu"), buf, ptrs), ptrs


def test_exchange_layout_and_argument_blocks():
    ex, ptrs = _exchange()
    slot = 4 * 2 * 1024 * 4
    assert ex.slot_bytes == slot and ex.record_off == 2 * slot
    assert PeerExchange.bytes_needed(4, 2, 1024) == ex.record_off + 2 * 16 * 8 * 8
    PeerExchange.clear(ex.buffer, 4, 2, 1024)
    words = ex.buffer.view(torch.int32)
    assert bool((words[: 2 * slot // 4] == -1).all()) and bool((words[2 * slot // 4:] == 0).all())
    push = ex.push_args(1)
    assert (push.mode, push.world, push.rank) == (native.TP_PUSH, 4, 1)
    assert push.data_offset == slot and push.peers == ex.peers.data_ptr()
    residual = torch.zeros(2, 1024, dtype=torch.bfloat16)
    ex.wait_cycles = 12345
    summ = ex.sum_args(1, residual)
    assert summ.mode == native.TP_SUM and summ.parts == ptrs[1] + slot
    assert summ.wait_cycles == 12345 and summ.residual == residual.data_ptr()
    rows = PeerExchange.empty_rows(2, 8, "cpu")
    assert rows.dtype == torch.bfloat16 and bool((rows.view(torch.int16) == -1).all())
    # the C struct: three ints, padding, then pointers and 64-bit fields
    assert native.GemvTp.peers.offset == 16 and ctypes.sizeof(native.GemvTp) == 56
    assert native.GemvArgs.tp.offset == 112 and native.GemvArgs.ldo.offset == 120
    assert native.GemvArgs.workspace.offset == 128 and ctypes.sizeof(native.GemvArgs) == 144


def test_exchange_refuses_a_missing_peer_a_small_buffer_and_ragged_rows():
    nbytes = PeerExchange.bytes_needed(2, 1, 1024)
    buf = torch.zeros(nbytes // 4, dtype=torch.float32)
    with pytest.raises(RuntimeError, match="one mapped buffer per rank"):
        PeerExchange(0, 2, 1, 1024, torch.device("cpu"), buf, [1 << 20])
    with pytest.raises(ValueError, match="too small"):
        PeerExchange(0, 2, 1, 1024, torch.device("cpu"), buf[:-8], [1 << 20, 2 << 20])
    with pytest.raises(ValueError, match="multiple of 4"):
        PeerExchange(0, 2, 1, 1022, torch.device("cpu"), buf, [1 << 20, 2 << 20])
    with pytest.raises(ValueError, match="at most 16 ranks"):
        PeerExchange(0, 17, 1, 1024, torch.device("cpu"), buf, [0] * 17)


def _vote_worker(rank, world, port, results):
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        ctx = tp.TPContext(rank, world)
        cpu = torch.device("cpu")
        everyone = tp.all_ranks_agree(ctx, True, cpu)
        one_failed = tp.all_ranks_agree(ctx, rank != 1, cpu)  # rank 1 could not set its buffer up
        results[rank] = (everyone, one_failed)
    finally:
        dist.destroy_process_group()


def test_a_rank_that_cannot_set_a_route_up_takes_every_rank_off_it():
    import socket

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    results = mp.Manager().dict()
    mp.spawn(_vote_worker, args=(2, port, results), nprocs=2, join=True)
    assert dict(results) == {0: (True, False), 1: (True, False)}
