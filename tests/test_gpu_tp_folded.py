"""The tensor-parallel decode step with the all-reduce folded into the GEMVs, on ONE GPU.

The ranks of a group live on one device and their launches are issued in lock step on one
stream (every pushing launch of all ranks before the launch that consumes the sums), so no
kernel ever waits for a kernel that has not been launched yet: the exchange buffers are plain
device memory mapped to themselves. What is checked is the multi-rank arithmetic and the
exchange protocol (partials that signal their own arrival, slots left empty for their next
use, the ready counters); the same kernels over NVLink peer memory are checked by tp_check.py on a
multi-GPU box.

Also here: every bounded device wait of the tensor-parallel kernels is made to run out (a flag
that nothing sets, a limit of about a millisecond) and must come back with its error word set
and the context usable."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import rel_l2, seeded
from llmquant_b200 import native
from llmquant_b200.core import QuantConfig, QuantizationArgs, QuantizationScheme, oneshot
from llmquant_b200.runtime import tp
from llmquant_b200.runtime.tp import PeerExchange

pytestmark = pytest.mark.gpu

SHORT_WAIT = 2_000_000  # SM clocks: about a millisecond


def _module(w, bits):
    from llmquant_b200.quantizers import KernelQuantLinear

    scheme = QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128), input_activations=None)
    linear = torch.nn.Linear(w.shape[1], w.shape[0], bias=False)
    linear.weight.data = w
    return KernelQuantLinear.from_linear(linear.cuda(), scheme)


@pytest.mark.parametrize("world,M,bits,k_shard", [(2, 1, 8, 256), (4, 2, 4, 512), (8, 1, 4, 1792), (8, 1, 8, 512),
                                                   (2, 2, 8, 2048)])
def test_pushed_partials_and_summing_consumer(world, M, bits, k_shard):
    """A row-parallel linear split over `world` ranks pushes its partial rows; the consumer
    builds bf16(bf16(sum in rank order) + residual), stores it and multiplies. Everything is
    compared bit for bit with the same arithmetic done by separate launches and torch ops,
    over several uses of a slot and two steps, and against the oracle's unsplit linear."""
    hidden, n_out, uses = 1024, 512, 3
    w_row = seeded((hidden, world * k_shard), 11, 0.02, torch.bfloat16)
    shards = [_module(w_row[:, r * k_shard:(r + 1) * k_shard].contiguous(), bits) for r in range(world)]
    consumer = _module(seeded((n_out, hidden), 12, 0.02, torch.bfloat16), 8 if bits == 4 else 4)
    gamma = (seeded((hidden,), 13) * 0.1 + 1).bfloat16().cuda()
    exs = PeerExchange.on_one_device(world, M, hidden, torch.device("cuda"))
    lib = native.library()
    for step in range(2):
        for use in range(uses):
            x = (seeded((M, world * k_shard), 100 + 10 * step + use)).bfloat16().cuda()
            residual = seeded((M, hidden), 200 + 10 * step + use).bfloat16().cuda()
            parts = []
            for r, (mod, ex) in enumerate(zip(shards, exs)):
                xr = x[:, r * k_shard:(r + 1) * k_shard].contiguous()
                mod.gemv(xr, out_dtype=torch.float32, pdl=True, tp=ex.push_args(0))
                parts.append(mod.gemv(xr, out_dtype=torch.float32))
            total = torch.zeros(M, hidden, dtype=torch.float32, device="cuda")
            for part in parts:  # rank order, from zero: the kernel's order
                total = total + part
            want_h = (total.bfloat16().float() + residual.float()).bfloat16()
            want_y = consumer.gemv(want_h, norm_weight=gamma, norm_eps=1e-5)
            for ex in exs:
                held = ex.buffer[: world * M * hidden].view(world, M, hidden)
                assert torch.equal(held, torch.stack(parts)), (step, use, ex.rank)
                h = PeerExchange.empty_rows(M, hidden, "cuda")
                residual_in = residual.clone()  # the consumer empties the residual rows it reads
                y = consumer.gemv(h, norm_weight=gamma, norm_eps=1e-5, pdl=True,
                                  tp=ex.sum_args(0, residual_in))
                assert torch.equal(h, want_h), (step, use, ex.rank)
                assert bool((residual_in.view(torch.int16) == -1).all())
                assert torch.equal(y, want_y), (step, use, ex.rank)
                # the consumer left the slot empty for its next use
                assert bool((ex.buffer[: world * M * hidden].view(torch.int32) == -1).all())
            if step == 0 and use == 0:  # the unsplit linear of the oracle
                q, scale = oracle.quantize_weight(w_row.float().numpy(), bits, 128)
                ref = oracle.real_linear(x.float().cpu().numpy(), q, scale, bits, 128)
                assert rel_l2(total.cpu().numpy(), ref) <= 1e-4
    assert lib.lq_gemv_device_error() == 0


def test_summing_consumer_gives_up_when_the_partials_never_arrive():
    hidden, M = 1024, 1
    consumer = _module(seeded((256, hidden), 1, 0.02, torch.bfloat16), 8)
    (ex,) = PeerExchange.on_one_device(1, M, hidden, torch.device("cuda"))
    ex.wait_cycles = SHORT_WAIT
    lib = native.library()
    assert lib.lq_gemv_device_error() == 0
    residual = torch.zeros(M, hidden, dtype=torch.bfloat16, device="cuda")
    h = PeerExchange.empty_rows(M, hidden, "cuda")
    consumer.gemv(h, tp=ex.sum_args(0, residual))  # nothing was pushed
    torch.cuda.synchronize()
    assert lib.lq_gemv_device_error() == 3
    # the context is intact: a complete exchange on fresh buffers works
    (ex2,) = PeerExchange.on_one_device(1, M, hidden, torch.device("cuda"))
    producer = _module(seeded((hidden, 256), 2, 0.02, torch.bfloat16), 8)
    x = seeded((M, 256), 3).bfloat16().cuda()
    producer.gemv(x, out_dtype=torch.float32, tp=ex2.push_args(0))
    PeerExchange.mark_empty(h)
    residual.zero_()
    y = consumer.gemv(h, tp=ex2.sum_args(0, residual))
    want_h = producer.gemv(x, out_dtype=torch.float32).bfloat16()
    assert torch.equal(h, want_h) and torch.equal(y, consumer.gemv(want_h))
    assert lib.lq_gemv_device_error() == 0


def test_allreduce_kernel_gives_up_on_a_missing_peer():
    """lq_allreduce_residual told of two ranks whose second buffer is its own: the second
    rank's flag is never written, the wait runs out, the call returns and reports it."""
    n = 1024
    lib = native.library()
    slot_floats = n
    flag_off = 2 * slot_floats * 4
    buf = torch.zeros(flag_off // 4 + 2 * lib.lq_allreduce_max_world(), dtype=torch.float32, device="cuda")
    peers = torch.tensor([buf.data_ptr(), buf.data_ptr()], dtype=torch.int64, device="cuda")
    seq = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    assert lib.lq_allreduce_device_error() == 0
    native.call("lq_allreduce_residual", peers.data_ptr(), 0, 2, 0, slot_floats, flag_off, seq.data_ptr(), 0,
                out.data_ptr(), n, SHORT_WAIT, 0, native.stream_ptr())
    torch.cuda.synchronize()
    assert lib.lq_allreduce_device_error() == 1
    # a one-rank group on a fresh buffer completes and sums what is there
    buf.zero_()
    buf[:n] = torch.arange(n, dtype=torch.float32, device="cuda")
    seq.zero_()
    native.call("lq_allreduce_residual", peers.data_ptr(), 0, 1, 0, slot_floats, flag_off, seq.data_ptr(), 0,
                out.data_ptr(), n, SHORT_WAIT, 0, native.stream_ptr())
    assert torch.equal(out.float(), torch.arange(n, dtype=torch.float32, device="cuda").bfloat16().float())
    assert lib.lq_allreduce_device_error() == 0 and int(seq) == 1


@pytest.mark.parametrize("B", [1, 2])
def test_token_exchange_picks_like_argmax_and_gives_up_on_a_missing_rank(B):
    V, hist = 4000, 16
    lib = native.library()
    logits = seeded((B, V), 5).bfloat16().cuda()
    logits[0, 3000] = 40.0
    logits[0, 12] = 40.0  # equal maxima: the lower index wins
    (ex,) = PeerExchange.on_one_device(1, B, 1024, torch.device("cuda"))
    tokens = torch.full((B,), -1, dtype=torch.long, device="cuda")
    pos = torch.tensor([4], dtype=torch.long, device="cuda")
    history = torch.zeros(B, hist, dtype=torch.long, device="cuda")
    ticket = torch.zeros(1, dtype=torch.int32, device="cuda")
    for rep in range(3):
        ex.next_token(logits, tokens, pos, history, ticket, pdl=False)
        assert torch.equal(tokens, torch.argmax(logits.float(), -1)) and int(tokens[0]) == 12
        assert int(pos) == 5 + rep and int(ex.step) == rep + 1 and int(ticket) == 0
        assert torch.equal(history[:, 5 + rep], tokens)
    # two ranks, the other's record written by hand: the larger value wins, then the lower index
    exs = PeerExchange.on_one_device(2, B, 1024, torch.device("cuda"))
    records = exs[0].buffer.view(torch.int64)[exs[0].record_off // 8:].view(2, 16, exs[0].max_batch)
    best = logits.float().max(-1).values
    for b in range(B):
        theirs = 60.0 if b == 0 else float(best[b])  # row 0: the other rank wins; row 1: a tie, rank 0's index is lower
        bits = int(torch.tensor(theirs).bfloat16().view(torch.int16)) & 0xFFFF
        records[0, 1, b] = ((V + 77) << 32) | (bits << 16) | 1
    exs[0].next_token(logits, tokens, pos, history, ticket, pdl=False)
    assert int(tokens[0]) == V + 77
    if B > 1:
        assert int(tokens[1]) == int(torch.argmax(logits[1].float()))
    assert lib.lq_glue_device_error() == 0
    # now nothing arrives from the second rank (the tag of step 1 is not there)
    exs[0].wait_cycles = SHORT_WAIT
    exs[0].next_token(logits, tokens, pos, history, ticket, pdl=False)
    torch.cuda.synchronize()
    assert lib.lq_glue_device_error() == 5


def _lockstep(decs):
    """One folded step of every rank, launch by launch; the token is picked on the host side
    of the test (the exchange kernel of one rank would wait for a launch still to come)."""
    gens = [d._folded_launches() for d in decs]
    for _ in zip(*gens):
        pass
    full = torch.cat([d.local_logits for d in decs], dim=1)
    tok = full.float().argmax(-1)
    for d in decs:
        d.logits.copy_(full)
        d.tokens.copy_(tok)
        d.pos.add_(1)
    return full


@pytest.mark.parametrize("world", [2, 4])
def test_folded_decode_of_a_tiny_llama_against_one_gpu_and_the_reference(golden, world):
    """A seeded tiny Llama split over 2 and 4 ranks (all on this GPU), decoded token by token
    from an empty cache with the reference's own tokens fed in: logits against the one-GPU
    fused decoder (split-K summation order is the only difference) and against the
    reference's real-mode logits (tests/golden/tiny_llama.npz)."""
    from llmquant_b200.runtime.decoder import FusedLlamaDecoder
    from oracle.real_mode import tiny_llama

    blob = golden("tiny_llama")
    want_tokens, want_logits = blob["hd128_tokens"], blob["hd128_logits"]
    n_prompt = blob["hd128_prompt"].shape[1]
    kw = dict(head_dim=128, hidden=512, inter=1024, heads=4, kv_heads=4 if world == 4 else 2)
    compare_reference = kw["kv_heads"] == 2  # the golden model has two KV heads
    quant = QuantConfig(attn_weight="int8", mlp_weight="int4", head_weight="int8", kv_cache="int8")
    ids = torch.from_numpy(want_tokens).cuda()
    B, total = ids.shape
    full = oneshot(tiny_llama(seed=0, **kw).cuda(), quant.to_modifier(mode="kernel"))
    single = FusedLlamaDecoder(full, B, total + 2, kv_bits=8, use_graph=False)
    exs = PeerExchange.on_one_device(world, B, kw["hidden"], torch.device("cuda"))
    decs = []
    for r in range(world):
        ctx = tp.TPContext(r, world)
        sharded = tp.shard_linears_(tiny_llama(seed=0, **kw), ctx).cuda()
        oneshot(sharded, quant.to_modifier(mode="kernel"))
        decs.append(FusedLlamaDecoder(sharded, B, total + 2, kv_bits=8, use_graph=False, tp=ctx, exchange=exs[r]))
        assert decs[-1].exchange is exs[r] and decs[-1].launches_per_step == single.launches_per_step
    for d in [single] + decs:
        d.start_empty(ids[:, 0])
    worst = 0.0
    got = []
    for s in range(total - 1):
        for d in [single] + decs:
            d.tokens.copy_(ids[:, s])
        single.step()
        logits = _lockstep(decs)
        worst = max(worst, rel_l2(logits.float().cpu().numpy(), single.logits.float().cpu().numpy()))
        if s >= n_prompt - 1:
            got.append(logits.float().cpu().numpy())
    assert worst <= 1e-2, worst
    for d in decs[1:]:  # every rank holds the same hidden state bit for bit (the other buffer is left empty)
        assert torch.equal(d.h[0].view(torch.int16), decs[0].h[0].view(torch.int16))
        assert bool((d.h[1].view(torch.int16) == -1).all())
    if compare_reference:
        got = np.stack(got, 1)
        assert rel_l2(got, want_logits) <= 2e-2
        top2 = np.sort(want_logits, -1)[..., -2:]
        decided = (top2[..., 1] - top2[..., 0]) > 4 * np.abs(got - want_logits).max(-1)
        assert (got.argmax(-1) == want_logits.argmax(-1))[decided].all()
    lib = native.library()
    assert lib.lq_gemv_device_error() == 0 and lib.lq_attn_device_error() == 0
