"""Run under torchrun with 2+ ranks (see test_gpu_tp.py): tensor-parallel fused decode of a
seeded tiny Llama, with every all-reduce route (folded into the GEMVs, the separate kernel over
peer memory, NCCL), against the single-GPU fused decoder and against the reference's real-mode
logits (tests/golden/tiny_llama.npz, when the group size divides the golden model's heads).
Prints TP_CHECK_OK on rank 0."""

import os
import sys

import numpy as np
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
    blob = dict(np.load(os.path.join(ROOT, "tests", "golden", "tiny_llama.npz")))
    golden_ok = world == 2  # the golden model: 4 query heads, 2 KV heads
    if golden_ok:
        kw = dict(head_dim=128, hidden=512, inter=1024)
        ids = torch.from_numpy(blob["hd128_tokens"]).to(device)
        n_prompt = blob["hd128_prompt"].shape[1]
        want_logits = blob["hd128_logits"]
    else:
        kw = dict(head_dim=128, hidden=1024, inter=2048, heads=8, kv_heads=world, vocab=512)
        g = torch.Generator().manual_seed(3)
        ids = torch.randint(0, 512, (2, 36), generator=g).to(device)
        n_prompt = 20
    B, total = ids.shape
    new = total - n_prompt

    # single-GPU fused decoder on rank 0, teacher-forced with `ids`
    ref_logits = []
    if rank == 0:
        full = oneshot(tiny_llama(seed=0, **kw).cuda(), quant.to_modifier(mode="kernel"))
        ref = FusedLlamaDecoder(full, B, total + 2, kv_bits=8, use_graph=False)
        ref.prefill(ids[:, :n_prompt])
        for i in range(new - 1):
            ref.tokens.copy_(ids[:, n_prompt + i])
            ref.step()
            ref_logits.append(ref.logits.float().cpu().numpy().copy())
        del ref, full

    ok = True
    notes = []
    routes = [("folded", dict(fused_allreduce=True, peer_allreduce=True)),
              ("kernel", dict(fused_allreduce=False, peer_allreduce=True)),
              ("nccl", dict(fused_allreduce=False, peer_allreduce=False))]
    for name, flags in routes:
        for use_graph in ((False, True) if name == "folded" else (True,)):
            ctx = tp.TPContext(rank, world, **flags)
            sharded = tp.shard_linears_(tiny_llama(seed=0, **kw), ctx).cuda()
            oneshot(sharded, quant.to_modifier(mode="kernel"))
            tp.wrap_for_prefill_(sharded, ctx)
            dec = FusedLlamaDecoder(sharded, B, total + 2, kv_bits=8, tp=ctx, use_graph=use_graph,
                                    gather_logits=True)
            got_route = "folded" if dec.exchange is not None else ("kernel" if dec.peer is not None else "nccl")
            if got_route != name:
                notes.append(f"rank {rank}: wanted {name}, got {got_route}: {dec.peer_error}")
                ok &= name != "folded" or got_route == "folded"
            dec.prefill(ids[:, :n_prompt])
            produced, logits = [], []
            for i in range(new - 1):
                dec.tokens.copy_(ids[:, n_prompt + i])
                dec.step()
                produced.append(dec.tokens.clone())
                logits.append(dec.logits.float().cpu().numpy().copy())
            mine = torch.stack(produced)
            theirs = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(theirs, mine)
            same = all(torch.equal(theirs[0], t) for t in theirs)  # every rank decodes the same tokens
            ok &= same
            if rank == 0:
                logits = np.stack(logits, 1)
                # the token the exchange picked is the argmax of the gathered logits
                picked = mine.T.cpu().numpy()
                ok &= bool((picked == logits.argmax(-1)).all())
                err = rel_l2(logits, np.stack(ref_logits, 1))
                ok &= err <= 1e-2
                line = f"{name} graph={use_graph}: ranks agree={same} rel-L2 vs one GPU {err:.2e}"
                if golden_ok:
                    want = want_logits[:, 1:new]
                    gerr = rel_l2(logits, want)
                    top2 = np.sort(want, -1)[..., -2:]
                    decided = (top2[..., 1] - top2[..., 0]) > 4 * np.abs(logits - want).max(-1)
                    agree = bool((logits.argmax(-1) == want.argmax(-1))[decided].all())
                    ok &= gerr <= 2e-2 and agree
                    line += f", vs the reference's real mode {gerr:.2e} (argmax where decided: {agree})"
                print(line, flush=True)
            try:
                dec.check_device_errors()
            except RuntimeError as exc:
                notes.append(f"rank {rank}: {exc}")
                ok = False
            del dec, sharded
    for n in notes:
        print(n, flush=True)
    flag = torch.tensor([1 if ok else 0], device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("TP_CHECK_OK" if int(flag) == 1 else "TP_CHECK_FAILED", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
