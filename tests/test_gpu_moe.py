"""The stacked-expert decode GEMV (`wq_gemv_batched`) and `KernelQuantExperts` on top of it:
bit-exact against the one-expert-at-a-time kernel path, and within the layer tolerance of
the numpy oracle's real-mode product per expert."""

import numpy as np
import pytest
import torch

import oracle
from gpu_util import rel_l2, seeded
from llmquant_b200.core import QuantizationArgs, QuantizationScheme

pytestmark = pytest.mark.gpu


def _scheme(bits):
    return QuantizationScheme(
        weights=QuantizationArgs(num_bits=bits, strategy="group", group_size=128), input_activations=None)


class _Experts(torch.nn.Module):
    def __init__(self, e, hidden, inter, seed):
        super().__init__()
        self.gate_up_proj = torch.nn.Parameter(seeded((e, 2 * inter, hidden), seed, 0.05, torch.bfloat16))
        self.down_proj = torch.nn.Parameter(seeded((e, hidden, inter), seed + 1, 0.05, torch.bfloat16))
        self.act_fn = torch.nn.functional.silu


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_batched_gemv_equals_the_looped_kernel_and_the_oracle(bits, dtype):
    from llmquant_b200.cuda import load_extension
    from llmquant_b200.quantizers import quantize_expert_stack

    kernels = load_extension()
    e, n, k = 6, 200, 300  # ragged: N not a multiple of 4, K padded to 384
    weights = seeded((e, n, k), 3, 0.05, torch.bfloat16).cuda()
    q, s = quantize_expert_stack(weights, _scheme(bits).weights)
    kp = q.shape[2] * q.shape[3]
    counts = [3, 0, 8, 1, 11, 2]  # expert 4 needs two blocks, expert 1 none
    rows = sum(counts)
    x = torch.nn.functional.pad(seeded((rows, k), 4).to(dtype), (0, kp - k)).cuda()
    limit = kernels.wq_gemv_batched_max_rows()
    be, b0, bn, start = [], [], [], 0
    for ex, c in enumerate(counts):
        for off in range(0, max(c, 1), limit):
            be.append(ex); b0.append(start + off); bn.append(max(0, min(limit, c - off)))
        start += c
    out = kernels.wq_gemv_batched(x, q, s, torch.tensor(be), torch.tensor(b0), torch.tensor(bn), 0)
    assert out.shape == (rows, n) and out.dtype == dtype
    start = 0
    for ex, c in enumerate(counts):
        if c == 0:
            continue
        rows_x = x[start:start + c]
        looped = torch.cat([kernels.wq_gemv(rows_x[i:i + 4], q[ex], s[ex], 0) for i in range(0, c, 4)])
        assert torch.equal(out[start:start + c], looped), ex
        qw, sc = oracle.quantize_weight(weights[ex].float().cpu().numpy(), bits, 128)
        want = oracle.real_linear(rows_x[:, :k].float().cpu().numpy(), qw, sc, bits, 128)
        assert rel_l2(out[start:start + c].float().cpu().numpy(), want) <= 2e-3, ex
        start += c


def test_batched_gemv_argument_checks():
    from llmquant_b200.cuda import load_extension

    kernels = load_extension()
    q = torch.zeros(2, 8, 1, 128, dtype=torch.int8, device="cuda")
    s = torch.ones(2, 8, 1, device="cuda")
    x = torch.zeros(1, 128, dtype=torch.bfloat16, device="cuda")
    idx = torch.zeros(1, dtype=torch.int32)
    with pytest.raises(RuntimeError, match=r"qweight must be \[E, N, groups, group_size\]"):
        kernels.wq_gemv_batched(x, q[0], s, idx, idx, idx + 1, 0)
    with pytest.raises(RuntimeError, match="x width must be groups"):
        kernels.wq_gemv_batched(x[:, :64], q, s, idx, idx, idx + 1, 0)
    empty = kernels.wq_gemv_batched(x, q, s, idx[:0], idx[:0], idx[:0], 0)
    assert empty.shape == (1, 8)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("tokens", [1, 3, 8, 20])
def test_experts_module_routes_like_a_per_expert_loop(bits, tokens):
    from llmquant_b200.quantizers import KernelQuantExperts

    e, hidden, inter, top_k = 8, 256, 384, 2
    experts = _Experts(e, hidden, inter, 20).cuda()
    module = KernelQuantExperts.from_experts(experts, _scheme(bits))
    h = seeded((tokens, hidden), 30).bfloat16().cuda()
    g = torch.Generator().manual_seed(tokens)
    index = torch.stack([torch.randperm(e, generator=g)[:top_k] for _ in range(tokens)]).cuda()
    weight = torch.rand(tokens, top_k, generator=g).bfloat16().cuda()
    got = module(h, index, weight)
    # the same arithmetic, one (token, expert) pair at a time through the one-expert kernel
    want = torch.zeros_like(h)
    for t in range(tokens):
        for j in range(top_k):
            ex = int(index[t, j])
            gate, up = module._gemv(h[t:t + 1], module.qgate_up[ex], module.sgate_up[ex], 0).chunk(2, dim=-1)
            out = module._gemv(torch.nn.functional.silu(gate) * up, module.qdown[ex], module.sdown[ex], 0)
            want[t] += (out * weight[t, j]).to(want.dtype)[0]
    # index_add_ sums a token's experts in routing-sorted order, the loop in slot order: bf16
    # additions in a different order, so compare at the layer tolerance, not bit for bit; with
    # more tokens than the stacked kernel takes, experts that see more than four rows go
    # through bf16-dequantized weights (the reference's choice too), hence the looser bound
    assert rel_l2(got.float().cpu().numpy(), want.float().cpu().numpy()) <= (4e-3 if tokens <= 8 else 1e-2)
    # and against the dequantized weights in fp32
    ref = torch.zeros(tokens, hidden)
    for t in range(tokens):
        for j in range(top_k):
            ex = int(index[t, j])
            wgu = (module.qgate_up[ex].float() * module.sgate_up[ex].unsqueeze(-1)).reshape(2 * inter, -1)[:, :hidden].cpu()
            wd = (module.qdown[ex].float() * module.sdown[ex].unsqueeze(-1)).reshape(hidden, -1)[:, :inter].cpu()
            gate, up = (h[t].float().cpu() @ wgu.T).chunk(2)
            ref[t] += (torch.nn.functional.silu(gate) * up) @ wd.T * weight[t, j].float().cpu()
    assert rel_l2(got.float().cpu().numpy(), ref.numpy()) <= 2e-2
