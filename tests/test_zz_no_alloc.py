"""The decode attention that brings its own scratch memory.

A host that cannot allocate on the device -- a plugin living inside another allocator's
process, a sandbox without cudaMalloc -- calls lq_attn_decode_kv_i8_static, which keeps the
slices' partial results in a fixed array inside the library. It must give what the regular
entry point gives with a caller-provided buffer, call after call (the array is reused and
keeps the previous call's contents), and refuse shapes the array cannot hold.

This file is collected last on purpose, so a run that stops at the first failure has already
run every other test. It does not depend on them: it also passes alone in a fresh process.
"""

import numpy as np
import pytest
import torch

from llmquant_b200 import native

pytestmark = pytest.mark.gpu


def _inputs(B, Hq, Hkv, D, T, Tmax, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(B, Hq, D, generator=g).bfloat16().cuda()
    kc = torch.randint(-127, 128, (B, Hkv, Tmax, D), generator=g, dtype=torch.int8).cuda()
    vc = torch.randint(-127, 128, (B, Hkv, Tmax, D), generator=g, dtype=torch.int8).cuda()
    ks = (torch.rand(B, Hkv, Tmax, 1, generator=g) * 0.02 + 0.001).cuda()
    vs = (torch.rand(B, Hkv, Tmax, 1, generator=g) * 0.02 + 0.001).cuda()
    return q, kc, vc, ks, vs


def _regular(q, kc, vc, ks, vs, T, splits):
    B, Hq, D = q.shape
    Hkv, Tmax = kc.shape[1], kc.shape[2]
    nbytes = native.library().lq_attn_decode_scratch_bytes(B, Hq, D, splits)
    scratch = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device="cuda")
    native.call("lq_attn_decode_kv_i8", q.data_ptr(), kc.data_ptr(), vc.data_ptr(), ks.data_ptr(),
                vs.data_ptr(), out.data_ptr(), scratch.data_ptr(), B, Hq, Hkv, D, Tmax, 0, T, 0,
                D ** -0.5, splits, 0, native.stream_ptr())
    return out


def _static(q, kc, vc, ks, vs, T, splits):
    B, Hq, D = q.shape
    Hkv, Tmax = kc.shape[1], kc.shape[2]
    out = torch.empty(B, Hq, D, dtype=torch.bfloat16, device="cuda")
    with torch.cuda.device(q.device):  # the built-in array is the current device's: make it the tensors'
        native.call("lq_attn_decode_kv_i8_static", q.data_ptr(), kc.data_ptr(), vc.data_ptr(),
                    ks.data_ptr(), vs.data_ptr(), out.data_ptr(), B, Hq, Hkv, D, Tmax, 0, T, 0,
                    D ** -0.5, splits, 0, native.stream_ptr(q.device))
    return out


def test_static_scratch_attention_matches_the_regular_entry_point_twice_in_a_row():
    assert native.library().lq_attn_decode_static_scratch_bytes() == 4 << 20
    # two different problems back to back: the second call meets the first one's leftovers
    first = _inputs(2, 8, 2, 128, 700, 768, seed=1)
    second = _inputs(1, 8, 2, 64, 333, 512, seed=2)
    for inputs, T, splits in ((first, 700, 9), (second, 333, 5), (first, 700, 9)):
        want = _regular(*inputs, T, splits)
        got = _static(*inputs, T, splits)
        torch.cuda.synchronize()
        # same kernels, same slicing: the results are bit-identical, well inside the 1e-2
        # rel-L2 the attention tests allow
        assert torch.equal(got, want)
        err = np.linalg.norm((got.float() - want.float()).cpu().numpy())
        assert err == 0.0


def test_static_scratch_rejects_what_it_cannot_hold():
    q, kc, vc, ks, vs = _inputs(8, 32, 8, 128, 64, 64, seed=3)
    with pytest.raises(RuntimeError, match="built-in array holds"):
        _static(q, kc, vc, ks, vs, 64, 64)  # 8 * 32 * 64 * 130 * 4 bytes > 4 MiB
