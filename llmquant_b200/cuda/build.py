"""`load_extension()` with the reference's contract (llmquant/cuda/build.py:112-135).

The reference compiles four source files on first use and returns a pybind module with
`fake_quant_group`, `wq_gemv`, `wq_gemv_batched` and `wq_gemv_batched_max_rows`. Here the
kernels are already compiled into libllmquant_b200.so; the returned object has the same four
callables with the same arguments, defaults, return values and error phrases
(llmquant/cuda/csrc/fake_quant.cpp:21-51), so `KernelQuantLinear` and `fake_quantize_cuda`
of the reference run on it unchanged.
"""

import functools

import torch

from llmquant_b200 import native


def _require_cuda(t, what):
    if not t.is_cuda:
        raise RuntimeError(f"{what} must be a CUDA tensor")


class _Kernels:
    """Tensor-level shim over the C ABI. Outputs come from torch's caching allocator, so
    the calls stay CUDA-graph capturable; nothing here synchronizes."""

    name = "llmquant_kernels"

    @staticmethod
    def fake_quant_group(x, num_bits, group_size, return_scale=False):
        _require_cuda(x, "x")
        if x.dim() < 1:
            raise RuntimeError("x must have at least one dimension")
        if x.dtype not in native.DTYPE_ID:
            raise RuntimeError(f"x must be float32, float16 or bfloat16, got {x.dtype}")
        if not 2 <= num_bits <= 8:
            raise RuntimeError(f"num_bits must be in [2, 8], got {num_bits}")
        if group_size <= 0:
            raise RuntimeError(f"group_size must be positive, got {group_size}")
        xc = x.contiguous()
        k = xc.shape[-1]
        if k % group_size:
            raise RuntimeError(f"last dim {k} is not divisible by group_size {group_size}")
        out = torch.empty_like(xc)
        if xc.numel() == 0:
            return out.reshape(x.shape), torch.empty(0, dtype=torch.float32, device=x.device)
        groups = xc.numel() // group_size
        if return_scale:
            scale = torch.empty(*xc.shape[:-1], k // group_size, dtype=torch.float32, device=x.device)
        else:
            scale = torch.empty(0, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            native.call("lq_fake_quant_group", xc.data_ptr(), out.data_ptr(),
                        scale.data_ptr() if return_scale else 0, groups, group_size, num_bits,
                        native.DTYPE_ID[x.dtype], native.stream_ptr(x.device))
        return out.reshape(x.shape), scale

    @staticmethod
    def wq_gemv(x, qweight, wscale, out_group=0):
        if not (x.is_cuda and qweight.is_cuda and wscale.is_cuda):
            raise RuntimeError("all tensors must be CUDA")
        if qweight.dim() != 3:
            raise RuntimeError(f"qweight must be [N, groups, group_size], got {qweight.dim()}D")
        if qweight.dtype != torch.int8:
            raise RuntimeError("qweight must be int8")
        if wscale.dtype != torch.float32:
            raise RuntimeError("wscale must be float32")
        if x.dtype not in native.DTYPE_ID:
            raise RuntimeError(f"x must be float32, float16 or bfloat16, got {x.dtype}")
        xc, wc, sc = x.contiguous(), qweight.contiguous(), wscale.contiguous()
        n, groups, group_size = wc.shape
        m = xc.numel() // xc.shape[-1] if xc.shape[-1] else 0
        if group_size % 4:
            raise RuntimeError(f"group_size must be a multiple of 4, got {group_size}")
        if xc.shape[-1] != groups * group_size:
            raise RuntimeError(
                f"x last dim {xc.shape[-1]} does not match qweight {groups}x{group_size}")
        scale_rows = -(-n // out_group) if out_group > 0 else n
        if sc.dim() != 2 or sc.shape[0] != scale_rows or sc.shape[1] != groups:
            raise RuntimeError(
                f"wscale must be [{scale_rows}, {groups}], got {list(sc.shape)}")
        out = torch.empty(m, n, dtype=x.dtype, device=x.device)
        if m == 0 or n == 0:
            return out
        with torch.cuda.device(x.device):
            native.call("lq_wq_gemv", xc.data_ptr(), wc.data_ptr(), sc.data_ptr(), out.data_ptr(),
                        m, n, groups, group_size, int(out_group), native.DTYPE_ID[x.dtype],
                        native.stream_ptr(x.device))
        return out

    @staticmethod
    def wq_gemv_batched_max_rows():
        return int(native.library().lq_wq_gemv_batched_max_rows())

    @staticmethod
    def wq_gemv_batched(x, qweight, wscale, block_expert, block_row0, block_rows, out_group=0):
        """Stacked-expert GEMV: rows of `x` grouped by expert, one (expert, first row, row
        count) triple per block (llmquant/cuda/csrc/wq_gemv_batched.cu:133-185)."""
        if not (x.is_cuda and qweight.is_cuda and wscale.is_cuda):
            raise RuntimeError("tensors must be CUDA")
        if qweight.dim() != 4:
            raise RuntimeError("qweight must be [E, N, groups, group_size]")
        if wscale.dim() != 3:
            raise RuntimeError("wscale must be [E, scale_rows, groups]")
        if qweight.dtype != torch.int8:
            raise RuntimeError("qweight must be int8")
        if wscale.dtype != torch.float32:
            raise RuntimeError("wscale must be float32")
        if x.dtype not in (torch.float16, torch.bfloat16):
            raise RuntimeError("wq_gemv_batched takes float16 or bfloat16 activations")
        xc, qw, ws = x.contiguous(), qweight.contiguous(), wscale.contiguous()
        dev = xc.device
        be = block_expert.to(device=dev, dtype=torch.int32).contiguous()
        br0 = block_row0.to(device=dev, dtype=torch.int32).contiguous()
        brn = block_rows.to(device=dev, dtype=torch.int32).contiguous()
        rows, n, groups, gs = xc.shape[0], qw.shape[1], qw.shape[2], qw.shape[3]
        if xc.shape[1] != groups * gs:
            raise RuntimeError("x width must be groups * group_size")
        if gs % 4 != 0 or gs // 4 > 32:
            raise RuntimeError("group_size must be a multiple of 4 and at most 128")
        out = torch.empty(rows, n, dtype=xc.dtype, device=dev)
        if be.numel() == 0 or rows == 0:
            return out
        with torch.cuda.device(dev):
            native.call("lq_wq_gemv_batched", xc.data_ptr(), qw.data_ptr(), ws.data_ptr(), be.data_ptr(),
                        br0.data_ptr(), brn.data_ptr(), out.data_ptr(), rows, n, groups, gs, ws.shape[1],
                        int(out_group), be.numel(), native.DTYPE_ID[xc.dtype], native.stream_ptr(dev))
        return out


@functools.lru_cache(maxsize=1)
def load_extension(verbose: bool = False):
    """Return the kernel object; raises without a GPU or without the built library."""
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA is not available; the kernels need a GPU to build and run")
    native.library()
    return _Kernels()
