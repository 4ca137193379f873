import torch
import torch.nn.functional as F

from llmquant_b200.cuda.build import load_extension


def fake_quantize_cuda(x: torch.Tensor, args, return_scale: bool = False):
    """Quant-dequant on the GPU, bit-exact with the reference's `fake_quantize`.

    Same contract as llmquant/cuda/ops.py:8-29: groups run along the last axis, "channel" and
    "token" are the one-group case, and a last axis that is not a whole number of groups is
    zero-padded for the kernel and trimmed afterwards (a zero cannot move an abs-max).
    """
    if args.strategy == "group":
        group_size = args.group_size
    elif args.strategy in ("channel", "token"):
        group_size = x.shape[-1]
    else:
        raise ValueError(f"unsupported strategy {args.strategy!r}")
    width = x.shape[-1]
    tail = width % group_size
    padded = F.pad(x, (0, group_size - tail)) if tail else x
    out, scale = load_extension().fake_quant_group(padded, args.num_bits, group_size, return_scale)
    if tail:
        out = out[..., :width]
    return (out, scale) if return_scale else out
