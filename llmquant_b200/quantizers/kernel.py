"""`KernelQuantLinear`: the drop-in Linear whose weight stays integer into the CUDA kernels.

Same constructor, `from_linear`, attributes and forward contract as the reference module
(llmquant/quantizers/kernel.py:31-103), so `save_packed_model` / `load_packed_model` and the
modifier treat it identically. What differs is underneath:

  * the weight is quantized on the GPU by the library (bit-identical codes and scales);
  * it is held in the streaming layout -- true nibbles for int4 (0.5 byte per weight in
    HBM, where the reference keeps one byte), head padding stripped, scales group-major --
    (`[N/4, groups, 4]` tiles) -- and the canonical `[N, groups, group_size]` int8 tensor is rebuilt on demand by an
    exact inverse (`.qweight`), so the file format is unchanged;
  * up to DECODE_MAX_ROWS activation rows go through the streaming GEMV; more rows take
    the prefill path.
"""

import ctypes

import torch
import torch.nn as nn

from llmquant_b200 import native
from llmquant_b200.core.scheme import QuantizationScheme

# rows the streaming GEMV accepts; the reference switches to its library-GEMM path above 4
# (llmquant/quantizers/kernel.py:27-28)
KERNEL_MAX_ROWS = 4
DECODE_MAX_ROWS = 8
GEMV_VARIANT = 0  # 0 = library default; see lq_wq_gemv_stream
# Prefill rows: up to PREFILL_EXACT_MAX_ROWS the tcgen05 GEMM keeps the real mode's arithmetic
# (exact integer sums per group, scaled in fp32); from there to PREFILL_TENSOR_CORE_MAX_ROWS it
# multiplies by bf16(code * scale) in one pass over K -- the same weights the reference's
# kernel mode dequantizes for its library GEMM (llmquant/quantizers/kernel.py:68-79), without
# materialising them; above that, and for narrow outputs (too few 128 x 128 tiles to fill the
# GPU), dequantize + library GEMM is still the faster of the two (measured crossover: between
# 512 and 768 rows at the Llama-3-8B shapes; 1024 output features lose at every row count).
DECODE_GEMM_MAX_ROWS = 64
# from this many rows the decode GEMM is the default (measured on B200 at the Llama-3-8B shapes,
# 8 rows: q|k|v 11 vs 25 us, o 9 vs 13, gate|up 32 vs 44, down 17 vs 45 for the GEMV variants)
DECODE_GEMM_MIN_ROWS = 5
# `forward` takes the decode GEMM up to this many rows, the prefill kernels above (measured at
# 128 rows, two passes: faster on down_proj, slower on gate/up and q/o)
FORWARD_DECODE_GEMM_MAX_ROWS = 64
PREFILL_EXACT_MAX_ROWS = 16
PREFILL_TENSOR_CORE_MAX_ROWS = 512
PREFILL_TENSOR_CORE_MIN_FEATURES = 2048


def _canonical_geometry(out_features, in_features, args):
    """Shape of the canonical tensor and its scale table for one Linear."""
    gs = args.group_size
    if args.head_dim:
        if in_features % args.head_dim:
            raise ValueError(
                f"last dim {in_features} is not a multiple of head_dim {args.head_dim}")
        groups = (in_features // args.head_dim) * -(-args.head_dim // gs)
    else:
        groups = -(-in_features // gs)
    scale_rows = -(-out_features // args.out_group) if args.out_group else out_features
    return groups, scale_rows


def quantize_weight_canonical(weight: torch.Tensor, args):
    """GPU quantizer: `[N, K]` weight -> canonical int8 `[N, G, gs]` and fp32 `[scale_rows, G]`.

    The device-side equivalent of quantize_weight + group_view as used by from_linear
    (llmquant/quantizers/real.py:29-47, llmquant/quantizers/kernel.py:60-66)."""
    if not weight.is_cuda:
        raise RuntimeError("weight must be a CUDA tensor: the kernel path has no CPU fallback")
    if weight.dtype not in native.DTYPE_ID:
        raise RuntimeError(f"weight must be float32, float16 or bfloat16, got {weight.dtype}")
    if args.strategy != "group":
        raise ValueError("the kernel path quantizes weights per group along the reduction axis")
    w = weight.detach().contiguous()
    n, k = w.shape
    groups, scale_rows = _canonical_geometry(n, k, args)
    canonical = torch.empty(n, groups, args.group_size, dtype=torch.int8, device=w.device)
    wscale = torch.empty(scale_rows, groups, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        native.call("lq_quantize_weight", w.data_ptr(), native.DTYPE_ID[w.dtype], n, k,
                    args.group_size, args.head_dim or 0, args.out_group or 0, args.num_bits,
                    canonical.data_ptr(), wscale.data_ptr(), native.stream_ptr(w.device))
    return canonical, wscale


def pad_activation(flat, args):
    """Pad x the way the canonical weight's K axis was padded (kernel.py:17-25 of the
    reference). Only the canonical-layout GEMV needs it; the streaming layout does not."""
    gs = args.group_size
    if args.head_dim:
        lead, k = flat.shape[:-1], flat.shape[-1]
        per_head = flat.reshape(*lead, k // args.head_dim, args.head_dim)
        tail = args.head_dim % gs
        if tail:
            per_head = nn.functional.pad(per_head, (0, gs - tail))
        return per_head.reshape(*lead, -1)
    tail = flat.shape[-1] % gs
    return nn.functional.pad(flat, (0, gs - tail)) if tail else flat


class KernelQuantLinear(nn.Module):
    """Linear backed by integer weights in HBM, dequantized inside the kernels."""

    def __init__(self, qweight, wscale, bias, scheme: QuantizationScheme, in_features: int):
        super().__init__()
        if not qweight.is_cuda:
            raise RuntimeError(
                "KernelQuantLinear needs CUDA tensors: the kernel path has no CPU fallback")
        native.library()  # fail here, loudly, if the library was not built
        args = scheme.weights
        self.scheme = scheme
        self.bias = bias
        self.out_features = qweight.shape[0]
        self.in_features = in_features
        self.canonical_shape = tuple(qweight.shape)
        self.padded_in_features = qweight.shape[1] * qweight.shape[2]
        self.out_group = args.out_group or 0
        self.num_bits = args.num_bits
        self._weight_args = args
        self._scale_rows = wscale.shape[0]
        n, groups, gs = qweight.shape
        qweight = qweight.contiguous()
        wscale = wscale.contiguous().float()
        try:
            if args.num_bits not in (4, 8):
                raise RuntimeError("unsupported")
            kd, span, npad = native.stream_layout_sizes(n, groups, gs, args.head_dim, args.num_bits)
            self._stream = True
        except RuntimeError:
            self._stream = False
        if self._stream:
            self._kd, self._span = kd, span
            codes = torch.empty(n, kd * args.num_bits // 8, dtype=torch.uint8, device=qweight.device)
            scale_tiles = torch.empty(npad // 4, groups, 4, dtype=torch.float32, device=qweight.device)
            with torch.cuda.device(qweight.device):
                native.call("lq_repack_stream", qweight.data_ptr(), wscale.data_ptr(),
                            codes.data_ptr(), scale_tiles.data_ptr(), n, groups, gs,
                            args.head_dim or 0, args.num_bits, self.out_group,
                            native.stream_ptr(qweight.device))
            self.register_buffer("codes", codes, persistent=False)
            self.register_buffer("scale_tiles", scale_tiles, persistent=False)
        else:
            # geometry the streaming GEMV does not cover: keep the canonical tensors and use
            # the canonical-layout kernel
            self.register_buffer("_qweight", qweight, persistent=False)
            self.register_buffer("_wscale", wscale, persistent=False)
        self._bias_bf16 = None
        self._tiled = None  # the weight in the decode GEMM's tile-major layout, built on first use

    # ---- construction -----------------------------------------------------------------
    @classmethod
    def from_linear(cls, linear: nn.Linear, scheme: QuantizationScheme):
        if scheme.weights is None:
            raise ValueError("the kernel path needs a weight scheme; bf16 weights stay nn.Linear")
        canonical, wscale = quantize_weight_canonical(linear.weight, scheme.weights)
        return cls(canonical, wscale, linear.bias, scheme, linear.in_features)

    # ---- the reference's tensors, rebuilt exactly -----------------------------------------
    def _unrepack(self):
        n, groups, gs = self.canonical_shape
        dev = self.codes.device
        qweight = torch.empty(n, groups, gs, dtype=torch.int8, device=dev)
        wscale = torch.empty(self._scale_rows, groups, dtype=torch.float32, device=dev)
        with torch.cuda.device(dev):
            native.call("lq_unrepack_stream", self.codes.data_ptr(), self.scale_tiles.data_ptr(),
                        qweight.data_ptr(), wscale.data_ptr(), n, groups, gs,
                        self._weight_args.head_dim or 0, self.num_bits, self.out_group,
                        native.stream_ptr(dev))
        return qweight, wscale

    def canonical_tensors(self):
        """(qweight, wscale) in the reference's layout with one pass of the inverse repack (the
        two properties below each run it)."""
        return self._unrepack() if self._stream else (self._qweight, self._wscale)

    @property
    def qweight(self):
        """Canonical `[N, groups, group_size]` int8 codes (what model.bin stores)."""
        return self._unrepack()[0] if self._stream else self._qweight

    @property
    def wscale(self):
        """`[scale_rows, groups]` fp32 scales."""
        return self._unrepack()[1] if self._stream else self._wscale

    def weight_bytes(self) -> int:
        """Bytes one decode step streams for this layer's weight and scales."""
        if self._stream:
            return self.codes.numel() + self._scale_rows * self.canonical_shape[1] * 4
        return self._qweight.numel() + self._wscale.numel() * 4

    # ---- state dict: the reference's two tensors, although they are not what is stored ----
    # (the reference registers qweight / wscale as persistent buffers, llmquant/quantizers/
    # kernel.py:36-37, so `model.state_dict()` carries the quantized weights there; here they are
    # rebuilt on the way out and repacked on the way in)
    emit_canonical_state = True  # save_packed_model switches this off: it writes them itself, packed

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        super()._save_to_state_dict(destination, prefix, keep_vars)
        if self.emit_canonical_state:
            qweight, wscale = self.canonical_tensors()
            destination[prefix + "qweight"] = qweight
            destination[prefix + "wscale"] = wscale

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys,
                              unexpected_keys, error_msgs):
        qweight, wscale = state_dict.pop(prefix + "qweight", None), state_dict.pop(prefix + "wscale", None)
        if qweight is not None and wscale is not None:
            if tuple(qweight.shape) != self.canonical_shape or wscale.shape[0] != self._scale_rows:
                error_msgs.append(f"{prefix}qweight / wscale: shapes {tuple(qweight.shape)} / "
                                  f"{tuple(wscale.shape)} do not match this layer")
            elif self._stream:
                dev = self.codes.device
                q = qweight.to(device=dev, dtype=torch.int8).contiguous()
                sc = wscale.to(device=dev, dtype=torch.float32).contiguous()
                n, groups, gs = self.canonical_shape
                with torch.cuda.device(dev):
                    native.call("lq_repack_stream", q.data_ptr(), sc.data_ptr(), self.codes.data_ptr(),
                                self.scale_tiles.data_ptr(), n, groups, gs, self._weight_args.head_dim or 0,
                                self.num_bits, self.out_group, native.stream_ptr(dev))
                    torch.cuda.current_stream(dev).synchronize()  # q and sc are temporaries
            else:
                self._qweight.copy_(qweight)
                self._wscale.copy_(wscale)
        elif strict and (qweight is None) != (wscale is None):
            missing_keys.append(prefix + ("qweight" if qweight is None else "wscale"))
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys,
                                      unexpected_keys, error_msgs)

    # ---- forward ------------------------------------------------------------------------
    def _dequantized_weight(self, dtype):
        """Dense `[out, in]` weight in the activation dtype for the library-GEMM path."""
        dev = self.codes.device if self._stream else self._qweight.device
        if not self._stream:
            n, groups, gs = self.canonical_shape
            out = torch.empty(n, groups * gs, dtype=dtype, device=dev)
            with torch.cuda.device(dev):
                native.call("lq_dequant_weight", self._qweight.data_ptr(), self._wscale.data_ptr(),
                            out.data_ptr(), native.DTYPE_ID[dtype], n, groups, gs, self.out_group,
                            native.stream_ptr(dev))
            return out
        out = torch.empty(self.out_features, self.in_features, dtype=dtype, device=dev)
        with torch.cuda.device(dev):
            native.call("lq_dequant_stream", self.codes.data_ptr(), self.scale_tiles.data_ptr(),
                        out.data_ptr(), native.DTYPE_ID[dtype], self.out_features, self.in_features,
                        self._kd, self._span, self.num_bits, native.stream_ptr(dev))
        return out

    def tensor_core_gemv_ok(self, m: int) -> bool:
        """Whether GEMV variant 4 (tensor-core integer products) serves `m` rows of this layer."""
        return bool(self._stream and native.library().lq_gemv_tensor_core_ok(m, self._kd, self._span, self.num_bits))

    def gemv(self, flat, out_dtype=None, residual=None, variant=None, norm_weight=None,
             norm_eps=1e-5, epilogue=0, pdl=False, out=None, tp=None, workspace=None):
        """Streaming GEMV on `[M, K]` bf16 rows -> `[M, N]` (bf16 or fp32), 8 rows per launch.

        Optional fusions (see `lq_wq_gemv_fused`): RMSNorm of the input rows by `norm_weight`,
        `epilogue=1` for silu(gate) * up over interleaved (gate, up) rows, a residual added to
        the output, and `pdl` to overlap the weight prefetch with the previous kernel.
        `tp` (a `native.GemvTp`) couples the launch to the other ranks of a tensor-parallel
        group: as a pushing row-parallel linear (no `out`: the partial rows go to the ranks'
        exchange buffers) or as the consumer that first builds `flat` from the ranks' partials.
        More than 8 rows (or `variant=5`) go through the tensor-core decode GEMM, which streams
        the weight once for up to 64 rows; `workspace` is its scratch (a uint8 tensor of
        `decode_workspace_bytes(rows)`; allocated per call when absent)."""
        m = flat.shape[0]
        out_dtype = out_dtype or torch.bfloat16
        n_out = self.out_features // 2 if epilogue == 1 else self.out_features
        pushing = tp is not None and tp.mode == native.TP_PUSH
        if out is None and not pushing:
            out = torch.empty(m, n_out, dtype=out_dtype, device=flat.device)
        if m == 0:
            return out
        gemm_rows = m > DECODE_MAX_ROWS or (m >= DECODE_GEMM_MIN_ROWS and variant in (None, 0) and tp is None
                                            and self._span == 128)
        if gemm_rows or variant == 5:
            if tp is not None:
                raise RuntimeError(f"the tensor-parallel coupling takes the rows of one pass ({m} given)")
            if variant == 5 and self._span != 128:
                raise RuntimeError(f"the decode GEMM needs scale groups of 128 stored codes (this weight: {self._span})")
            if self._span == 128 and variant in (None, 0, 5):
                return self._decode_gemm(flat, out, out_dtype, residual, norm_weight, norm_eps, epilogue, pdl,
                                         workspace)
            return self._gemv_row_blocks(flat, out, out_dtype, residual, variant, norm_weight, norm_eps,
                                         epilogue, pdl)
        bias = None
        if self.bias is not None:
            if self._bias_bf16 is None or self._bias_bf16.device != flat.device:
                self._bias_bf16 = self.bias.detach().to(device=flat.device, dtype=torch.bfloat16).contiguous()
            bias = self._bias_bf16
        if flat.stride(-1) != 1:
            flat = flat.contiguous()
        args = native.GemvArgs(
            x=flat.data_ptr(), ldx=flat.stride(0), norm_weight=native.ptr(norm_weight),
            norm_eps=norm_eps, codes=self.codes.data_ptr(), scale_tiles=self.scale_tiles.data_ptr(),
            bias=native.ptr(bias), residual=native.ptr(residual), out=native.ptr(out),
            out_dtype=native.DTYPE_ID[out_dtype], M=m, N=self.out_features, K=self.in_features,
            Kd=self._kd, span=self._span, bits=self.num_bits, epilogue=epilogue,
            variant=GEMV_VARIANT if variant is None else variant, pdl=1 if pdl else 0,
            tp=ctypes.addressof(tp) if tp is not None else None)
        with torch.cuda.device(flat.device):
            native.call("lq_wq_gemv_fused", ctypes.byref(args), native.stream_ptr(flat.device))
        return out

    def decode_workspace_bytes(self, rows: int) -> int:
        """Scratch bytes of the decode GEMM for up to `rows` activation rows per call."""
        rows = min(max(rows, 1), DECODE_GEMM_MAX_ROWS)
        return int(native.library().lq_decode_gemm_workspace_bytes(rows, self.out_features, self._kd))

    def tiled_weight(self):
        """The weight in the tile-major layout the decode GEMM streams (`lq_tile_weight`): a
        second copy of the codes (with their scales), built on first use and kept with the module."""
        if self._tiled is None or self._tiled.device != self.codes.device:
            dev = self.codes.device
            nbytes = native.library().lq_tile_weight_bytes(self.out_features, self._kd, self.num_bits)
            tiled = torch.empty(nbytes, dtype=torch.uint8, device=dev)
            with torch.cuda.device(dev):
                native.call("lq_tile_weight", self.codes.data_ptr(), self.scale_tiles.data_ptr(), tiled.data_ptr(),
                            self.out_features, self._kd, self.num_bits, native.stream_ptr(dev))
            self._tiled = tiled
        return self._tiled

    def _decode_gemm(self, flat, out, out_dtype, residual, norm_weight, norm_eps, epilogue, pdl, workspace):
        """Rows through the tensor-core decode GEMM (variant 5 of `lq_wq_gemv_fused`), 64 per
        call: activation planes, one pass over the weight, finish -- three launches."""
        m = flat.shape[0]
        tiled = self.tiled_weight()
        bias = None
        if self.bias is not None:
            if self._bias_bf16 is None or self._bias_bf16.device != flat.device:
                self._bias_bf16 = self.bias.detach().to(device=flat.device, dtype=torch.bfloat16).contiguous()
            bias = self._bias_bf16
        if flat.stride(-1) != 1:
            flat = flat.contiguous()
        need = self.decode_workspace_bytes(m)
        if workspace is None:
            workspace = torch.empty(need, dtype=torch.uint8, device=flat.device)
        elif workspace.numel() * workspace.element_size() < need or workspace.device != flat.device:
            raise ValueError(f"the decode GEMM needs {need} bytes of workspace on {flat.device}")
        es, n_out = out.element_size(), out.shape[1]
        stream = native.stream_ptr(flat.device)
        with torch.cuda.device(flat.device):
            for m0 in range(0, m, DECODE_GEMM_MAX_ROWS):
                rows = min(DECODE_GEMM_MAX_ROWS, m - m0)
                off = m0 * n_out * es
                args = native.GemvArgs(
                    x=flat.data_ptr() + m0 * flat.stride(0) * 2, ldx=flat.stride(0),
                    norm_weight=native.ptr(norm_weight), norm_eps=norm_eps, codes=tiled.data_ptr(),
                    scale_tiles=tiled.data_ptr(), bias=native.ptr(bias),
                    residual=(residual.data_ptr() + off) if residual is not None else None,
                    out=out.data_ptr() + off, out_dtype=native.DTYPE_ID[out_dtype], M=rows, N=self.out_features,
                    K=self.in_features, Kd=self._kd, span=self._span, bits=self.num_bits, epilogue=epilogue,
                    variant=5, pdl=1 if pdl else 0, tp=None, ldo=n_out, workspace=workspace.data_ptr(),
                    workspace_bytes=workspace.numel() * workspace.element_size())
                native.call("lq_wq_gemv_fused", ctypes.byref(args), stream)
        return out

    def _gemv_row_blocks(self, flat, out, out_dtype, residual, variant, norm_weight, norm_eps, epilogue, pdl):
        """More activation rows than one GEMV launch takes (8) on a weight the decode GEMM does
        not serve (scale groups other than 128 codes): one pass over the weight per 8 rows."""
        for m0 in range(0, flat.shape[0], DECODE_MAX_ROWS):
            rows = slice(m0, m0 + DECODE_MAX_ROWS)
            self.gemv(flat[rows], out_dtype=out_dtype, residual=None if residual is None else residual[rows],
                      variant=variant, norm_weight=norm_weight, norm_eps=norm_eps, epilogue=epilogue, pdl=pdl,
                      out=out[rows])
        return out

    def gemm(self, flat, a8: bool = False, fold_scales: bool = False, serial: bool = False):
        """Prefill GEMM on the tensor cores for any number of rows: `[M, K]` bf16 -> `[M, N]`
        bf16. `a8=True` quantizes the activations per token per group to int8 first (the
        reference's dynamic activation scheme) and multiplies integers. `fold_scales=True`
        (bf16 activations only) multiplies by `bf16(code * scale)`, the weight the reference's
        kernel mode dequantizes for its library GEMM, instead of scaling exact integer sums
        per group: faster, with that mode's rounding. `serial=True` runs the unpipelined kernel
        (fill, MMA and drain in turn), which otherwise only serves shapes the warp-specialized
        kernels do not take; same results."""
        m = flat.shape[0]
        out = torch.empty(m, self.out_features, dtype=torch.bfloat16, device=flat.device)
        if m == 0:
            return out
        flat = flat.contiguous()
        bias = None
        if self.bias is not None:
            if self._bias_bf16 is None or self._bias_bf16.device != flat.device:
                self._bias_bf16 = self.bias.detach().to(device=flat.device, dtype=torch.bfloat16).contiguous()
            bias = self._bias_bf16
        x_codes = x_scales = None
        if a8:
            if self._kd != self.in_features:
                flat = nn.functional.pad(flat, (0, self._kd - self.in_features))
            groups = self._kd // self._span
            x_codes = torch.empty(m, self._kd, dtype=torch.int8, device=flat.device)
            x_scales = torch.empty(m, groups, dtype=torch.float32, device=flat.device)
            with torch.cuda.device(flat.device):
                native.call("lq_quantize_group_i8", flat.data_ptr(), x_codes.data_ptr(),
                            x_scales.data_ptr(), m * groups, self._span, 8, native.LQ_BF16,
                            native.stream_ptr(flat.device))
        with torch.cuda.device(flat.device):
            native.call("lq_wq_gemm_prefill", flat.data_ptr(), flat.stride(0), native.ptr(x_codes),
                        native.ptr(x_scales), self.codes.data_ptr(), self.scale_tiles.data_ptr(),
                        native.ptr(bias), out.data_ptr(), m, self.out_features, self.in_features,
                        self._kd, self._span, self.num_bits,
                        (native.GEMM_FOLD_SCALES if (fold_scales and not a8) else 0)
                        | (native.GEMM_SERIAL if serial else 0),
                        native.stream_ptr(flat.device))
        return out

    def forward(self, x):
        if not x.is_cuda:
            raise RuntimeError("x must be a CUDA tensor: the kernel path has no CPU fallback")
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        m = flat.shape[0]
        if self._stream and flat.dtype == torch.bfloat16 and (
                m <= DECODE_MAX_ROWS or (m <= FORWARD_DECODE_GEMM_MAX_ROWS and self._span == 128)):
            # up to 8 rows the GEMV, up to 64 the decode GEMM (one pass over the weight; faster
            # than the prefill kernels' 128-token tiles at these row counts)
            out = self.gemv(flat)
        elif (self._stream and m <= PREFILL_TENSOR_CORE_MAX_ROWS and flat.dtype == torch.bfloat16
              and (self.out_features >= PREFILL_TENSOR_CORE_MIN_FEATURES or m <= PREFILL_EXACT_MAX_ROWS)
              and self._span in (64, 128)):
            out = self.gemm(flat, fold_scales=m > PREFILL_EXACT_MAX_ROWS)
        elif not self._stream and m <= DECODE_MAX_ROWS:
            from llmquant_b200.cuda.build import load_extension

            padded = pad_activation(flat, self._weight_args)
            out = load_extension().wq_gemv(padded, self._qweight, self._wscale, self.out_group)
            if self.bias is not None:
                out = out + self.bias.to(out.dtype)
        else:
            weight = self._dequantized_weight(flat.dtype)
            if not self._stream:
                flat = pad_activation(flat, self._weight_args)
            out = flat @ weight.T
            if self.bias is not None:
                out = out + self.bias.to(out.dtype)
        return out.reshape(*shape[:-1], self.out_features).to(x.dtype)

    def extra_repr(self):
        act = self.scheme.input_activations
        return (
            f"in_features={self.in_features}, out_features={self.out_features}, "
            f"w{self.num_bits}a{act.num_bits if act else 16}, "
            f"group_size={self._weight_args.group_size}, layout="
            f"{'stream' if self._stream else 'canonical'}"
        )
