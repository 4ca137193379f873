"""`KernelQuantExperts`: a stack of Mixture-of-Experts feed-forward weights held as integers,
with every routed (token, expert) product of a decode step done by ONE stacked-expert GEMV
launch per projection.

Same constructor arguments, buffers (`qgate_up`, `sgate_up`, `qdown`, `sdown`), `from_experts`
and `forward(hidden_states, top_k_index, top_k_weights)` contract as the reference module
(llmquant/quantizers/kernel.py:128-289). The routing plan -- rows sorted by expert, one
(expert, first row, row count) triple per block -- is built with device-side tensor ops only,
so a step never waits for the host and can be captured in a CUDA graph.
"""

import torch
import torch.nn as nn

from llmquant_b200.core.scheme import QuantizationScheme
from llmquant_b200.cuda import load_extension
from llmquant_b200.quantizers.kernel import KERNEL_MAX_ROWS, pad_activation, quantize_weight_canonical


def quantize_expert_stack(weights: torch.Tensor, args):
    """`[E, N, K]` expert weights -> canonical int8 `[E, N, G, gs]` and fp32 `[E, rows, G]`,
    each expert quantized exactly as a Linear of its own would be."""
    codes, scales = zip(*(quantize_weight_canonical(w, args) for w in weights))
    return torch.stack(codes), torch.stack(scales)


class KernelQuantExperts(nn.Module):
    """Stands in for a fused experts module (gate_up_proj `[E, 2I, H]`, down_proj `[E, H, I]`)."""

    def __init__(self, qgate_up, sgate_up, qdown, sdown, scheme: QuantizationScheme, hidden_dim,
                 intermediate_dim, act_fn):
        super().__init__()
        self.register_buffer("qgate_up", qgate_up)  # [E, 2I, G, gs] int8
        self.register_buffer("sgate_up", sgate_up)  # [E, scale_rows, G] fp32
        self.register_buffer("qdown", qdown)
        self.register_buffer("sdown", sdown)
        self.scheme = scheme
        self.num_experts = qgate_up.shape[0]
        self.hidden_dim = hidden_dim
        self.intermediate_dim = intermediate_dim
        self.act_fn = act_fn
        self._weight_args = scheme.weights
        kernels = load_extension()
        self._gemv = kernels.wq_gemv
        self._gemv_batched = kernels.wq_gemv_batched
        self._batched_max_rows = kernels.wq_gemv_batched_max_rows()

    @classmethod
    def from_experts(cls, experts: nn.Module, scheme: QuantizationScheme):
        if scheme.weights is None:
            raise ValueError("the kernel path needs a weight scheme")
        qgate_up, sgate_up = quantize_expert_stack(experts.gate_up_proj.data, scheme.weights)
        qdown, sdown = quantize_expert_stack(experts.down_proj.data, scheme.weights)
        return cls(qgate_up, sgate_up, qdown, sdown, scheme,
                   hidden_dim=experts.gate_up_proj.shape[2], intermediate_dim=experts.down_proj.shape[2],
                   act_fn=experts.act_fn)

    # ---- helpers ----------------------------------------------------------------------------
    def _padded(self, x, qweight):
        """x widened to the canonical K axis of `qweight` (zero columns where it was padded)."""
        if x.shape[-1] != qweight.shape[-2] * qweight.shape[-1]:
            x = pad_activation(x, self._weight_args)
        return x

    def _plan(self, top_k_index):
        """Sort order of the routed rows by expert and the kernel's block list, all on device.

        Every expert gets ceil(rows / limit) block slots; slots beyond its share carry zero
        rows and cost nothing. Sizes depend on shapes only, never on the routing itself."""
        flat = top_k_index.reshape(-1)
        order = torch.argsort(flat, stable=True)
        counts = torch.zeros(self.num_experts, dtype=torch.int64, device=flat.device)
        counts.scatter_add_(0, flat, torch.ones_like(flat))
        first = torch.cumsum(counts, 0) - counts
        limit = self._batched_max_rows
        slots = -(-flat.numel() // limit)
        step = torch.arange(slots, device=flat.device, dtype=torch.int64) * limit
        block_expert = torch.arange(self.num_experts, device=flat.device).repeat_interleave(slots)
        taken = step.repeat(self.num_experts)
        block_row0 = first.repeat_interleave(slots) + taken
        block_rows = (counts.repeat_interleave(slots) - taken).clamp(0, limit)
        return order, (block_expert.int(), block_row0.int(), block_rows.int())

    def _one_expert(self, x, qweight, wscale):
        """One expert's projection of a few rows (kernel) or many rows (dense product)."""
        x = self._padded(x, qweight)
        if x.shape[0] <= KERNEL_MAX_ROWS:
            return self._gemv(x, qweight, wscale, 0)
        spread = wscale.repeat_interleave(qweight.shape[0] // wscale.shape[0], dim=0).unsqueeze(-1)
        dense = (qweight * spread).to(x.dtype).reshape(qweight.shape[0], -1)
        return x @ dense.T

    # ---- forward ----------------------------------------------------------------------------
    def forward(self, hidden_states, top_k_index, top_k_weights):
        # a token never picks one expert twice, so no expert sees more rows than there are
        # tokens: the shape alone says whether the stacked kernel applies
        if hidden_states.shape[0] > self._batched_max_rows:
            return self._forward_per_expert(hidden_states, top_k_index, top_k_weights)
        with torch.no_grad():
            order, plan = self._plan(top_k_index)
        k = top_k_index.shape[-1]
        token_of_row, slot_of_row = order // k, order % k
        rows = hidden_states[token_of_row]
        fused = self._gemv_batched(self._padded(rows, self.qgate_up), self.qgate_up, self.sgate_up, *plan, 0)
        gate, up = fused.chunk(2, dim=-1)
        mid = self.act_fn(gate) * up
        out = self._gemv_batched(self._padded(mid, self.qdown), self.qdown, self.sdown, *plan, 0)
        out = out * top_k_weights[token_of_row, slot_of_row, None]
        final = torch.zeros_like(hidden_states)
        final.index_add_(0, token_of_row, out.to(final.dtype))
        return final

    def _forward_per_expert(self, hidden_states, top_k_index, top_k_weights):
        """Prefill-sized inputs: one expert at a time."""
        final = torch.zeros_like(hidden_states)
        for expert in torch.unique(top_k_index).tolist():
            token_idx, slot = torch.where(top_k_index == expert)
            tokens = hidden_states[token_idx]
            gate, up = self._one_expert(tokens, self.qgate_up[expert], self.sgate_up[expert]).chunk(2, dim=-1)
            out = self._one_expert(self.act_fn(gate) * up, self.qdown[expert], self.sdown[expert])
            final.index_add_(0, token_idx, (out * top_k_weights[token_idx, slot, None]).to(final.dtype))
        return final

    def extra_repr(self):
        return (f"num_experts={self.num_experts}, hidden={self.hidden_dim}, intermediate={self.intermediate_dim}, "
                f"w{self.scheme.weights.num_bits}, group_size={self.scheme.weights.group_size}")
