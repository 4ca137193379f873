"""Save a kernel-mode model into one `model.bin` and load it back without a bf16 copy.

File contents and metadata keys are those of llmquant/packing/model_io.py:40-231: per
quantized layer `{name}.qweight` (canonical codes, nibble-packed for int4), `{name}.wscale`,
optional `{name}.bias`, and a `layers` record (in/out features, canonical_shape, weights and
input_activations args, bias flag); every other state tensor as bf16; non-persistent buffers
in their own dtype; `kv_cache_bits`. Loading differs only in where the work happens: packed
bytes are uploaded as they are and unpacked on the GPU.
"""

import torch
import torch.nn as nn

from llmquant_b200.core.scheme import QuantizationArgs, QuantizationScheme
from llmquant_b200.packing.format import read_header, read_packed, write_packed
from llmquant_b200.packing.packing import pack_weight, unpack_weight
from llmquant_b200.quantizers.experts import KernelQuantExperts
from llmquant_b200.quantizers.kernel import KernelQuantLinear

_ARG_FIELDS = ("num_bits", "strategy", "group_size", "head_dim", "out_group", "symmetric", "dynamic")


def _args_to_dict(args):
    return None if args is None else {field: getattr(args, field) for field in _ARG_FIELDS}


def _args_from_dict(payload):
    return None if payload is None else QuantizationArgs(**payload)


def save_packed_model(model: nn.Module, path, model_id: str, kv_cache_bits=None, extra=None):
    tensors, layers = {}, {}
    for name, module in model.named_modules():
        if not isinstance(module, KernelQuantLinear):
            continue
        args = module.scheme.weights
        qweight, wscale = module.canonical_tensors()  # one un-repack per layer
        tensors[f"{name}.qweight"] = pack_weight(qweight, args.num_bits)
        tensors[f"{name}.wscale"] = wscale
        layers[name] = {
            "in_features": module.in_features,
            "out_features": module.out_features,
            "canonical_shape": list(module.canonical_shape),
            "weights": _args_to_dict(args),
            "input_activations": _args_to_dict(module.scheme.input_activations),
            "bias": module.bias is not None,
        }
        if module.bias is not None:
            tensors[f"{name}.bias"] = module.bias

    # a Mixture-of-Experts block is one module holding every expert: one record with its two
    # stacked tensors, packed along the group axis like a single weight
    # (llmquant/packing/model_io.py:67-95 of the reference)
    experts = {}
    for name, module in model.named_modules():
        if not isinstance(module, KernelQuantExperts):
            continue
        args = module.scheme.weights
        tensors[f"{name}.qgate_up"] = pack_weight(module.qgate_up, args.num_bits)
        tensors[f"{name}.sgate_up"] = module.sgate_up
        tensors[f"{name}.qdown"] = pack_weight(module.qdown, args.num_bits)
        tensors[f"{name}.sdown"] = module.sdown
        experts[name] = {
            "num_experts": module.num_experts,
            "hidden_dim": module.hidden_dim,
            "intermediate_dim": module.intermediate_dim,
            "gate_up_shape": list(module.qgate_up.shape),
            "down_shape": list(module.qdown.shape),
            "weights": _args_to_dict(args),
            "input_activations": _args_to_dict(module.scheme.input_activations),
        }

    owned = tuple(f"{layer}." for layer in (*layers, *experts))
    KernelQuantLinear.emit_canonical_state = False  # already written above, packed
    try:
        state = model.state_dict()
    finally:
        KernelQuantLinear.emit_canonical_state = True
    for name, tensor in state.items():
        if (owned and name.startswith(owned)) or name in tensors:
            continue
        tensors[name] = tensor.detach().to(torch.bfloat16)

    non_persistent = []
    for name, buffer in model.named_buffers():
        if (owned and name.startswith(owned)) or name in state or name in tensors:
            continue
        tensors[name] = buffer.detach()
        non_persistent.append(name)

    meta = {
        "model_id": model_id,
        "layers": layers,
        "experts": experts,
        "non_persistent_buffers": non_persistent,
        "kv_cache_bits": kv_cache_bits,
        **(extra or {}),
    }
    return write_packed(path, tensors, meta)


def build_quant_linear(spec: dict, stored, wscale, bias, device, dtype=torch.bfloat16):
    """One KernelQuantLinear from its file record: upload packed bytes, unpack on the GPU."""
    args = _args_from_dict(spec["weights"])
    scheme = QuantizationScheme(weights=args,
                                input_activations=_args_from_dict(spec["input_activations"]))
    qweight = unpack_weight(stored.to(device), args.num_bits).reshape(spec["canonical_shape"])
    if bias is not None:
        bias = nn.Parameter(bias.to(device=device, dtype=dtype), requires_grad=False)
    return KernelQuantLinear(qweight, wscale.to(device), bias, scheme, spec["in_features"])


def _replace(model, name, module):
    parent_name, _, child = name.rpartition(".")
    parent = model.get_submodule(parent_name) if parent_name else model
    setattr(parent, child, module)


def _materialize_remaining(model, device, dtype, provided):
    """Storage for whatever is still on `meta` and will not be assigned from the file."""
    for prefix, module in model.named_modules():
        for name, param in list(module.named_parameters(recurse=False)):
            full = f"{prefix}.{name}" if prefix else name
            if param is not None and param.is_meta and full not in provided:
                setattr(module, name, nn.Parameter(
                    torch.empty(param.shape, dtype=dtype, device=device),
                    requires_grad=param.requires_grad))
        for name, buffer in list(module.named_buffers(recurse=False)):
            full = f"{prefix}.{name}" if prefix else name
            if buffer is not None and buffer.is_meta and full not in provided:
                persistent = name not in getattr(module, "_non_persistent_buffers_set", set())
                module.register_buffer(
                    name, torch.empty(buffer.shape, dtype=buffer.dtype, device=device),
                    persistent=persistent)


def load_packed_model(path, device="cuda", dtype=torch.bfloat16, config=None):
    """Rebuild the model from a packed file; nothing is ever allocated at bf16 width for a
    quantized layer. `config` overrides the lookup of `meta["model_id"]` (a local directory
    or an already-built transformers config)."""
    from transformers import AutoConfig, AutoModelForCausalLM

    tensors, meta = read_packed(path)
    if config is None:
        config = AutoConfig.from_pretrained(meta["model_id"])
    with torch.device("meta"):
        model = AutoModelForCausalLM.from_config(config)

    for name, spec in meta["layers"].items():
        module = build_quant_linear(spec, tensors[f"{name}.qweight"], tensors[f"{name}.wscale"],
                                    tensors.get(f"{name}.bias"), device, dtype)
        _replace(model, name, module)

    for name, spec in (meta.get("experts") or {}).items():
        args = _args_from_dict(spec["weights"])
        scheme = QuantizationScheme(weights=args,
                                    input_activations=_args_from_dict(spec["input_activations"]))
        qgate_up = unpack_weight(tensors[f"{name}.qgate_up"].to(device), args.num_bits)
        qdown = unpack_weight(tensors[f"{name}.qdown"].to(device), args.num_bits)
        # the activation is architecture, not weights: take it from the block being replaced
        module = KernelQuantExperts(
            qgate_up.reshape(spec["gate_up_shape"]), tensors[f"{name}.sgate_up"].to(device),
            qdown.reshape(spec["down_shape"]), tensors[f"{name}.sdown"].to(device), scheme,
            spec["hidden_dim"], spec["intermediate_dim"], model.get_submodule(name).act_fn)
        _replace(model, name, module)

    provided = set(tensors)
    _materialize_remaining(model, device, dtype, provided)
    non_persistent = set(meta.get("non_persistent_buffers", []))
    owned = tuple(f"{layer}." for layer in (*meta["layers"], *(meta.get("experts") or {})))
    remaining = {
        name: tensor.to(device=device, dtype=dtype)
        for name, tensor in tensors.items()
        if name not in non_persistent and not (owned and name.startswith(owned))
    }
    _, unexpected = model.load_state_dict(remaining, strict=False, assign=True)
    unexpected = [n for n in unexpected if not (owned and n.startswith(owned))]
    if unexpected:
        raise ValueError(f"packed file has tensors the model does not want: {unexpected[:5]}")
    for name in non_persistent:
        parent_name, _, attribute = name.rpartition(".")
        parent = model.get_submodule(parent_name) if parent_name else model
        parent.register_buffer(attribute, tensors[name].to(device), persistent=False)
    if getattr(config, "tie_word_embeddings", False) and hasattr(model, "tie_weights"):
        model.tie_weights()
    return model.eval()


def packed_dtypes(path) -> dict:
    """The dtype each config axis has in a packed file (model_io.py:240-274 of the reference)."""
    meta = read_header(path)["meta"]
    seen = {"attn_weight": set(), "mlp_weight": set(), "head_weight": set()}
    for name, spec in (meta.get("layers") or {}).items():
        key = ("attn_weight" if ".self_attn." in name else "mlp_weight" if ".mlp." in name
               else "head_weight" if "lm_head" in name else None)
        bits = (spec.get("weights") or {}).get("num_bits")
        if key and bits:
            seen[key].add(bits)

    def label(bits_set):
        if not bits_set:
            return "bf16"
        return "mixed" if len(bits_set) > 1 else f"int{next(iter(bits_set))}"

    kv_bits = meta.get("kv_cache_bits")
    return {**{k: label(v) for k, v in seen.items()},
            "kv_cache": f"int{kv_bits}" if kv_bits else "bf16", "activation": "bf16"}


def describe_packed(path) -> dict:
    header = read_header(path)
    entries = header["tensors"]
    return {
        "model_id": header["meta"]["model_id"],
        "quantized_layers": len(header["meta"]["layers"]),
        "expert_blocks": len(header["meta"].get("experts") or {}),
        "tensors": len(entries),
        "bytes": sum(e["nbytes"] for e in entries.values()),
    }
