"""Loaders with the signatures of the reference's ``core/eoq_linear.py``, and the module they produce.

``load_eoq_to_quantized_model`` is the loading path the reference describes and leaves as a TODO
(core/eoq_linear.py:15-54: ".eoq -> rANS decode -> pack to INT4 -> QuantizedLinear"): here the ``.eoq`` container is
read, every tensor's wire-format blocks are decoded on the GPU, and each linear layer of the model whose weight the
file holds becomes an :class:`EOQLinear` -- a module that keeps the weight entropy-coded in HBM and runs the fused
decode + GEMV / GEMM kernels in ``forward``.  The weights never exist as fp32; parameters the fused kernels do not
serve (norms, embeddings, biases, matrices with odd shapes) are dequantised on the GPU and copied into place.
"""
from __future__ import annotations

import os
import time
from typing import Dict, Optional, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..eoq_file import EOQTensorRecord, fusable, read_eoq
from ..fused import EOQWeight, require_cuda
from .quantized_linear import get_model_memory, replace_linear_with_quantized


class EOQLinear(nn.Module):
    """A linear layer whose weight is an :class:`EOQWeight` (entropy-coded tiles resident in HBM).

    Same call contract as ``QuantizedLinear.forward`` (core/quantized_linear.py:222-228): ``x`` of shape
    ``(..., in_features)`` in any of fp16 / bf16 / fp32, result ``(..., out_features)`` in ``x.dtype``, fp32 accumulation.
    Up to 8 rows run the fused decode + GEMV kernel, more rows of 16-bit activations the fused decode + tensor-core
    kernel, fp32 activations beyond 8 rows one dequantisation and a library GEMM.
    """

    def __init__(self, weight: EOQWeight, bias: Optional[torch.Tensor] = None, bits: int = 4, block_size: int = 128):
        super().__init__()
        self.eoq = weight
        self.out_features, self.in_features = weight.rows, weight.cols
        self.bits, self.block_size = bits, block_size
        self.register_buffer("bias_param", None if bias is None else bias.detach().float().to(weight.device))

    @classmethod
    def from_record(cls, rec: EOQTensorRecord, bias: Optional[torch.Tensor] = None, device="cuda") -> "EOQLinear":
        """From one tensor of an ``.eoq`` file: its `RANS` container is decoded on the GPU and tiled once, here."""
        if not fusable(rec):
            raise ValueError(f"{rec.name}: shape {rec.shape} / {rec.bits} bits is not served by the fused kernels")
        with torch.cuda.device(device):
            w = EOQWeight.from_rans(rec.rans_data, rec.scales, rec.shape, group=rec.quant_block_size)
        return cls(w, bias, rec.bits, rec.quant_block_size)

    @property
    def bias(self) -> Optional[torch.Tensor]:
        return self.bias_param

    def _dequantize_weight(self) -> torch.Tensor:
        """float32 (out_features, in_features), as QuantizedLinear._dequantize_weight."""
        return self.eoq.dequantize(torch.float32)

    _dequantize = _dequantize_weight

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        require_cuda(x, "EOQLinear.forward")
        return self.eoq.linear(x, self.bias_param)

    def memory_bytes(self) -> dict:
        info = self.eoq.info
        total = int(info.stream_bytes + info.table_bytes + info.scale_bytes + info.desc_bytes)
        return {"packed_bytes": int(info.stream_bytes), "scales_bytes": int(info.scale_bytes),
                "bias_bytes": 0 if self.bias_param is None else self.bias_param.numel() * 4, "total_bytes": total,
                "original_fp32_bytes": self.out_features * self.in_features * 4}

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias_param is not None}, "
                f"bits={self.bits}, block_size={self.block_size}, {self.eoq.info.bits_per_weight:.2f} bit/weight in HBM")


def _dense_from_record(rec: EOQTensorRecord, device) -> torch.Tensor:
    """Decode (GPU) and dequantise one tensor of the container: (sym - qmax) * scale per block (core/utils.py:130-161)."""
    import numpy as np
    from .rans_blocked import BlockedRANSDecoder, deserialize_blocked_rans
    qmax = (1 << (rec.bits - 1)) - 1
    sym = BlockedRANSDecoder().decode_all(deserialize_blocked_rans(rec.rans_data))
    codes = torch.from_numpy((sym - qmax).astype(np.float32)).to(device)
    scales = torch.from_numpy(np.frombuffer(rec.scales, np.float16).astype(np.float32)).to(device)
    n, bs = codes.numel(), rec.quant_block_size
    pad = (-n) % bs
    if pad:
        codes = torch.cat([codes, torch.zeros(pad, device=device)])
    return (codes.view(-1, bs) * scales[:, None]).flatten()[:n].view(rec.shape)


def fill_model_from_eoq(model: nn.Module, eoq_path: Union[str, os.PathLike], device="cuda") -> Dict[str, int]:
    """Move `model` to `device` and give it the tensors of an ``.eoq`` file.  A record named ``<path>.weight`` whose
    module is a linear layer (``nn.Linear`` or a layer with ``in_features`` / ``out_features``) and whose shape the fused
    kernels serve replaces that module by an :class:`EOQLinear`; every other record is dequantised and copied into the
    parameter or buffer of the same name.  Returns counts: layers replaced, tensors copied, records with no home."""
    _, records = read_eoq(eoq_path)
    by_name = {r.name: r for r in records}
    model.to(device)
    modules = dict(model.named_modules())
    stats = {"layers_replaced": 0, "tensors_copied": 0, "unmatched": 0}
    done = set()
    with torch.cuda.device(device):
        for name, rec in by_name.items():
            path, _, leaf = name.rpartition(".")
            mod = modules.get(path)
            is_linear = leaf == "weight" and mod is not None and hasattr(mod, "in_features") and hasattr(mod, "out_features")
            if is_linear and tuple(rec.shape) == (mod.out_features, mod.in_features) and fusable(rec):
                bias = None
                brec = by_name.get(path + ".bias")
                if brec is not None:
                    bias = _dense_from_record(brec, device)
                    done.add(path + ".bias")
                elif getattr(mod, "bias", None) is not None:
                    bias = mod.bias.detach()
                parent_path, _, attr = path.rpartition(".")
                setattr(modules[parent_path] if parent_path else model, attr, EOQLinear.from_record(rec, bias, device))
                stats["layers_replaced"] += 1
                done.add(name)
        targets = dict(model.named_parameters())
        targets.update(dict(model.named_buffers()))
        for name, rec in by_name.items():
            if name in done:
                continue
            dst = targets.get(name)
            if dst is None or tuple(dst.shape) != tuple(rec.shape):
                stats["unmatched"] += 1
                continue
            with torch.no_grad():
                dst.copy_(_dense_from_record(rec, device).to(dst.dtype))
            stats["tensors_copied"] += 1
    return stats


def load_eoq_to_quantized_model(eoq_path: str, model_name, device: str = "cpu") -> tuple:
    """(model, tokenizer, stats) (core/eoq_linear.py:15-54).  `model_name` is a Hugging Face identifier, as in the
    reference, or an already-built ``nn.Module`` (then the tokenizer returned is None).  When `eoq_path` exists the
    model's tensors come from it (see :func:`fill_model_from_eoq`; the GPU is required, `device` "cpu" means the
    default CUDA device); otherwise, as in the reference, the pretrained weights are quantised in place."""
    tokenizer = None
    if isinstance(model_name, nn.Module):
        model = model_name
    else:
        from transformers import AutoModelForCausalLM, AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(model_name, trust_remote_code=True)
        model = AutoModelForCausalLM.from_pretrained(model_name, torch_dtype=torch.float32, trust_remote_code=True)
    if eoq_path and os.path.exists(eoq_path):
        dev = "cuda" if str(device) == "cpu" else device
        stats = fill_model_from_eoq(model, eoq_path, dev)
        model.eval()
        return model, tokenizer, stats
    n = replace_linear_with_quantized(model, bits=4)
    model.eval()
    return model.to(device), tokenizer, {"layers_replaced": n}


def load_quantized_model(model_name: str, bits: int = 4, block_size: int = 128, device: str = "cpu") -> tuple:
    """(model, tokenizer, stats) (core/eoq_linear.py:58-103)."""
    from transformers import AutoModelForCausalLM, AutoTokenizer
    tokenizer = AutoTokenizer.from_pretrained(model_name, trust_remote_code=True)
    t0 = time.time()
    model = AutoModelForCausalLM.from_pretrained(model_name, torch_dtype=torch.float32, trust_remote_code=True)
    n = replace_linear_with_quantized(model, bits=bits, block_size=block_size)
    load_time = time.time() - t0
    model.eval()
    mem = get_model_memory(model)
    stats = {"model": model_name, "bits": bits, "layers_replaced": n, "load_time": load_time,
             "ram_mb": mem["total_bytes"] / 1024 / 1024, "compression": mem["compression_ratio"]}
    return model.to(device), tokenizer, stats
