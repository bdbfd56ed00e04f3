"""Loaders with the signatures of the reference's ``core/eoq_linear.py``.  Both need a
Hugging Face checkpoint (``transformers`` plus the model files); the layer replacement they
perform is :func:`replace_linear_with_quantized` of this package, whose forward is the fused
GPU path."""
from __future__ import annotations

import time

import torch

from .quantized_linear import get_model_memory, replace_linear_with_quantized


def load_eoq_to_quantized_model(eoq_path: str, model_name: str, device: str = "cpu") -> tuple:
    """(model, tokenizer, stats) (core/eoq_linear.py:15-54).  As in the reference the weights come
    from the pretrained checkpoint and are re-quantised; `eoq_path` is accepted for signature parity."""
    from transformers import AutoModelForCausalLM, AutoTokenizer
    tokenizer = AutoTokenizer.from_pretrained(model_name, trust_remote_code=True)
    model = AutoModelForCausalLM.from_pretrained(model_name, torch_dtype=torch.float32, trust_remote_code=True)
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
