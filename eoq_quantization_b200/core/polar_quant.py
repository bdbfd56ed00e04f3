"""PolarQuant surface of the reference (core/polar_quant.py:42-264): per-block L2 norm, normalise, Walsh-Hadamard
rotation, scale to N(0, 1), nearest of the 2^bits Lloyd-Max centroids; the inverse for dequantisation.

Quantisation is the encode side of the path (done once, when a model is converted) and runs as torch operations
on whatever device the weight is on; the decode side -- centroid look-up, rotation, norm and the dot product -- is
the fused kernel behind ``kernels.polar_engine.PolarLinear`` / ``EOQWeight(kind=KIND_Q5_POLAR)``.
``polar_dequantize`` is kept for callers that want the dense matrix and follows the reference's order of operations.
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional

import numpy as np
import torch

#: Lloyd-Max centroids of N(0, 1) by bit width; 2 and 3 bits are the reference's tabulated values
#: (core/polar_quant.py:32-40), wider ones are computed on first use.
GAUSSIAN_CENTROIDS: dict = {
    2: torch.tensor([-1.5104, -0.4528, 0.4528, 1.5104]),
    3: torch.tensor([-2.1520, -1.3440, -0.7560, -0.2451, 0.2451, 0.7560, 1.3440, 2.1520]),
    4: None, 5: None, 6: None,
}


def compute_lloyd_max_centroids(n_levels: int, n_iter: int = 100) -> torch.Tensor:
    """Lloyd-Max quantiser of N(0, 1) (core/polar_quant.py:42-83): start from uniform boundaries on [-4, 4] with
    open ends, then alternate centroid = E[X | cell] = (phi(a) - phi(b)) / (Phi(b) - Phi(a)) and boundary =
    midpoint of neighbouring centroids, ``n_iter`` times; float64 throughout, float32 result."""
    from scipy.stats import norm

    edges = np.linspace(-4.0, 4.0, n_levels + 1)
    edges[0], edges[-1] = -np.inf, np.inf
    cent = np.zeros(n_levels)
    for _ in range(n_iter):
        lo, hi = edges[:-1], edges[1:]
        mass = norm.cdf(hi) - norm.cdf(lo)
        with np.errstate(invalid="ignore", divide="ignore"):
            mean = (norm.pdf(lo) - norm.pdf(hi)) / mass
        cent = np.where(mass > 1e-10, mean, (lo + hi) / 2)
        edges = np.concatenate(([-np.inf], (cent[:-1] + cent[1:]) / 2, [np.inf]))
    return torch.tensor(cent, dtype=torch.float32)


def _ensure_centroids(bits: int) -> torch.Tensor:
    if GAUSSIAN_CENTROIDS.get(bits) is None:
        GAUSSIAN_CENTROIDS[bits] = compute_lloyd_max_centroids(1 << bits)
    return GAUSSIAN_CENTROIDS[bits]


_hadamard_cache: dict = {}


def hadamard_matrix(n: int, device: Optional[torch.device] = None) -> torch.Tensor:
    """Normalised Walsh-Hadamard matrix of order n (a power of two), Sylvester construction with a division by
    sqrt(2) per doubling (core/polar_quant.py:104-120); symmetric and its own inverse."""
    if n not in _hadamard_cache:
        if n < 1 or n & (n - 1):
            raise ValueError(f"Hadamard order must be a power of two, got {n}")
        h = torch.tensor([[1.0]])
        while h.shape[0] < n:
            h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0) / math.sqrt(2)
        _hadamard_cache[n] = h
    h = _hadamard_cache[n]
    return h.to(device) if device is not None else h


@dataclass
class PolarQuantResult:
    """Fields of the reference's result type (core/polar_quant.py:127-138)."""
    codes: torch.Tensor            # int8 centroid indices, flat, n_elements
    norms: torch.Tensor            # fp16 per-block norms
    bits: int
    block_size: int
    shape: tuple
    n_elements: int
    use_qjl: bool
    qjl_signs: Optional[torch.Tensor] = None


def _qjl_directions(block_size: int, device) -> torch.Tensor:
    # the reference draws its +-1 projection from a generator re-seeded with 42 at every call (core/polar_quant.py:197-198)
    torch.manual_seed(42)
    return torch.randint(0, 2, (block_size,), device=device).float() * 2 - 1


def polar_quantize(weight: torch.Tensor, bits: int = 4, block_size: int = 128, use_qjl: bool = True,
                   chunk_blocks: int = 1 << 16) -> PolarQuantResult:
    """core/polar_quant.py:141-213.  The nearest-centroid search runs over ``chunk_blocks`` blocks at a time so that
    the [blocks, block_size, levels] distance tensor of a large matrix never exists as a whole."""
    cent = _ensure_centroids(bits).to(weight.device)
    H = hadamard_matrix(block_size, weight.device)
    flat = weight.detach().float().flatten()
    n = flat.numel()
    pad = (block_size - n % block_size) % block_size
    if pad:
        flat = torch.nn.functional.pad(flat, (0, pad))
    blocks = flat.view(-1, block_size)
    norms = blocks.norm(dim=1, keepdim=True).clamp(min=1e-10)
    root = math.sqrt(block_size)
    codes = torch.empty(blocks.shape, dtype=torch.int8, device=weight.device)
    signs = torch.empty(blocks.shape[0], dtype=torch.uint8, device=weight.device) if use_qjl else None
    dirs = _qjl_directions(block_size, weight.device) if use_qjl else None
    for lo in range(0, blocks.shape[0], chunk_blocks):
        hi = min(blocks.shape[0], lo + chunk_blocks)
        scaled = ((blocks[lo:hi] / norms[lo:hi]) @ H) * root
        idx = (scaled.unsqueeze(-1) - cent.view(1, 1, -1)).abs().argmin(dim=-1)
        codes[lo:hi] = idx.to(torch.int8)
        if use_qjl:
            signs[lo:hi] = (((scaled - cent[idx]) * dirs.unsqueeze(0)).sum(dim=1) >= 0).to(torch.uint8)
    return PolarQuantResult(codes=codes.flatten()[:n], norms=norms.squeeze(1).to(torch.float16), bits=bits,
                            block_size=block_size, shape=tuple(weight.shape), n_elements=n, use_qjl=use_qjl, qjl_signs=signs)


def polar_dequantize(result: PolarQuantResult, device: Optional[torch.device] = None) -> torch.Tensor:
    """core/polar_quant.py:216-264: centroids[codes] (+ the QJL nudge) / sqrt(d) @ H * norm -> float16 of result.shape."""
    device = result.codes.device if device is None else device
    cent = _ensure_centroids(result.bits).to(device)
    bs, n = result.block_size, result.n_elements
    H = hadamard_matrix(bs, device)
    codes = result.codes.to(device).long()
    pad = (bs - n % bs) % bs
    if pad:
        codes = torch.nn.functional.pad(codes, (0, pad))
    rec = cent[codes.view(-1, bs)]
    if result.use_qjl and result.qjl_signs is not None:
        step = _qjl_directions(bs, device).unsqueeze(0) / math.sqrt(bs)
        rec = rec + 0.5 * (result.qjl_signs.float().to(device) * 2 - 1).unsqueeze(1) * step
    rec = ((rec / math.sqrt(bs)) @ H) * result.norms.float().to(device).unsqueeze(1)
    return rec.flatten()[:n].view(result.shape).half()
