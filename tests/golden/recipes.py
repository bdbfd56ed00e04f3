"""Seeded synthetic inputs of the benchmark configurations, shared by the fixture generator (which feeds them to the
imported reference) and by the tests (which feed them to the library and compare with what the reference made of
them).  CPU generators only, so both sides see the same numbers wherever they run."""
from __future__ import annotations

import hashlib

import numpy as np
import torch

#: name -> (rows, cols, seed, sigma); INT4 symmetric absmax, group 128, as the benchmark set words configurations 1, 2 and 5
INT4_SHAPES = {
    "square_4096x4096": (4096, 4096, 101, 0.02),          # config 1
    "up_11008x4096": (11008, 4096, 102, 0.02),            # config 2
    "down_4096x11008": (4096, 11008, 103, 0.02),          # config 2, transposed layer
    "gate_shard_3584x8192": (3584, 8192, 104, 0.015),     # config 5: 28672 x 8192 over eight ranks
    "down_shard_1024x28672": (1024, 28672, 105, 0.015),   # config 5: 8192 x 28672 over eight ranks
}
#: config 3: 14336 x 4096, N(0, 0.015), 0.1 % of the entries at +-8 sigma
POLAR_SHAPE = ("polar_14336x4096", 14336, 4096, 106, 0.015)
SLICE_ROWS = 512       # rows of a large matrix whose reference output is stored or hashed
BRIDGE_ROWS = 128      # rows of config 1 that go through the reference's tensor bridge (block 256, p 14)


def weight(rows: int, cols: int, seed: int, sigma: float) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, cols, generator=g) * sigma


def polar_weight(rows: int, cols: int, seed: int, sigma: float) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(rows, cols, generator=g) * sigma
    hit = torch.rand(rows, cols, generator=g) < 0.001
    sign = torch.where(torch.rand(rows, cols, generator=g) < 0.5, -1.0, 1.0)
    return torch.where(hit, sign * 8 * sigma, w)


def activations(rows: int, cols: int, seed: int, dtype=torch.float16) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randn(rows, cols, generator=g).to(dtype)


def sha(a) -> str:
    a = a.detach().cpu().numpy() if isinstance(a, torch.Tensor) else np.asarray(a)
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()
