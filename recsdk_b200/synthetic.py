"""Seeded synthetic workloads with the shapes and value distributions of the benchmark configs.

The reference measures on Criteo-style data (26 categorical fields, one id per field) that is not
available offline; these generators stand in for it: Zipf-distributed ids over log-uniformly sized
tables, uniform table init, N(0,1) upstream gradients.  Everything is generated on the device.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List

import numpy as np
import torch


def table_rows_log_uniform(seed: int, n_tables: int, lo: float, hi: float) -> List[int]:
    rng = np.random.default_rng(seed)
    return [int(r) for r in np.round(10 ** rng.uniform(math.log10(lo), math.log10(hi), n_tables)).astype(np.int64)]


def zipf_ids(gen: torch.Generator, n: int, vocab: int, alpha: float, device) -> torch.Tensor:
    """n ids ~ Zipf(alpha) over [0, vocab) by inverse CDF; rank r is mapped to id (r * A + C) mod vocab with
    A coprime to vocab, so hot rows are spread over the table instead of sitting in its first pages."""
    ranks = torch.arange(1, vocab + 1, dtype=torch.float64, device=device)
    cdf = torch.cumsum(ranks.pow_(-alpha), 0)
    u = torch.rand(n, generator=gen, dtype=torch.float64, device=device) * cdf[-1]
    r = torch.searchsorted(cdf, u).clamp_(max=vocab - 1)
    del cdf, ranks
    a = 2654435761 % vocab
    while math.gcd(a, vocab) != 1:
        a += 1
    return (r * a + 12345) % vocab


@dataclass
class TbeLayout:
    rows: List[int]
    dims: List[int]
    weights_offsets: torch.Tensor = field(default=None)
    D_offsets: torch.Tensor = field(default=None)
    hash_size_cumsum: torch.Tensor = field(default=None)
    total_D: int = 0
    max_D: int = 0
    total_rows: int = 0
    total_elems: int = 0
    total_hash_size_bits: int = 0


def make_layout(rows: List[int], dims: List[int], device) -> TbeLayout:
    lay = TbeLayout(rows=list(rows), dims=list(dims))
    wo = np.concatenate([[0], np.cumsum([r * d for r, d in zip(rows, dims)])]).astype(np.int64)
    do = np.concatenate([[0], np.cumsum(dims)]).astype(np.int32)
    hs = np.concatenate([[0], np.cumsum(rows)]).astype(np.int64)
    lay.weights_offsets = torch.from_numpy(wo[:-1].copy()).to(device)
    lay.D_offsets = torch.from_numpy(do).to(device)
    lay.hash_size_cumsum = torch.from_numpy(hs).to(device)
    lay.total_D, lay.max_D = int(do[-1]), int(max(dims))
    lay.total_rows, lay.total_elems = int(hs[-1]), int(wo[-1])
    lay.total_hash_size_bits = max(1, int(hs[-1]).bit_length())
    return lay


def one_hot_batch(gen: torch.Generator, rows: List[int], B: int, alpha: float, device):
    """indices [T*B] (feature-major) and offsets [T*B+1] for one id per (field, sample)."""
    idx = torch.cat([zipf_ids(gen, B, r, alpha, device) for r in rows])
    offsets = torch.arange(len(rows) * B + 1, dtype=torch.int64, device=device)
    return idx.contiguous(), offsets


def multi_hot_batch(gen: torch.Generator, rows: List[int], B: int, max_len: int, alpha: float, device):
    """bag length ~ UniformInt[1, max_len] per (sample, field), CSR offsets feature-major."""
    T = len(rows)
    lens = torch.randint(1, max_len + 1, (T * B,), generator=gen, device=device)
    offsets = torch.zeros(T * B + 1, dtype=torch.int64, device=device)
    offsets[1:] = torch.cumsum(lens, 0)
    per_table = lens.view(T, B).sum(1).tolist()
    idx = torch.cat([zipf_ids(gen, int(n), r, alpha, device) for n, r in zip(per_table, rows)])
    return idx.contiguous(), offsets
