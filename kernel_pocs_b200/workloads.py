"""Synthetic benchmark workloads of the SwiGLU path and their row partition across GPUs.

Every workload is a token-major matrix ``[tokens, width]`` for gate, up and dh.  Data are
drawn per CHUNK of ``CHUNK_ROWS`` token rows from a generator seeded with
``seed * 2**32 + chunk_index``, so any contiguous row range can be produced on its own
device, bit-identical to the same rows of the whole matrix, without ever materialising the
whole matrix anywhere.  The shapes carry the names of the models whose MLP widths they are;
no model weights or data sets are involved.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

CHUNK_ROWS = 8192


@dataclass(frozen=True)
class Workload:
    name: str
    tokens: int
    width: int
    dtype: torch.dtype
    seed: int
    std: float = 1.0
    note: str = ""

    @property
    def elements(self) -> int:
        return self.tokens * self.width

    def bytes_fwd(self, tokens: int | None = None) -> int:
        """Algorithmic bytes of the forward: read gate, up; write h."""
        t = self.tokens if tokens is None else tokens
        return 3 * t * self.width * _ITEMSIZE[self.dtype]

    def bytes_bwd(self, tokens: int | None = None) -> int:
        """Algorithmic bytes of the backward: read dh, gate, up; write dgate, dup."""
        t = self.tokens if tokens is None else tokens
        return 5 * t * self.width * _ITEMSIZE[self.dtype]


_ITEMSIZE = {torch.float32: 4, torch.float16: 2, torch.bfloat16: 2}


def varlen_lengths(seed: int = 2, sequences: int = 16, max_len: int = 8192) -> list[int]:
    """Sequence lengths of the variable-length packed batch: uniform on [1, max_len]."""
    g = torch.Generator().manual_seed(seed)
    return torch.randint(1, max_len + 1, (sequences,), generator=g).tolist()


def workloads() -> dict[str, Workload]:
    varlen_tokens = sum(varlen_lengths())
    return {
        "c1": Workload("c1", 256, 1024, torch.float32, 0, note="fp32 [2,128,1024]: the CPU-runnable parity case"),
        "c2": Workload("c2", 32768, 14336, torch.bfloat16, 1, note="Llama-3-8B MLP activation, batch 8 x seq 4096"),
        "c3": Workload("c3", varlen_tokens, 11008, torch.bfloat16, 2, std=2.0,
                       note="16 packed variable-length sequences, Llama-2-7B width, N(0, 2^2)"),
        "c3-fp32": Workload("c3-fp32", varlen_tokens, 11008, torch.float32, 2, std=2.0,
                            note="same in fp32"),
        "c5": Workload("c5", 65536, 28672, torch.bfloat16, 4, note="Llama-3-70B MLP activation"),
    }


def row_shard(total_rows: int, world_size: int, rank: int) -> tuple[int, int]:
    """Contiguous, balanced partition of token rows: ranks [0, total % world) get one extra."""
    if not (0 <= rank < world_size):
        raise ValueError(f"rank {rank} outside world of {world_size}")
    base, extra = divmod(total_rows, world_size)
    lo = rank * base + min(rank, extra)
    hi = lo + base + (1 if rank < extra else 0)
    return lo, hi


def generate_rows(w: Workload, lo: int, hi: int, device: torch.device | str):
    """gate, up, dh for token rows [lo, hi) of workload ``w`` on ``device``."""
    device = torch.device(device)
    gate, up, dh = (torch.empty((hi - lo, w.width), dtype=w.dtype, device=device) for _ in range(3))
    first, last = lo // CHUNK_ROWS, (max(hi, lo + 1) - 1) // CHUNK_ROWS
    for chunk in range(first, last + 1):
        c_lo, c_hi = chunk * CHUNK_ROWS, (chunk + 1) * CHUNK_ROWS
        g = torch.Generator(device=device).manual_seed(w.seed * 2**32 + chunk)
        a, b = max(lo, c_lo), min(hi, c_hi)
        for t in (gate, up, dh):
            full = torch.randn((CHUNK_ROWS, w.width), generator=g, device=device, dtype=torch.float32)
            if a < b:
                t[a - lo:b - lo] = (full[a - c_lo:b - c_lo] * w.std).to(w.dtype)
            del full
    return gate, up, dh
