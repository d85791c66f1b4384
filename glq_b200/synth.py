"""Seeded synthetic GLQ layers of the benchmark shapes (no checkpoint is needed: any bit pattern is
a valid 3INST stream and any 16-bit value a valid E8 index — the reference's own kernel benchmarks
use random int16 the same way, benchmarks/_trellis_moe_grouped_parity.py:53-56)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from . import _lib
from .plan import LinearSpec, block_decompose

# (name, out_features m, in_features n) per decoder layer
SMOLLM3_3B = dict(layers=36, hidden=2048, proj=[("q", 2048, 2048), ("k", 512, 2048), ("v", 512, 2048),
                                                 ("o", 2048, 2048), ("gate", 11008, 2048), ("up", 11008, 2048),
                                                 ("down", 2048, 11008)])
LLAMA3_8B = dict(layers=32, hidden=4096, proj=[("q", 4096, 4096), ("k", 1024, 4096), ("v", 1024, 4096),
                                                ("o", 4096, 4096), ("gate", 14336, 4096), ("up", 14336, 4096),
                                                ("down", 4096, 14336)])
DENSE_62L = dict(layers=62, hidden=5376, proj=[("q", 4096, 5376), ("k", 2048, 5376), ("v", 2048, 5376),
                                               ("o", 5376, 4096), ("gate", 21504, 5376), ("up", 21504, 5376),
                                               ("down", 5376, 21504)])
COLUMN_PARALLEL = ("q", "k", "v", "gate", "up")    # output rows are split across ranks
ROW_PARALLEL = ("o", "down")                       # input columns are split; outputs are summed


@dataclass
class SynthLayer:
    name: str
    m: int
    n: int
    fmt: int
    codes: list
    bits: list
    tables: list
    stage_scale: list
    su: torch.Tensor
    sv: torch.Tensor
    wscale: float

    def code_bytes(self) -> int:
        return sum(c.numel() * c.element_size() for c in self.codes)

    def spec(self, batch=1, x_dtype=torch.bfloat16, y_dtype=torch.bfloat16, **kw) -> LinearSpec:
        return LinearSpec(format=self.fmt, m_pad=self.m, n_pad=self.n, in_features=self.n, out_features=self.m,
                          codes=self.codes, bits=self.bits, tables=self.tables, stage_scale=self.stage_scale,
                          su=self.su, sv=self.sv, wscale=self.wscale, blocks_n=block_decompose(self.n),
                          blocks_m=block_decompose(self.m), batch=batch, x_dtype=x_dtype, y_dtype=y_dtype, **kw)


def _signs(n: int, gen: torch.Generator, device) -> torch.Tensor:
    return (torch.randint(0, 2, (n,), generator=gen, device=device, dtype=torch.int32) * 2 - 1).to(torch.float16)


def _rand_i16(shape, gen: torch.Generator, device) -> torch.Tensor:
    return torch.randint(-32768, 32768, shape, generator=gen, device=device, dtype=torch.int32).to(torch.int16)


def _scale(gen: torch.Generator, device) -> float:
    u = torch.rand((), generator=gen, device=device).item()
    return float(torch.tensor((0.5 + u) * 0.02, dtype=torch.float16).item())


def trellis_layer(name, m, n, bits, gen, device, inv_resid_scale2=0.21) -> SynthLayer:
    """bits = [K] or [K, K2]; packed bit-streams are uniform random 16-bit words."""
    codes = [_rand_i16(((m // 16) * (n // 16), 16 * k), gen, device) for k in bits]
    return SynthLayer(name, m, n, _lib.FMT_TRELLIS_3INST, codes, list(bits), [],
                      [inv_resid_scale2] if len(bits) > 1 else [], _signs(m, gen, device), _signs(n, gen, device),
                      _scale(gen, device))


def e8_layer(name, m, n, stages, table, gen, device, inv_resid_scale=0.1) -> SynthLayer:
    """stages x uniform uint16 index matrices; stage s+1 is scaled by inv_resid_scale**s."""
    codes = [_rand_i16((m, n // 8), gen, device) for _ in range(stages)]
    scales = [inv_resid_scale ** (s + 1) for s in range(stages - 1)]
    return SynthLayer(name, m, n, _lib.FMT_E8_SHELL, codes, [], [table] * stages, scales,
                      _signs(m, gen, device), _signs(n, gen, device), _scale(gen, device))


def shard_shape(name: str, m: int, n: int, world: int) -> tuple[int, int]:
    """Tensor-parallel shard of a projection: rows split for q/k/v/gate/up, columns for o/down.
    Each shard is a GLQ layer of its own (its own sign vectors and Hadamard blocks)."""
    if world == 1:
        return m, n
    if name in COLUMN_PARALLEL:
        assert m % world == 0
        return m // world, n
    assert n % world == 0
    return m, n // world


def load_e8_table(device) -> torch.Tensor:
    """The nibble-packed E8 shell table shipped with the package, as an int32 CUDA tensor."""
    import os
    import numpy as np
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "e8_shell_packed.npy")
    return torch.from_numpy(np.load(path).view(np.int32)).to(device)
