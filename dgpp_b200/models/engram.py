"""Hashed n-gram memory ("Engram") sites for models whose residual path is a set of streams.

At an Engram site every token hashes its last 2 .. max_ngram token classes (a many-to-one map of the vocabulary; a
pad class before the start of the sequence) into one table row per (n-gram size, head), concatenates the rows,
projects them to one key per stream plus one value, and every stream adds the value through its own gate
(`ops.engram_embed`, a linear, `ops.engram_gate`).  The constants of the hash (class map, per-layer multipliers, a
prime modulus and a row offset per (size, head)) ship with the checkpoint; `random_init` draws a consistent set.
A request remembers its last max_ngram - 1 tokens between passes (`history`), the only state of the mechanism.
(reference counterparts: src/models/dsv41/engram_layer.cpp, engram_tables.cpp, src/kernels/dsv41_engram.cu.  The
 reference keeps the tables on NVMe and gathers on the host; this build keeps them in device memory.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List

import torch

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize

BF = torch.bfloat16


@dataclass
class EngramConfig:
    max_ngram: int = 4            # 2-, 3- and 4-grams
    heads: int = 2
    head_dim: int = 64
    bucket: int = 1000            # rows per (size, head) range, rounded down to a prime
    classes: int = 0              # size of the compressed vocabulary (0: vocab // 2)

    @property
    def slots(self) -> int:
        return (self.max_ngram - 1) * self.heads


@dataclass
class EngramLayer:
    multipliers: torch.Tensor     # [max_ngram] int64
    primes: torch.Tensor          # [max_ngram - 1, heads] int64
    offsets: torch.Tensor         # [max_ngram - 1, heads] int64
    table: torch.Tensor           # [rows, D] uint8 (e4m3)
    table_sf: torch.Tensor        # [rows, D / 32] uint8 (e8m0)
    wkv: QuantLinear              # [(hc + 1) * H, slots * D]
    q_weight: torch.Tensor        # [hc, H] bf16
    k_weight: torch.Tensor        # [hc, H] bf16


def _primes_below(n: int, count: int) -> List[int]:
    out, v = [], n
    while len(out) < count and v > 2:
        if all(v % q for q in range(2, int(v ** 0.5) + 1)):
            out.append(v)
        v -= 1
    return out


class Engram:
    def __init__(self, cfg: EngramConfig, token_map: torch.Tensor, pad_class: int, layers: Dict[int, EngramLayer], eps: float):
        self.cfg, self.token_map, self.pad_class, self.layers, self.eps = cfg, token_map, pad_class, layers, eps

    @staticmethod
    def random_init(cfg: EngramConfig, layer_ids, vocab: int, hc: int, hidden: int, device, seed: int = 0, std: float = 0.05,
                    eps: float = 1e-6) -> "Engram":
        g = torch.Generator(device="cpu")
        g.manual_seed(seed * 31 + 7)
        classes = cfg.classes or max(2, vocab // 2)
        token_map = torch.randint(0, classes, (vocab,), generator=g, dtype=torch.int32)
        layers = {}
        per = cfg.slots
        assert cfg.head_dim % 32 == 0 and (per * cfg.head_dim) % 64 == 0, "the projection reads rows of a multiple of 64 values"
        for li in layer_ids:
            pr = torch.tensor(_primes_below(cfg.bucket, per), dtype=torch.int64).view(cfg.max_ngram - 1, cfg.heads)
            off = torch.cumsum(pr.flatten(), 0) - pr.flatten()
            rows = int(pr.sum())
            payload = (torch.randn(rows, cfg.head_dim, generator=g)).to(torch.float8_e4m3fn).view(torch.uint8)
            sf = torch.randint(122, 126, (rows, cfg.head_dim // 32), generator=g, dtype=torch.int32).to(torch.uint8)
            mult = torch.randint(1, 2 ** 31, (cfg.max_ngram,), generator=g, dtype=torch.int64) * 2 + 1
            wkv = quantize(torch.randn((hc + 1) * hidden, per * cfg.head_dim, generator=g) * std, "bf16").to(device)
            layers[li] = EngramLayer(mult.to(device), pr.to(device), off.view_as(pr).contiguous().to(device), payload.to(device),
                                     sf.to(device), wkv, (1 + 0.1 * torch.randn(hc, hidden, generator=g)).to(BF).to(device),
                                     (1 + 0.1 * torch.randn(hc, hidden, generator=g)).to(BF).to(device))
        return Engram(cfg, token_map.to(device), classes, layers, eps)

    # ---- token history
    def prev_rows(self, tokens: List[int], history: List[int]) -> List[List[int]]:
        """Rows k = 0 .. max_ngram - 2 of the `prev` operand for consecutive `tokens` of one request whose newest earlier
        tokens are `history` (newest last)."""
        seq = list(history) + list(tokens)
        h = len(history)
        return [[seq[h + t - k - 1] if h + t - k - 1 >= 0 else -1 for t in range(len(tokens))]
                for k in range(self.cfg.max_ngram - 1)]

    def keep(self, history: List[int], tokens: List[int]) -> List[int]:
        return (list(history) + list(tokens))[-(self.cfg.max_ngram - 1):]

    # ---- the site
    def apply_reference(self, li: int, streams: torch.Tensor, tokens: torch.Tensor, prev: torch.Tensor) -> torch.Tensor:
        L = self.layers[li]
        e = ref.engram_embed(tokens, prev, self.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf, self.pad_class)
        return ref.engram_gate(streams, ref.linear(e, L.wkv), L.q_weight, L.k_weight, self.eps)

    def apply(self, li: int, streams: torch.Tensor, tokens: torch.Tensor, prev: torch.Tensor) -> torch.Tensor:
        L = self.layers[li]
        e = ops.engram_embed(tokens, prev, self.token_map, L.multipliers, L.primes, L.offsets, L.table, L.table_sf, self.pad_class)
        return ops.engram_gate(streams, ops.linear(e, L.wkv), L.q_weight, L.k_weight, self.eps)
