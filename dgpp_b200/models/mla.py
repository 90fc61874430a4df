"""Multi-head latent attention (absorbed form) and the sparse-attention index, as PyTorch oracles next to the
kernel wrappers in ``ops.core`` (``mla_decode``, ``dsa_index``, ``topk_select``).

Cache row per token: [latent c (dc) | rotary key (dr)].  With W_uk absorbed into the query and W_uv applied after
the attention, every head reads the same row: score = q_abs . c + q_rot . k_rot, output = sum_t p_t c_t.
Sparse attention keeps, per query row, the top-k cached positions by the lightning-indexer score
sum_h w_h relu(q_idx_h . k_idx_t); ties go to the lower position.
(reference counterparts: src/models/dsa_layer.cu, dsa_reference.cpp, src/kernels/dsa.cu.)
"""
from __future__ import annotations

from typing import Optional

import torch


def gather_rows(cache: torch.Tensor, block_table_row: torch.Tensor, n: int) -> torch.Tensor:
    """First n token rows of a request from a paged [blocks, page, d] pool."""
    page = cache.shape[1]
    tok = torch.arange(n, device=cache.device)
    return cache[block_table_row.long()[tok // page], tok % page]


def mla_reference(q: torch.Tensor, latent: torch.Tensor, scale: float, dc: int,
                  sel: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q: [heads, dc + dr]; latent: [n, dc + dr] (tokens 0..n-1, the query's own token last).  fp32."""
    lat = latent.float()
    if sel is not None:
        idx = sel[sel >= 0].long()
        lat = lat[idx]
    s = (q.float() @ lat.t()) * scale
    p = torch.softmax(s, -1)
    return p @ lat[:, :dc]


def index_scores_reference(q_idx: torch.Tensor, w_idx: torch.Tensor, k_idx: torch.Tensor) -> torch.Tensor:
    """q_idx [hi, di], w_idx [hi], k_idx [n, di] -> [n] fp32 scores."""
    return (torch.relu(q_idx.float() @ k_idx.float().t()) * w_idx.float().unsqueeze(-1)).sum(0)


def topk_reference(scores: torch.Tensor, k: int) -> torch.Tensor:
    """Positions of the k best scores, ties to the lower position, ascending; -1 padded."""
    n = scores.numel()
    if n <= k:
        out = torch.full((k,), -1, dtype=torch.int32, device=scores.device)
        out[:n] = torch.arange(n, dtype=torch.int32, device=scores.device)
        return out
    order = torch.argsort(-scores, stable=True)[:k]
    return torch.sort(order).values.to(torch.int32)
