"""Gated DeltaNet linear-attention layer (the recurrent 3-of-4 layers of the hybrid family): input projections,
causal depthwise convolution + SiLU, gated delta-rule recurrence with a per-head fp32 state, gated RMSNorm, output
projection.  ``gdn_reference`` is the PyTorch oracle (token by token); ``GdnLayer.forward`` launches the sm_100a
kernels (`csrc/kernels/gdn.cu`) for a prefill chunk of one request or for a batch of single decode tokens.
(reference counterparts: src/kernels/gdn_chunk.cu, src/kernels/kda.cu, src/models/qwen/model35.cpp GDN layers.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch
import torch.nn.functional as F

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize

BF = torch.bfloat16


@dataclass
class GdnConfig:
    hidden: int = 2048
    k_heads: int = 16
    v_heads: int = 32
    dk: int = 128
    dv: int = 128
    conv_width: int = 4
    eps: float = 1e-6

    @property
    def conv_channels(self) -> int:
        return 2 * self.k_heads * self.dk + self.v_heads * self.dv

    @property
    def proj_cols(self) -> int:      # q | k | v | z | alpha | beta
        return self.conv_channels + self.v_heads * self.dv + 2 * self.v_heads


@dataclass
class GdnWeights:
    cfg: GdnConfig
    in_proj: QuantLinear         # [proj_cols, hidden]
    conv_w: torch.Tensor         # [conv_channels, W] bf16
    conv_b: Optional[torch.Tensor]
    A_log: torch.Tensor          # [hv] fp32
    dt_bias: torch.Tensor        # [hv] fp32
    norm_w: torch.Tensor         # [dv] bf16
    out_proj: QuantLinear        # [hidden, hv * dv]

    @staticmethod
    def random_init(cfg: GdnConfig, device, seed: int = 0, std: float = 0.02, fmt: str = "bf16") -> "GdnWeights":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        rnd = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        return GdnWeights(cfg, quantize(rnd(cfg.proj_cols, cfg.hidden) * std * 4, fmt),
                          (rnd(cfg.conv_channels, cfg.conv_width) * 0.5).to(BF), None,
                          torch.log(torch.rand(cfg.v_heads, device=device, generator=g) * 4 + 0.5),
                          rnd(cfg.v_heads) * 0.5, (1 + 0.1 * rnd(cfg.dv)).to(BF),
                          quantize(rnd(cfg.hidden, cfg.v_heads * cfg.dv) * std, fmt))


class GdnState:
    """Per-slot recurrent state: convolution tail + delta-rule memory (fp32)."""

    def __init__(self, cfg: GdnConfig, slots: int, device, conv: Optional[torch.Tensor] = None,
                 ssm: Optional[torch.Tensor] = None):
        """conv / ssm: views into a pool shared by all recurrent layers (one commit kernel then serves every layer)."""
        self.conv = conv if conv is not None else torch.zeros(slots, cfg.conv_width - 1, cfg.conv_channels,
                                                              dtype=torch.float32, device=device)
        self.ssm = ssm if ssm is not None else torch.zeros(slots, cfg.v_heads, cfg.dk, cfg.dv, dtype=torch.float32,
                                                           device=device)

    def reset(self, slot: int) -> None:
        self.conv[slot].zero_()
        self.ssm[slot].zero_()

    def snapshot(self, slot: int):
        return self.conv[slot].clone(), self.ssm[slot].clone()

    def restore(self, slot: int, snap) -> None:
        self.conv[slot].copy_(snap[0])
        self.ssm[slot].copy_(snap[1])


def _split(cfg: GdnConfig, proj: torch.Tensor):
    nq = cfg.k_heads * cfg.dk
    nv = cfg.v_heads * cfg.dv
    c = cfg.conv_channels
    return proj[:, :c], proj[:, c:c + nv], proj[:, c + nv:c + nv + cfg.v_heads], proj[:, c + nv + cfg.v_heads:], nq, nv


def gdn_reference(x: torch.Tensor, w: GdnWeights, conv_state: torch.Tensor, ssm_state: torch.Tensor) -> torch.Tensor:
    """x [T, hidden] (normed, bf16): consecutive tokens of one request.  conv_state [W-1, C] and ssm_state
    [hv, dk, dv] (fp32) are updated in place.  Rounding points follow the kernels: bf16 after the projection, after
    the convolution activation, after the recurrence output and after the gated norm."""
    c = w.cfg
    proj = ref.linear(x, w.in_proj)
    mixed, z, al, be, nq, nv = _split(c, proj)
    T = x.shape[0]
    hist = torch.cat([conv_state, mixed.float()], 0)                       # [W-1+T, C]
    cw = w.conv_w.float()
    conv = torch.zeros(T, c.conv_channels, device=x.device)
    for i in range(c.conv_width):
        conv += hist[i:i + T] * cw[:, i]
    if w.conv_b is not None:
        conv += w.conv_b.float()
    conv_state.copy_(hist[T:])
    act = ref.act(F.silu(conv)).float()
    q = act[:, :nq].view(T, c.k_heads, c.dk)
    k = act[:, nq:2 * nq].view(T, c.k_heads, c.dk)
    v = act[:, 2 * nq:].view(T, c.v_heads, c.dv)
    rep = c.v_heads // c.k_heads
    q = (q * torch.rsqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * c.dk ** -0.5).repeat_interleave(rep, 1)
    k = (k * torch.rsqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, 1)
    g = -torch.exp(w.A_log.float()) * F.softplus(al.float() + w.dt_bias.float())   # [T, hv]
    beta = torch.sigmoid(be.float())
    out = torch.zeros(T, c.v_heads, c.dv, device=x.device)
    S = ssm_state
    for t in range(T):
        S.mul_(torch.exp(g[t]).view(-1, 1, 1))
        mem = torch.einsum("hkv,hk->hv", S, k[t])
        u = beta[t].unsqueeze(-1) * (v[t] - mem)
        S.add_(torch.einsum("hk,hv->hkv", k[t], u))
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = ref.act(out).float()
    rstd = torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + c.eps)
    n = ref.act(o * rstd).float() * w.norm_w.float()
    gated = ref.act(n * F.silu(z.float().view(T, c.v_heads, c.dv))).reshape(T, nv)
    return ref.linear(gated, w.out_proj)


class GdnLayer:
    def __init__(self, w: GdnWeights, max_rows: int, device):
        c = w.cfg
        self.w, self.c = w, c
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        self.proj, self.conv = e(max_rows, c.proj_cols), e(max_rows, c.conv_channels)
        self.o, self.gated = e(max_rows, c.v_heads * c.dv), e(max_rows, c.v_heads * c.dv)
        self.prep = torch.empty(max_rows * (2 * c.k_heads * c.dk + 2 * c.v_heads), dtype=torch.float32, device=device)

    def forward(self, x: torch.Tensor, state: GdnState, out: torch.Tensor, slot: int = 0,
                row_slot: Optional[torch.Tensor] = None, seg: int = 0, snap=None, xa=None, dq=None) -> torch.Tensor:
        """x [rows, hidden] bf16.  row_slot None: the rows are consecutive tokens of request `slot` (prefill chunk);
        otherwise one decode token per row, row r belonging to state slot row_slot[r].  seg > 0 (with row_slot): runs of
        `seg` consecutive tokens per request (speculative verify rows); snap = (conv_snap [rows, W - 1, C], ssm_snap
        [rows, hv, dk, dv]) then receives the state after every row."""
        c, w = self.c, self.w
        rows = x.shape[0]
        seq = row_slot is None
        # xa / dq: the rows' NVFP4 terms and the decode quantiser (decode widths): both projections run block-scaled
        proj = ops.gemm_fp4(xa, w.in_proj, out=self.proj[:rows]) if xa is not None else ops.linear(x, w.in_proj, out=self.proj[:rows])
        mixed, z, al, be, nq, nv = _split(c, proj)
        cs, ss = snap if snap is not None else (None, None)
        conv = ops.gdn_conv(mixed, w.conv_w, w.conv_b, state.conv, self.conv[:rows], row_slot, slot, seq, seg=seg, snap=cs)
        ops.gdn_recurrent(conv[:, :nq], conv[:, nq:2 * nq], conv[:, 2 * nq:], al, be, w.A_log, w.dt_bias, state.ssm,
                          self.o[:rows], c.k_heads, c.v_heads, c.dk, c.dv, row_slot, slot, seq, prep=self.prep, seg=seg,
                          snap=ss)
        ops.gated_rmsnorm(self.o[:rows], z, w.norm_w, self.gated[:rows], c.v_heads, c.dv, c.eps)
        if xa is not None and dq is not None and dq.usable(rows, w.out_proj):
            return ops.gemm_fp4(dq.plain(self.gated[:rows], "g"), w.out_proj, out=out)
        return ops.linear(self.gated[:rows], w.out_proj, out=out)
