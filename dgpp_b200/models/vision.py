"""Vision tower: a ViT encoder that turns an image canvas into rows of the text model's hidden size, one row per
visual token, spliced into the prompt's embedding rows at the image's pad tokens.

Structure (the Qwen-VL / GLM-V family shape): patch embedding (a p x p convolution as one GEMM over flattened
patches) -> L pre-norm blocks [LayerNorm -> qkv (+bias) -> 2-D RoPE (first half of a head rotates by the patch row,
second half by the patch column) -> full (non-causal) attention -> proj (+bias) -> residual; LayerNorm -> fc1 -> GELU
-> fc2 -> residual] -> spatial merge of m x m neighbouring patches (patch rows are ordered so that a merge group is
contiguous, the merge is a reshape) -> LayerNorm -> MLP projector to the text hidden size.

CUDA path: every linear and both attention products run on the tcgen05 GEMM (`ops.gemm_tc`, bf16 operands: per head
S = Q.K^T with K as the [T, d] "weight", then O = P.V with V^T as the [d, T_pad] "weight"); the kernels in
csrc/kernels/vision.cu prepare the operands.  `forward_reference` is the fp32 PyTorch statement of the same math.
(reference counterparts: src/models/glm/vision.cpp, src/models/qwen/vision.cpp, src/kernels/*_vision.cu.)
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional, Tuple

import torch

from ..quant.formats import QuantLinear

BF = torch.bfloat16


@dataclass
class VisionConfig:
    patch: int = 14
    merge: int = 2
    hidden: int = 256
    heads: int = 4
    layers: int = 2
    mlp: int = 512
    out_hidden: int = 256           # the text model's hidden size
    eps: float = 1e-6
    rope_theta: float = 10000.0
    act: str = "gelu"               # "gelu" (erf) or "gelu_tanh"
    mean: Tuple[float, float, float] = (0.48145466, 0.4578275, 0.40821073)
    std: Tuple[float, float, float] = (0.26862954, 0.26130258, 0.27577711)

    @property
    def head_dim(self) -> int:
        return self.hidden // self.heads

    @property
    def grid(self) -> int:
        return self.patch * self.merge


@dataclass
class VisionBlock:
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    qkv: QuantLinear
    qkv_b: torch.Tensor
    proj: QuantLinear
    proj_b: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor
    fc1: QuantLinear
    fc1_b: torch.Tensor
    fc2: QuantLinear
    fc2_b: torch.Tensor


@dataclass
class VisionTower:
    cfg: VisionConfig
    patch_embed: QuantLinear            # [hidden, 3 * p * p]
    patch_b: torch.Tensor
    blocks: List[VisionBlock]
    merge_ln_w: torch.Tensor
    merge_ln_b: torch.Tensor
    merge_fc1: QuantLinear              # [out_hidden, merge^2 * hidden]
    merge_fc1_b: torch.Tensor
    merge_fc2: QuantLinear              # [out_hidden, out_hidden]
    merge_fc2_b: torch.Tensor
    _scratch: dict = field(default_factory=dict)

    @staticmethod
    def random_init(cfg: VisionConfig, device="cuda", seed: int = 0, std: float = 0.05) -> "VisionTower":
        assert cfg.hidden % cfg.heads == 0 and cfg.head_dim % 4 == 0
        g = torch.Generator(device="cpu")
        g.manual_seed(seed)

        def lin(n, k):
            return QuantLinear("bf16", n, k, (torch.randn(n, k, generator=g) * std).to(BF).to(device))

        def vec(n, base=0.0, s=0.02):
            return (base + torch.randn(n, generator=g) * s).to(BF).to(device)

        h, p = cfg.hidden, cfg.patch
        blocks = [VisionBlock(vec(h, 1.0), vec(h), lin(3 * h, h), vec(3 * h), lin(h, h), vec(h), vec(h, 1.0), vec(h),
                              lin(cfg.mlp, h), vec(cfg.mlp), lin(h, cfg.mlp), vec(h)) for _ in range(cfg.layers)]
        mh = cfg.merge * cfg.merge * h
        return VisionTower(cfg, lin(h, 3 * p * p), vec(h), blocks, vec(mh, 1.0), vec(mh),
                           lin(cfg.out_hidden, mh), vec(cfg.out_hidden), lin(cfg.out_hidden, cfg.out_hidden),
                           vec(cfg.out_hidden))

    # ------------------------------------------------------------------ geometry
    def tokens_of(self, canvas_h: int, canvas_w: int) -> int:
        g = self.cfg.grid
        assert canvas_h % g == 0 and canvas_w % g == 0
        return (canvas_h // g) * (canvas_w // g)

    def patch_positions(self, canvas_h: int, canvas_w: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
        """(row, column) of every patch in the tower's row order (merge groups contiguous)."""
        c = self.cfg
        ph, pw, m = canvas_h // c.patch, canvas_w // c.patch, c.merge
        gy, gx, my, mx = torch.meshgrid(torch.arange(ph // m), torch.arange(pw // m), torch.arange(m), torch.arange(m),
                                        indexing="ij")
        py = (gy * m + my).reshape(-1).to(torch.int32).to(device)
        px = (gx * m + mx).reshape(-1).to(torch.int32).to(device)
        return py, px

    # ------------------------------------------------------------------ fp32 oracle
    @torch.no_grad()
    def forward_reference(self, canvas: torch.Tensor) -> torch.Tensor:
        """canvas: uint8 [H, W, 3] -> fp32 [tokens, out_hidden].  Activations are rounded to bf16 where the CUDA path
        stores them, so the two agree to bf16 rounding noise."""
        c = self.cfg
        dev = canvas.device
        H, W, _ = canvas.shape
        p, m = c.patch, c.merge
        py, px = self.patch_positions(H, W, dev)
        x = canvas.float() / 255.0
        x = (x - torch.tensor(c.mean, device=dev)) / torch.tensor(c.std, device=dev)
        # [H, W, 3] -> patches [ph, pw, 3, p, p] -> tower order
        x = x.view(H // p, p, W // p, p, 3).permute(0, 2, 4, 1, 3)
        x = x[py.long(), px.long()].reshape(-1, 3 * p * p)
        r = lambda t: t.to(BF).float()
        lin = lambda t, w, b: r(r(t) @ w.payload.float().T) + b.float()
        ln = lambda t, w, b: torch.nn.functional.layer_norm(t, (t.shape[-1],), w.float(), b.float(), c.eps)
        act = (lambda t: torch.nn.functional.gelu(t)) if c.act == "gelu" else \
            (lambda t: torch.nn.functional.gelu(t, approximate="tanh"))
        x = r(lin(r(x), self.patch_embed, self.patch_b))
        T, d, nh = x.shape[0], c.head_dim, c.heads
        half, quarter = d // 2, d // 4
        inv = c.rope_theta ** (-torch.arange(quarter, device=dev).float() / quarter)

        def rope(t):                              # t [T, heads, d]
            out = t.clone()
            for seg, pos in ((0, py), (1, px)):
                ang = pos.float().unsqueeze(-1) * inv
                cs, sn = ang.cos().unsqueeze(1), ang.sin().unsqueeze(1)
                a = t[..., seg * half:seg * half + quarter]
                b = t[..., seg * half + quarter:(seg + 1) * half]
                out[..., seg * half:seg * half + quarter] = a * cs - b * sn
                out[..., seg * half + quarter:(seg + 1) * half] = b * cs + a * sn
            return out

        for B in self.blocks:
            h1 = r(ln(x, B.ln1_w, B.ln1_b))
            qkv = r(h1 @ B.qkv.payload.float().T)       # (the bias joins in the split kernel, before the rotation)
            qkv = qkv + B.qkv_b.float()
            q, k, v = (qkv[:, i * c.hidden:(i + 1) * c.hidden].view(T, nh, d) for i in range(3))
            q, k, v = r(rope(q)), r(rope(k)), r(v)
            s = r(torch.einsum("thd,shd->hts", q, k) / math.sqrt(d))
            pr = r(torch.softmax(s, dim=-1))
            o = r(torch.einsum("hts,shd->thd", pr, v)).reshape(T, c.hidden)
            x = r(lin(o, B.proj, B.proj_b) + x)
            h2 = r(ln(x, B.ln2_w, B.ln2_b))
            f = r(act(lin(h2, B.fc1, B.fc1_b)))
            x = r(lin(f, B.fc2, B.fc2_b) + x)
        x = x.view(T // (m * m), m * m * c.hidden)
        x = r(ln(x, self.merge_ln_w, self.merge_ln_b))
        x = r(act(lin(x, self.merge_fc1, self.merge_fc1_b)))
        return r(lin(x, self.merge_fc2, self.merge_fc2_b))

    # ------------------------------------------------------------------ CUDA path
    def _buf(self, name: str, shape, dtype=BF, zero: bool = False):
        key = (name, tuple(shape), dtype)
        t = self._scratch.get(key)
        if t is None:
            dev = self.patch_embed.payload.device
            t = (torch.zeros if zero else torch.empty)(*shape, dtype=dtype, device=dev)
            self._scratch[key] = t
        return t

    @torch.no_grad()
    def forward(self, canvas: torch.Tensor) -> torch.Tensor:
        """canvas: uint8 [H, W, 3] on the tower's device -> bf16 [tokens, out_hidden]."""
        from ..ops import core as ops

        c = self.cfg
        H, W, _ = canvas.shape
        dev = canvas.device
        p, m, h, nh, d = c.patch, c.merge, c.hidden, c.heads, c.head_dim
        assert d % 64 == 0, "the tensor-core attention products need head_dim % 64 == 0"
        T = (H // p) * (W // p)
        T_pad = (T + 63) // 64 * 64
        act = 1 if c.act == "gelu" else 2
        py, px = self.patch_positions(H, W, dev)
        patches = self._buf("patches", (T, (3 * p * p + 63) // 64 * 64), zero=True)
        feat = 3 * p * p
        if patches.shape[1] == feat:
            ops.vis_patchify(canvas, patches, p, m, c.mean, c.std)
            x = ops.gemm_tc(patches, self.patch_embed)
        else:
            # the GEMM wants K % 64 == 0: patch rows and the embedding's columns are zero-padded once
            tmp = self._buf("patches_raw", (T, feat))
            ops.vis_patchify(canvas, tmp, p, m, c.mean, c.std)
            patches[:, :feat].copy_(tmp)
            x = ops.gemm_tc(patches, self._padded_patch_embed(patches.shape[1]))
        ops.bias_act(x, self.patch_b)
        q_h = self._buf("q_h", (nh, T, d))
        k_h = self._buf("k_h", (nh, T, d))
        vt_h = self._buf("vt_h", (nh, d, T_pad), zero=True)
        s = self._buf("scores", (T, T_pad))
        o = self._buf("attn_out", (T, h))
        scale = 1.0 / math.sqrt(d)
        for B in self.blocks:
            h1 = ops.layernorm(x, B.ln1_w, B.ln1_b, c.eps)
            qkv = ops.gemm_tc(h1, B.qkv)
            ops.vis_qkv_split_rope(qkv, B.qkv_b, py, px, q_h, k_h, vt_h, nh, d, c.rope_theta)
            for hd in range(nh):
                # S = scale * Q.K^T on the tensor cores (K rows as the weight operand), softmax, O = P.V
                ops.gemm_tc(q_h[hd], QuantLinear("bf16", T, d, k_h[hd], alpha=scale), out=s[:, :T])
                ops.softmax_rows(s, T)
                ops.gemm_tc(s, QuantLinear("bf16", d, T_pad, vt_h[hd]), out=o[:, hd * d:(hd + 1) * d])
            y = ops.gemm_tc(o, B.proj)
            ops.bias_act(y, B.proj_b, resid=x)
            x = y
            h2 = ops.layernorm(x, B.ln2_w, B.ln2_b, c.eps)
            f = ops.gemm_tc(h2, B.fc1)
            ops.bias_act(f, B.fc1_b, act=act)
            y = ops.gemm_tc(f, B.fc2)
            ops.bias_act(y, B.fc2_b, resid=x)
            x = y
        x = x.view(T // (m * m), m * m * h)
        x = ops.layernorm(x, self.merge_ln_w, self.merge_ln_b, c.eps)
        x = ops.gemm_tc(x, self.merge_fc1)
        ops.bias_act(x, self.merge_fc1_b, act=act)
        x = ops.gemm_tc(x, self.merge_fc2)
        ops.bias_act(x, self.merge_fc2_b)
        return x

    def _padded_patch_embed(self, k_pad: int) -> QuantLinear:
        w = self._scratch.get("patch_embed_padded")
        if w is None:
            pe = self.patch_embed
            pay = torch.zeros(pe.n, k_pad, dtype=BF, device=pe.payload.device)
            pay[:, :pe.k] = pe.payload
            w = QuantLinear("bf16", pe.n, k_pad, pay)
            self._scratch["patch_embed_padded"] = w
        return w
