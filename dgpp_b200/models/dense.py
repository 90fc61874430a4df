"""Dense GQA decoder (Llama/Qwen-style): RMSNorm -> fused QKV -> RoPE -> GQA attention -> o_proj ->
RMSNorm -> SwiGLU MLP, with quantised linear layers in checkpoint layout.

Tensor parallel sharding (reference contract: lines 344-400 of the reference tree's top-level design document -- heads sharded,
q/kv/gate-up column-split, o_proj/down row-split, hidden replicated at block boundaries):
rank r owns q heads [r*hq/W, (r+1)*hq/W), the matching kv heads, and rows [r*I/W, (r+1)*I/W) of the
MLP intermediate; the two row-split projections are followed by an all-reduce.

``DenseModel.forward_reference`` is the PyTorch oracle (any device); ``DenseRunner`` in
``dgpp_b200.engine.runner`` executes the same math with the sm_100a kernels.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize, random_quant_linear

BF = torch.bfloat16


@dataclass
class DenseConfig:
    layers: int = 64
    hidden: int = 5120
    q_heads: int = 40
    kv_heads: int = 8
    head_dim: int = 128
    ffn: int = 17408
    vocab: int = 151936
    rope_theta: float = 1e6
    rot_dim: Optional[int] = None
    eps: float = 1e-6
    qk_norm: bool = False
    weight_fmt: str = "nvfp4"
    head_fmt: str = "bf16"
    kv_fp8: bool = True
    page: int = 64
    yarn_factor: float = 1.0
    yarn_original_max_pos: int = 0
    # sliding-window + sink attention families: layers attend to the last `sliding_window` positions, except every
    # `global_every`-th layer (1-based) which stays global; `attn_sinks` adds a learned per-head sink logit (a
    # value-less softmax column) to every layer
    sliding_window: int = 0
    global_every: int = 0
    attn_sinks: bool = False
    name: str = "dense-27b-nvfp4"

    def layer_window(self, li: int) -> int:
        if self.sliding_window <= 0 or (self.global_every > 0 and (li + 1) % self.global_every == 0):
            return 0
        return self.sliding_window

    @staticmethod
    def dense_27b(**kw) -> "DenseConfig":
        return DenseConfig(**kw)

    @staticmethod
    def plumbing_fp32(**kw) -> "DenseConfig":
        """The CPU-plumbing model: 2 layers, hidden 256, 4 q / 2 kv heads of 64, SwiGLU 688, RoPE 1e4, fp32."""
        base = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=688, vocab=4096, rope_theta=1e4,
                    weight_fmt="fp32", head_fmt="fp32", kv_fp8=False, page=16, name="plumbing-fp32")
        base.update(kw)
        return DenseConfig(**base)

    @staticmethod
    def tiny(**kw) -> "DenseConfig":
        base = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, ffn=768, vocab=4096,
                    rope_theta=1e4, weight_fmt="nvfp4", name="dense-tiny")
        base.update(kw)
        return DenseConfig(**base)

    def param_count(self) -> int:
        per = self.hidden * (self.q_heads + 2 * self.kv_heads) * self.head_dim
        per += self.q_heads * self.head_dim * self.hidden + 3 * self.hidden * self.ffn
        return self.layers * per + 2 * self.vocab * self.hidden


@dataclass
class DenseLayer:
    in_norm: torch.Tensor
    post_norm: torch.Tensor
    qkv: QuantLinear          # [(hq + 2 hkv) * d / W, hidden]
    o: QuantLinear            # [hidden, hq * d / W]
    gate_up: QuantLinear      # [2 * ffn / W, hidden] (gate rows then up rows)
    down: QuantLinear         # [hidden, ffn / W]
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    sink: Optional[torch.Tensor] = None    # [local q heads] fp32 sink logits
    window: int = 0                        # sliding window of this layer (0 = global)


@dataclass
class DenseModel:
    cfg: DenseConfig
    embed: torch.Tensor       # [vocab, hidden] bf16 (replicated)
    layers: List[DenseLayer]
    final_norm: torch.Tensor
    head: QuantLinear         # [vocab / W, hidden]
    tp_rank: int = 0
    tp_size: int = 1
    inv_freq: torch.Tensor = field(default=None)
    mscale: float = 1.0

    # ------------------------------------------------------------------ construction
    @staticmethod
    def random_init(cfg: DenseConfig, device="cuda", seed: int = 0, tp_rank: int = 0, tp_size: int = 1,
                    std: float = 0.02) -> "DenseModel":
        """N(0, std) weights quantised to cfg.weight_fmt.  Every rank draws the full matrices from the same
        seed and keeps its shard, so shards of different world sizes describe the same model."""
        W = tp_size
        assert cfg.q_heads % W == 0 and cfg.kv_heads % W == 0 and cfg.ffn % W == 0 and cfg.vocab % W == 0
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        d, H = cfg.head_dim, cfg.hidden

        def full(n, k):
            return torch.randn(n, k, device=device, dtype=torch.float32, generator=g) * std

        def make(n, k, fmt, row_slices=None, col_slice=None, pad_rows=0, pad_cols=0, pad_first=0):
            w = full(n, k)
            if W > 1 and row_slices is not None:
                parts = [w[a:b] for a, b in row_slices]
                if pad_rows:   # zero rows after every slice (the padded intermediate channels stay exactly zero)
                    parts = [torch.cat([q, q.new_zeros(pad_rows, k)]) for q in parts]
                if pad_first:  # zero rows after the first slice only (padding query heads)
                    parts[0] = torch.cat([parts[0], parts[0].new_zeros(pad_first, k)])
                w = torch.cat(parts)
            if W > 1 and col_slice is not None:
                w = w[:, col_slice[0]:col_slice[1]]
                if pad_cols:
                    w = torch.cat([w, w.new_zeros(n, pad_cols)], dim=1)
                w = w.contiguous()
            return quantize_like_random(w, fmt, std)

        hq_l, hkv_l, ffn_l = cfg.q_heads // W, cfg.kv_heads // W, cfg.ffn // W
        # a rank's slice of the intermediate dimension is padded with zero channels up to the K granule of the
        # block-scaled tensor-core GEMM (256), e.g. 17408 / 8 = 2176 -> 2304
        ffn_pad = (-ffn_l) % 256 if (W > 1 and cfg.weight_fmt in ("nvfp4", "mxfp4")) else 0
        q_pad = (padded_q_heads(cfg, W) - hq_l) * d
        r = tp_rank
        adt = torch.float32 if cfg.weight_fmt == "fp32" else BF
        embed = (torch.randn(cfg.vocab, H, device=device, dtype=torch.float32, generator=g) * std).to(adt)
        layers = []
        ones = lambda n: torch.ones(n, device=device, dtype=adt)
        for _ in range(cfg.layers):
            nq, nkv = cfg.q_heads * d, cfg.kv_heads * d
            qkv = make(nq + 2 * nkv, H, cfg.weight_fmt, pad_first=q_pad,
                       row_slices=[(r * hq_l * d, (r + 1) * hq_l * d),
                                   (nq + r * hkv_l * d, nq + (r + 1) * hkv_l * d),
                                   (nq + nkv + r * hkv_l * d, nq + nkv + (r + 1) * hkv_l * d)])
            o = make(H, nq, cfg.weight_fmt, col_slice=(r * hq_l * d, (r + 1) * hq_l * d), pad_cols=q_pad)
            gu = make(2 * cfg.ffn, H, cfg.weight_fmt, pad_rows=ffn_pad,
                      row_slices=[(r * ffn_l, (r + 1) * ffn_l), (cfg.ffn + r * ffn_l, cfg.ffn + (r + 1) * ffn_l)])
            dn = make(H, cfg.ffn, cfg.weight_fmt, col_slice=(r * ffn_l, (r + 1) * ffn_l), pad_cols=ffn_pad)
            sink = None
            if cfg.attn_sinks:
                full_sink = torch.randn(cfg.q_heads, device=device, dtype=torch.float32, generator=g)
                sink = torch.full((padded_q_heads(cfg, W),), -1e4, device=device, dtype=torch.float32)
                sink[:hq_l] = full_sink[r * hq_l:(r + 1) * hq_l]
            layers.append(DenseLayer(ones(H), ones(H), qkv, o, gu, dn,
                                     ones(d) if cfg.qk_norm else None, ones(d) if cfg.qk_norm else None,
                                     sink, cfg.layer_window(len(layers))))
        vl = cfg.vocab // W
        head = make(cfg.vocab, H, cfg.head_fmt, row_slices=[(r * vl, (r + 1) * vl)])
        m = DenseModel(cfg, embed, layers, ones(H), head, tp_rank, tp_size)
        m._init_rope(device)
        return m

    def _init_rope(self, device):
        c = self.cfg
        inv, ms = ref.rope_inv_freq(c.rot_dim or c.head_dim, c.rope_theta, device, c.yarn_factor,
                                    c.yarn_original_max_pos)
        self.inv_freq, self.mscale = inv.contiguous(), ms

    @property
    def hq_local(self) -> int:
        """Query heads computed on this rank, padding heads included (see `padded_q_heads`)."""
        return padded_q_heads(self.cfg, self.tp_size)

    @property
    def hkv_local(self) -> int:
        return self.cfg.kv_heads // self.tp_size

    def pack_bf12(self) -> int:
        """Swap the bf16 matrices of the model (the lm head) for their lossless 12-bit resident form where it pays
        (see quant.formats.bf12_encode); the outputs do not change by a bit.  Returns the bytes saved."""
        from ..quant.formats import bf12_encode
        saved = 0
        if self.head.fmt == "bf16" and self.head.k % 128 == 0:
            q = bf12_encode(self.head.payload)
            if q is not None:
                saved += self.head.nbytes - q.nbytes
                self.head = q
        return saved

    def weight_bytes(self) -> int:
        b = self.head.nbytes
        for l in self.layers:
            b += l.qkv.nbytes + l.o.nbytes + l.gate_up.nbytes + l.down.nbytes
        return b

    # ------------------------------------------------------------------ PyTorch oracle
    @torch.no_grad()
    def forward_reference(self, tokens: torch.Tensor, start_pos: int = 0, kv: Optional[list] = None,
                          all_reduce=None, return_hidden: bool = False, lora=None, embed_spans=None, capture=None):
        """Full-precision-accumulate reference of one request: tokens [T] at positions start_pos.. .
        `kv` is a list (per layer) of (k, v) fp32 tensors [Tk, hkv, d] that is extended in place; KV
        values go through the same FP8 round trip as the paged cache when cfg.kv_fp8.  `lora`: a bound
        ``adapters.lora.LoraAdapter`` whose updates are added to the bf16 outputs of the projections.  `capture`: a dict
        whose integer keys name layers; each gets the bf16 residual stream entering that layer [T, hidden] (key
        `layers`: the stream entering the final norm)."""
        from ..adapters.lora import lora_reference

        def adapt(li, proj, xin, out):
            if lora is not None:
                for p in lora.pairs(li, proj):
                    sl = slice(p.col0, p.col0 + p.b.shape[0])
                    out[:, sl] = lora_reference(xin, p.a, p.b, out[:, sl], lora.scale)
            return out

        c = self.cfg
        T = tokens.numel()
        dev = self.embed.device
        d, hq, hkv = c.head_dim, self.hq_local, self.hkv_local
        pos = torch.arange(start_pos, start_pos + T, device=dev)
        x = ref.embed_gather(tokens.to(dev), self.embed)
        # embed_spans: [(absolute start position, rows [n, hidden])] -- rows of an image (or any precomputed input
        # embedding) replace the token embeddings of the positions they cover
        for p0, rows in embed_spans or ():
            a, b = max(p0, start_pos), min(p0 + rows.shape[0], start_pos + T)
            if a < b:
                x[a - start_pos:b - start_pos] = rows[a - p0:b - p0].to(x.dtype).to(dev)
        delta = None
        if kv is None:
            kv = [None] * c.layers
        scale = 1.0 / math.sqrt(d)  # the YaRN attention factor is carried by cos/sin (mscale)
        for li, L in enumerate(self.layers):
            xn, x = ref.rmsnorm(x, L.in_norm, c.eps, delta)
            if capture is not None and li in capture:
                capture[li] = x.clone()
            qkv = adapt(li, "qkv", xn, ref.linear(xn, L.qkv)).float()
            q = qkv[:, :hq * d].view(T, hq, d)
            k = qkv[:, hq * d:(hq + hkv) * d].view(T, hkv, d)
            v = qkv[:, (hq + hkv) * d:].view(T, hkv, d)
            if L.q_norm is not None:
                q = ref.head_norm(q, L.q_norm, c.eps)
                k = ref.head_norm(k, L.k_norm, c.eps)
            q = ref.apply_rope(q, pos, self.inv_freq, c.rot_dim or d, self.mscale)
            k = ref.apply_rope(k, pos, self.inv_freq, c.rot_dim or d, self.mscale)
            if c.kv_fp8:
                kq, ks = ref.quant_kv_fp8(k)
                vq, vs = ref.quant_kv_fp8(v)
                k = kq.view(torch.float8_e4m3fn).float() * ks.unsqueeze(-1)
                v = vq.view(torch.float8_e4m3fn).float() * vs.unsqueeze(-1)
            else:
                v = ref._r(v)
            if kv[li] is not None:
                k = torch.cat([kv[li][0], k])
                v = torch.cat([kv[li][1], v])
            kv[li] = (k, v)
            a = ref.act(ref.attention(q, k, v, scale, causal_offset=start_pos, window=L.window,
                                      sink=L.sink).reshape(T, hq * d))
            o = adapt(li, "o", a, ref.linear(a, L.o))
            if all_reduce is not None:
                o = all_reduce(o)
            xn, x = ref.rmsnorm(x, L.post_norm, c.eps, o)
            act = ref.swiglu(adapt(li, "gate_up", xn, ref.linear(xn, L.gate_up)))
            delta = adapt(li, "down", act, ref.linear(act, L.down))
            if all_reduce is not None:
                delta = all_reduce(delta)
        xn, x = ref.rmsnorm(x, self.final_norm, c.eps, delta)
        if capture is not None and c.layers in capture:
            capture[c.layers] = x.clone()
        if return_hidden:
            return xn, kv
        logits = ref.linear(xn, self.head, out_fp32=True)
        return logits, kv


def padded_q_heads(cfg: "DenseConfig", tp_size: int) -> int:
    """Local query heads.  With NVFP4 weights under tensor parallelism the o_proj K dimension (heads * head_dim)
    must be a multiple of the block-scaled GEMM's K granule (256) and the q-per-kv group one the tensor-core
    attention supports; otherwise zero heads are appended (zero q rows in qkv, zero columns in o_proj: they add
    exact zeros).  40 heads / 8 ranks = 5 heads of 128 (K = 640) becomes 8 heads (K = 1024)."""
    hq, hkv = cfg.q_heads // tp_size, max(cfg.kv_heads // tp_size, 1)
    if tp_size == 1 or cfg.weight_fmt not in ("nvfp4", "mxfp4") or (hq * cfg.head_dim) % 256 == 0:
        return hq
    for cand in range(hq + 1, 8 * hkv + 1):
        if (cand * cfg.head_dim) % 256 == 0 and cand % hkv == 0 and cand // hkv in (1, 2, 4, 5, 8):
            return cand
    return hq


def quantize_like_random(w: torch.Tensor, fmt: str, std: float) -> QuantLinear:
    """Quantise a shard with the same analytic nvfp4 tensor scale that `random_quant_linear` uses, so the
    shards of every world size decode to the same values."""
    if fmt != "nvfp4":
        return quantize(w, fmt)
    from ..quant.formats import e2m1_encode, pack_nibbles
    n, k = w.shape
    gs = (5.5 * std) / (6.0 * 448.0)
    blk = w.view(n, k // 16, 16)
    sb8 = (blk.abs().amax(-1) / 6.0 / gs).clamp(max=448.0).to(torch.float8_e4m3fn)
    sbf = sb8.float().clamp_min(2.0 ** -9).unsqueeze(-1)
    codes = e2m1_encode(blk / (sbf * gs))
    return QuantLinear("nvfp4", n, k, pack_nibbles(codes.view(n, k)).contiguous(),
                       sb8.view(torch.uint8).contiguous(), gs)
