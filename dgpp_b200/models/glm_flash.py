"""KDA + MLA + hyper-connection + MoE decoder family (GLM-Flash style).

The residual path is `streams` parallel copies of the hidden state (manifold-constrained hyper-connections).  Every
sub-block (token mixer, FFN) reads ONE row collapsed from the streams with per-token coefficients, and its output is
written back to all streams through a per-token placement vector and a doubly-stochastic stream mixer:

    pre, post, comb = coefficients(streams)            (flattened-stream RMS norm, (2 + n) n dots, sigmoid / Sinkhorn)
    h               = block(rmsnorm(sum_j pre_j streams_j))
    streams_i       = post_i h + sum_j comb[j, i] streams_j

Token mixers: three of every `mla_every` layers are KDA (delta-rule linear attention with a per-key-channel decay,
a causal depthwise convolution in front, an output gate and a per-head RMS norm behind; fp32 state per request), the
remaining one is multi-head latent attention over a paged latent cache (optionally with the sparse lightning index).
FFN: dense SwiGLU in the first `dense_layers` layers, mixture of experts after.  The head reads a final collapse.
Optional hashed n-gram memory sites (`engram`, `engram_layers`): in front of a listed layer every stream takes in a
value looked up by a hash of the token's last 2 .. max_ngram tokens (`models/engram.py`).

``GlmFlashModel.forward_reference`` is the PyTorch oracle (token by token recurrence, plain non-absorbed attention);
``GlmFlashRunner`` launches the sm_100a kernels: `mhc_compute` / `mhc_fold`, `gdn_conv` + `kda_recurrent` +
`gated_rmsnorm`, the absorbed MLA sequence of `MlaCaches`, the MoE block, tensor-core linears; decode passes are
captured into CUDA graphs per batch width.
(reference counterparts: src/models/glm/forward.cpp, decode.cpp, src/models/kda_layer.cu, src/kernels/kda.cu,
 src/kernels/glm_mhc.cu, src/models/dsa_layer.cu, src/models/glm/moe_layer.cpp.)
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch
import torch.nn.functional as F

from ..ops import core as ops
from ..ops import reference as ref
from ..quant.formats import QuantLinear, quantize
from .engram import Engram, EngramConfig
from .mla_moe import MlaCaches, MlaLayer, mla_attention_reference
from .moe import MoEBlock, MoEConfig, MoEWeights, moe_reference

BF = torch.bfloat16


@dataclass
class GlmFlashConfig:
    layers: int = 4
    hidden: int = 512
    vocab: int = 2048
    mla_every: int = 4           # layer i is MLA when (i + 1) % mla_every == 0, KDA otherwise
    streams: int = 4             # hyper-connection streams (2, 4 or 8)
    sinkhorn_iters: int = 20
    # KDA
    k_heads: int = 4
    v_heads: int = 4
    dk: int = 128
    dv: int = 128
    conv_width: int = 4
    lower_bound: float = -5.0
    # MLA (field names shared with the MLA + MoE family: `MlaCaches` and the oracle read them from this object)
    heads: int = 8
    q_lora: int = 256
    kv_lora: int = 128
    nope: int = 64
    rope: int = 32
    v_dim: int = 64
    index_heads: int = 0
    index_dim: int = 64
    index_topk: int = 64
    # FFN
    ffn: int = 1024
    dense_layers: int = 1
    moe: Optional[MoEConfig] = None
    eps: float = 1e-6
    rope_theta: float = 1e4
    page: int = 64
    engram: Optional[EngramConfig] = None      # hashed n-gram memory in front of the layers listed in engram_layers
    engram_layers: tuple = ()

    def is_mla(self, i: int) -> bool:
        return (i + 1) % self.mla_every == 0

    @property
    def conv_channels(self) -> int:
        return 2 * self.k_heads * self.dk + self.v_heads * self.dv

    @property
    def kda_cols(self) -> int:      # q | k | v (convolved) | z (output gate) | beta | per-channel gate
        return self.conv_channels + self.v_heads * self.dv + self.v_heads + self.v_heads * self.dk


@dataclass
class HcSite:
    """Hyper-connection coefficients of one sub-block."""
    fn: torch.Tensor             # [(2 + n) n, n H] bf16
    base: torch.Tensor           # [(2 + n) n] fp32
    scale: torch.Tensor          # [3] fp32
    norm: torch.Tensor           # [H] bf16: RMSNorm weight of the collapsed row


@dataclass
class KdaWeights:
    in_proj: QuantLinear         # [kda_cols, H]
    conv_w: torch.Tensor         # [conv_channels, W] bf16
    A_log: torch.Tensor          # [hv] fp32
    dt_bias: torch.Tensor        # [hv * dk] fp32
    norm_w: torch.Tensor         # [dv] bf16
    out_proj: QuantLinear        # [H, hv * dv]


@dataclass
class GlmFlashLayer:
    att_hc: HcSite
    ffn_hc: HcSite
    kda: Optional[KdaWeights] = None
    mla: Optional[MlaLayer] = None
    gate_up: Optional[QuantLinear] = None
    down: Optional[QuantLinear] = None
    moe: Optional[MoEWeights] = None


def _kda_split(c: GlmFlashConfig, proj: torch.Tensor):
    cc, nv = c.conv_channels, c.v_heads * c.dv
    o = cc + nv
    return proj[:, :cc], proj[:, cc:o], proj[:, o:o + c.v_heads], proj[:, o + c.v_heads:]


def kda_layer_reference(c: GlmFlashConfig, w: KdaWeights, x: torch.Tensor, conv_state: torch.Tensor,
                        ssm_state: torch.Tensor) -> torch.Tensor:
    """x [T, H] normed bf16 rows of one request; conv_state [W - 1, C] and ssm_state [hv, dk, dv] fp32 in place."""
    T = x.shape[0]
    proj = ref.linear(x, w.in_proj)
    mixed, z, beta, gate = _kda_split(c, proj)
    hist = torch.cat([conv_state, mixed.float()], 0)
    cw = w.conv_w.float()
    conv = torch.zeros(T, c.conv_channels, device=x.device)
    for i in range(c.conv_width):
        conv += hist[i:i + T] * cw[:, i]
    conv_state.copy_(hist[T:])
    act = ref.act(F.silu(conv))
    nq = c.k_heads * c.dk
    o = ref.kda_recurrent(act[:, :nq], act[:, nq:2 * nq], act[:, 2 * nq:], gate, beta, w.A_log, w.dt_bias, c.lower_bound,
                          ssm_state, c.k_heads, c.v_heads, c.dk, c.dv).float().view(T, c.v_heads, c.dv)
    rstd = torch.rsqrt(o.pow(2).mean(-1, keepdim=True) + c.eps)
    n = ref.act(o * rstd).float() * w.norm_w.float()
    gated = ref.act(n * F.silu(z.float().view(T, c.v_heads, c.dv))).reshape(T, c.v_heads * c.dv)
    return ref.linear(gated, w.out_proj)


class GlmFlashModel:
    def __init__(self, cfg: GlmFlashConfig, embed, layers: List[GlmFlashLayer], final_hc: HcSite, head: QuantLinear,
                 inv_freq):
        self.cfg, self.embed, self.layers, self.final_hc, self.head, self.inv_freq = cfg, embed, layers, final_hc, head, inv_freq
        self.engram: Optional[Engram] = None

    @staticmethod
    def random_init(cfg: GlmFlashConfig, device, seed: int = 0, std: float = 0.05, fmt: str = "bf16") -> "GlmFlashModel":
        g = torch.Generator(device=device)
        g.manual_seed(seed)
        c, H, n = cfg, cfg.hidden, cfg.streams
        rnd = lambda *s: torch.randn(*s, device=device, dtype=torch.float32, generator=g)
        lin = lambda rows, k: quantize(rnd(rows, k) * std, fmt if (k % 256 == 0 or fmt == "bf16") else "bf16")
        ones = lambda k: torch.ones(k, device=device, dtype=BF)

        def site():
            return HcSite((rnd((2 + n) * n, n * H) * 0.05).to(BF), rnd((2 + n) * n) * 0.5,
                          torch.tensor([1.0, 1.0, 1.0], device=device), (1 + 0.1 * rnd(H)).to(BF))

        layers = []
        for i in range(c.layers):
            L = GlmFlashLayer(site(), site())
            if c.is_mla(i):
                L.mla = MlaLayer(ones(H), ones(H), lin(c.q_lora, H), ones(c.q_lora), lin(c.heads * (c.nope + c.rope), c.q_lora),
                                 lin(c.kv_lora + c.rope, H), ones(c.kv_lora),
                                 (rnd(c.heads, c.nope, c.kv_lora) * std * 2).to(BF),
                                 (rnd(c.heads, c.v_dim, c.kv_lora) * std * 2).to(BF), lin(H, c.heads * c.v_dim))
                if c.index_heads:
                    L.mla.idx_q = quantize(rnd(c.index_heads * c.index_dim, H) * std * 4, fmt)
                    L.mla.idx_k = quantize(rnd(c.index_dim, H) * std * 4, "bf16")
                    L.mla.idx_w = quantize(rnd(c.index_heads, H) * std, "bf16")
            else:
                L.kda = KdaWeights(quantize(rnd(c.kda_cols, H) * std * 4, fmt), (rnd(c.conv_channels, c.conv_width) * 0.5).to(BF),
                                   torch.log(torch.rand(c.v_heads, device=device, generator=g) * 2 + 0.5),
                                   rnd(c.v_heads * c.dk) * 0.5, (1 + 0.1 * rnd(c.dv)).to(BF), lin(H, c.v_heads * c.dv))
            if c.moe is not None and i >= c.dense_layers:
                L.moe = MoEWeights.random_init(c.moe, device, seed=seed * 1000 + i, std=std)
            else:
                L.gate_up, L.down = lin(2 * c.ffn, H), lin(H, c.ffn)
            layers.append(L)
        embed = (rnd(c.vocab, H) * std * 8).to(BF)
        inv = 1.0 / (c.rope_theta ** (torch.arange(0, c.rope, 2, device=device).float() / c.rope))
        m = GlmFlashModel(cfg, embed, layers, site(), quantize(rnd(c.vocab, H) * std, "bf16"), inv)
        if c.engram is not None and c.engram_layers:
            m.engram = Engram.random_init(c.engram, c.engram_layers, c.vocab, n, H, device, seed=seed, std=std, eps=c.eps)
        return m

    # ------------------------------------------------------------------ oracle
    def forward_reference(self, tokens: torch.Tensor) -> torch.Tensor:
        """fp32 logits [T, V] of one request from position 0."""
        c, n = self.cfg, self.cfg.streams
        dev = self.embed.device
        T = tokens.numel()
        pos = torch.arange(T, device=dev)
        streams = ref.embed_gather(tokens.to(dev), self.embed).unsqueeze(1).repeat(1, n, 1).contiguous()

        def site(hc: HcSite, block):
            nonlocal streams
            col, post, comb = ref.mhc_compute(streams, hc.fn, hc.base, hc.scale, c.sinkhorn_iters, 1e-6, c.eps)
            xn = ref.rmsnorm(col, hc.norm, c.eps)[0]
            streams = ref.mhc_fold(streams, block(xn), post, comb)

        prev = None
        if self.engram is not None:
            prev = torch.tensor(self.engram.prev_rows(tokens.tolist(), []), dtype=torch.int32, device=dev)
        for i, L in enumerate(self.layers):
            if self.engram is not None and i in self.engram.layers:
                streams = self.engram.apply_reference(i, streams, tokens.to(dev), prev)
            if L.mla is not None:
                site(L.att_hc, lambda xn: mla_attention_reference(c, self.inv_freq, L.mla, xn, pos))
            else:
                conv = torch.zeros(c.conv_width - 1, c.conv_channels, device=dev)
                ssm = torch.zeros(c.v_heads, c.dk, c.dv, device=dev)
                site(L.att_hc, lambda xn: kda_layer_reference(c, L.kda, xn, conv, ssm))
            if L.moe is not None:
                site(L.ffn_hc, lambda xn: moe_reference(xn, L.moe))
            else:
                site(L.ffn_hc, lambda xn: ref.linear(ref.swiglu(ref.linear(xn, L.gate_up)), L.down))
        hc = self.final_hc
        col, _, _ = ref.mhc_compute(streams, hc.fn, hc.base, hc.scale, c.sinkhorn_iters, 1e-6, c.eps)
        return ref.linear(ref.rmsnorm(col, hc.norm, c.eps)[0], self.head, out_fp32=True)


class GlmFlashRunner:
    """Kernel execution.  Rows are a prefill chunk of one request (consecutive tokens) or one decode token per request.
    State per request: one latent-cache row per token and MLA layer, one convolution tail and one [hv, dk, dv] fp32
    memory per KDA layer (pooled over the layers: `conv_pool`, `ssm_pool`)."""

    def __init__(self, model: GlmFlashModel, max_rows: int, slots: int, max_seq_len: int, device):
        c = model.cfg
        self.m, self.c, self.dev, self.max_rows, self.slots = model, c, device, max_rows, slots
        self.mla_index = {i: j for j, i in enumerate(i for i in range(c.layers) if c.is_mla(i))}
        self.kda_index = {i: j for j, i in enumerate(i for i in range(c.layers) if not c.is_mla(i))}
        self.att = MlaCaches(c, len(self.mla_index), [model.layers[i].mla.idx_q is not None for i in self.mla_index],
                             max_rows, slots, max_seq_len, device)
        Lk = max(len(self.kda_index), 1)
        self.ssm_pool = torch.zeros(Lk, slots, c.v_heads, c.dk, c.dv, dtype=torch.float32, device=device)
        self.conv_pool = torch.zeros(Lk, slots, c.conv_width - 1, c.conv_channels, dtype=torch.float32, device=device)
        pool = {}
        self.moe = {i: MoEBlock(L.moe, min(max_rows, 16), device, pool=pool) for i, L in enumerate(model.layers)
                    if L.moe is not None and L.moe.gu_q is not None}
        e = lambda *s: torch.empty(*s, dtype=BF, device=device)
        H = c.hidden
        self.streams = e(max_rows, c.streams, H)
        self.h, self.xn = e(max_rows, H), e(max_rows, H)
        self.proj, self.conv = e(max_rows, c.kda_cols), e(max_rows, c.conv_channels)
        self.o, self.gated = e(max_rows, c.v_heads * c.dv), e(max_rows, c.v_heads * c.dv)
        self.prep = torch.empty(max_rows * (2 * c.k_heads * c.dk + 2 * c.v_heads + c.v_heads * c.dk), dtype=torch.float32,
                                device=device)
        self.lengths = [0] * slots
        self.history = [[] for _ in range(slots)]      # the newest tokens of every request (the n-gram memory's lookback)
        self.use_graphs, self._graphs, self._static = True, {}, {}
        self.pdl_graphs = True      # programmatic-dependent-launch edges between this library's kernels in captured passes

    def reset(self, slot: int) -> None:
        self.lengths[slot] = 0
        self.history[slot] = []
        self.ssm_pool[:, slot].zero_()
        self.conv_pool[:, slot].zero_()

    def _state_tensors(self):
        return [self.conv_pool, self.ssm_pool]

    def _site(self, hc: HcSite, rows: int, block) -> None:
        c = self.c
        st = self.streams[:rows]
        col, post, comb = ops.mhc_compute(st, hc.fn, hc.base, hc.scale, c.sinkhorn_iters, 1e-6, c.eps)
        xn = ops.rmsnorm(col, hc.norm, c.eps, out=self.xn[:rows])
        block(xn, self.h[:rows])
        ops.mhc_fold(st, self.h[:rows], post, comb, out=st)

    def _kda(self, i: int, w: KdaWeights, xn: torch.Tensor, out: torch.Tensor, chunk_slot, row_req) -> None:
        c, j = self.c, self.kda_index[i]
        rows = xn.shape[0]
        seq = chunk_slot is not None
        proj = ops.linear(xn, w.in_proj, out=self.proj[:rows])
        mixed, z, beta, gate = _kda_split(c, proj)
        conv = ops.gdn_conv(mixed, w.conv_w, None, self.conv_pool[j], self.conv[:rows], None if seq else row_req,
                            chunk_slot or 0, seq)
        nq = c.k_heads * c.dk
        ops.kda_recurrent(conv[:, :nq], conv[:, nq:2 * nq], conv[:, 2 * nq:], gate, beta, w.A_log, w.dt_bias, c.lower_bound,
                          self.ssm_pool[j], self.o[:rows], c.k_heads, c.v_heads, c.dk, c.dv,
                          row_slot=None if seq else row_req, slot=chunk_slot or 0, sequential=seq, prep=self.prep)
        ops.gated_rmsnorm(self.o[:rows], z, w.norm_w, self.gated[:rows], c.v_heads, c.dv, c.eps)
        ops.linear(self.gated[:rows], w.out_proj, out=out)

    def _ffn(self, i: int, L: GlmFlashLayer, xn: torch.Tensor, out: torch.Tensor) -> None:
        if L.moe is None:
            ops.linear(ops.swiglu(ops.linear(xn, L.gate_up)), L.down, out=out)
            return
        blk = self.moe.get(i)
        if blk is not None and xn.shape[0] <= blk.max_rows:
            blk.forward(xn, out)
        elif blk is not None:
            out.copy_(blk.forward_gathered(xn))
        else:
            out.copy_(moe_reference(xn, L.moe))

    @torch.no_grad()
    def forward(self, tokens: torch.Tensor, positions: torch.Tensor, row_req: torch.Tensor,
                chunk_slot: Optional[int] = None, all_logits: bool = True, select: bool = True,
                prev: Optional[torch.Tensor] = None) -> torch.Tensor:
        """int32 [rows] device tensors -> fp32 logits [rows, V] (all_logits=False: the last row's, [1, V]).  chunk_slot
        given: the rows are consecutive tokens of that request (prefill chunk); otherwise one decode token per row."""
        m, c = self.m, self.c
        rows = tokens.shape[0]
        st = self.streams[:rows]
        ops.embed_gather(tokens, m.embed, out=self.h[:rows])
        st.copy_(self.h[:rows].unsqueeze(1).expand(rows, c.streams, c.hidden))
        for i, L in enumerate(m.layers):
            if m.engram is not None and i in m.engram.layers:
                m.engram.apply(i, st, tokens, prev)
            if L.mla is not None:
                j = self.mla_index[i]
                self._site(L.att_hc, rows, lambda xn, out: self.att.attention(j, L.mla, m.inv_freq, xn, positions, row_req,
                                                                              select, out))
            else:
                self._site(L.att_hc, rows, lambda xn, out: self._kda(i, L.kda, xn, out, chunk_slot, row_req))
            self._site(L.ffn_hc, rows, lambda xn, out: self._ffn(i, L, xn, out))
        hc = m.final_hc
        col, _, _ = ops.mhc_compute(st, hc.fn, hc.base, hc.scale, c.sinkhorn_iters, 1e-6, c.eps)
        xn = ops.rmsnorm(col, hc.norm, c.eps, out=self.xn[:rows])
        sel = xn if all_logits else xn[rows - 1:rows]
        return ops.gemm_tc(sel, m.head, out32=torch.empty(sel.shape[0], c.vocab, dtype=torch.float32, device=self.dev))

    @torch.no_grad()
    def prefill(self, slot: int, tokens: List[int], chunk: int = 64) -> torch.Tensor:
        """Appends `tokens` to request `slot`; returns the logits of the last token [1, V]."""
        start = self.lengths[slot]
        assert start + len(tokens) <= self.att.max_ctx - self.att.page
        out = None
        for o in range(0, len(tokens), chunk):
            part = tokens[o:o + chunk]
            t = torch.tensor(part, dtype=torch.int32, device=self.dev)
            pos = torch.arange(start + o, start + o + len(part), dtype=torch.int32, device=self.dev)
            req = torch.full((len(part),), slot, dtype=torch.int32, device=self.dev)
            prev = None
            if self.m.engram is not None:
                prev = torch.tensor(self.m.engram.prev_rows(part, self.history[slot]), dtype=torch.int32, device=self.dev)
                self.history[slot] = self.m.engram.keep(self.history[slot], part)
            out = self.forward(t, pos, req, chunk_slot=slot, all_logits=False,
                               select=start + o + len(part) > self.c.index_topk, prev=prev)
        self.lengths[slot] = start + len(tokens)
        return out

    @torch.no_grad()
    def decode(self, slots: List[int], tokens: List[int]) -> torch.Tensor:
        """One token per listed request -> fp32 logits [len(slots), V].  On a GPU the pass is captured once per batch
        width into a CUDA graph over static id / position / request tensors and replayed; the warm-up and capture
        passes must not move the recurrent state, so it is saved before them and put back after."""
        b = len(slots)
        positions = [self.lengths[s] for s in slots]
        select = bool(self.c.index_heads) and max(positions) + 1 > self.c.index_topk
        rows3 = [tokens, positions, slots]
        eng = self.m.engram
        if eng is not None:
            per = [eng.prev_rows([t], self.history[s]) for s, t in zip(slots, tokens)]
            rows3 = rows3 + [[per[r][k][0] for r in range(b)] for k in range(eng.cfg.max_ngram - 1)]
        host = torch.tensor(rows3, dtype=torch.int32)
        rest = lambda t: t[3:] if t.shape[0] > 3 else None
        if not (self.use_graphs and torch.device(self.dev).type == "cuda"):
            d = host.to(self.dev)
            out = self.forward(d[0], d[1], d[2], select=select, prev=rest(d))
        else:
            key = (b, select)
            st = self._static.get(key)
            if st is None:
                st = self._static[key] = torch.zeros(host.shape[0], b, dtype=torch.int32, device=self.dev)
            st.copy_(host, non_blocking=True)
            g = self._graphs.get(key)
            if g is None:
                saved = [t.clone() for t in self._state_tensors()]
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.forward(st[0], st[1], st[2], select=select, prev=rest(st))
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                from ..engine.graph import capture_with_pdl
                graph, out, _ = capture_with_pdl(lambda: self.forward(st[0], st[1], st[2], select=select, prev=rest(st)),
                                                 self.pdl_graphs)
                for t, s0 in zip(self._state_tensors(), saved):
                    t.copy_(s0)
                g = self._graphs[key] = (graph, out)
            graph, out = g
            graph.replay()
        for s, t in zip(slots, tokens):
            self.lengths[s] += 1
            if eng is not None:
                self.history[s] = eng.keep(self.history[s], [t])
        return out
