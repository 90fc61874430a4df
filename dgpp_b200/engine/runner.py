"""Kernel-path execution of the dense decoder: one `DenseRunner` owns the static activation buffers
and issues the sm_100a kernels for a batch of rows (prefill chunk or decode batch).

Every buffer is allocated once, so a forward pass is a pure sequence of kernel launches on the
current stream: it can be captured into a CUDA graph as is (no allocation, no host sync).
Row-split projections (o_proj, down) are followed by the tensor-parallel reduction supplied by a
`Reducer` (``dgpp_b200.parallel``): the fused peer-memory kernel, or NCCL as the baseline.
(reference call stack being replaced: src/models/qwen/model35.cpp:2066-2399 run_rows.)
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..models.dense import DenseModel
from ..ops import core as ops
from .kv_cache import PagedKV

BF = torch.bfloat16


class DenseRunner:
    def __init__(self, model: DenseModel, kv: PagedKV, max_rows: int, reducer=None, decode_splits: int = 8,
                 decode_fp4: bool = True, act_terms: int = 3, attn_tc: bool = True,
                 decode_rows: Optional[int] = None, fuse_ar: bool = True, fused_decode: bool = False,
                 l2_prefetch: bool = False, fuse_combine: bool = True, seq_parallel: bool = True):
        self.m, self.kv, self.max_rows, self.reducer = model, kv, max_rows, reducer
        # tensor parallel at prefill sizes: keep the residual stream sharded by token tile between the blocks (fold +
        # norm at the owner, normed rows all-gathered straight into the next projection); False: every boundary folds
        # and gathers the residual rows themselves
        self.seq_parallel = seq_parallel
        # decode rows (<= 64) run the linears on the block-scaled FP4 tensor-core path with the activations
        # expanded into `act_terms` residual NVFP4 terms; attention reads the FP8 cache through tcgen05
        self.decode_fp4 = decode_fp4 and model.cfg.weight_fmt in ("nvfp4", "mxfp4")
        # MXFP4 checkpoints: the decode path sees the same bytes through exact block-scaled views (e2m1 codes shared,
        # e8m0 scales re-expressed as e4m3 per 16 + tensor scale); a layer that cannot be re-expressed keeps the
        # whole model on the converter GEMM
        self.layers_fp4 = model.layers
        if self.decode_fp4 and model.cfg.weight_fmt == "mxfp4":
            import dataclasses
            from ..quant.formats import mxfp4_as_nvfp4
            views = []
            for L in model.layers:
                conv = {nm: mxfp4_as_nvfp4(getattr(L, nm)) for nm in ("qkv", "o", "gate_up", "down")}
                if any(v is None for v in conv.values()):
                    views = None
                    break
                views.append(dataclasses.replace(L, **conv))
            if views is None:
                self.decode_fp4 = False
            else:
                self.layers_fp4 = views
        self.act_terms = act_terms
        self.chunk = None
        self.embed_spans = None        # [(absolute start position, bf16 rows [n, hidden])] of the request in prefill
        self._li = 0
        # decode: a projection can ask L2 for the next projection's weights while the small kernels between them
        # leave HBM idle.  Measured on the 27B-class model at C8 the hint LOSES (7.70 vs 7.43 ms per step: the requests
        # compete with the issuing kernel's own weight stream), so it is off unless the engine options turn it on.
        self.l2_prefetch = l2_prefetch
        # fold the split-KV partials of decode attention inside the o projection's quantiser (one launch per layer
        # less); off keeps the stand-alone combine kernel
        self.fuse_combine = fuse_combine
        # fused GEMM -> all-reduce (peer-memory push in the GEMM epilogue, fold in the next norm kernel)
        self.fuse_ar = fuse_ar and reducer is not None and getattr(reducer, "comm", None) is not None and \
            model.cfg.hidden % 128 == 0 and model.cfg.hidden // 128 <= 64
        self.attn_tc = attn_tc and model.cfg.kv_fp8 and model.cfg.head_dim == 128 and \
            (model.cfg.q_heads // model.cfg.kv_heads) in (1, 2, 4, 5, 8)
        c = model.cfg
        dev = model.embed.device
        d = c.head_dim
        self.hq, self.hkv, self.d = model.hq_local, model.hkv_local, d
        self.qkv_cols = (self.hq + 2 * self.hkv) * d
        H, I = c.hidden, model.layers[0].down.k       # local intermediate width (padded to the GEMM's K granule)
        R = max_rows
        # every activation buffer is a view into the runner's arena (no allocation after construction; the report()
        # of the arena is the runner's activation footprint)
        from ..utils.arena import Arena
        self.arena = Arena(dev, slab_bytes=32 << 20)
        e = lambda *s: self.arena.alloc(s, BF, "device_hot")
        self.x, self.xn, self.delta = e(R, H), e(R, H), e(R, H)
        self.qkv, self.attn = e(R, self.qkv_cols), e(R, self.hq * d)
        self.gu, self.act = e(R, 2 * I), e(R, I)
        self.vocab_local = c.vocab // model.tp_size
        self.max_logit_rows = min(R, 256)
        self.logits = torch.empty(self.max_logit_rows, self.vocab_local, dtype=torch.float32, device=dev)
        self.pick_id = torch.zeros(self.max_logit_rows, dtype=torch.int32, device=dev)
        self.pick_val = torch.zeros(self.max_logit_rows, dtype=torch.float32, device=dev)
        self.scale = 1.0 / math.sqrt(d)
        self.decode_splits = decode_splits
        self.att_ml = torch.empty(R * self.hq * decode_splits * 2, dtype=torch.float32, device=dev)
        self.att_acc = torch.empty(min(R, 256) * self.hq * decode_splits * d, dtype=torch.float32, device=dev)
        self.ws = ops.default_workspace(dev)
        # runtime low-rank adapter (adapters.lora.LoraAdapter) applied after every adapted projection; the fused
        # GEMM -> all-reduce push is bypassed while one is installed (the update is added to the partial output)
        self.lora = None
        self.lora_scratch = torch.empty(R * 256, dtype=torch.float32, device=dev)
        self.qa = {}
        # decode through the persistent per-layer kernel (ops.decode_layer) where it applies.  Off by default: measured
        # on the 27B-class model at 8 rows it is slower than the per-operator sequence (7.67 vs 7.10 ms per step on one
        # GPU, 8.33 vs 7.74 ms on two, 7.39 vs 7.10 ms on eight); every grid-barrier phase costs about as much as a
        # programmatic-launch kernel boundary, so only fewer dependent steps per layer can make it pay
        self.fused_decode = fused_decode
        self._fused_plans, self._fused_bufs = {}, None
        self.fp4_rows = min(64, decode_rows or max_rows)
        if self.decode_fp4:
            bn = min(64, ops.pick_bn(self.fp4_rows))
            for k in {H, self.hq * d, I}:
                self.qa[k] = ops.QuantAct(bn, k, act_terms, bn, dev)

    # ------------------------------------------------------------------ persistent decode-layer kernel
    def _fused_ok(self, rows: int) -> bool:
        """The persistent per-layer kernel serves decode batches of up to 16 rows of NVFP4 models with head_dim 128
        and an FP8 cache; everything else (adapters, sink layers, NCCL reducer, wider batches) keeps the per-operator
        launch sequence."""
        m, c = self.m, self.m.cfg
        if not (self.fused_decode and self.decode_fp4 and self.attn_tc and self.lora is None):
            return False
        if rows > 16 or self.d != 128 or not c.kv_fp8:
            return False
        if self.reducer is not None and getattr(self.reducer, "comm", None) is None:
            return False
        L0 = self.layers_fp4[0]
        H, A, I = c.hidden, self.hq * self.d, L0.down.k
        if any(k % 256 or k > 16384 for k in (H, A)) or I % 256 or L0.gate_up.n != 2 * I:
            return False
        return all(L.sink is None and w.fmt == "nvfp4" for L in self.layers_fp4
                   for w in (L.qkv, L.o, L.gate_up, L.down))

    def _fused_plan(self, rows: int, positions, row_req, splits: int):
        key = (rows, positions.data_ptr(), row_req.data_ptr(), splits)
        plan = self._fused_plans.get(key)
        if plan is not None:
            return plan
        from ..ops.decode_layer import LayerLaunch
        m, c, kv = self.m, self.m.cfg, self.kv
        dev = m.embed.device
        H, A, I = c.hidden, self.hq * self.d, self.layers_fp4[0].down.k
        if self._fused_bufs is None:
            qa = {nm: ops.QuantAct(16, k, 3, 16, dev) for nm, k in (("a", A), ("h", H), ("i", I))}
            f32 = dict(dtype=torch.float32, device=dev)
            self._fused_bufs = dict(qa=qa, ws=torch.empty(16 * 160 * 128, **f32), stats=torch.zeros(256, **f32),
                                    hbuf=torch.empty(16, I, dtype=BF, device=dev),
                                    amax=torch.zeros((I // 128) * 16, **f32))
        fb = self._fused_bufs
        qa = fb["qa"]
        comm = getattr(self.reducer, "comm", None) if self.reducer is not None else None
        tp = comm is not None
        x, xn, qkv, attn = self.x[:rows], self.xn[:rows], self.qkv[:rows], self.attn[:rows]
        layers = self.layers_fp4
        n = len(layers)

        def new():
            ll = LayerLaunch(rows, x, H, c.eps, fb["ws"], fb["stats"], comm=comm)
            ll.set_act(0, qa["a"]); ll.set_act(1, qa["h"]); ll.set_act(2, qa["i"])
            return ll

        def qkv_tail(ll, li):
            """... in_norm of layer li -> qkv projection -> RoPE + KV append"""
            L = layers[li]
            ll.set_gemm(3, L.qkv, act=1)
            ll.gemm(3)
            ll.rope(3, qkv, positions, row_req, kv.block_table, m.inv_freq, kv.layers[li], self.hq, self.hkv, self.d,
                    c.rot_dim or self.d, m.mscale, L.q_norm, L.k_norm)

        launches = []
        head = new()
        head.rowq(2, mode=2, out_act=1, norm_w=layers[0].in_norm)
        qkv_tail(head, 0)
        launches.append(head)
        for li, L in enumerate(layers):
            ll = new()
            if splits > 1:
                ll.set_attention(self.att_ml, self.att_acc, splits, self.hq, self.d)
                ll.rowq(0, mode=3, out_act=0)
            else:
                ll.set_attention(None, None, 1, self.hq, self.d)
                ll.rowq(0, mode=0, out_act=0, inp=attn)
            ll.set_gemm(0, L.o, act=0)
            ll.gemm(0)
            ll.rowq(1, mode=2, out_act=1, src_gemm=0, tp_fold=tp, norm_w=L.post_norm)
            ll.set_gemm(1, L.gate_up, act=1, pair=True)
            ll.set_swiglu(fb["hbuf"], fb["amax"], I, 2)
            ll.gemm(1)
            ll.unitq()
            ll.set_gemm(2, L.down, act=2)
            ll.gemm(2)
            if li + 1 < n:
                ll.rowq(2, mode=2, out_act=1, src_gemm=2, tp_fold=tp, norm_w=layers[li + 1].in_norm)
                qkv_tail(ll, li + 1)
            else:
                ll.rowq(2, mode=2, out_act=-1, src_gemm=2, tp_fold=tp, norm_w=m.final_norm, x_out=xn)
            launches.append(ll)
        self._fused_plans[key] = launches
        return launches

    def _forward_fused(self, rows: int, tokens, positions, row_req, splits: int):
        """Decode pass through the persistent per-layer kernels: 2 launches per layer (attention + everything
        else).  Leaves the final-norm output in self.xn[:rows]."""
        m, kv = self.m, self.kv
        plan = self._fused_plan(rows, positions, row_req, splits)
        plan[0].launch()                      # (self.x[:rows] already holds the gathered embeddings)
        qkv, attn = self.qkv[:rows], self.attn[:rows]
        for li, L in enumerate(self.layers_fp4):
            if splits > 1:
                ops.attn_decode_tc(qkv, qkv.stride(0), kv.layers[li], kv.block_table, row_req, positions, self.hq,
                                   self.hkv, self.d, self.scale, splits=splits, scratch=(self.att_ml, self.att_acc),
                                   window=L.window, partials_only=True)
            else:
                ops.attn_decode_tc(qkv, qkv.stride(0), kv.layers[li], kv.block_table, row_req, positions, self.hq,
                                   self.hkv, self.d, self.scale, splits=1, out=attn, window=L.window)
            plan[li + 1].launch()

    def linear(self, x, w, out, fp4: bool):
        if fp4 and w.fmt == "nvfp4" and w.k % 256 == 0:
            xa = ops.act_quant_nvfp4(x, self.act_terms, out=self.qa[w.k])
            return ops.gemm_fp4(xa, w, out=out)
        return ops.linear(x, w, out=out)

    def _layer_fp4(self, L, cache, x, delta, have_delta, qkv, attn, gu, positions, row_req, rows, splits,
                   pending_fold=False, last=False):
        """One decoder layer on the block-scaled FP4 path: every linear consumes NVFP4 residual terms written by
        the kernel that produces its input (add + RMSNorm, attention output, SwiGLU)."""
        m, c = self.m, self.m.cfg
        H = c.hidden
        lora, li = self.lora, self._li
        xn = self.xn[:rows] if lora is not None else None       # bf16 input of the adapted projections
        if pending_fold:
            xa = ops.act_quant_nvfp4(x, out=self.qa[H], mode="rmsnorm", norm_w=L.in_norm, eps=c.eps,
                                     fold_comm=self.reducer.comm)
        else:
            xa = ops.act_quant_nvfp4(x, out=self.qa[H], mode="rmsnorm", delta=delta if have_delta else None,
                                     norm_w=L.in_norm, eps=c.eps, x_out=xn)
        pf = self.l2_prefetch
        ops.gemm_fp4(xa, L.qkv, out=qkv, prefetch=L.o if pf else None)
        if lora is not None:
            lora.apply(li, "qkv", xn, qkv, self.lora_scratch)
        ops.rope_kv_write(qkv, positions, row_req, self.kv.block_table, m.inv_freq, cache, self.hq, self.hkv, self.d,
                          rot_dim=c.rot_dim or self.d, mscale=m.mscale, q_norm_w=L.q_norm, k_norm_w=L.k_norm, eps=c.eps)
        if self.fuse_combine and splits > 1 and self.attn_tc and self.chunk is None and L.sink is None:
            # split-KV decode attention leaves its partials; the quantiser of the o projection folds them
            ops.attn_decode_tc(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                               self.d, self.scale, splits=splits, scratch=(self.att_ml, self.att_acc),
                               window=L.window, partials_only=True)
            xa = ops.attn_combine_quant((self.att_ml, self.att_acc), rows, splits, self.hq, self.d,
                                        out=self.qa[self.hq * self.d], x_out=attn if lora is not None else None)
        else:
            self.attention(qkv, cache, row_req, positions, rows, splits, attn, L)
            xa = ops.act_quant_nvfp4(attn, out=self.qa[self.hq * self.d], mode="plain")
        # tensor parallel, peer memory: the GEMM epilogue pushes its tiles to every rank and the next
        # add + RMSNorm + quantise kernel folds them (no separate all-reduce launch)
        fuse = getattr(self.reducer, "comm", None) if (self.fuse_ar and lora is None) else None
        if fuse:
            ops.gemm_fp4(xa, L.o, push_comm=fuse, prefetch=L.gate_up if pf else None)
            xa = ops.act_quant_nvfp4(x, out=self.qa[H], mode="rmsnorm", norm_w=L.post_norm, eps=c.eps, fold_comm=fuse)
        else:
            ops.gemm_fp4(xa, L.o, out=delta, prefetch=L.gate_up if pf else None)
            if lora is not None:
                lora.apply(li, "o", attn, delta, self.lora_scratch)
            if self.reducer is not None:
                self.reducer.all_reduce(delta)
            xa = ops.act_quant_nvfp4(x, out=self.qa[H], mode="rmsnorm", delta=delta, norm_w=L.post_norm, eps=c.eps,
                                     x_out=xn)
        ops.gemm_fp4(xa, L.gate_up, out=gu, prefetch=L.down if pf else None)
        act = None
        if lora is not None:
            lora.apply(li, "gate_up", xn, gu, self.lora_scratch)
            act = self.act[:rows]
        xa = ops.act_quant_nvfp4(gu, out=self.qa[gu.shape[1] // 2], mode="swiglu", x_out=act)
        nxt = self.layers_fp4[li + 1].qkv if (pf and li + 1 < len(self.layers_fp4)) else None
        if fuse and not last:
            ops.gemm_fp4(xa, L.down, push_comm=fuse, prefetch=nxt)
            return True            # the next layer's first kernel folds the pushed tiles
        ops.gemm_fp4(xa, L.down, out=delta, prefetch=nxt)
        if lora is not None:
            lora.apply(li, "down", act, delta, self.lora_scratch)
        if self.reducer is not None:
            self.reducer.all_reduce(delta)
        return False

    # ------------------------------------------------------------------
    def forward(self, rows: int, tokens, positions, row_req, logits_rows: Optional[slice] = None,
                decode: bool = False, pick: bool = True, chunk: Optional[tuple] = None):
        """Run `rows` rows through the model.  tokens/positions/row_req: int32 device tensors [rows].
        Logits (fp32, this rank's vocab slice) are produced for `logits_rows` (default: all rows when
        decode, else only the last row) and the greedy pick of those rows lands in self.pick_id."""
        m, c, kv = self.m, self.m.cfg, self.kv
        # chunk = (slot, first position): all rows are consecutive positions of ONE request -> flash-attention prefill
        self.chunk = None if decode else chunk
        x, xn, delta = self.x[:rows], self.xn[:rows], self.delta[:rows]
        qkv, attn, gu, act = self.qkv[:rows], self.attn[:rows], self.gu[:rows], self.act[:rows]
        ops.embed_gather(tokens, m.embed, out=x)
        if self.embed_spans and self.chunk is not None:
            # precomputed input rows (image tokens) replace the gathered embeddings of the positions they cover
            pos0 = self.chunk[1]
            for p0, src in self.embed_spans:
                a, b = max(p0, pos0), min(p0 + src.shape[0], pos0 + rows)
                if a < b:
                    x[a - pos0:b - pos0].copy_(src[a - p0:b - p0])
        have_delta = False
        pending = False
        sp_in = False
        splits = self.decode_splits if (decode and rows <= 256) else 1
        fp4 = self.decode_fp4 and decode and rows <= self.fp4_rows and all(
            w.k % 256 == 0 for w in (m.layers[0].qkv, m.layers[0].o, m.layers[0].down))
        lora = self.lora
        fused = fp4 and decode and self.embed_spans is None and self._fused_ok(rows)
        if fused:
            self._forward_fused(rows, tokens, positions, row_req, splits)
        for li, L in enumerate(m.layers if not fused else ()):
            self._li = li
            if fp4:
                pending = self._layer_fp4(self.layers_fp4[li], kv.layers[li], x, delta, have_delta, qkv, attn, gu, positions, row_req,
                                          rows, splits, pending_fold=pending, last=li == len(m.layers) - 1)
                have_delta = True
                continue
            if sp_in:
                # the previous block's boundary left the normed rows of every token tile in the symmetric region
                ops.gemm_tc_ag(L.qkv, self.reducer.comm, rows, out=qkv)
            else:
                ops.rmsnorm(x, L.in_norm, c.eps, delta=delta if have_delta else None, out=xn)
                self.linear(xn, L.qkv, qkv, fp4)
            sp_in = False
            if lora is not None:
                lora.apply(li, "qkv", xn, qkv, self.lora_scratch)
            cache = kv.layers[li]
            ops.rope_kv_write(qkv, positions, row_req, kv.block_table, m.inv_freq, cache, self.hq, self.hkv, self.d,
                              rot_dim=c.rot_dim or self.d, mscale=m.mscale, q_norm_w=L.q_norm, k_norm_w=L.k_norm,
                              eps=c.eps)
            self.attention(qkv, cache, row_req, positions, rows, splits, attn, L)
            # tensor parallel at prefill sizes: GEMM epilogue -> reduce-scatter push, fold at the owner + all-gather
            rs = (self.fuse_ar and lora is None and not fp4 and rows > 64 and
                  getattr(self.reducer, "can_rs", lambda *a: False)(rows, c.hidden, ops.pick_bn(rows)))
            sp = rs and self.seq_parallel and hasattr(self.reducer, "rs_norm_push")
            if sp:
                # sequence-parallel boundary: fold + residual + norm at the tile's owner, normed rows all-gathered into
                # every rank's region, the gate / up projection waits per token tile inside its kernel
                bn = ops.gemm_tc_push(attn, L.o, self.reducer.comm)
                self.reducer.rs_norm_push(x, L.post_norm, c.eps, bn)
            elif rs:
                # (x already holds the residual stream: the input norm above folded the previous block's output in)
                self.reducer.rs_ag(x, ops.gemm_tc_push(attn, L.o, self.reducer.comm))
                ops.rmsnorm(x, L.post_norm, c.eps, out=xn)
            else:
                self.linear(attn, L.o, delta, fp4)
                if lora is not None:
                    lora.apply(li, "o", attn, delta, self.lora_scratch)
                if self.reducer is not None:
                    self.reducer.all_reduce(delta)
                ops.rmsnorm(x, L.post_norm, c.eps, delta=delta, out=xn)
            if sp:
                ops.gemm_tc_ag(L.gate_up, self.reducer.comm, rows, out=gu)
            else:
                self.linear(xn, L.gate_up, gu, fp4)
            if lora is not None:
                lora.apply(li, "gate_up", xn, gu, self.lora_scratch)
            ops.swiglu(gu, out=act)
            if sp and li + 1 < len(m.layers):
                bn = ops.gemm_tc_push(act, L.down, self.reducer.comm)
                self.reducer.rs_norm_push(x, m.layers[li + 1].in_norm, c.eps, bn)
                have_delta, sp_in = False, True
                continue
            if rs:
                # (the last block gathers the residual rows themselves: the final norm needs the last row everywhere)
                self.reducer.rs_ag(x, ops.gemm_tc_push(act, L.down, self.reducer.comm))
                have_delta = False                     # the block's output is already in the residual stream
                continue
            self.linear(act, L.down, delta, fp4)
            if lora is not None:
                lora.apply(li, "down", act, delta, self.lora_scratch)
            if self.reducer is not None:
                self.reducer.all_reduce(delta)
            have_delta = True
        if not fused:
            ops.rmsnorm(x, m.final_norm, c.eps, delta=delta if have_delta else None, out=xn)
        if logits_rows is None:
            logits_rows = slice(0, rows) if decode else slice(rows - 1, rows)
        hx = xn[logits_rows]
        n = hx.shape[0]
        assert n <= self.max_logit_rows
        logits = self.logits[:n]
        ops.gemm_tc(hx, m.head, out32=logits)
        if pick:
            ops.argmax(logits, id_base=m.tp_rank * self.vocab_local, out_id=self.pick_id[:n],
                       out_val=self.pick_val[:n])
            if self.reducer is not None and m.tp_size > 1:
                self.reducer.merge_picks(self.pick_id[:n], self.pick_val[:n])
        return logits

    def attention(self, qkv, cache, row_req, positions, rows, splits, out, layer=None):
        """Attention of `rows` query rows against the paged cache (their own K/V already appended).  `layer` carries
        the sliding window and the sink logits of windowed-sink families; sink layers run on the CUDA-core kernel
        (the sink column is folded into its final normalisation), the tensor-core kernels take the window."""
        window = layer.window if layer is not None else 0
        sink = layer.sink if layer is not None else None
        if sink is not None:
            sp = splits if rows <= 256 else 1
            ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                            self.d, self.scale, splits=sp, scratch=(self.att_ml, self.att_acc) if sp > 1 else None,
                            out=out, window=window, sink=sink)
        elif self.chunk is not None and self.attn_tc and self.d == 128 and cache.fp8:
            slot, pos0 = self.chunk
            ops.attn_prefill_tc(qkv, qkv.stride(0), cache, self.kv.block_table[slot], pos0, self.hq, self.hkv, self.d,
                                self.scale, out=out, rows=rows, window=window)
        elif self.attn_tc:
            ops.attn_decode_tc(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                               self.d, self.scale, splits=splits,
                               scratch=(self.att_ml, self.att_acc) if splits > 1 else None, out=out, window=window)
        elif splits > 1:
            ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                            self.d, self.scale, splits=splits, scratch=(self.att_ml, self.att_acc), out=out,
                            window=window)
        else:
            ops.attn_decode(qkv, qkv.stride(0), cache, self.kv.block_table, row_req, positions, self.hq, self.hkv,
                            self.d, self.scale, splits=1, out=out, window=window)
