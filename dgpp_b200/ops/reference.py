"""Plain PyTorch fp32 restatements of every CUDA op: the oracle for kernel tests and the execution
path on hosts without a GPU (CPU plumbing runs, gloo multi-rank tests)."""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..quant.formats import QuantLinear

BF = torch.bfloat16

# Activation dtype of the reference path.  bf16 reproduces the rounding points of the kernels; float32 turns every
# rounding point into the identity (used by the fp32 CPU-plumbing model).
_ACT = {"dtype": torch.bfloat16}


class activation_dtype:
    """Context manager: run the reference ops with another activation dtype (torch.float32 or torch.bfloat16)."""

    def __init__(self, dtype):
        self.dtype, self.prev = dtype, None

    def __enter__(self):
        self.prev = _ACT["dtype"]
        _ACT["dtype"] = self.dtype

    def __exit__(self, *a):
        _ACT["dtype"] = self.prev


def act(x: torch.Tensor) -> torch.Tensor:
    return x.to(_ACT["dtype"])


def _r(x: torch.Tensor) -> torch.Tensor:
    """Round fp32 to the activation dtype and come back (marks a rounding point)."""
    return x.to(_ACT["dtype"]).float()


def embed_gather(ids, table):
    return table[ids.long().clamp(0, table.shape[0] - 1)]


def rmsnorm(x, w, eps=1e-6, delta=None, one_plus_w=False):
    """Returns (out, new_residual).  out = bf16(w * bf16(x * rstd))."""
    xf = x.float()
    if delta is not None:
        xf = _r(xf + delta.float())
    rstd = torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    g = w.float() + (1.0 if one_plus_w else 0.0)
    return act(_r(xf * rstd) * g), act(xf)


def swiglu(gate_up, limit: float = 0.0, alpha: float = 0.0):
    """alpha = 0: silu(gate) * up; alpha > 0: gate * sigmoid(alpha * gate) * (up + 1).  limit > 0 clamps gate above and
    up on both sides first."""
    inter = gate_up.shape[-1] // 2
    g, u = gate_up[..., :inter].float(), gate_up[..., inter:].float()
    if limit > 0:
        g = g.clamp(max=limit)
        u = u.clamp(-limit, limit)
    if alpha > 0:
        return act(_r(g * torch.sigmoid(alpha * g)) * (u + 1.0))
    return act(_r(g * torch.sigmoid(g)) * u)


def argmax(logits, id_base=0):
    v, i = logits.float().max(-1)
    # torch.max returns the first maximal index on CPU and CUDA for 1-D reductions; make it explicit
    eq = logits.float() == v.unsqueeze(-1)
    first = torch.argmax(eq.to(torch.int8), dim=-1)
    return (first + id_base).to(torch.int32), v


def linear(x, w: QuantLinear, resid=None, out_fp32=False):
    """out = alpha * x @ dequant(w)^T in fp32, one bf16 rounding (+ residual add with a second one)."""
    y = x.float() @ w.dequant().t().to(x.device)
    if out_fp32:
        return y
    y = act(y)
    if resid is not None:
        y = act(resid.float() + y.float())
    return y


def rope_inv_freq(rot_dim: int, theta: float, device=None, yarn_factor: float = 1.0,
                  original_max_pos: int = 0, beta_fast: float = 32.0, beta_slow: float = 1.0):
    """fp32 inverse frequencies [rot_dim/2]; with yarn_factor > 1 returns the YaRN-blended table and the
    attention scale (mscale) that multiplies cos/sin."""
    inv = 1.0 / (theta ** (torch.arange(0, rot_dim, 2, dtype=torch.float32, device=device) / rot_dim))
    if yarn_factor <= 1.0:
        return inv, 1.0

    def corr_dim(rot):
        return (rot_dim * math.log(original_max_pos / (rot * 2 * math.pi))) / (2 * math.log(theta))

    low = max(math.floor(corr_dim(beta_fast)), 0)
    high = min(math.ceil(corr_dim(beta_slow)), rot_dim // 2 - 1)
    ramp = ((torch.arange(rot_dim // 2, dtype=torch.float32, device=device) - low) / max(high - low, 1e-3)).clamp(0, 1)
    mask = 1.0 - ramp
    inv_yarn = inv / yarn_factor * (1 - mask) + inv * mask
    mscale = 0.1 * math.log(yarn_factor) + 1.0
    return inv_yarn, mscale


def apply_rope(x, positions, inv_freq, rot_dim, mscale=1.0):
    """x: [rows, heads, d] fp32; rotate-half pairing on the first rot_dim dims, one bf16 rounding."""
    ang = positions.float().unsqueeze(-1) * inv_freq.unsqueeze(0)      # [rows, rot/2]
    cs, sn = (torch.cos(ang) * mscale).unsqueeze(1), (torch.sin(ang) * mscale).unsqueeze(1)
    h = rot_dim // 2
    x0, x1 = x[..., :h], x[..., h:rot_dim]
    out = x.clone()
    out[..., :h] = x0 * cs - x1 * sn
    out[..., h:rot_dim] = x1 * cs + x0 * sn
    return _r(out)


def head_norm(x, w, eps, one_plus_w=False):
    rstd = torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps)
    g = w.float() + (1.0 if one_plus_w else 0.0)
    return _r(_r(x * rstd) * g)


def quant_kv_fp8(x):
    """x: [..., d] fp32 -> (e4m3 codes uint8, fp32 scale [...]) with scale = amax / 448."""
    amax = x.abs().amax(-1)
    scale = torch.where(amax > 0, amax / 448.0, torch.ones_like(amax))
    q = (x * (1.0 / scale).unsqueeze(-1)).clamp(-448, 448).to(torch.float8_e4m3fn)
    return q.view(torch.uint8), scale


def attention(q, k, v, scale, causal_offset: Optional[int] = None, window: int = 0, sink=None):
    """q: [Tq, hq, d], k/v: [Tk, hkv, d] fp32.  causal_offset = position of q row 0 (None: no mask).
    sink: optional [hq] logits of a value-less extra softmax column (sliding-window + sink attention)."""
    tq, hq, d = q.shape
    tk, hkv, _ = k.shape
    g = hq // hkv
    kk = k.repeat_interleave(g, 1)
    vv = v.repeat_interleave(g, 1)
    s = torch.einsum("qhd,khd->hqk", q, kk) * scale
    if causal_offset is not None:
        qpos = torch.arange(tq, device=q.device).unsqueeze(-1) + causal_offset
        kpos = torch.arange(tk, device=q.device).unsqueeze(0)
        mask = kpos > qpos
        if window > 0:
            mask = mask | (kpos <= qpos - window)
        s = s.masked_fill(mask.unsqueeze(0), float("-inf"))
    if sink is not None:
        s = torch.cat([s, sink.float().view(hq, 1, 1).expand(hq, tq, 1)], dim=-1)
        p = torch.softmax(s, -1)[..., :-1]
    else:
        p = torch.softmax(s, -1)
    return torch.einsum("hqk,khd->qhd", p, vv)


def hadamard32(x: torch.Tensor) -> torch.Tensor:
    """Oracle of ops.hadamard32_rows: five butterfly stages at strides 1, 2, 4, 8, 16 in fp32 (element j takes
    v_j + v_{j^s} when bit s of j is clear, v_{j^s} - v_j when set), times fp32(1 / sqrt(32)), one bf16 rounding."""
    rows, k = x.shape
    v = x.float().view(rows, k // 32, 32).clone()
    j = torch.arange(32, device=x.device)
    for s in (1, 2, 4, 8, 16):
        o = v[..., j ^ s]
        v = torch.where((j & s) != 0, o - v, v + o)
    return (v * torch.tensor(0.17677669529663687, dtype=torch.float32, device=x.device)).to(torch.bfloat16).view(rows, k)


def hadamard32_quant_int8(x: torch.Tensor):
    """Oracle of ops.hadamard32_quant_int8: rotated bf16 values, per 128: scale = max(amax / 127, 1e-30), rint codes."""
    rows, k = x.shape
    r = hadamard32(x).float().view(rows, k // 128, 128)
    sc = (r.abs().amax(-1) / 127.0).clamp_min(1e-30)
    codes = torch.clamp(torch.round(r / sc.unsqueeze(-1)), -128, 127).to(torch.int8).view(rows, k)
    return codes, sc


def moe_hash_routes(tokens, tid2eid, scores, scaling: float = 1.0, norm_topk: bool = True):
    """Oracle of ops.moe_hash_routes."""
    ids = tid2eid[tokens.long().clamp(0, tid2eid.shape[0] - 1)].long()
    w = scores.gather(1, ids)
    if norm_topk:
        denom = torch.zeros(w.shape[0], dtype=torch.float32, device=w.device)
        for i in range(w.shape[1]):
            denom = denom + w[:, i]
        w = w / (denom + 1e-20).unsqueeze(-1)
    return ids.to(torch.int32), w * scaling


def kda_recurrent(q, k, v, gate, beta, A_log, dt_bias, lower_bound: float, state, hk: int, hv: int, dk: int, dv: int):
    """Oracle of ops.kda_recurrent for consecutive tokens of one request.  q / k [T, hk * dk], v [T, hv * dv], gate
    [T, hv * dk], beta [T, hv]; state [hv, dk, dv] fp32 updated in place.  Returns bf16 [T, hv * dv]."""
    T = q.shape[0]
    rep = hv // hk
    qf = q.float().view(T, hk, dk)
    kf = k.float().view(T, hk, dk)
    qf = (qf * torch.rsqrt(qf.pow(2).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5).repeat_interleave(rep, 1)
    kf = (kf * torch.rsqrt(kf.pow(2).sum(-1, keepdim=True) + 1e-6)).repeat_interleave(rep, 1)
    vf = v.float().view(T, hv, dv)
    x = gate.float().view(T, hv, dk) + dt_bias.float().view(1, hv, dk)
    g = lower_bound / (1.0 + torch.exp(-torch.exp(A_log.float()).view(1, hv, 1) * x))
    decay = torch.exp(g)
    b = torch.sigmoid(beta.float())
    out = torch.zeros(T, hv, dv, device=q.device)
    S = state
    for t in range(T):
        S.mul_(decay[t].unsqueeze(-1))
        mem = torch.einsum("hkv,hk->hv", S, kf[t])
        u = b[t].unsqueeze(-1) * (vf[t] - mem)
        S.add_(torch.einsum("hk,hv->hkv", kf[t], u))
        out[t] = torch.einsum("hkv,hk->hv", S, qf[t])
    return out.to(torch.bfloat16).view(T, hv * dv)


def _bf(x):
    return x.to(torch.bfloat16).float()


def justnorm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    xf = x.float()
    rstd = 1.0 / torch.sqrt(xf.double().pow(2).sum(-1, keepdim=True).float() + eps)
    return (xf * rstd).to(torch.bfloat16)


def slerp_alpha(a, b, alpha, s: float, eps: float = 1e-6) -> torch.Tensor:
    an, bn = justnorm(a, eps).float(), justnorm(b, eps).float()
    lr = (alpha.float() * s).abs()
    m = an + lr * (bn - an)
    rstd = 1.0 / torch.sqrt(m.double().pow(2).sum(-1, keepdim=True).float() + eps)
    return (m * rstd).to(torch.bfloat16)


def gr_gate_act(t: torch.Tensor, hc: int) -> torch.Tensor:
    v = _bf(t.float() / hc)
    return (v * torch.sigmoid(v)).to(torch.bfloat16)


def gr_mix_finish(logits, rn, hc: int) -> torch.Tensor:
    rows = logits.shape[0]
    H = logits.shape[1] // hc
    g = _bf(torch.sigmoid(logits.float())).view(rows, hc, H)
    prod = _bf(g * rn.float().view(rows, hc, H))
    acc = torch.zeros(rows, H, device=logits.device)
    for i in range(hc):
        acc = acc + prod[:, i]
    return (acc / hc).to(torch.bfloat16)


def gr_combine(r_state, rn, w_inject, y, hc: int) -> torch.Tensor:
    rows, H = y.shape
    dots = rn.float() @ w_inject.float().t()                                   # [rows, hc]
    s = 2.0 * _bf(torch.sigmoid(_bf(dots / hc)))
    add = _bf(y.float().unsqueeze(1) * s.unsqueeze(-1))                        # [rows, hc, H]
    return (r_state.float().view(rows, hc, H) + add).to(torch.bfloat16).view(rows, hc * H)


def mhc_compute(streams, fn, base, scale, iters: int = 20, hc_eps: float = 1e-6, norm_eps: float = 1e-5):
    """Oracle of ops.mhc_compute (fp32 throughout, bf16 at the outputs)."""
    tokens, n, D = streams.shape
    x = streams.float().view(tokens, n * D)
    flat = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + norm_eps)
    logits = flat @ fn.float().t()
    pre = torch.sigmoid(logits[:, :n] * scale[0] + base[:n]) + hc_eps
    post = 2.0 * torch.sigmoid(logits[:, n:2 * n] * scale[1] + base[n:2 * n])
    comb = torch.softmax(logits[:, 2 * n:].view(tokens, n, n) * scale[2] + base[2 * n:].view(n, n), -1) + hc_eps
    comb = comb / (comb.sum(-2, keepdim=True) + hc_eps)
    for _ in range(iters - 1):
        comb = comb / (comb.sum(-1, keepdim=True) + hc_eps)
        comb = comb / (comb.sum(-2, keepdim=True) + hc_eps)
    collapsed = torch.einsum("tj,tjd->td", pre, streams.float())
    return collapsed.to(torch.bfloat16), post.to(torch.bfloat16), comb.to(torch.bfloat16)


def mhc_fold(streams, h, post, comb):
    """Oracle of ops.mhc_fold."""
    placed = _bf(post.float().unsqueeze(-1) * h.float().unsqueeze(1))                      # [t, n, D]
    mix = _bf(torch.einsum("tji,tjd->tid", comb.float(), streams.float()))
    return (placed + mix).to(torch.bfloat16)


def engram_ids(tokens, prev, token_map, multipliers, primes, offsets, pad_class: int):
    """Oracle of the hash of ops.engram_embed -> int64 [rows, (max_ngram - 1) * heads] table rows.  64-bit wrapping
    products (torch int64 arithmetic wraps), XOR-accumulated over the lookback, modulo the per-(size, head) prime with a
    non-negative remainder, plus the per-(size, head) offset."""
    vocab = token_map.numel()

    def cls(t):
        t = t.long()
        ok = (t >= 0) & (t < vocab)
        return torch.where(ok, token_map.long()[t.clamp(0, vocab - 1)], torch.full_like(t, pad_class))

    rolling = cls(tokens) * multipliers[0]
    out = []
    for n in range(1, multipliers.numel()):
        rolling = rolling ^ (cls(prev[n - 1]) * multipliers[n])
        out.append(torch.remainder(rolling.unsqueeze(-1), primes[n - 1].unsqueeze(0)) + offsets[n - 1].unsqueeze(0))
    return torch.cat(out, -1)


def engram_embed(tokens, prev, token_map, multipliers, primes, offsets, table, table_sf, pad_class: int):
    ids = engram_ids(tokens, prev, token_map, multipliers, primes, offsets, pad_class)
    rows, d = ids.shape[0], table.shape[1]
    val = table[ids].view(torch.float8_e4m3fn).float()                                    # [rows, slots, D]
    sc = torch.exp2(table_sf[ids].float() - 127.0).repeat_interleave(32, dim=-1)
    return act(val * sc).reshape(rows, -1)


def engram_gate(streams, kv, q_weight, k_weight, eps: float = 1e-6):
    rows, hc, h = streams.shape
    x = streams.float()
    key = kv[:, :hc * h].float().view(rows, hc, h)
    val = kv[:, hc * h:].float().view(rows, 1, h)
    w = q_weight.float() * k_weight.float()
    rstd = torch.rsqrt(x.pow(2).mean(-1) + eps) * torch.rsqrt(key.pow(2).mean(-1) + eps)
    dot = (x * w * key).sum(-1) * rstd / math.sqrt(h)
    sgn = torch.where(torch.signbit(dot), -torch.ones_like(dot), torch.ones_like(dot))      # copysign: +0 counts as positive
    gate = torch.sigmoid(sgn * torch.sqrt(dot.abs().clamp_min(1e-6)))
    return act(x + gate.unsqueeze(-1) * val)
