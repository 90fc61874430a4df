"""The fixed-scratch decode attention entry point (dgpp_attn_decode_static): called through the exported C symbol,
it must give the same bits as dgpp_attn_decode with caller-owned scratch, on two calls in a row (the shared array
keeps the previous call's contents), and must refuse sizes beyond the array.  Collected last on purpose: it has to
pass alone and after every other GPU test has used the device."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

BF = torch.bfloat16
P, I, L, F = C.c_void_p, C.c_int, C.c_int64, C.c_float
SIG = [P, L, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P]
SCRATCH_FLOATS = 1 << 20


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    return torch.device("cuda:0")


def _static_fn():
    from dgpp_b200.ops import _lib

    lib = _lib.load()
    fn = lib.dgpp_attn_decode_static
    fn.argtypes, fn.restype = SIG, I
    return lib, fn


def _case(dev, hq, hkv, d, ctx, page, fp8, seed):
    from dgpp_b200.engine.kv_cache import PagedKV
    from dgpp_b200.ops import core as ops, reference as ref

    torch.manual_seed(seed)
    kv = PagedKV(1, hkv, d, 4 * (ctx // page + 2), 4, ctx // page + 2, page, fp8, dev)
    inv_freq, _ = ref.rope_inv_freq(d, 1e4, dev)
    qkv = torch.randn(ctx, (hq + 2 * hkv) * d, device=dev).to(BF)
    pos = torch.arange(ctx, device=dev, dtype=torch.int32)
    req = torch.full((ctx,), 3, device=dev, dtype=torch.int32)
    assert kv.reserve(3, ctx)
    ops.rope_kv_write(qkv, pos, req, kv.block_table, inv_freq, kv.layers[0], hq, hkv, d)
    sel = torch.tensor([ctx - 1, ctx // 3, 0, ctx // 2], device=dev)
    return kv, qkv[sel].contiguous(), pos[sel].contiguous(), req[sel].contiguous()


def _call_static(fn, q, cache, kv, req, pos, out, hq, hkv, d, splits, scale):
    from dgpp_b200.ops._lib import ptr, stream_ptr

    return fn(ptr(q), q.stride(0), ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale),
              ptr(kv.block_table), ptr(req), ptr(pos), ptr(out), pos.numel(), hq, hkv, d, cache.page,
              kv.block_table.shape[1], splits, int(cache.fp8), float(scale), 0, stream_ptr())


@pytest.mark.parametrize("hq,hkv,d,ctx,page,fp8,splits", [(10, 2, 128, 700, 64, True, 4), (8, 2, 64, 333, 16, False, 3),
                                                          (16, 2, 256, 500, 32, True, 2), (4, 4, 128, 90, 16, True, 1)])
def test_static_scratch_matches_caller_scratch_twice(dev, hq, hkv, d, ctx, page, fp8, splits):
    from dgpp_b200.ops import core as ops

    lib, fn = _static_fn()
    scale = 1.0 / math.sqrt(d)
    for rep in range(2):          # second case reuses the array after a call with other sizes and data
        kv, q, pos, req = _case(dev, hq, hkv, d, ctx - 17 * rep, page, fp8, seed=10 + rep)
        cache = kv.layers[0]
        want = ops.attn_decode(q, q.stride(0), cache, kv.block_table, req, pos, hq, hkv, d, scale, splits=splits)
        out1 = torch.full_like(want, float("nan"))
        out2 = torch.full_like(want, float("nan"))
        assert _call_static(fn, q, cache, kv, req, pos, out1, hq, hkv, d, splits, scale) == 0, lib.dgpp_last_error().decode()
        assert _call_static(fn, q, cache, kv, req, pos, out2, hq, hkv, d, splits, scale) == 0, lib.dgpp_last_error().decode()
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.equal(out1.view(torch.int16), want.view(torch.int16))
        assert torch.equal(out2.view(torch.int16), want.view(torch.int16))


def test_static_scratch_rejects_oversize(dev):
    lib, fn = _static_fn()
    hq, hkv, d, splits = 64, 8, 256, 16
    kv, q, pos, req = _case(dev, 8, 2, 128, 100, 16, True, seed=3)
    rows = SCRATCH_FLOATS // (hq * splits * (d + 2)) + 1          # one row too many for the array
    out = torch.zeros(4, 8 * 128, device=dev, dtype=BF)
    from dgpp_b200.ops._lib import ptr, stream_ptr

    cache = kv.layers[0]
    rc = fn(ptr(q), q.stride(0), ptr(cache.k), ptr(cache.v), ptr(cache.k_scale), ptr(cache.v_scale), ptr(kv.block_table),
            ptr(req), ptr(pos), ptr(out), rows, hq, hkv, d, cache.page, kv.block_table.shape[1], splits, 1, 0.1, 0,
            stream_ptr())
    assert rc != 0
    msg = lib.dgpp_last_error().decode()
    assert "scratch floats" in msg and str(SCRATCH_FLOATS) in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0                   # nothing was launched
