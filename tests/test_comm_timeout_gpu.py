"""A peer that never raises its flag: the collective kernel's bounded wait runs out, the kernel returns, the host
reads an error status and the CUDA context stays usable.  The missing peer is made on the host (a world of two whose
second rank does not exist); nothing faults, traps or hangs."""
import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_all_reduce_with_a_missing_peer_reports_status_and_returns():
    from dgpp_b200.ops import _lib, core as ops
    from dgpp_b200.ops._lib import I, L, P, call, ptr, stream_ptr
    from dgpp_b200.parallel import peer  # noqa: F401  (declares the comm entry points)
    _lib.declare("dgpp_comm_loopback", [P])
    lib = _lib.load()
    lib.dgpp_comm_create.restype = P
    lib.dgpp_comm_create.argtypes = [I, I, L, P]
    torch.cuda.set_device(0)
    ops.check_status()
    handle = (C.c_ubyte * 64)()
    comm = lib.dgpp_comm_create(2, 0, 8 * 5120 * 2, C.cast(handle, P))
    assert comm
    try:
        call("dgpp_comm_loopback", comm)
        x = torch.randn(8, 5120, device="cuda").to(torch.bfloat16)
        before = x.clone()
        t0 = time.time()
        call("dgpp_comm_all_reduce", comm, ptr(x), None, x.numel(), 4, stream_ptr())
        torch.cuda.synchronize()
        waited = time.time() - t0
        assert 0.5 < waited < 20.0, waited                      # a bounded wait, not a hang
        buf = (C.c_int * 4)()
        call("dgpp_status_read", C.cast(buf, P))
        assert buf[0] == 4 and buf[2] == 1 and buf[1] >= 1      # kTimeoutPeerFlag, missing source rank 1
        with pytest.raises(RuntimeError, match="code=4"):
            ops.check_status()                                  # raises and clears
        assert torch.equal(x, before)                           # nothing was folded from a rank that never arrived
        # the context is alive: an ordinary kernel still runs and the status is clean again
        w = torch.ones(5120, device="cuda", dtype=torch.bfloat16)
        y = ops.rmsnorm(x, w, 1e-6)
        torch.cuda.synchronize()
        ops.check_status()
        assert torch.isfinite(y.float()).all()
    finally:
        call("dgpp_comm_destroy", comm)
