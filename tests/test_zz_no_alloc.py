"""The allocation-free attention entry point (sdv2_attn_kvcache_static), for callers that cannot
provide scratch memory: it must give the same result as the workspace entry point, call after
call, although every call reuses the same built-in device array.  Collected last on purpose."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _inputs(seed, B, N, H, S, dev):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(torch.bfloat16).to(dev)
    return mk(B, N, H, 128), mk(B, S, H, 128), mk(B, S, H, 128)


def _call_static(q, k, v, lens):
    from streamdiffusionv2_b200 import _native as N
    out = torch.full_like(q, float("nan"))
    views = [N.view(t) for t in (q, k, v, out)]
    status = C.c_void_p(0)
    rc = N.lib().sdv2_attn_kvcache_static(*[C.byref(x) for x in views], q.shape[0], q.shape[1], q.shape[2], 128,
                                          k.shape[1], N.i32_array(lens), 128 ** -0.5, C.byref(status),
                                          N.stream_ptr(q.device))
    return rc, out, status


def test_static_scratch_entry_matches_workspace_entry_twice_in_a_row():
    from streamdiffusionv2_b200 import _native as N
    from streamdiffusionv2_b200 import ops
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    # long enough key ranges and a small grid, so that the tail split (the part that needs scratch) runs;
    # the second call has other data, other lengths and fewer rows: leftovers of call 1 must not show
    for seed, (B, n_q, H, S, lens) in enumerate([(2, 300, 3, 5000, [5000, 2100]), (1, 700, 2, 6000, [4321])]):
        q, k, v = _inputs(40 + seed, B, n_q, H, S, dev)
        want = ops.attn_kvcache(q, k, v, lens)
        rc, got, status = _call_static(q, k, v, lens)
        assert rc == 0, N.lib().sdv2_strerror(rc)
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        err = (got.float() - want.float()).abs()
        assert err.max().item() <= 2e-2 and err.mean().item() <= 1e-3, (seed, err.max().item())
        assert torch.equal(got, want), "same kernels, same split: results should be bit-identical"
        detail = C.c_int(0)
        assert N.lib().sdv2_read_status(status, C.byref(detail), N.stream_ptr(dev)) == 0


def test_static_scratch_entry_refuses_oversized_calls():
    dev = torch.device("cuda", 0)
    q, k, v = _inputs(7, 1, 16, 1, 128, dev)
    q65 = q.expand(65, -1, -1, -1).contiguous()
    k65 = k.expand(65, -1, -1, -1).contiguous()
    rc, _, _ = _call_static(q65, k65, k65, [128] * 65)
    assert rc == -2          # more cache rows than one call supports
    rc, _, _ = _call_static(q, k, v, [129])
    assert rc == -1          # length beyond the cache
