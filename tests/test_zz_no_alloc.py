"""Attention forward through b200k_attn_fwd_bf16_noalloc, the entry point for callers that cannot
allocate device memory (hosts bound to a fixed memory pool, plugins that only receive buffers, warm
serving loops).  It keeps the row statistics and the status word in a static device array inside the
library, so the caller passes only q, k, v and o.  The output must be bit-identical to what
b200k_attn_fwd_bf16 produces (the arithmetic of a tile does not depend on the order in which the tiles are
scheduled), on two calls in a row (the second call reuses the array with the first call's contents in it),
and within the attention tolerance of the CPU oracle.

This file sorts last on purpose: a run that stops at the first failure has then already executed
every other test."""
import ctypes

import pytest
import torch

import golden_inputs as gi
from oracle import cpu_oracle as oracle
from triton_tenstorrent_b200 import _lib

pytestmark = pytest.mark.gpu

ATTN_MAX_ABS = 2e-2   # the attention tolerance used throughout tests/test_gpu_parity.py


def _existing(lib, q, k, v, causal, scale):
    o = torch.empty_like(q)
    Z, H, S, D = q.shape
    m = torch.empty((Z, H, S), device=q.device, dtype=torch.float32)
    _lib.check(lib.b200k_attn_fwd_bf16(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), m.data_ptr(), Z, H, S, D,
                                       int(causal), scale, torch.cuda.current_stream().cuda_stream))
    return o


def _noalloc(lib, q, k, v, causal, scale, o=None):
    if o is None:
        o = torch.full_like(q, float("nan"))     # every element must be overwritten
    Z, H, S, D = q.shape
    _lib.check(lib.b200k_attn_fwd_bf16_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), Z, H, S, D,
                                               int(causal), scale, torch.cuda.current_stream().cuda_stream))
    return o


def _status(lib):
    code = ctypes.c_uint32(0xFFFFFFFF)
    rc = lib.b200k_attn_noalloc_status(torch.cuda.current_stream().cuda_stream, ctypes.byref(code))
    return rc, code.value


def test_noalloc_matches_existing_entry_point_twice():
    assert torch.cuda.is_available()
    torch.cuda.set_device(0)
    lib = _lib.load()
    scale = 128 ** -0.5
    # two different problems back to back: the second call finds the first call's data in the shared array
    for call, (Z, H, S, causal, seed) in enumerate([(2, 3, 512, True, 41), (1, 4, 1024, False, 42)]):
        qh, kh, vh = gi.attn_inputs(Z, H, S, 128, seed=seed)
        q, k, v = qh.cuda(), kh.cuda(), vh.cuda()
        got = _noalloc(lib, q, k, v, causal, scale)
        ref = _existing(lib, q, k, v, causal, scale)
        torch.cuda.synchronize()
        assert not torch.isnan(got.float()).any(), f"call {call}: output not fully written"
        assert torch.equal(got.view(torch.int16), ref.view(torch.int16)), f"call {call}: not bit-identical to b200k_attn_fwd_bf16"
        ref_o, _ = oracle.attention(qh, kh, vh, causal, scale)
        err = float((got.cpu().float() - ref_o.float()).abs().max())
        assert err <= ATTN_MAX_ABS, f"call {call}: max-abs difference to the CPU oracle {err}"
    assert _status(lib) == (_lib.OK, 0)


def test_noalloc_allocates_nothing_once_warm():
    # the claim in the entry point's name: the device's free memory is the same before and after warm calls
    lib = _lib.load()
    q, k, v = (t.cuda() for t in gi.attn_inputs(1, 2, 512, 128, seed=43))
    o = torch.empty_like(q)
    _noalloc(lib, q, k, v, True, 0.1, o)           # first call on the device: looks up the array's address
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for causal in (False, True, False):
        _noalloc(lib, q, k, v, causal, 0.1, o)
    rc, code = _status(lib)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert (rc, code) == (_lib.OK, 0)
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes"


def test_noalloc_at_the_static_capacity_leaves_neighbours_untouched():
    # exactly 524288 query rows (the limit), HEAD_DIM 64; O sits inside a canary-filled buffer
    lib = _lib.load()
    Z, H, S, D = 1, 32, 16384, 64
    assert Z * H * S == 524288
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn(Z, H, S, D, device="cuda", generator=g).bfloat16()
    k = torch.randn(Z, H, S, D, device="cuda", generator=g).bfloat16()
    v = torch.randn(Z, H, S, D, device="cuda", generator=g).bfloat16()
    pad = 4096
    buf = torch.full((q.numel() + 2 * pad,), -7.0, device="cuda", dtype=torch.bfloat16)
    o = buf[pad:pad + q.numel()].view(Z, H, S, D)
    _noalloc(lib, q, k, v, True, D ** -0.5, o)
    ref = _existing(lib, q, k, v, True, D ** -0.5)
    torch.cuda.synchronize()
    assert torch.equal(o.view(torch.int16), ref.view(torch.int16))
    assert bool((buf[:pad] == -7.0).all()) and bool((buf[pad + q.numel():] == -7.0).all())
    assert _status(lib) == (_lib.OK, 0)


def test_noalloc_status_reports_a_wait_that_gave_up():
    # a bounded wait that runs out on this path must be visible without b200k_device_status (which allocates on a
    # device's first use): the self-test kernel waits about a millisecond on a barrier nothing completes, gives up
    # and returns normally, reporting into the static array
    lib = _lib.load()
    stream = torch.cuda.current_stream().cuda_stream
    assert _status(lib) == (_lib.OK, 0)
    _lib.check(lib.b200k_attn_noalloc_selftest(2_000_000, stream))
    rc, code = _status(lib)
    assert rc == _lib.ERR_DEVICE_TIMEOUT and (code & 0xFF) == 1 and (code >> 8) == 99
    assert "gave up" in _lib.last_error()
    assert _status(lib) == (_lib.OK, 0)          # reported once, then cleared
    # the context is still usable and the entry point still works
    q, k, v = (t.cuda() for t in gi.attn_inputs(1, 1, 256, 128, seed=44))
    got = _noalloc(lib, q, k, v, False, 0.1)
    ref = _existing(lib, q, k, v, False, 0.1)
    torch.cuda.synchronize()
    assert torch.equal(got.view(torch.int16), ref.view(torch.int16))


def test_noalloc_rejects_problems_beyond_the_static_capacity():
    lib = _lib.load()
    q = torch.zeros(16, dtype=torch.bfloat16, device="cuda")   # never read: the size check comes first
    rc = lib.b200k_attn_fwd_bf16_noalloc(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 8, 32, 4096, 128, 0,
                                         0.1, None)            # 1 048 576 rows > 524 288
    assert rc == _lib.ERR_INVALID_ARG
    assert "524288" in _lib.last_error()
    # a product that would overflow 64 bits if it were formed carelessly
    rc = lib.b200k_attn_fwd_bf16_noalloc(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 2 ** 31 - 1, 2 ** 31 - 1,
                                         2 ** 31 - 128, 128, 0, 0.1, None)
    assert rc == _lib.ERR_INVALID_ARG
    rc = lib.b200k_attn_fwd_bf16_noalloc(q.data_ptr(), q.data_ptr(), q.data_ptr(), q.data_ptr(), 1, 1, 128, 48, 0, 0.1, None)
    assert rc == _lib.ERR_UNSUPPORTED                           # same shape rules as the existing entry point
