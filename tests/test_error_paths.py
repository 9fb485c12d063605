"""The bounded waits, made to run out without hanging anything: a self-test kernel of the library waits on a barrier
that nothing completes, with the kernels' own wait loop and a small try limit, gives up, records the error code the
attention kernels would record and returns.  The host then reads the code and the context stays usable."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_expiry_is_reported_and_the_context_survives():
    from kernels import _native, flash_attention_v2

    lib = _native.lib()
    dev = torch.device("cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    ws = torch.zeros(256, dtype=torch.uint8, device=dev)
    _native.check(lib.b200attn_selftest_wait_expiry(torch.cuda.current_device(), C.c_void_p(ws.data_ptr()), 1 << 12, stream),
                  "b200attn_selftest_wait_expiry")
    code = C.c_int32(0)
    rc = lib.b200attn_check_workspace(C.c_void_p(ws.data_ptr()), stream, C.byref(code))
    assert rc == -6 and code.value == 1, (rc, code.value, _native.last_error())
    assert "bounded wait expired" in _native.last_error()
    # the word was cleared, and a second check is clean
    assert lib.b200attn_check_workspace(C.c_void_p(ws.data_ptr()), stream, C.byref(code)) == 0 and code.value == 0
    # the context is intact: a following attention call runs and is right
    g = torch.Generator().manual_seed(0)
    q = torch.randn((1, 4, 40, 64), generator=g).half().to(dev)
    k = torch.randn((1, 4, 40, 64), generator=g).half().to(dev)
    v = torch.randn((1, 4, 40, 64), generator=g).half().to(dev)
    out = flash_attention_v2(q, k, v, is_causal=True)
    ref = torch.nn.functional.scaled_dot_product_attention(q.float(), k.float(), v.float(), is_causal=True)
    torch.testing.assert_close(out.float(), ref, atol=1e-2, rtol=1e-2)


def test_wait_expiry_selftest_rejects_unbounded_limits():
    from kernels import _native

    lib = _native.lib()
    ws = torch.zeros(256, dtype=torch.uint8, device="cuda")
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert lib.b200attn_selftest_wait_expiry(torch.cuda.current_device(), C.c_void_p(ws.data_ptr()), 0, stream) == -1
    assert lib.b200attn_selftest_wait_expiry(torch.cuda.current_device(), C.c_void_p(ws.data_ptr()), (1 << 20) + 1, stream) == -1
    assert lib.b200attn_selftest_wait_expiry(torch.cuda.current_device(), None, 16, stream) == -1
