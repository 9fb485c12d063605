"""b200attn_decode_static: decode for callers that may not allocate device memory (a server whose HBM is
all spoken for after start-up, a plug-in inside another framework's pool).  Its scratch is an 8 MiB array
built into the library instead of a caller workspace.  The test drives it through the C ABI and requires
the same output as b200attn_decode, twice in a row with different inputs so that whatever the first call
left in the shared array cannot leak into the second.  Collected last on purpose."""
import ctypes as C
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEVICE = "cuda"
PAGE = 16


def _problem(seed, lens, qh=32, kvh=8, d=128, m=1, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(seed)
    blocks = [(n + PAGE - 1) // PAGE for n in lens]
    pages = sum(blocks) + 3
    width = max(blocks)
    kc = torch.randn((pages * PAGE, kvh, d), generator=gen).to(dtype).to(DEVICE)
    vc = torch.randn((pages * PAGE, kvh, d), generator=gen).to(dtype).to(DEVICE)
    tables = []
    for _ in range(2):
        perm = torch.randperm(pages, generator=gen).to(torch.int32)
        t = torch.full((len(lens), width), -1, dtype=torch.int32)
        cur = 0
        for i, nb in enumerate(blocks):
            t[i, :nb] = perm[cur: cur + nb]
            cur += nb
        tables.append(t.to(DEVICE))
    q = torch.randn((len(lens), qh, m, d), generator=gen).to(dtype).to(DEVICE)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=DEVICE)
    return q, kc, vc, tables[0], tables[1], lens_t


def _args(q, kc, vc, kt, vt, lens_t, out, causal):
    from kernels import _native

    b, qh, m, d = q.shape
    a = _native.DecodeArgs()
    a.q, a.k, a.v, a.out = q.data_ptr(), kc.data_ptr(), vc.data_ptr(), out.data_ptr()
    a.kv_indptr, a.k_table, a.v_table = lens_t.data_ptr(), kt.data_ptr(), vt.data_ptr()
    a.total_kv, a.table_stride = kc.shape[0], kt.shape[1]
    a.dtype, a.layout, a.indptr_is_i64 = _native.DTYPE_CODE[q.dtype], _native.PAGED, 0
    a.batch, a.q_heads, a.kv_heads, a.q_len = b, qh, kc.shape[1], m
    a.max_kv, a.head_dim, a.page_size = kt.shape[1] * PAGE, d, PAGE
    a.causal_drafts, a.device = int(causal), torch.cuda.current_device()
    a.sm_scale = 1.0 / math.sqrt(d)
    return a


def _run_both(prob, causal=False):
    from kernels import _native

    lib = _native.lib()
    q = prob[0]
    stream = torch.cuda.current_stream().cuda_stream
    out_ws = torch.zeros_like(q)
    a = _args(*prob, out_ws, causal)
    need = lib.b200attn_decode_workspace_bytes(C.byref(a))
    ws = torch.zeros(need, dtype=torch.uint8, device=DEVICE)
    a.workspace, a.workspace_bytes = ws.data_ptr(), need
    _native.check(lib.b200attn_decode(C.byref(a), C.c_void_p(stream)), "b200attn_decode")
    out_static = torch.zeros_like(q)
    s = _args(*prob, out_static, causal)      # workspace fields stay null: the entry point ignores them
    _native.check(lib.b200attn_decode_static(C.byref(s), C.c_void_p(stream)), "b200attn_decode_static")
    torch.cuda.synchronize()
    return out_ws, out_static


def test_static_scratch_decode_matches_workspace_decode_twice():
    # long sequences: several KV chunks each, so partials and the ticket merge go through the scratch
    first = _problem(1, [5000, 333, 2049, 4097])
    a_ws, a_static = _run_both(first)
    assert torch.isfinite(a_static.float()).all()
    torch.testing.assert_close(a_static.float(), a_ws.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(a_static, a_ws)  # same kernels, same plan: bit-identical
    second = _problem(2, [777, 6001, 64], qh=16, kvh=8, m=4)
    b_ws, b_static = _run_both(second, causal=True)
    torch.testing.assert_close(b_static.float(), b_ws.float(), atol=2e-2, rtol=2e-2)
    assert torch.equal(b_static, b_ws)
    # and against the CPU oracle, so that "equal" cannot mean "equally wrong"
    from benchmarks.workloads import gather_paged
    from oracle import sdpa_ref

    q, kc, vc, kt, vt, lens_t = second
    lens = lens_t.tolist()
    ks = [gather_paged(kc, kt[i], lens[i], PAGE) for i in range(len(lens))]
    vs = [gather_paged(vc, vt[i], lens[i], PAGE) for i in range(len(lens))]
    refs = sdpa_ref.spec_decode_reference([q[i] for i in range(len(lens))], ks, vs, 16, 8, True)
    for i in range(len(lens)):
        torch.testing.assert_close(b_static[i].float().cpu(), refs[i].cpu(), atol=2e-2, rtol=2e-2)


def _static_only(prob, causal):
    """One b200attn_decode_static call on pre-allocated tensors; returns the output."""
    from kernels import _native

    out = torch.zeros_like(prob[0])
    a = _args(*prob, out, causal)
    _native.check(_native.lib().b200attn_decode_static(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                  "b200attn_decode_static")
    return out


def test_static_scratch_call_takes_no_device_memory():
    """The property the entry point exists for: once the first call on the device has loaded the module and
    looked up the array, a call neither allocates through torch nor changes the device's free memory."""
    from kernels import _native

    prob = _problem(5, [3000, 1500, 700])
    _static_only(prob, False)                      # first call on this device in this process, or a repeat
    out = torch.zeros_like(prob[0])
    a = _args(*prob, out, False)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    allocated, reserved, free = torch.cuda.memory_allocated(), torch.cuda.memory_reserved(), torch.cuda.mem_get_info()[0]
    _native.check(_native.lib().b200attn_decode_static(C.byref(a), stream), "b200attn_decode_static")
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == allocated and torch.cuda.memory_reserved() == reserved
    assert torch.cuda.mem_get_info()[0] == free
    code = C.c_int32(-1)
    assert _native.lib().b200attn_decode_static_check(torch.cuda.current_device(), stream, C.byref(code)) == 0
    assert code.value == 0
    assert torch.cuda.mem_get_info()[0] == free


@pytest.mark.parametrize("case", ["tcgen05_rows_18", "fp32", "fp32_drafts"])
def test_static_scratch_other_kernels_match_workspace_decode(case):
    """The shared array under the two other decode kernels: the tcgen05 kernel (more than 16 q rows per KV head) and
    the fp32 kernel; each twice in a row with different problems.  fp32 inputs with draft rows take the fp32 kernel
    here (the array has no room for fp16 copies) and the tensor-core kernels with a workspace: same answer to the
    16-bit class bar, not bit for bit."""
    from kernels import _native

    for seed, lens in [(11, [4000, 90, 1300]), (12, [2500, 2600])]:
        if case == "fp32":
            prob, causal = _problem(seed, lens, qh=8, kvh=2, m=1, dtype=torch.float32), True
        elif case == "fp32_drafts":
            prob, causal = _problem(seed, lens, qh=8, kvh=2, m=2, dtype=torch.float32), True
            ws_out, static_out = _run_both(prob, causal)
            assert torch.isfinite(static_out).all()
            torch.testing.assert_close(static_out, ws_out, atol=4e-3, rtol=1e-2)
            continue
        else:
            prob, causal = _problem(seed, lens, qh=12, kvh=2, m=3), True     # 6 x 3 = 18 rows per KV head
            a = _args(*prob, torch.zeros_like(prob[0]), causal)
            assert _native.lib().b200attn_decode_workspace_bytes(C.byref(a)) <= (8 << 20)
        ws_out, static_out = _run_both(prob, causal)
        assert torch.isfinite(static_out.float()).all()
        assert torch.equal(static_out, ws_out)
    code = C.c_int32(-1)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert _native.lib().b200attn_decode_static_check(torch.cuda.current_device(), stream, C.byref(code)) == 0


def test_static_scratch_rejects_problems_beyond_its_size():
    from kernels import _native

    lib = _native.lib()
    prob = _problem(3, [100, 50], qh=64, kvh=8, m=5)   # 40 rows per KV head: partial slots exceed 8 MiB
    out = torch.zeros_like(prob[0])
    a = _args(*prob, out, True)
    assert lib.b200attn_decode_workspace_bytes(C.byref(a)) > (8 << 20)
    rc = lib.b200attn_decode_static(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == -4
    assert "8388608" in _native.last_error() and "b200attn_decode" in _native.last_error()
