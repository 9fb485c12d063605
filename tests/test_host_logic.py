"""CPU tests: the C-ABI library loads and exports what include/b200attn.h declares, the ctypes structs
match the C structs, the planners obey their bounds, the validators reject what the reference rejects."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200attn.h")


def test_library_loads_and_exports_every_declared_symbol():
    from kernels import _native

    handle = _native.lib()
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(b200attn_[a-z_]+)\s*\(", text))
    assert declared, "no declarations found in the header"
    assert declared == set(_native.EXPORTS)
    for name in declared:
        assert hasattr(handle, name), name
    assert handle.b200attn_abi_version() == _native.ABI_VERSION


def test_ctypes_structs_match_the_header(tmp_path):
    """Compile the header as plain C and compare sizes and a few offsets with the ctypes mirrors."""
    from kernels import _native

    src = tmp_path / "sizes.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "b200attn.h"\n'
        "int main(void){printf(\"%zu %zu %zu %zu %zu %zu %zu\\n\", sizeof(b200attn_prefill_args_t),"
        "sizeof(b200attn_decode_args_t), sizeof(b200attn_device_info_t), offsetof(b200attn_prefill_args_t, sm_scale),"
        "offsetof(b200attn_decode_args_t, sm_scale), offsetof(b200attn_prefill_args_t, total_q),"
        "offsetof(b200attn_decode_args_t, q_len));return 0;}\n"
    )
    exe = tmp_path / "sizes"
    subprocess.run(["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)], check=True)
    got = [int(x) for x in subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.split()]
    want = [C.sizeof(_native.PrefillArgs), C.sizeof(_native.DecodeArgs), C.sizeof(_native.DeviceInfo),
            _native.PrefillArgs.sm_scale.offset, _native.DecodeArgs.sm_scale.offset,
            _native.PrefillArgs.total_q.offset, _native.DecodeArgs.q_len.offset]
    assert got == want


def test_native_rejects_bad_arguments_without_a_gpu():
    from kernels import _native

    handle = _native.lib()
    assert handle.b200attn_prefill(None, None) != 0
    assert "null" in _native.last_error()
    args = _native.DecodeArgs()
    args.dtype, args.layout, args.batch, args.q_heads, args.kv_heads, args.head_dim = 1, 0, 1, 8, 3, 64
    assert handle.b200attn_decode(C.byref(args), None) == -1  # q_heads % kv_heads
    args.kv_heads, args.head_dim = 2, 96
    assert handle.b200attn_decode(C.byref(args), None) == -2  # head_dim not built
    assert "head_dim" in _native.last_error()


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from kernels import _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setenv("B200ATTN_LIBRARY", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="not found"):
        _native.lib()


def test_product_path_never_imports_the_oracle():
    pkg = os.path.join(ROOT, "triton-kernels_b200")
    for base, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(base, f)).read()
                assert "oracle" not in text, os.path.join(base, f)


@pytest.mark.parametrize("qh,kvh,m", [(32, 8, 1), (64, 8, 5), (8, 1, 16), (8, 8, 1), (64, 1, 2), (32, 1, 5), (48, 1, 16)])
def test_decode_plan_bounds(qh, kvh, m):
    from utils.launch_config import decode_chunk_tokens, decode_items, decode_plan

    g = torch.Generator().manual_seed(qh + m)
    for batch, lo, hi in [(1, 1, 10), (64, 512, 8192), (32, 1024, 32768), (300, 0, 5), (7, 100000, 200000)]:
        lens = torch.randint(lo, hi + 1, (batch,), generator=g).tolist()
        plan = decode_plan(148, batch, qh, kvh, m)
        items = decode_items(plan, lens)
        chunk = decode_chunk_tokens(plan, lens)
        assert chunk % 64 == 0 and chunk >= plan.min_chunk
        assert sum(items) <= plan.max_items
        assert all(i >= 1 for i in items)
        assert all((i - 1) * chunk < max(n, 1) for i, n in zip(items, lens))
        from utils.launch_config import decode_pass_group

        sub = decode_pass_group(qh // kvh, m)
        assert (qh // kvh) % sub == 0 and sub * m <= 128 and plan.mma_tiles * 16 >= sub * m


def test_prefill_grid_and_boxes():
    from utils.launch_config import paged_box_rows, prefill_items

    assert prefill_items("dense", 2, 32, 8, max_q=2048) == 2 * 16 * 16       # head pairs x 128-row tiles
    assert prefill_items("dense", 2, 8, 8, max_q=2048) == 2 * 8 * 8          # MHA: 256-row blocks per head
    lens = [2638, 3890, 2767, 3581]
    assert prefill_items("ragged", len(lens), 1, 1, total_q=sum(lens)) >= sum(-(-n // 256) for n in lens)
    assert prefill_items("ragged", len(lens), 2, 1, total_q=sum(lens)) >= sum(-(-n // 128) for n in lens)
    assert [paged_box_rows(p) for p in (1, 8, 16, 24, 48, 128, 256, 384)] == [1, 8, 16, 8, 16, 128, 128, 128]
    for p in (1, 8, 16, 24, 48, 128, 256, 384):
        assert p % paged_box_rows(p) == 0 or paged_box_rows(p) == 128 and p % 128 == 0


def test_layout_detection_follows_the_reference():
    from utils.validation import DENSE, PAGED, RAGGED, detect_layout

    t = torch.zeros(1)
    assert detect_layout(None, None, None, prefill=True) == DENSE
    assert detect_layout(t, t, None, prefill=True) == RAGGED
    assert detect_layout(None, t, None, prefill=True) == DENSE      # kernels/attention.py:767: ragged keys on q_indptr
    assert detect_layout(t, t, t, prefill=True) == PAGED
    assert detect_layout(None, t, None, prefill=False) == RAGGED    # kernels/decode.py:241
    assert detect_layout(None, t, t, prefill=False) == PAGED


def test_validators_raise_assertion_errors_on_cpu_tensors():
    from utils.validation import validate_decode, validate_prefill

    q = torch.zeros((2, 8, 16, 64))
    k = torch.zeros((2, 2, 16, 64))
    with pytest.raises(AssertionError, match="CUDA"):
        validate_prefill(q, k, k, None, None, None, None, None)
    with pytest.raises(AssertionError, match="dtype"):
        validate_prefill(q, k.half(), k, None, None, None, None, None)
    with pytest.raises(AssertionError):
        validate_decode(q[:, :, 0], k, k, None, None, None, None, spec=False)


def test_sequence_balancing_and_shards():
    from sharding.planner import balance_sequences, batch_head_units, contiguous_shard, kv_head_shard

    lens = [2638, 3890, 2767, 3581, 1368, 1124, 2178, 516, 3513, 3836, 1369, 1444, 2159, 2597, 3378, 2974]
    for world in (1, 2, 4, 8):
        bins = balance_sequences(lens, world)
        assert sorted(i for b in bins for i in b) == list(range(16))
        cost = [sum(lens[i] * (lens[i] + 1) // 2 for i in b) for b in bins]
        assert max(cost) <= 1.35 * (sum(cost) / world)
        covered = []
        for r in range(world):
            covered += list(range(*contiguous_shard(64, world, r)))
            units = batch_head_units(2, 8, world, r)
            assert len(units) == 16 // world
        assert covered == list(range(64))
    assert [kv_head_shard(8, 8, r) for r in range(8)] == [(r, r + 1) for r in range(8)]
    assert kv_head_shard(8, 2, 1) == (4, 8)


@pytest.mark.gpu
@pytest.mark.parametrize("qh,kvh,m,batch,d,fp32", [(32, 8, 1, 64, 128, False), (64, 8, 5, 32, 128, False), (8, 2, 1, 4, 64, True),
                                                   (32, 1, 5, 3, 128, False), (48, 1, 16, 2, 64, False), (8, 8, 16, 300, 64, False),
                                                   (8, 1, 10, 16, 64, True)])
def test_planning_mirror_agrees_with_the_library(qh, kvh, m, batch, d, fp32):
    """utils/launch_config.py restates the library's decode planning; the scratch size both derive from it must be
    the same number, or the mirror (and the CPU tests built on it) no longer describes the library."""
    import ctypes as C

    from kernels import _native
    from utils.launch_config import decode_pass_group, decode_plan, decode_workspace_bytes

    info = _native.device_info(torch.cuda.current_device())
    a = _native.DecodeArgs()
    a.batch, a.q_heads, a.kv_heads, a.q_len, a.head_dim = batch, qh, kvh, m, d
    a.dtype = _native.F32 if fp32 else _native.BF16
    a.layout, a.device = _native.RAGGED, torch.cuda.current_device()
    a.total_kv = 5000
    want = _native.lib().b200attn_decode_workspace_bytes(C.byref(a))
    plan = decode_plan(info.sm_count, batch, qh, kvh, m, fp32=fp32)
    rows = decode_pass_group(qh // kvh, m) * m
    cast = fp32 and (rows > 16 or m > 1)      # fp16 copies of q, k, v for the tensor-core kernels
    assert decode_workspace_bytes(plan, batch, kvh, d, rows, batch * qh * m * d if cast else 0,
                                  a.total_kv * kvh * d if cast else 0) == want


@pytest.mark.gpu
@pytest.mark.parametrize("qh,kvh,m,lens", [
    (32, 8, 1, [8192]),                                   # one sequence: a single wave of short items
    (32, 8, 1, [8192] * 16),                              # uniform batch that fits one wave of three-resident CTAs
    (32, 8, 1, [4096] * 32),                              # ... and one that stays with two waves
    (64, 8, 5, [8192] * 32),                              # speculative decode, uniform: one item per sequence
    (64, 8, 5, [8192] * 4),
    (8, 1, 5, [1500, 9000, 31000, 700, 16000, 12000]),    # one KV head (the eight-GPU shard)
    (32, 8, 1, [600, 8000, 512, 4100, 7777, 2300, 900, 5000] * 8),   # uneven lengths, more sequences than one wave holds
])
def test_planner_chunk_matches_the_mirror(qh, kvh, m, lens):
    """The chunk size and item count the device planner wrote into the workspace header are the ones
    utils/launch_config.py derives from the same lengths (several waves or a single one)."""
    from kernels import _native
    from kernels.decode import decode_attention
    from kernels.speculative_decode import speculative_decode_attention
    from utils.launch_config import decode_chunk_tokens, decode_items, decode_plan

    dev = torch.device("cuda")
    info = _native.device_info(torch.cuda.current_device())
    gen = torch.Generator().manual_seed(5)
    total = sum(lens)
    k = torch.randn((total, kvh, 64), generator=gen).to(torch.bfloat16).to(dev)
    v = torch.randn((total, kvh, 64), generator=gen).to(torch.bfloat16).to(dev)
    indptr = torch.tensor([0] + lens, dtype=torch.int64).cumsum(0).to(torch.int32).to(dev)
    if m == 1:
        q = torch.randn((len(lens), qh, 64), generator=gen).to(torch.bfloat16).to(dev)
        decode_attention(q, k, v, kv_indptr=indptr)
    else:
        q = torch.randn((len(lens), qh, m, 64), generator=gen).to(torch.bfloat16).to(dev)
        speculative_decode_attention(q, k, v, kv_indptr=indptr, causal=False)
    torch.cuda.synchronize()
    ws = _native._workspaces[(torch.cuda.current_device(), int(torch.cuda.current_stream().cuda_stream))]
    header = ws[:16].view(torch.int32).tolist()
    plan = decode_plan(info.sm_count, len(lens), qh, kvh, m)
    assert header[0] == 0
    assert header[1] == decode_chunk_tokens(plan, lens)
    assert header[2] == sum(decode_items(plan, lens))


@pytest.mark.gpu
def test_fp32_copies_are_capped_by_scratch_size():
    """fp32 speculative decode asks for room for fp16 copies of q, k, v - unless the cache is so large that the copies
    would pass 8 GiB, where the call stays on the fp32 kernel and the scratch need does not grow with the cache."""
    import ctypes as C

    from kernels import _native

    def need(total_kv):
        a = _native.DecodeArgs()
        a.batch, a.q_heads, a.kv_heads, a.q_len, a.head_dim = 8, 64, 8, 5, 128
        a.dtype, a.layout, a.device = _native.F32, _native.PAGED, torch.cuda.current_device()
        a.page_size, a.total_kv, a.table_stride = 16, total_kv, 64
        return _native.lib().b200attn_decode_workspace_bytes(C.byref(a))

    small, large = need(100_000), need(10_000_000)
    assert small >= 2 * 2 * 100_000 * 8 * 128            # fp16 copies of k and v
    assert large < small                                 # 41 GB of fp32 cache: no copies, fp32 kernel
