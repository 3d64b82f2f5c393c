"""The routing entry point that allocates nothing, through the C ABI.

Who needs it: a host that drives the single ops of include/tei_b200_ops.h from inside a runtime
that owns all device memory - an inference server with a fixed arena sized at start-up, where a
cudaMalloc on the request path is forbidden because it stalls every stream of the device and can
fail once the arena has taken the memory - or an operator plugin that is only ever handed the
input and output tensors of its operator.  tei_b200_op_moe_route asks such a caller for a small
counter buffer it cannot provide; tei_b200_op_moe_route_noalloc keeps those counters in an array
inside the library instead.

What is checked: the new entry point gives what the existing one gives on the same logits, twice
in a row (the built-in counters keep the previous call's contents and must be cleared by the
call), with different sizes in between, and it refuses more experts than its array holds.  It
shares one device array with every other caller in the process, so it runs after the other GPU
tests (pytest collects this file last) and alone in a fresh process alike.
"""
import ctypes
import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

pytestmark = pytest.mark.gpu


def _logits(T, E, seed, dtype):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    width = (E + 7) // 8 * 8  # the row stride the router GEMM produces
    return (torch.randn(T, width, device="cuda", generator=g) * 2.0).to(dtype)


def _check_same(ref, got, E):
    import torch
    te, tw, pos, counts = ref
    te2, tw2, pos2, counts2 = got
    assert torch.equal(te, te2)          # same picks (both apply the same tie rule)
    assert torch.equal(tw, tw2)          # same weights, bit for bit: same arithmetic
    assert torch.equal(counts, counts2)  # same number of tokens per expert
    # rows inside an expert are handed out in arrival order, which may differ between two
    # launches; what must hold is that each expert's rows are 0 .. count-1, each exactly once
    for e in range(E):
        rows = pos2[te2 == e].long().sort().values
        assert torch.equal(rows, torch.arange(int(counts2[e]), device="cuda"))


def test_noalloc_routing_matches_the_allocating_entry_point(lib):
    import torch
    from tei_b200 import ops
    for dtype in (torch.float16, torch.bfloat16):
        # call 1: 8 experts, top 2
        a = _logits(3000, 8, 1, dtype)
        _check_same(ops.moe_route(a, 8, 2), ops.moe_route_noalloc(a, 8, 2), 8)
        # call 2 directly after it, other logits and sizes: stale counters would show here
        b = _logits(517, 5, 2, dtype)
        _check_same(ops.moe_route(b, 5, 3), ops.moe_route_noalloc(b, 5, 3), 5)
        # call 3: the first shapes again, into buffers that already hold old results
        out = ops.moe_route_noalloc(b, 5, 3)
        c = _logits(517, 5, 3, dtype)
        _check_same(ops.moe_route(c, 5, 3), ops.moe_route_noalloc(c, 5, 3, out=out), 5)
        # the full 64 experts the built-in array can hold
        d = _logits(1000, 64, 4, dtype)
        _check_same(ops.moe_route(d, 64, 8), ops.moe_route_noalloc(d, 64, 8), 64)


def test_noalloc_routing_refuses_what_does_not_fit(lib):
    import torch
    from tei_b200 import ops
    a = _logits(16, 72, 5, torch.float16)
    with pytest.raises(RuntimeError) as e:
        ops.moe_route_noalloc(a, 65, 2)
    assert "at most 64 experts" in str(e.value)
    # counts_out may be NULL, and so may the message buffer
    te = torch.empty((16, 2), dtype=torch.int32, device="cuda")
    tw = torch.empty((16, 2), dtype=torch.float32, device="cuda")
    pos = torch.empty((16, 2), dtype=torch.int32, device="cuda")
    rc = lib.tei_b200_op_moe_route_noalloc(ctypes.c_void_p(a.data_ptr()), a.stride(0), 16, 64, 2,
                                           ctypes.c_void_p(te.data_ptr()), ctypes.c_void_p(tw.data_ptr()),
                                           ctypes.c_void_p(pos.data_ptr()), None, 0, None, None, 0)
    assert rc == 0
    torch.cuda.synchronize()
    ref = ops.moe_route(a, 64, 2)
    assert torch.equal(ref[0], te) and torch.equal(ref[1], tw)
    assert lib.tei_b200_op_moe_route_noalloc(ctypes.c_void_p(a.data_ptr()), a.stride(0), 16, 0, 2, None, None, None,
                                             None, 0, None, None, 0) != 0
