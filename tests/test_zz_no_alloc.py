"""The allocation-free Muon entry point (`b200_muon_rms_noalloc`, csrc/optim/optim_noalloc.h).

It serves callers that cannot allocate device memory when they call into the library (the device
allocator is frozen for them, or they only hold pointers handed over by another runtime), so the
per-segment scratch is a fixed array inside the library instead of a caller-provided buffer. The
test drives it through its exported C symbol with raw device pointers only and checks it against
the regular entry point, which takes its scratch from the caller, on two consecutive calls - the
second call sees the scratch left behind by the first. This file sorts last on purpose, so a run
that stops at the first failure has already executed every other test.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_SEGMENTS = 4096          # B200_NOALLOC_MAX_SEGMENTS
TOO_MANY_SEGMENTS = -10      # B200_NOALLOC_TOO_MANY_SEGMENTS


def _symbols():
    from rust_neural_network_b200 import _native as nv
    lib = nv.cuda()
    noalloc = lib.b200_muon_rms_noalloc
    noalloc.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_float, C.c_float, C.c_float, C.c_void_p]
    noalloc.restype = C.c_int
    regular = lib.b200_muon_rms
    regular.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_float, C.c_float, C.c_float, C.c_void_p]
    regular.restype = C.c_int
    return noalloc, regular


@pytest.mark.parametrize("index", range(max(1, torch.cuda.device_count())))
def test_noalloc_matches_regular_entry_point_on_two_calls(index):
    """On every visible device: the built-in scratch is one array per GPU, looked up on that GPU's first call."""
    noalloc, regular = _symbols()
    dev = torch.device("cuda", index)
    torch.cuda.set_device(dev)
    torch.manual_seed(0)
    sizes = [1000, 64, 7, 4096, 333]
    offs, begin = [], 0
    for s in sizes:
        offs.append([begin, begin + s]); begin += s + 13          # gaps between segments stay untouched
    n = begin
    seg = torch.tensor(offs, dtype=torch.int64, device=dev)
    p0 = torch.randn(n, device=dev)
    grads = [torch.randn(n, device=dev) * (i + 1) for i in range(2)]

    pa, bufa = p0.clone(), torch.zeros(n, device=dev)
    sha = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    pb, bufb = p0.clone(), torch.zeros(n, device=dev)
    shb = torch.zeros(n, dtype=torch.bfloat16, device=dev)
    scratch = torch.empty(len(sizes), device=dev)                 # caller-provided scratch of the regular entry
    stream = torch.cuda.current_stream(dev).cuda_stream
    for g in grads:                                               # two calls in a row
        rc = noalloc(pa.data_ptr(), g.data_ptr(), bufa.data_ptr(), sha.data_ptr(), seg.data_ptr(), len(sizes), 0.02, 0.95, 1e-8, stream)
        assert rc == 0
        rc = regular(pb.data_ptr(), g.data_ptr(), bufb.data_ptr(), shb.data_ptr(), seg.data_ptr(), len(sizes), scratch.data_ptr(), 0.02, 0.95, 1e-8, stream)
        assert rc == 0
        torch.cuda.synchronize()
        assert torch.allclose(pa, pb, atol=1e-5, rtol=1e-4)
        assert torch.allclose(bufa, bufb, atol=1e-5, rtol=1e-4)
        assert torch.equal(sha, shb)
    assert not torch.equal(pa, p0)                                # the update really happened
    gap = torch.ones(n, dtype=torch.bool, device=dev)
    for a, b in offs:
        gap[a:b] = False
    assert torch.equal(pa[gap], p0[gap])                          # elements outside the segments are not touched
    torch.cuda.set_device(0)


def test_noalloc_rejects_more_segments_than_the_builtin_scratch():
    noalloc, _ = _symbols()
    dev = torch.device("cuda")
    nseg = MAX_SEGMENTS + 1
    seg = torch.zeros((nseg, 2), dtype=torch.int64, device=dev)
    p = torch.zeros(8, device=dev)
    rc = noalloc(p.data_ptr(), p.data_ptr(), p.data_ptr(), None, seg.data_ptr(), nseg, 0.1, 0.9, 1e-8,
                 torch.cuda.current_stream().cuda_stream)
    assert rc == TOO_MANY_SEGMENTS
    torch.cuda.synchronize()
