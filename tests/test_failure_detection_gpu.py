"""Failure detection on the device without faulting it: a kernel that waits for a peer's flag gets a
flag nothing ever sets, its bounded wait runs out, the kernel returns, the host reads the status
word, and the context stays usable for the next launch."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_peer_flag_wait_expires_and_context_survives():
    from rust_neural_network_b200 import _native as nv
    from rust_neural_network_b200.parallel.sp import StateExchangeArgs, SX_MAX_CTAS, SX_MAX_WORLD
    dev = torch.device("cuda", 0)
    lib = nv.cuda()
    n = 1024
    slot0 = torch.zeros(n, device=dev)
    slot1 = torch.zeros(n, device=dev)                       # stands in for the absent peer's slot (local memory)
    flags0 = torch.zeros(2 * SX_MAX_WORLD * SX_MAX_CTAS, dtype=torch.int32, device=dev)
    flags1 = torch.zeros_like(flags0)                        # the "peer's" flag area: this kernel writes it, nobody answers
    inp, out = torch.ones(n, device=dev), torch.full((n,), -7.0, device=dev)
    a = StateExchangeArgs()
    a.slot[0], a.slot[1] = slot0.data_ptr(), slot1.data_ptr()
    a.flags[0], a.flags[1] = flags0.data_ptr(), flags1.data_ptr()
    a.inp, a.out, a.numel = inp.data_ptr(), out.data_ptr(), n
    a.rank, a.world, a.mode, a.epoch = 0, 2, 2, 1
    clock_hz = torch.cuda.get_device_properties(dev).clock_rate * 1000
    a.wait_cycles = int(0.05 * clock_hz)                     # 50 ms budget
    a.status = nv.status_word(dev).data_ptr()
    nv.check(lib.b200_state_exchange(C.byref(a), 4, nv.stream_ptr()), "state_exchange")
    torch.cuda.synchronize()                                 # the kernel came back by itself
    with pytest.raises(RuntimeError, match="status 5"):
        nv.check_status()
    assert float(out[0]) == -7.0                             # it returned before the sum: no partial result
    assert int(flags1[0 * SX_MAX_WORLD * SX_MAX_CTAS + 0 * SX_MAX_CTAS]) == 1      # its own signal did go out
    # the context is alive: status is clear again and ordinary kernels run
    nv.check_status()
    from rust_neural_network_b200.ops import gemm as G
    x = torch.randn(128, 64, device=dev, dtype=torch.bfloat16)
    y = G.gemm(x, x)
    torch.cuda.synchronize()
    assert torch.allclose(y.float(), x.float() @ x.float().t(), rtol=2e-2, atol=2e-1)
    nv.check_status()
