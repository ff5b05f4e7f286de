"""Arenas allocated with the driver's virtual memory management (what `use_fabric=True` selects) on one GPU: the
allocation, its views and its release, and the layer giving the same bits as on cudaMalloc arenas.  Sharing between
processes is covered by the `fdpass` (CPU) and `vmm` (multi-GPU) cases of test_multiprocess.py."""
import os

import pytest
import torch

import teramoe_b200 as tm
from helpers import make_problem

pytestmark = pytest.mark.gpu


def test_vmm_arena_allocates_views_and_closes():
    from teramoe_b200._build import load_ext
    ext = load_ext()
    a = ext.SymmetricArena(0, 1, 3 * 128 * 1000, vmm=True)          # not a multiple of the 2 MB granularity
    assert a.is_vmm() and a.bytes() == 3 * 128 * 1000 and a.local_ptr() % 256 == 0
    a.adopt_peer_pointers([a.local_ptr()])
    v = a.view(256, [1000], torch.int32)
    assert int(v.abs().sum()) == 0                                   # zero-filled like the cudaMalloc arena
    v.copy_(torch.arange(1000, dtype=torch.int32, device="cuda"))
    assert int(a.view(256 + 4 * 996, [4], torch.int32)[3]) == 999     # views start on 16-byte boundaries
    fd = a.export_fd()
    assert fd >= 0 and a.export_fd() == fd                           # one descriptor, owned by the arena
    with pytest.raises(RuntimeError):
        a.export_handle()                                            # no CUDA IPC handle for this kind
    del v
    torch.cuda.synchronize()
    a.close()
    with pytest.raises(OSError):
        os.fstat(fd)                                                 # closed with the arena
    b = ext.SymmetricArena(0, 1, 1 << 20)
    with pytest.raises(RuntimeError):
        b.export_fd()
    b.close()


def test_layer_on_vmm_arena_matches_ipc_arena_bitwise():
    prob = make_problem(1, 700, 512, 1536, 8, 4, seed=21, dtype=torch.bfloat16, device="cuda", x_scale=0.5, w_scale=0.05)
    r = prob["ranks"][0]
    res = []
    for fabric in (False, True):
        buf = tm.Buffer(None, int(1e6) // 128 * 128, explicitly_destroy=True, use_fabric=fabric)
        assert buf._world.control.is_vmm() == fabric
        x = r["x"].clone().requires_grad_(True)
        Wg = prob["W_gateup"].clone().requires_grad_(True)
        Wd = prob["W_down"].clone().requires_grad_(True)
        out = buf.teramoe_autograd(x, r["idx"], r["w"], Wg, Wd, prob["E"])
        out.backward(r["go"])
        assert buf._world.data.is_vmm() == fabric
        res.append((out.detach().clone(), x.grad.clone(), Wg.grad.clone(), Wd.grad.clone()))
        buf.check_status()
        buf.destroy()
    for a, b in zip(*res):
        assert torch.equal(a, b)
    assert res[0][0].float().abs().max().item() > 0
