"""Multi-process runs: gloo ranks on CPU (host-side logic), nccl ranks on GPUs (real peer stores)."""
import os
import subprocess
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    """A port nobody listens on right now (asked from the kernel), so consecutive launches never meet a socket in TIME_WAIT."""
    import socket
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _launch(backend, case, world, timeout=300, extra_env=None):
    port = _free_port()
    procs = []
    for r in range(world):
        env = dict(os.environ, RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, os.path.join(HERE, "mp_worker.py"), backend, case], env=env,
                                      stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True))
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=timeout)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for r, (p, out) in enumerate(zip(procs, outs)):
        assert p.returncode == 0 and f"WORKER_OK {r}" in out, f"rank {r} failed (rc={p.returncode}):\n{out[-3000:]}"


@pytest.mark.parametrize("world", [2, 3])
def test_gloo_layer(world):
    _launch("gloo", "layer", world)


def test_gloo_bootstrap_from_an_mpi_style_communicator(tmp_path):
    """`Buffer(comm=...)`: no process group exists, the communicator (a file-based stand-in for mpi4py) carries the rendezvous."""
    _launch("gloo", "mpi_comm", 2, timeout=180, extra_env={"FILECOMM_DIR": str(tmp_path)})


def test_gloo_mismatched_arguments_raise():
    _launch("gloo", "mismatch", 2)


def test_gloo_absent_rank_is_detected():
    """Host-side failure detection: a rank that leaves makes the others raise instead of hanging."""
    _launch("gloo", "absent", 2, timeout=120)


@pytest.mark.parametrize("world", [2, 4])
def test_descriptor_exchange_between_processes(world):
    """SCM_RIGHTS plumbing of the virtual-memory arenas, with anonymous memory files standing in for allocations."""
    _launch("gloo", "fdpass", world, timeout=120)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_layer_on_vmm_arenas():
    """cuMemCreate arenas mapped through shared descriptors give the same bits as cudaMalloc + CUDA IPC arenas."""
    _launch("nccl", "vmm", _world(), timeout=300)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_layer_all_gpus():
    world = torch.cuda.device_count()
    world = 8 if world >= 8 else 4 if world >= 4 else 2
    _launch("nccl", "layer", world, timeout=600)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_layer_fused_dispatch_and_combine():
    """The one-kernel dispatch + GEMM path and the combine pushed from the GEMM epilogues, forced on for the small test shapes."""
    world = torch.cuda.device_count()
    world = 8 if world >= 8 else 4 if world >= 4 else 2
    _launch("nccl", "layer", world, timeout=600, extra_env={"TERAMOE_FUSED_COMBINE": "1", "TERAMOE_FUSED_DISPATCH": "1"})


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_layer_default_rules_pick_fused_kernels():
    """A shape with I >= 1536 and no environment switches: the default rules must take the fused dispatch + GEMM kernel and
    the pushed combine, match the fp32 oracle and repeat bit for bit."""
    world = torch.cuda.device_count()
    world = 8 if world >= 8 else 4 if world >= 4 else 2
    _launch("nccl", "layer_auto", world, timeout=600)


def _world():
    world = torch.cuda.device_count()
    return 8 if world >= 8 else 4 if world >= 4 else 2


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_layer_kernel_one_row_per_rank_on_the_wire():
    _launch("nccl", "wire_rank", _world(), timeout=300)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_soak_changing_routing_interleaved_layers():
    """Race / reuse soak (the reference's accuracy script repeats 10,000 identical steps,
    tests/test_teramoe_accuracy.py:296-305; here every step is different): see the "soak" case of mp_worker.py."""
    _launch("nccl", "soak", _world(), timeout=1500, extra_env={"SOAK_STEPS": os.environ.get("SOAK_STEPS", "200")})


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_cached_dispatch_behind_a_slow_rank():
    _launch("nccl", "cached_race", _world(), timeout=300)


@pytest.mark.gpu
@pytest.mark.multigpu
def test_nccl_low_latency_round_trip():
    _launch("nccl", "ll", _world(), timeout=300)
