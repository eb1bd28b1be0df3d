"""Multi-GPU checks (2+ GPUs on one node), run as torchrun child processes."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def _run(nproc, models, port, env_extra=None):
    env = dict(os.environ)
    env.update(env_extra or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port), os.path.join(HERE, "mp_fused_check.py"), models]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=420, env=env)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_path_two_gpus():
    r = _run(2, "gt,graphormer,graphgps,exphormer", 29611)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK ") == 4, r.stdout[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_path_two_gpus_plain_peer_loads():
    """Same with NVSwitch multimem disabled: the all-reduce takes the peer load/store kernel."""
    r = _run(2, "gt", 29612, {"BF_DISABLE_MULTIMEM": "1", "NCCL_NVLS_ENABLE": "0"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_fused_path_two_gpus_narrow_column_slices():
    """hidden 64 on 2 ranks: a rank's slice of q|k|v is 96 columns and of d(context) 32, so the GEMM epilogue stages
    destination-wide (unswizzled) panels and bulk-stores them into the peer's buffer - the path 4 and 8 ranks take at
    hidden 128."""
    r = _run(2, "gt,graphgps", 29615, {"BF_TEST_HIDDEN": "64"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert r.stdout.count("OK ") == 2, r.stdout[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_cpu_edge_build_two_gpus():
    """Each rank builds the rows of its own queries on the CPU; the shards are all-gathered as device tensors over NCCL
    and give the graph of a whole build."""
    r = _run(2, "sharded_build", 29616)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "OK sharded host build" in r.stdout, r.stdout[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_sharded_device_edge_build_two_gpus():
    """Each rank selects the rows of its own queries on its GPU and fetches the other shards through symmetric memory:
    the graph equals the one every rank would build whole, in the step and one epoch ahead on the side stream."""
    r = _run(2, "sharded_device_build", 29617)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "OK sharded device build" in r.stdout, r.stdout[-2000:]


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_watchdog_rank_leaves_between_steps_two_gpus():
    """Rank 1 finishes step 2, drains its queue, announces its departure and exits (code 0, so that the launcher leaves
    rank 0 alone); rank 0 gets PeerLost at its next step boundary, with a clean device status.  Host-side failure only:
    no kernel or collective is in flight when the rank leaves, NVLS and multimem are off."""
    import json
    r = _run(2, "watchdog_leave", 29618, {"BF_FAULT_EXIT_CODE": "0"})
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("WATCHDOG ")]
    assert lines, r.stdout[-2000:] + r.stderr[-3000:]
    out = json.loads(lines[0][len("WATCHDOG "):])
    if out["outcome"] == "multicast_bound":
        pytest.skip("symmetric allocations are still bound to a multicast object on this machine: no rank may leave")
    assert out["outcome"] == "peer_lost" and "rank 1 left" in out["message"], out
    assert out["epoch"] == 2 and out["status"] == 0, out


@pytest.mark.skipif(torch.cuda.device_count() < 4, reason="needs 4 GPUs")
def test_fused_path_four_gpus():
    r = _run(4, "gt,graphormer", 29613)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


@pytest.mark.skipif(torch.cuda.device_count() < 8, reason="needs 8 GPUs")
def test_fused_path_eight_gpus():
    r = _run(8, "gt,graphgps", 29614)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]


def test_barrier_wait_expires_and_reports_status():
    """A peer that never raises its flag: the bounded spin gives up, writes a status word and the context stays
    usable (no trap, no hang)."""
    from budgetformer_b200.ops import _ext, gemm
    ext = _ext.load()
    dev = torch.device("cuda")
    mine = torch.zeros(64 * 8, dtype=torch.int32, device=dev)
    silent_peer = torch.zeros(64 * 8, dtype=torch.int32, device=dev)
    status = gemm.status_tensor(dev)
    status.zero_()
    ext.peer_barrier([mine.data_ptr(), silent_peer.data_ptr()], 0, 3, 1, status)
    torch.cuda.synchronize()
    assert int(status[0]) == 16 + 1 and int(status[1]) == 1          # waited for rank 1, epoch 1
    assert int(silent_peer[3 * 8 + 0]) == 1                           # our own flag was raised in the peer's page
    with pytest.raises(RuntimeError):
        gemm.check_status(dev)
    assert int(status[0]) == 0
    x = torch.ones(8, device=dev) * 2                                 # context still healthy
    assert float(x.sum()) == 16.0
