"""Multi-process CPU tests over gloo (world size 2): sequence-parallel equivalence, end-to-end training of the
2,048-node SBM configuration, voted OOM recovery with a host-injected fault."""
import json
import os
import subprocess
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _spawn(nproc, mode, out, port):
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = "2"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "mp_cpu_check.py"), mode, out]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]


def test_sp_two_ranks_equals_single_process(tmp_path):
    one, two = str(tmp_path / "one.json"), str(tmp_path / "two.json")
    _spawn(1, "equiv", one, 29801)
    _spawn(2, "equiv", two, 29802)
    a, b = json.load(open(one)), json.load(open(two))
    for model in a:
        assert a[model]["edges"] == b[model]["edges"] and a[model]["cols"] == b[model]["cols"], model
        assert torch.allclose(torch.tensor(a[model]["out"]), torch.tensor(b[model]["out"]), atol=2e-5), model
        for name in a[model]["grads"]:
            ga, gb = torch.tensor(a[model]["grads"][name]), torch.tensor(b[model]["grads"][name])
            assert torch.allclose(ga, gb, atol=2e-5 + 1e-3 * float(ga.abs().max())), (model, name)


def test_sbm_config_trains_on_two_cpu_ranks(tmp_path):
    out = str(tmp_path / "train.json")
    _spawn(2, "train", out, 29803)
    res = json.load(open(out))
    assert res["epochs"] == 4 and res["best"]["valid"] > 0.15


def test_voted_oom_recovery_is_symmetric(tmp_path):
    out = str(tmp_path / "oom.json")
    _spawn(2, "oom", out, 29804)
    r0, r1 = json.load(open(out + ".0")), json.load(open(out + ".1"))
    assert [e["modes"] for e in r0] == [e["modes"] for e in r1]          # ranks agree on every tier decision
    assert r0[0]["modes"] == ["retain", "retain"]
    assert r0[1]["modes"] == ["keep_mha", "retain"]                        # one tier demoted after the injected OOM
    assert r0[1]["dropped"] == 0.0 and r0[1]["loss"] == r0[1]["loss"]      # fault hit before backward: step retried
    assert r0[2]["dropped"] == 1.0 and r1[2]["dropped"] == 1.0             # fault after backward on rank 1: both drop
    assert r0[2]["modes"] == ["recompute", "retain"]
    assert r0[3]["dropped"] == 0.0 and r0[3]["modes"] == r0[2]["modes"]
    assert [e["weights"] for e in r0] == [e["weights"] for e in r1]        # no rank applied an update the other dropped
    assert r0[2]["weights"] == r0[1]["weights"] and r0[3]["weights"] != r0[2]["weights"]


def test_sync_batchnorm_two_ranks_equals_single_process(tmp_path):
    one, two = str(tmp_path / "bn1.json"), str(tmp_path / "bn2.json")
    _spawn(1, "syncbn", one, 29805)
    _spawn(2, "syncbn", two, 29806)
    a, b = json.load(open(one)), json.load(open(two))
    assert torch.allclose(torch.tensor(a["out"]), torch.tensor(b["out"]), atol=5e-5)
    assert torch.allclose(torch.tensor(a["running_mean"]), torch.tensor(b["running_mean"]), atol=1e-5)
    for name in a["grads"]:
        ga, gb = torch.tensor(a["grads"][name]), torch.tensor(b["grads"][name])
        assert torch.allclose(ga, gb, atol=5e-5 + 2e-3 * float(ga.abs().max())), name


def _spawn_raw(nproc, mode, out, port, env_extra):
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = "2"
    env.update(env_extra)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(HERE, "mp_cpu_check.py"), mode, out]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=240, env=env)


def _watchdog_outcome(out, r):
    """Either the main thread raised PeerLost between steps (JSON written), or it was already inside a collective and
    the watchdog thread ended the process with its message."""
    if os.path.exists(out + ".0"):
        res = json.load(open(out + ".0"))
        assert res["outcome"] == "peer_lost", res
        return res["message"]
    assert "[watchdog] rank 0" in r.stderr, r.stderr[-2000:]
    return r.stderr


def test_watchdog_reports_a_rank_that_left_between_steps(tmp_path):
    """Host-side failure only: rank 1 announces its departure before step 3 and exits (exit code 0, so that the
    launcher leaves rank 0 alone); rank 0 learns of it from the store."""
    out = str(tmp_path / "wd_leave.json")
    r = _spawn_raw(2, "watchdog", out, 29807, {"BF_WD_CASE": "leave", "BF_FAULT_EXIT_CODE": "0"})
    assert "rank 1 left" in _watchdog_outcome(out, r)
    assert not os.path.exists(out + ".1")                                   # rank 1 exited inside the injected fault


def test_watchdog_aborts_when_a_peer_stalls_silently(tmp_path):
    """Rank 1 stops making progress without a word; rank 0 is already inside the step's collectives.  Its watchdog thread
    sees the heartbeat stand still for the deadline and ends the process (or the main thread gets PeerLost first if it
    was between steps)."""
    out = str(tmp_path / "wd_stall.json")
    r = _spawn_raw(2, "watchdog", out, 29808, {"BF_WD_CASE": "stall", "BF_FAULT_STALL_SECONDS": "40"})
    msg = _watchdog_outcome(out, r)
    assert "silent" in msg or "did not reach step" in msg, msg


def test_watchdog_ends_a_step_that_exceeds_its_deadline(tmp_path):
    """Rank 1 stalls in the middle of step 3, after its heartbeat: both ranks sit in the same step (rank 0 inside the
    gradient collective), so no heartbeat is behind.  The step deadline ends the job with a message on every rank."""
    out = str(tmp_path / "wd_mid.json")
    r = _spawn_raw(2, "watchdog", out, 29809, {"BF_WD_CASE": "midstep", "BF_FAULT_STALL_SECONDS": "60"})
    assert not os.path.exists(out + ".0") and not os.path.exists(out + ".1")
    assert "has not reached a step boundary" in r.stderr or "abort requested" in r.stderr, r.stderr[-2000:]
    assert "[watchdog] rank" in r.stderr


def test_sharded_cpu_edge_build_equals_whole_build(tmp_path):
    """Two gloo ranks each build the rows of their own queries; the all-gathered graph is the graph of a whole build
    (typed, virtual-node and fan-out variants included) and a training run on it completes."""
    out = str(tmp_path / "shard.json")
    _spawn(2, "shard", out, 29811)
    res = json.load(open(out))
    for name in ("gt", "exphormer", "graphormer", "gt_fanout"):
        assert res[name]["equal"], (name, res[name])
        assert res[name]["totals"] == res[name]["totals_whole"], (name, res[name])
    assert res["fit"]["epochs"] == 4 and 0.0 <= res["fit"]["valid"] <= 1.0


def test_a_raising_rank_ends_the_job_promptly(tmp_path):
    """Rank 1 raises after two steps while rank 0 walks into the next step's collectives: the failing rank must leave
    with status 1 at once (traceback on stderr), and the launcher then ends the job - no hang until a timeout."""
    import time
    env = dict(os.environ)
    env["OMP_NUM_THREADS"] = "2"
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29811", os.path.join(HERE, "mp_cpu_check.py"), "raise", str(tmp_path / "unused.json")]
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=180, env=env)
    assert r.returncode != 0
    assert "injected failure on rank 1" in r.stderr
    assert time.time() - t0 < 120
