"""Child program of tests/test_gpu_multi.py: run under torchrun with one rank per GPU.

Checks, on every rank: (1) the peer-memory mean all-reduce equals NCCL's; (2) the fused sequence-parallel
layer path (GEMM epilogue push, peer pull, device barriers) reproduces the portable NCCL all-to-all path:
same loss, same parameter gradients after reduction; (3) a few fused training steps stay finite and the
device status word stays clean."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from budgetformer_b200.config import parse_fullgraph_args  # noqa: E402
from budgetformer_b200.graph.synthetic import sbm_graph  # noqa: E402
from budgetformer_b200.ops import gemm  # noqa: E402
from budgetformer_b200.parallel import symm  # noqa: E402
from budgetformer_b200.train.data import GraphData, random_split_idx  # noqa: E402
from budgetformer_b200.train.engine import FullGraphTrainer  # noqa: E402


def trainer(model, fused, extra=()):
    n = 4096
    x, y, ei = sbm_graph(n, feat_dim=64, seed=3)
    data = GraphData(x, y, ei, random_split_idx(n, 3), n, 7)
    hidden = int(os.environ.get("BF_TEST_HIDDEN", "128"))           # 64: column slices per rank that are not multiples of 64
    argv = ["--model", model, "--dataset", "t", "--n_layers", "2", "--hidden_dim", str(hidden), "--num_heads", str(hidden // 16),
            "--ffn_dim", str(2 * hidden), "--fixed_real_edges_per_query", "4", "--fixed_rw_edges_per_query", "4",
            "--amp_dtype", "bf16", "--force_random_split", "--fused_sp", "on" if fused else "off",
            "--dropout_rate", "0.0", "--attention_dropout_rate", "0.0", "--input_dropout_rate", "0.0", "--seed", "5"]
    return FullGraphTrainer(parse_fullgraph_args(argv + list(extra)), data=data, log=lambda *a, **k: None)


def check_sharded_host_build():
    """--shard_cpu_edge_build over NCCL: the graph all-gathered from the per-rank shards (device tensors) equals the
    graph every rank builds whole, for a plain and a typed (Exphormer) model."""
    for model in ("gt", "exphormer"):
        whole = trainer(model, fused=False, extra=["--edge_build_device", "cpu"])
        shard = trainer(model, fused=False, extra=["--edge_build_device", "cpu", "--shard_cpu_edge_build"])
        assert shard.edge_engine.sharded_host_build() and not whole.edge_engine.sharded_host_build()
        a, b = whole.build_edges(1), shard.build_edges(1)
        torch.cuda.synchronize()
        assert b.rowptr.is_cuda and torch.equal(a.rowptr, b.rowptr) and torch.equal(a.col, b.col), f"{model}: graphs differ"
        assert a.etype is None or torch.equal(a.etype, b.etype)
        loss = shard.train_step(1)["loss"]
        assert loss == loss
        whole.edge_engine.shutdown()
        shard.edge_engine.shutdown()
    if dist.get_rank() == 0:
        print("OK sharded host build", flush=True)


def check_sharded_device_build():
    """GPU edge policy on several ranks: every rank selects the rows of its own queries, the shards are fetched over
    NVLink - same graph as the build every rank repeats for itself (plain, typed and virtual-node models), both for
    the build inside a step and for the one that runs one epoch ahead on the side stream."""
    for model in ("gt", "exphormer", "graphormer"):
        whole = trainer(model, fused=True, extra=["--replicate_gpu_edge_build"])
        shard = trainer(model, fused=True)
        st = shard.budget_state()
        assert shard.edge_engine.sharded_device_build(st) and not whole.edge_engine.sharded_device_build(st)
        for epoch in (1, 2, 3):                       # epoch 1 is built in the step, 2 and 3 one epoch ahead
            a = whole.build_edges(epoch)
            out = shard.train_step(epoch)
            b = shard.last_graph
            torch.cuda.synchronize()
            assert torch.equal(a.rowptr, b.rowptr) and torch.equal(a.col, b.col), f"{model}: graphs differ at epoch {epoch}"
            assert a.etype is None or torch.equal(a.etype, b.etype)
            assert out["loss"] == out["loss"]
        gemm.check_status(shard.device)
        whole.edge_engine.shutdown()
        shard.edge_engine.shutdown()
    if dist.get_rank() == 0:
        print("OK sharded device build", flush=True)


def check_watchdog_departure():
    """A rank leaves between steps (host-injected exit, nothing of it in flight); the survivor learns of it on the host
    before its next launch.  The trainer switches NVLS and multimem off for such a run before any group exists."""
    from budgetformer_b200.utils.watchdog import PeerLost
    import json
    t = trainer("gt", fused=True, extra=["--watchdog_seconds", "5", "--fault_inject", "exit@step:3:rank1", "--epochs", "6",
                                        "--eval_every", "100"])
    assert os.environ.get("NCCL_NVLS_ENABLE") == "0" and os.environ.get("BF_DISABLE_MULTIMEM") == "1"
    sw = symm.get_world(t.sp_group, t.device)
    assert t.fused_sp and not sw.use_multimem
    # a rank may only leave when no allocation of the job is bound to an NVSwitch multicast object: verify it on every
    # rank before anything departs; if a binding is still there, nobody leaves and the parent skips the test
    bound = torch.tensor([1.0 if sw.multicast_bound() else 0.0], device=t.device)
    dist.all_reduce(bound, op=dist.ReduceOp.MAX)
    if float(bound) > 0:
        print("WATCHDOG " + json.dumps({"outcome": "multicast_bound"}), flush=True)
        t.edge_engine.shutdown()
        dist.barrier()
        dist.destroy_process_group()
        return
    try:
        t.fit()
        out = {"outcome": "finished"}
    except PeerLost as e:
        torch.cuda.synchronize()                     # the survivor's own queue drains: nothing waits for the lost rank
        code = int(gemm.status_tensor(t.device)[0])
        out = {"outcome": "peer_lost", "message": str(e), "epoch": t.epoch, "status": code}
    print("WATCHDOG " + json.dumps(out), flush=True)
    os._exit(0)                                      # the peer is gone: skip the collective teardown


def main():
    if len(sys.argv) > 1 and sys.argv[1] == "watchdog_leave":
        return check_watchdog_departure()
    if len(sys.argv) > 1 and sys.argv[1] in ("sharded_build", "sharded_device_build"):
        check_sharded_host_build() if sys.argv[1] == "sharded_build" else check_sharded_device_build()
        dist.barrier()
        dist.destroy_process_group()
        return
    models = sys.argv[1].split(",") if len(sys.argv) > 1 else ["gt"]
    first = trainer(models[0], fused=False)
    rank, world, dev = first.rank, first.sp_world, first.device
    # ---- (1) all-reduce ---------------------------------------------------------------------------
    sw = symm.get_world(first.sp_group, dev)
    buf = sw.alloc((1 << 20,), torch.float32)
    torch.manual_seed(100 + rank)
    buf.tensor.copy_(torch.randn(1 << 20, device=dev))
    ref = buf.tensor.clone()
    dist.all_reduce(ref)
    ref /= world
    class B: pass
    b = B(); b.symm = (sw, buf)
    symm.bucket_all_reduce_mean(b)
    torch.cuda.synchronize()
    err = float((buf.tensor - ref).abs().max())
    assert err < 1e-5, f"rank {rank}: all-reduce mismatch {err} (multimem={bool(buf.multicast_ptr)})"
    # ---- (2) fused vs portable ----------------------------------------------------------------------
    for m in models:
        a = first if m == models[0] else trainer(m, fused=False)
        f = trainer(m, fused=True)
        assert f.fused_sp and not a.fused_sp
        f.model.load_state_dict(a.model.state_dict())
        g = a.build_edges(1)
        la, oa = a._loss(g, a.local_idx["train"])
        lf, of = f._loss(g, f.local_idx["train"])
        assert torch.allclose(oa.float(), of.float(), atol=6e-2, rtol=6e-2), f"{m}: forward mismatch on rank {rank}"
        a.reducer.prepare_backward(); f.reducer.prepare_backward()
        la.backward(); lf.backward()
        a.reducer.finalize_backward(); f.reducer.finalize_backward()
        torch.cuda.synchronize()
        gemm.check_status(dev)
        # the all-reduce kernel also leaves the squared norm of the averaged gradients (one part per rank) everywhere
        norms = [getattr(b, "norm", None) for b in f.reducer.buckets]
        assert all(n is not None and n["ready"] for n in norms), "fused gradient norm missing"
        got = float(norms[0]["all"].double().sum())
        want = sum(float((b.flat.double() ** 2).sum()) for b in f.reducer.buckets)
        assert abs(got - want) <= 1e-4 * max(want, 1e-12), f"{m}: fused grad norm^2 {got} vs {want} on rank {rank}"
        gmax = max(float(p.grad.abs().max()) for p in a.model.parameters())
        nmax = max(float(p.grad.float().norm()) for p in a.model.parameters())
        for (na, pa), (_, pf) in zip(a.model.named_parameters(), f.model.named_parameters()):
            e = float((pa.grad - pf.grad).abs().max())
            assert e <= 0.12 * max(float(pa.grad.abs().max()), 1e-6) or e <= 5e-3 * gmax, \
                f"{m}: grad mismatch on {na} rank {rank}: {e} vs {float(pa.grad.abs().max())}"
            # both paths store bf16 activations: per tensor the difference, relative to the tensor's own norm, is a few
            # rounding steps (2^-8 each); tensors whose gradient is analytically ~0 are left to the check above
            norm = float(pa.grad.float().norm())
            if norm >= 1e-3 * nmax:
                rel = float((pa.grad.float() - pf.grad.float()).norm()) / norm
                assert rel < 0.08, f"{m}: relative gradient error {rel:.4f} on {na} rank {rank}"
        # ---- (3) a few fused steps ------------------------------------------------------------------
        losses = [f.train_step(e)["loss"] for e in range(1, 6)]
        gemm.check_status(dev)
        assert all(l == l for l in losses), losses
        if rank == 0:
            print(f"OK {m}: world={world} loss {float(la):.4f}/{float(lf):.4f} allreduce_err={err:.2e} "
                  f"multimem={bool(buf.multicast_ptr)} steps={['%.3f' % l for l in losses]}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    from budgetformer_b200.utils.rank_main import run_rank_main
    run_rank_main(main)
