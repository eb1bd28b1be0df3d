"""Mini-batch sequence-parallel training (legacy mode): sequences of ``--seq_len`` nodes, Graphormer / GT.

    torchrun --standalone --nproc_per_node=P main_node_sp.py --model gt --dataset <name> --seq_len 4096 ...

Counterpart of the reference's ``main_node_sp.py`` (:370-647): per-epoch shuffle of the training nodes, one
optimizer step per sequence, gradient averaging over the SP group, periodic validation / test with the
sparse evaluator, best-by-validation checkpoint ``<model_dir>/<dataset>.pkl``."""
import os
import sys
import time

import torch
import torch.nn.functional as F

from budgetformer_b200.config import build_batch_parser, normalize_main_node_sp_args
from budgetformer_b200.graph.attn_graph import Topology
from budgetformer_b200.parallel.initialize import (destroy_distributed, get_sequence_parallel_group, get_sequence_parallel_rank,
                                                   get_sequence_parallel_world_size, initialize_distributed)
from budgetformer_b200.parallel.reducer import build_gradient_reducer, sync_params_and_buffers
from budgetformer_b200.train.data import load_data
from budgetformer_b200.train.engine import build_model
from budgetformer_b200.train.legacy_batch import get_batch_blockize
from budgetformer_b200.train.legacy_eval import collect_hop_stats, sparse_eval_gpu
from budgetformer_b200.utils.lr import PolynomialDecayLR
from budgetformer_b200.utils.misc import autocast_context, resolve_amp_dtype, set_seed


def main(argv=None):
    args = normalize_main_node_sp_args(build_batch_parser().parse_args(argv))
    if args.model not in ("graphormer", "gt"):
        raise SystemExit("main_node_sp.py supports --model graphormer|gt")
    if args.model != "graphormer":
        args.num_global_node = 0
    initialize_distributed(args)
    device = torch.device(args.device)
    rank, p, r = args.rank, get_sequence_parallel_world_size(), get_sequence_parallel_rank()
    set_seed(args.seed)
    data = load_data(args)
    n = data.num_nodes
    if getattr(args, "attn_bias_mode", "none") == "local_spd":
        args.attn_bias_dim = int(args.attn_bias_max_dist) + 1
    topo = Topology.from_edge_index(data.edge_index, n) if args.batch_subgraph_mode == "seed_rw" else None
    model = build_model(args, int(data.x.size(1)), data.output_dim).to(device)
    sync_params_and_buffers(model, get_sequence_parallel_group())
    reducer = build_gradient_reducer(model, get_sequence_parallel_group(), 25.0, p)
    opt = torch.optim.AdamW(model.parameters(), lr=args.peak_lr, weight_decay=args.weight_decay)
    sched = PolynomialDecayLR(opt, warmup=args.warmup_updates, tot=args.epochs, lr=args.peak_lr, end_lr=args.end_lr, power=1.0)
    amp = resolve_amp_dtype(getattr(args, "amp_dtype", "none"), device)
    seed_bs = int(args.seed_batch_size or args.seq_len)
    train_idx = data.split_idx["train"]
    best = {"valid": 0.0, "test": 0.0, "epoch": -1}
    times = []
    for epoch in range(1, args.epochs + 1):
        t0 = time.time()
        model.train()
        g = torch.Generator().manual_seed(args.seed + epoch)
        losses = []
        for batch in torch.split(train_idx[torch.randperm(train_idx.numel(), generator=g)], seed_bs):
            x_i, y_i, graph, bias, ok = get_batch_blockize(args, data.x, data.y, batch, data.edge_index, n, r, p, topo=topo,
                                                           epoch_seed=args.seed + epoch)
            with autocast_context(device, amp):
                out = model(x_i.to(device), None if bias is None else bias.to(device), graph.to(device), attn_type=args.attn_type)
            m = (ok & (y_i >= 0)).to(device)
            loss = F.nll_loss(out[m].float(), y_i.to(device)[m]) if bool(m.any()) else out.sum() * 0
            reducer.prepare_backward()
            loss.backward()
            reducer.finalize_backward()
            opt.step()
            losses.append(float(loss.detach()))
        sched.step()
        times.append(time.time() - t0)
        if rank == 0:
            print(f"Epoch {epoch:04d} | loss={sum(losses) / max(1, len(losses)):.4f} | t={times[-1]:.2f}s", flush=True)
        if epoch % max(1, int(args.eval_every)) == 0 or epoch == args.epochs:
            val = sparse_eval_gpu(args, model, data.x, data.y, data.split_idx["valid"], data.edge_index, n, device, topo)
            test = sparse_eval_gpu(args, model, data.x, data.y, data.split_idx["test"], data.edge_index, n, device, topo)
            if getattr(args, "full_attn_hop_stats", False):
                path = collect_hop_stats(args, model, data.x, data.y, data.split_idx["valid"], data.edge_index, n, device,
                                         epoch, topo)
                if rank == 0 and path:
                    print(f"[hop_stats] wrote {path}", flush=True)
            if rank == 0:
                print(f"  eval epoch {epoch:04d} | valid={val:.4f} test={test:.4f}", flush=True)
                if val > best["valid"]:
                    best = {"valid": val, "test": test, "epoch": epoch}
                    if args.save_model:
                        os.makedirs(args.model_dir, exist_ok=True)
                        torch.save(model.state_dict(), os.path.join(args.model_dir, f"{args.dataset}.pkl"))
    if rank == 0:
        print(f"Best by validation: epoch={best['epoch']} valid={best['valid']:.4f} test={best['test']:.4f} | "
              f"avg epoch {sum(times[1:] or times) / max(1, len(times[1:] or times)):.2f}s")
    destroy_distributed()
    return best


def cli() -> int:
    """Console-script entry point (the return value of ``main`` is a result dict, not an exit status)."""
    main(sys.argv[1:])
    return 0


if __name__ == "__main__":
    main(sys.argv[1:])
