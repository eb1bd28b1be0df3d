"""Full-graph sequence-parallel Graph Transformer training on B200.

    torchrun --standalone --nproc_per_node=P main_node_fullgraph_sp.py --model gt --dataset <name> ...

Accepts the command-line surface of the reference driver of the same name
(main_node_fullgraph_sp.py:184-1911 there); see ``budgetformer_b200/config.py`` for the flags."""
import sys

from budgetformer_b200.config import parse_fullgraph_args
from budgetformer_b200.parallel.initialize import destroy_distributed
from budgetformer_b200.train.engine import FullGraphTrainer
from budgetformer_b200.train.report import print_git_version
from budgetformer_b200.utils.rank_main import run_rank_main


def main(argv=None):
    args = parse_fullgraph_args(argv)
    trainer = FullGraphTrainer(args)
    if trainer.rank == 0:
        print_git_version(print)
    try:
        best = trainer.fit()
    finally:
        trainer.edge_engine.shutdown()
    destroy_distributed()                        # collective: only after a run that every rank finished
    return best


def cli() -> int:
    """Console-script entry point (the return value of ``main`` is a result dict, not an exit status)."""
    run_rank_main(main, sys.argv[1:])
    return 0


if __name__ == "__main__":
    run_rank_main(main, sys.argv[1:])
