"""Entry-point guard for one rank of a multi-process job.

A rank whose program raises must leave at once: the launcher (``torchrun``) ends the other ranks when it sees the exit
status.  Interpreter shutdown can instead wait for ever in the destructors of communicators and peer-memory mappings
whose owners never reached their collective teardown, so the traceback is printed and the process ends with
``os._exit``.  Single-process runs re-raise as usual."""
from __future__ import annotations

import os
import sys
import traceback


def run_rank_main(fn, *args, **kwargs):
    try:
        return fn(*args, **kwargs)
    except SystemExit:
        raise
    except BaseException:
        if int(os.environ.get("WORLD_SIZE", "1")) <= 1:
            raise
        traceback.print_exc()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(1)
