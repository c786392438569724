"""The N > 1 path on CPU: two gloo ranks each run their shard of the sessions (the CPU oracle
stands in for the GPU engine here) and the gathered token ids equal a single process running all
sessions in one packed step. No collective touches the data path; only ids are gathered."""
import os
import sys

import numpy as np
import pytest
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, out):
    sys.path.insert(0, ROOT); sys.path.insert(0, os.path.join(ROOT, "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="2")
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import splosh_b200 as S
    from splosh_b200 import sharding
    from helpers import Pair, tokens_for
    from oracle import oracle as O
    g = S.Geometry(4, 256, 512, 2048, 4, 2, 128, 32, 2, 4, 128, 1e-6, 1e7)
    toks = tokens_for(0xC0FFEE00, 1024, 2048)
    sessions = list(range(4))
    mine = sharding.assign_sessions(sessions, world)[rank]
    pair = Pair(g, S.EngineConfig(max_slots=4, max_rows=64, kv_pages=8, max_context=512), gpu=False)
    rows = []
    for sid in mine:
        slot = sharding.local_slot(sid, world)
        rows += [S.EngineRow(slot, toks[100 * sid + i], i, i == 9 + sid) for i in range(10 + sid)]
    _, logits = pair.step(rows)
    ids = O.argmax(logits, 2048)
    gathered = sharding.gather_ids([(sid, int(ids[i])) for i, sid in enumerate(mine)], dist)
    dist.barrier()
    if rank == 0:
        out.put(gathered)
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_process_tokens():
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import splosh_b200 as S
    from splosh_b200 import sharding
    from helpers import Pair, tokens_for
    from oracle import oracle as O
    assert sharding.assign_sessions(list(range(5)), 2) == [[0, 2, 4], [1, 3]]
    g = S.Geometry(4, 256, 512, 2048, 4, 2, 128, 32, 2, 4, 128, 1e-6, 1e7)
    toks = tokens_for(0xC0FFEE00, 1024, 2048)
    pair = Pair(g, S.EngineConfig(max_slots=4, max_rows=64, kv_pages=8, max_context=512), gpu=False)
    rows = []
    for sid in range(4):
        rows += [S.EngineRow(sid, toks[100 * sid + i], i, i == 9 + sid) for i in range(10 + sid)]
    _, logits = pair.step(rows)
    single = [(sid, int(t)) for sid, t in enumerate(O.argmax(logits, 2048))]
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    gathered = out.get(timeout=180)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert gathered == single
