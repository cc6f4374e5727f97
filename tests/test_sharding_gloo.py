"""The multi-GPU host path on CPU: two gloo ranks shard a jagged batch by token-balanced sequence
ranges, each computes its shard (the oracle stands in for the CUDA operator, which has no CPU path),
the outputs are gathered for validation and must equal the unsharded result; the step time is
reduced with MAX over the ranks."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gdpa_oracle as orc


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ads_model_kernel_library_b200.gdpa.sharding import gather_rows, max_over_ranks, shard_inputs

        rng = np.random.default_rng(0)
        lq, lk = rng.integers(1, 60, 11), rng.integers(1, 80, 11)
        qo = torch.tensor(np.concatenate([[0], np.cumsum(lq)]))
        ko = torch.tensor(np.concatenate([[0], np.cumsum(lk)]))
        g = torch.Generator().manual_seed(0)
        q = torch.randn(int(qo[-1]), 2, 16, generator=g)
        k = torch.randn(int(ko[-1]), 2, 16, generator=g)
        v = torch.randn(int(ko[-1]), 2, 16, generator=g)
        q_r, k_r, v_r, qo_r, ko_r, seqs, rows = shard_inputs(q, k, v, qo, ko, rank, world)
        assert int(qo_r[0]) == 0 and int(ko_r[0]) == 0 and int(qo_r[-1]) == q_r.shape[0]
        o_r = orc.gdpa_forward(q_r, k_r, v_r, qo_r, ko_r, "gelu_approx", 0.1)
        o_all = gather_rows(o_r)
        t = max_over_ranks(float(rank + 1), torch.device("cpu"))
        if rank == 0:
            full = orc.gdpa_forward(q, k, v, qo, ko, "gelu_approx", 0.1)
            ret["max_err"] = float((o_all - full).abs().max())
            ret["shape_ok"] = o_all.shape == full.shape
            ret["tmax"] = t
    finally:
        dist.destroy_process_group()


def test_two_rank_sharded_forward_equals_unsharded():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert ret["shape_ok"]
    assert ret["max_err"] < 1e-6
    assert ret["tmax"] == 2.0
