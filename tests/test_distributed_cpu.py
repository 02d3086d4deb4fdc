"""CPU, world_size 2 over gloo: the multi-GPU partitioning logic without a GPU.

Rank processes use the CPU oracle as the stand-in for the local CUDA SpMM; what is under
test is the sharding and the reassembly (row ranges with no collective, column slabs with
an all-gather), which is the same code the GPU ranks run.
"""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _oracle_spmm(values, row_indices, row_offsets, column_indices, dense, m):
    from oracle import oracle as orc
    out = orc.spmm(row_indices.numpy(), values.numpy(), row_offsets.numpy(), column_indices.numpy(),
                   dense.numpy(), m)[0]
    return torch.from_numpy(out)


def _worker(rank, world, port, results):
    sys.path.insert(0, REPO)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from intrasm_engine_b200 import synthetic as syn
        from intrasm_engine_b200.pytorch import distributed as D
        from intrasm_engine_b200.pytorch import utils as U

        # (1) row split, no collective: each rank computes its rows; rank 0 checks the union
        a, b = syn.spmm_fp32_case(7, 96, 80, 24, 0.2)
        v, ro, ci = (torch.from_numpy(x) for x in (a.values, a.row_offsets, a.column_indices))
        lv, lri, lro, lci, (beg, end) = D.shard_csr_rows(v, ro, ci, rank, world)
        local = _oracle_spmm(lv, lri, lro, lci, torch.from_numpy(b), end - beg)
        full = _oracle_spmm(v, torch.from_numpy(a.row_indices), ro, ci, torch.from_numpy(b), 96)
        ok_rows = torch.equal(local, full[beg:end])
        ranges = [None] * world
        dist.all_gather_object(ranges, (beg, end))  # test bookkeeping only, not the data path

        # (2) column-sharded down projection + all-gather
        act, w = syn.relu_ffn_layer_case(3, layer=1, tokens=16, k=64, n=32, density=0.3)
        av, ari, aro, aci = (torch.from_numpy(x) for x in
                             (act.values.astype(np.float32), act.row_indices, act.row_offsets,
                              act.column_indices))
        wt = torch.from_numpy(w.astype(np.float32))
        layer = D.ColumnShardedDownProj(wt, rank, world, _oracle_spmm)
        out = layer(av, ari, aro, aci, 16)
        ref = _oracle_spmm(av, ari, aro, aci, wt, 16)
        ok_cols = torch.equal(out, ref) and out.shape == (16, 32)
        results[rank] = (ok_rows, ok_cols, ranges)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_row_split_and_column_allgather_gloo(world):
    mgr = mp.Manager()
    results = mgr.dict()
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(world, port, results), nprocs=world, join=True)
    assert len(results) == world
    for rank in range(world):
        ok_rows, ok_cols, ranges = results[rank]
        assert ok_rows and ok_cols
        assert ranges[0][0] == 0 and ranges[-1][1] == 96
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))


def test_all_gather_columns_single_rank():
    from intrasm_engine_b200.pytorch import distributed as D
    w = torch.arange(24.0).reshape(4, 6)
    assert torch.equal(D.column_slab(w, 1, 3), w[:, 2:4])
