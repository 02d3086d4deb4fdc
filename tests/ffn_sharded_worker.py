"""One rank of the column-sharded ReLU-sparse FFN down projection check; launched by
test_ffn_sharded_gpu.py under ``python -m torch.distributed.run --nproc-per-node G``.
Every rank runs the benchmark-shaped layer (256 tokens, 11008 -> 4096) on its weight slab with
both gather methods (the kernel's peer stores, NCCL all-gather) and compares the gathered
result with torch.sparse.mm on CPU.  Prints FFN_SHARDED_OK on success."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

REPO = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, REPO)


def main() -> int:
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    from intrasm_engine_b200 import _lib, synthetic as syn
    from intrasm_engine_b200.pytorch.ffn import ReluSparseDownProj
    from oracle import oracle

    tokens, k, n = 256, 11008, 4096
    n_local = n // world
    bad = 0
    layers = {g: ReluSparseDownProj(tokens, k, n, rank, world, dev, gather=g) for g in ("peer", "nccl")}
    for layer_idx in range(3):
        a, w = syn.relu_ffn_layer_case(0, layer_idx, tokens, k, n)
        up = lambda z: torch.as_tensor(np.ascontiguousarray(z)).to(dev)
        vals, ro, ci = up(a.values), up(a.row_offsets), up(a.column_indices)
        slab = up(w[:, rank * n_local:(rank + 1) * n_local].T)
        ref = oracle.torch_spmm(a.row_offsets, a.column_indices, a.values, w, tokens)
        sabs = oracle.torch_spmm(a.row_offsets, a.column_indices, np.abs(a.values), np.abs(w), tokens)
        bound = 2.0 ** -10 * np.abs(ref) + 1e-5 * sabs + 1e-7
        outs = {}
        for g, layer in layers.items():
            outs[g] = layer(vals, ro, ci, slab).clone()
            torch.cuda.synchronize()
            if not np.all(np.abs(outs[g].float().cpu().numpy().astype(np.float64) - ref) <= bound):
                bad += 1
        if not torch.equal(outs["peer"], outs["nccl"]):  # same kernels, same part order
            bad += 1
    status = _lib.lib.iex_last_device_status(1)
    flag = torch.tensor([bad + (1 if status != 0 else 0)], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("FFN_SHARDED_OK" if int(flag.item()) == 0 else f"FFN_SHARDED_FAILED bad={int(flag.item())} status={status}",
              flush=True)
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
