"""One rank of the peer-store all-gather check; launched by test_peer_gather_gpu.py under
``python -m torch.distributed.run --nproc-per-node G`` (one process per GPU, NCCL for the
rendezvous only).  Every rank multiplies a replicated activation with its column slab of a
replicated weight through ``iex_linear_f16_splitk_gather`` + ``iex_peer_barrier`` and
compares the gathered result with the CPU oracle.  Prints PEER_GATHER_OK on success."""
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
    from intrasm_engine_b200 import _lib
    from intrasm_engine_b200.pytorch.distributed import PeerGather
    from oracle import oracle

    tokens, k, n = 64, 1024, 1024
    n_local = n // world
    rng = np.random.default_rng(7)
    layers = 5
    acts = [(rng.standard_normal((tokens, k)) * 0.5).astype(np.float16) for _ in range(layers)]
    w = (rng.standard_normal((n, k)) * 0.05).astype(np.float16)          # [out, in], replicated
    slab = torch.as_tensor(w[rank * n_local:(rank + 1) * n_local]).to(dev).contiguous()
    pg = PeerGather(tokens, n, rank, world, dev)
    st = torch.cuda.current_stream().cuda_stream
    bad = 0
    for parts in (1, 4):
        need = _lib.lib.iex_tc_workspace_bytes(0, 1, n_local, parts, tokens)
        ws = torch.empty(max(need, 256), dtype=torch.uint8, device=dev)
        got = []
        for layer in range(layers):
            x = torch.as_tensor(acts[layer]).to(dev)
            pg.linear(layer % 2, x, slab, parts, ws, st)
            pg.barrier(st)
            got.append(pg.result(layer % 2).clone())  # stream-ordered after the barrier
        torch.cuda.synchronize()
        for layer in range(layers):
            ref = oracle.linear(acts[layer].astype(np.float32), w.astype(np.float32))
            g = got[layer].float().cpu().numpy().astype(np.float64)
            # fp16 in / fp32 accumulate against the fp32 oracle: the final fp16 rounding plus
            # 1e-5 of the sum of the terms' magnitudes (far inside the 1e-2 relative bar)
            sabs = np.abs(acts[layer].astype(np.float32)) @ np.abs(w.astype(np.float32)).T
            bound = 2.0 ** -10 * np.abs(ref) + 1e-5 * sabs + 1e-7
            if not np.all(np.abs(g - ref) <= bound):
                bad += 1
    status = _lib.lib.iex_last_device_status(1)
    flag = torch.tensor([bad + (1 if status != 0 else 0)], device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print("PEER_GATHER_OK" if int(flag.item()) == 0 else f"PEER_GATHER_FAILED bad={int(flag.item())} status={status}",
              flush=True)
    dist.destroy_process_group()
    return 0 if int(flag.item()) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
