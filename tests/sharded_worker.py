"""Worker of tests/test_gpu_sharded_nccl.py: one process per GPU (RANK / WORLD_SIZE / LOCAL_RANK from the
launcher).  Every rank builds the same IVF-SQ8 model, keeps the lists it owns, and runs the library's own
sharded step (vb200_ivf_search_sharded / vb200_bf_search_sharded over a vb200_comm); the result on every
rank must be the unsharded index's, bit for bit.  Exit code 0 = all checks passed on this rank."""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def main() -> int:
    from conftest import mixture

    from vsag_b200 import engine, parallel

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    comm = parallel.Comm(dist, rank, world, device)
    assert (comm.rank, comm.world) == (rank, world)

    # ---- IVF-SQ8, lists dealt round-robin ----
    n, dim, nlist, nq, k, nprobe = 120_000, 32, 256, 1003, 10, 16
    base = mixture(21, n, dim, 300, 0.15)
    queries = mixture(22, nq, dim, 300, 0.15)
    ids = np.arange(n, dtype=np.int64) * 7 + 3
    whole = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    whole.train(base[:40_000], iters=4, init=base[:nlist].copy())
    whole.add(base, ids)
    shard = engine.IvfHandle(dim, engine.METRIC_L2, nlist, engine.QUANT_SQ8)
    shard.set_shard(rank, world)
    shard.set_centroids(whole.get_centroids())
    shard.set_sq8_model(*whole.get_sq8_model())
    shard.add(base, ids)
    want_i, want_d = whole.search(queries, k, nprobe)
    for q_in in (queries, torch.from_numpy(queries).to(device)):
        got_i, got_d = shard.search_sharded(comm, q_in, k, nprobe)
        if torch.is_tensor(got_i):
            got_i, got_d = got_i.cpu().numpy(), got_d.cpu().numpy()
        assert np.array_equal(got_d, want_d), "sharded IVF distances differ from the unsharded index"
        assert np.array_equal(got_i, want_i), "sharded IVF ids differ from the unsharded index"
    # without list pruning the exchange of bounds is the only pruning left: same result again
    shard.set_list_pruning(False)
    got_i, got_d = shard.search_sharded(comm, queries, k, nprobe)
    assert np.array_equal(got_d, want_d) and np.array_equal(got_i, want_i)
    # a batch smaller than the world, and a mismatch between shard and communicator
    got_i, got_d = shard.search_sharded(comm, queries[:1], k, nprobe)
    assert np.array_equal(got_d, want_d[:1]) and np.array_equal(got_i, want_i[:1])
    try:
        whole.search_sharded(comm, queries, k, nprobe)
        raise AssertionError("an unsharded index was accepted by the sharded step")
    except engine.VsagB200Error as err:
        assert "communicator" in str(err)

    # ---- BruteForce, rows dealt as contiguous ranges ----
    nb, kb = 50_000, 20
    bf_whole = engine.BfHandle(dim, engine.METRIC_L2, engine.QUANT_FP32)
    bf_whole.add(base[:nb], ids[:nb])
    lo, hi = parallel.row_range(nb, rank, world)
    bf_shard = engine.BfHandle(dim, engine.METRIC_L2, engine.QUANT_FP32)
    bf_shard.add(base[lo:hi], ids[lo:hi])
    want_i, want_d = bf_whole.search(queries, kb)
    got_i, got_d = bf_shard.search_sharded(comm, queries, kb)
    assert np.array_equal(got_d, want_d), "sharded BruteForce distances differ"
    assert np.array_equal(got_i, want_i), "sharded BruteForce ids differ"

    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print(f"rank {rank}: sharded searches equal the unsharded ones", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
