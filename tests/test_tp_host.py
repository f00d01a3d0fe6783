"""CPU, world size 2 over gloo: the tensor-parallel decomposition the runtime uses — row-split
projections concatenated, column-split projections summed with rank 0 carrying the residual — gives the
unsharded reference result when every rank runs the reference operator on its shard."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank: int, world: int, port: int, out_dir: str):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from oracle import ref as R
    from skainet_b200 import tp
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    rng = np.random.default_rng(42)                       # same seed on every rank: same full tensors
    d, f = 512, 1024
    w_up = R.quantize_q4k((0.05 * rng.standard_normal((f, d))).astype(np.float32))      # row split
    w_down = R.quantize_q4k((0.05 * rng.standard_normal((d, f))).astype(np.float32))    # column split
    x = rng.standard_normal(d).astype(np.float32)
    resid = rng.standard_normal(d).astype(np.float32)
    # column-parallel: each rank computes its rows; all-gather = the full vector
    r_up, c_up = tp.shard_shape("up", f, d, world)
    h_part = R.matmul("Q4_K", x, tp.shard_packed("up", w_up, "Q4_K", f, d, rank, world), c_up, r_up, "rm")
    parts = [torch.zeros(r_up) for _ in range(world)]
    dist.all_gather(parts, torch.from_numpy(h_part))
    h = torch.cat(parts).numpy()
    # row-parallel: each rank contracts its column slice of h; rank 0 adds the residual; all-reduce sums
    r_dn, c_dn = tp.shard_shape("down", d, f, world)
    y_part = R.matmul("Q4_K", h[rank * c_dn:(rank + 1) * c_dn].copy(), tp.shard_packed("down", w_down, "Q4_K", d, f, rank, world), c_dn, r_dn, "rm")
    if rank == 0:
        y_part = y_part + resid
    y = torch.from_numpy(y_part.copy())
    dist.all_reduce(y)
    if rank == 0:
        h_full = R.matmul("Q4_K", x, w_up, d, f, "rm")
        y_full = resid + R.matmul("Q4_K", h_full, w_down, f, d, "rm")
        np.savez(os.path.join(out_dir, "out.npz"), h=h, h_full=h_full, y=y.numpy(), y_full=y_full)
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_decomposition_matches_unsharded_reference(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + os.getpid() % 2000
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    r = np.load(tmp_path / "out.npz")
    np.testing.assert_array_equal(r["h"], r["h_full"])                  # rows are independent: bit-identical
    # K shards quantize their activation slice identically; only the fp32 order of the block sum differs
    np.testing.assert_allclose(r["y"], r["y_full"], rtol=0, atol=1e-5 * float(np.abs(r["y_full"]).max()))


def test_shard_planner_shapes_and_errors():
    sys.path.insert(0, ROOT)
    from skainet_b200 import tp
    assert tp.shard_shape("q", 8192, 8192, 8) == (1024, 8192)
    assert tp.shard_shape("down", 8192, 28672, 8) == (8192, 3584)       # 14 blocks of 256 per rank
    assert tp.shard_shape("embed", 128256, 8192, 8) == (128256, 8192)
    with pytest.raises(ValueError):
        tp.shard_shape("k", 1000, 512, 3)
    packed = np.arange(4 * 2 * 144, dtype=np.uint8 if False else np.int64).astype(np.uint8)
    with pytest.raises(ValueError, match="whole number"):
        tp.shard_packed("o", np.zeros(4 * 3 * 144, np.uint8), "Q4_K", 4, 768, 0, 2)
    full = np.random.default_rng(0).integers(0, 256, 4 * 2 * 144, dtype=np.uint8)
    a, b = (tp.shard_packed("o", full, "Q4_K", 4, 512, r, 2) for r in (0, 1))
    assert np.array_equal(np.concatenate([a.reshape(4, 1, 144), b.reshape(4, 1, 144)], axis=1).reshape(-1), full)
