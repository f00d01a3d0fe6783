"""Tensor parallelism on 2 GPUs: each rank holds its row/column shard of the same seeded model, two
all-reduces per layer and one arg-max all-gather per step; the result must match the single-GPU run."""
import os
import subprocess
import sys
import tempfile

import numpy as np
import pytest

from conftest import rel_err_ok

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


def run_world(world: int, d_model: int, extra_env: dict | None = None) -> dict:
    work = tempfile.mkdtemp(prefix=f"tp{world}_")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", **(extra_env or {}))
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py"), str(r), str(world), work, str(d_model)], env=env,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            for q in procs:
                q.kill()
            raise
        outs.append(out)
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{outs[r][-3000:]}"
    return dict(np.load(os.path.join(work, "out.npz")))


def check_against_single(one: dict, many: dict, what: str) -> None:
    # same seeded tensors, sharded: logits agree to fp32 summation order (K-shards quantize their slice
    # of the activation exactly as the unsharded kernel does), tokens identical unless a near tie
    rel_err_ok(many["logits0"], one["logits0"], 2e-3)
    assert list(many["firsts"]) == list(one["firsts"]), what
    if not np.array_equal(many["toks"], one["toks"]):
        lg = one["logits"]
        srt = np.sort(lg, axis=1)
        margin = float(((srt[:, -1] - srt[:, -2]) / np.sqrt((lg ** 2).mean(axis=1))).min())
        assert margin < 0.05, f"{what}: tokens differ without a near tie (margin {margin:.3f})"


_single = {}


def single(d_model: int) -> dict:
    if d_model not in _single:
        _single[d_model] = run_world(1, d_model)
    return _single[d_model]


# d_model 1024: group sums by the plain peer-memory all-reduce, norm separately. d_model 4096 (two CTAs per row in one
# cluster): by default the row-parallel matvecs store their partial rows into the peers' inboxes from their own epilogue
# and a gather kernel sums + normalises + quantizes; SKAINET_TP_FUSE=1 keeps the exchange inside that kernel (what rows of
# a batch or of a prompt use), =0 separates sum and norm, SKAINET_TP_ALLREDUCE=nccl takes every sum through NCCL.
@pytest.mark.parametrize("d_model,env", [(1024, {}), (4096, {}), (4096, {"SKAINET_TP_FUSE": "1"}), (4096, {"SKAINET_TP_FUSE": "0"}),
                                         (4096, {"SKAINET_TP_ALLREDUCE": "nccl"})])
def test_tp2_matches_single_gpu(gpu, d_model, env):
    if gpu.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    check_against_single(single(d_model), run_world(2, d_model, env), f"TP2 {env}")


def test_tp2_exchange_timing_entry_leaves_the_group_consistent(gpu):
    """skainet_cuda_llama_tp_exchange_time (what the bench's tp_collective workload and `tp_exchange` key call) returns a
    positive device time for the peer-memory sum, the fused store + gather + norm + quantize kernel and the NCCL sum, and a
    decode after those exchange rounds still matches the single-GPU run."""
    if gpu.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    out = run_world(2, 4096, {"SKAINET_TEST_EXCHANGE": "1"})
    assert (out["exchange_us"] > 0).all() and (out["exchange_us"] < 1e4).all(), out["exchange_us"]
    check_against_single(single(4096), out, "TP2 after exchange timing")


def test_tp4_matches_single_gpu(gpu):
    if gpu.device_count() < 4:
        pytest.skip("needs 4 GPUs")
    check_against_single(single(4096), run_world(4, 4096), "TP4")


def test_two_models_on_two_gpus_from_one_thread(gpu, cuda_lib):
    """One host thread drives a model on each of two GPUs: every call must use the flag, the SM count and the scratch of
    the device its kernels run on. Same seed, same prompt: both models give the same tokens, and neither device reports
    a bounded wait that gave up."""
    if gpu.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    from skainet_b200.llama import Llama, LlamaConfig
    models = []
    for dev in (0, 1):
        gpu.set_device(dev)
        m = Llama(LlamaConfig(2, 512, 8, 4, 64, 1024, 1000, max_seq=64))
        m.synth(seed=9, std=0.05); m.finalize()
        models.append(m)
    outs = []
    for rounds in range(2):                      # interleave the two devices
        for m in models:
            if rounds == 0:
                outs.append([m.prefill([3, 1, 4, 1, 5])])
            else:
                outs[models.index(m)] += [int(t) for t in m.generate([outs[models.index(m)][0]], 6)[:, 0]]
    assert outs[0] == outs[1]
    for dev in (0, 1):
        gpu.set_device(dev)
        assert cuda_lib.skainet_cuda_device_status() == 0
    for m in models:
        m.free()
    gpu.set_device(0)
