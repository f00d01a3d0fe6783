"""One tensor-parallel rank of the decoder (run as a child process by tests/test_gpu_tp.py).

    python tests/tp_worker.py RANK WORLD WORKDIR [D_MODEL]

Builds this rank's shard of a seeded small model, joins the TP group (rank 0 writes the NCCL unique id
to WORKDIR/id.bin), prefills a prompt, generates greedily, and rank 0 writes tokens + logits to WORKDIR/out.npz.
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank, world, work = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    from skainet_b200 import device
    from skainet_b200.llama import Llama, LlamaConfig
    device.set_device(rank if device.device_count() > rank else 0)
    d_model = int(sys.argv[4]) if len(sys.argv) > 4 else 1024
    cfg = LlamaConfig(2, d_model, 16, 4, 64, 2048, 1000, max_seq=64, max_batch=2, tp_rank=rank, tp_world=world)
    m = Llama(cfg)
    m.synth(seed=77, std=0.05)
    m.finalize()
    if world > 1:
        idf = os.path.join(work, "id.bin")
        if rank == 0:
            uid = Llama.tp_unique_id()
            with open(idf + ".tmp", "wb") as f:
                f.write(uid)
            os.rename(idf + ".tmp", idf)
        else:
            t0 = time.time()
            while not os.path.exists(idf):
                if time.time() - t0 > 120:
                    raise TimeoutError("rank 0 never published the unique id")
                time.sleep(0.05)
            uid = open(idf, "rb").read()
        m.tp_init(uid)
    # The exchange timing entry runs real exchange rounds on both inbox channels: the decode that follows must be unaffected.
    xt = np.zeros(3, np.float32)
    if world > 1 and os.environ.get("SKAINET_TEST_EXCHANGE") == "1":
        xt = np.array([m.tp_exchange_time(mode, 7, 3) for mode in (0, 1, 2)], np.float32)
    prompts = [[5, 17, 900, 33, 2, 640], [7, 7, 123]]
    firsts = [m.prefill(p, seq=i) for i, p in enumerate(prompts)]
    logits0 = m.logits(1)
    toks = m.generate(firsts, 6)
    logits = m.logits(2)
    if rank == 0:
        np.savez(os.path.join(work, "out.npz"), firsts=np.array(firsts), toks=toks, logits=logits, logits0=logits0, exchange_us=xt)
    m.free()


if __name__ == "__main__":
    main()
