"""Host-side tensor-parallel shard planner: which slice of a canonical packed [out, in] tensor a rank
holds, matching the shapes the decoder runtime expects (skainet_cuda_llama.h). Rows split on row
boundaries; columns split on whole blocks, which is also the granule of the reference's activation
quantizer (native/src/q4k_matmul.c:334-337), so a column shard quantizes its slice of the activation
exactly as the unsharded kernel would."""
from __future__ import annotations

import numpy as np

from ._lib import BLOCK_BYTES, BLOCK_ELEMS

ROW_SPLIT = ("q", "k", "v", "gate", "up", "head")     # column-parallel linears: output rows are sharded
COL_SPLIT = ("o", "down")                             # row-parallel linears: the contraction is sharded
REPLICATED = ("embed",)


def shard_shape(name: str, rows: int, cols: int, world: int) -> tuple[int, int]:
    if name in ROW_SPLIT:
        if rows % world:
            raise ValueError(f"{name}: {rows} rows do not divide by {world}")
        return rows // world, cols
    if name in COL_SPLIT:
        if cols % world:
            raise ValueError(f"{name}: {cols} columns do not divide by {world}")
        return rows, cols // world
    return rows, cols


def shard_packed(name: str, packed: np.ndarray, encoding: str, rows: int, cols: int, rank: int, world: int) -> np.ndarray:
    """The bytes of `rank`'s shard of a canonical row-major packed tensor."""
    bb, be = BLOCK_BYTES[encoding], BLOCK_ELEMS[encoding]
    bpr = cols // be
    blocks = np.ascontiguousarray(packed, dtype=np.uint8).reshape(rows, bpr, bb)
    if name in ROW_SPLIT:
        r, _ = shard_shape(name, rows, cols, world)
        return np.ascontiguousarray(blocks[rank * r:(rank + 1) * r]).reshape(-1)
    if name in COL_SPLIT:
        _, c = shard_shape(name, rows, cols, world)
        if c % be:
            raise ValueError(f"{name}: a shard of {c} columns is not a whole number of {be}-element blocks")
        b = c // be
        return np.ascontiguousarray(blocks[:, rank * b:(rank + 1) * b]).reshape(-1)
    return blocks.reshape(-1)
