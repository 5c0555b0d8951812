"""Layer split over several GPUs, one process per GPU: the reference's multi-GPU mode.

In the reference one Java thread walks the devices in order and carries the activation vector x from
one device to the next through a host array (Run.java:368-413, ContextCUDA.java:269-280).  Here every
rank owns one stage (a contiguous layer range from LayerAllocation) and the hand-off is a
point-to-point send/recv of `dim` floats between neighbouring ranks; the last rank owns the
classifier and sends the chosen token back to rank 0.  No collective is involved.

The per-stage compute is passed in as a callable so that the hand-off protocol can be tested on CPU
ranks (gloo) without a GPU; on GPUs the callable is `Transformer.forward_stage`.
"""
from __future__ import annotations

from typing import Callable, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist

from .layer_allocation import LayerAllocation


def stage_range(alloc: LayerAllocation, rank: int):
    """(first_layer, last_layer) of the stage a rank owns."""
    if not alloc.covers_model():
        raise ValueError("the layer allocation does not tile the model")
    if rank < 0 or rank >= alloc.device_count:
        raise ValueError(f"rank {rank} outside the {alloc.device_count} devices of the allocation")
    return alloc.first_layer[rank], alloc.last_layer[rank]


def pipeline_step(stage_fn: Callable, rank: int, world: int, token: int, pos: int, dim: int,
                  device: str = "cpu", group=None) -> Optional[int]:
    """One token through all stages.  `stage_fn(token, pos, x_in)` returns x (ndarray of `dim` floats) on a
    stage that is not the last and the chosen token (int) on the last one.  Returns the chosen token on
    every rank (the last rank broadcasts it the way the reference's host loop sees the logits)."""
    x_in = None
    if rank > 0:
        buf = torch.empty(dim, dtype=torch.float32, device=device)
        dist.recv(buf, src=rank - 1, group=group)
        x_in = buf.cpu().numpy()
    out = stage_fn(token if rank == 0 else 0, pos, x_in)
    if rank < world - 1:
        x = torch.from_numpy(np.ascontiguousarray(out, dtype=np.float32)).to(device)
        if x.numel() != dim:
            raise ValueError(f"stage returned {x.numel()} floats, expected {dim}")
        dist.send(x, dst=rank + 1, group=group)
    nxt = torch.zeros(1, dtype=torch.int64, device=device)
    if rank == world - 1:
        nxt[0] = int(out)
    if world > 1:
        dist.broadcast(nxt, src=world - 1, group=group)
    return int(nxt.item())


def pipeline_greedy(stage_fn: Callable, rank: int, world: int, prompt: Sequence[int], steps: int, dim: int,
                    device: str = "cpu", group=None) -> np.ndarray:
    """The token loop of Run.java:609-685 (greedy) over a layer split: BOS first, forced prompt tokens,
    then the arg-max of the last stage.  Every rank returns the same sequence."""
    token, chosen = 1, []
    prompt = [int(t) for t in prompt]
    for pos in range(steps):
        nxt = pipeline_step(stage_fn, rank, world, token, pos, dim, device, group)
        if pos < len(prompt):
            nxt = prompt[pos]
        chosen.append(nxt)
        token = nxt
    return np.asarray(chosen, dtype=np.int32)
