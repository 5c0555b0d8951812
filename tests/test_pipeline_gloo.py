"""The layer-split hand-off protocol on two CPU ranks (gloo): stage ranges from the layer allocation,
x passed rank to rank, the chosen token broadcast back.  The stage compute is a stand-in (the real one
needs a GPU); what is checked is that the two-rank pipeline computes the same function as one rank."""
import os
import socket

import numpy as np
import torch.distributed as dist
import torch.multiprocessing as mp

from llama2j_b200.layer_allocation import LayerAllocation
from llama2j_b200.model_files import ModelConfig
from llama2j_b200.pipeline import pipeline_greedy, stage_range

CFG = ModelConfig(dim=32, hidden_dim=64, n_layers=6, n_heads=4, n_kv_heads=4, vocab_size=50, seq_len=16)


def _layer(l, x, pos):
    """A deterministic stand-in for one transformer layer."""
    w = np.random.default_rng(100 + l).normal(0, 0.3, (CFG.dim, CFG.dim)).astype(np.float32)
    return np.tanh(w @ x + 0.01 * pos).astype(np.float32)


def _make_stage(first, last):
    emb = np.random.default_rng(1).normal(0, 1, (CFG.vocab_size, CFG.dim)).astype(np.float32)
    cls = np.random.default_rng(2).normal(0, 1, (CFG.vocab_size, CFG.dim)).astype(np.float32)

    def stage(token, pos, x_in):
        x = emb[token].copy() if first == 0 else np.asarray(x_in, dtype=np.float32)
        for l in range(first, last + 1):
            x = _layer(l, x, pos)
        if last == CFG.n_layers - 1:
            return int(np.argmax(cls @ x))
        return x
    return stage


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    alloc = LayerAllocation.equal_split(world, CFG)
    first, last = stage_range(alloc, rank)
    toks = pipeline_greedy(_make_stage(first, last), rank, world, [7, 9, 11], 12, CFG.dim)
    out[rank] = toks.tolist()
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_layer_split_equals_single_rank():
    single = []
    stage = _make_stage(0, CFG.n_layers - 1)
    token = 1
    prompt = [7, 9, 11]
    for pos in range(12):
        nxt = stage(token, pos, None)
        if pos < len(prompt):
            nxt = prompt[pos]
        single.append(nxt)
        token = nxt
    mgr = mp.Manager()
    out = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), out), nprocs=2, join=True)
    assert out[0] == single and out[1] == single


def test_stage_ranges_follow_the_layer_allocation():
    alloc = LayerAllocation.equal_split(3, CFG)
    assert [stage_range(alloc, r) for r in range(3)] == [(0, 1), (2, 3), (4, 5)]
