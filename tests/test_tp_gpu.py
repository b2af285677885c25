"""Tensor parallelism on two GPUs: the sharded executor (NCCL all-reduce and all-gather
captured in the step graph) produces the single-GPU greedy ids."""

from __future__ import annotations

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank: int, world: int, port: int, out_dir: str) -> None:
    import datetime
    import faulthandler

    import torch.distributed as dist

    # a rank that stops making progress dumps its stack and exits instead of holding the box
    faulthandler.dump_traceback_later(240, exit=True)
    from gpu.decodev2 import (MEDIUM_LLAMA, Comm, DecodeV2Loop, DeviceWeights, build, shard_weights)

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=90))
    try:
        model = build(MEDIUM_LLAMA, 0)
        full = DeviceWeights.from_synth(model, f"cuda:{rank}")
        prompt = [1, 3, 5, 7, 2, 9]
        want = DecodeV2Loop.from_weights(full).generate_device_window(prompt, 12).tokens
        shard = shard_weights(full, rank, world)
        loop = DecodeV2Loop.from_weights(shard, comm=Comm.from_env())
        eager = loop.generate_device_window(prompt, 12).tokens
        mode = loop.capture_graphs()
        graphed = loop.generate_device_window(prompt, 12).tokens
        chunked = loop.generate_device_window(prompt, 12, chunk=4).tokens
        # the same shard with the row-split sums done over peer memory inside the GEMV launch
        how = loop.state.enable_peer_exchange()
        loop._graph, loop.graph_mode = None, "off"
        p2p_eager = loop.generate_device_window(prompt, 12).tokens
        p2p_mode = loop.capture_graphs()
        p2p_graphed = loop.generate_device_window(prompt, 12).tokens
        p2p = (how, p2p_eager, p2p_mode, loop.graph_error, p2p_graphed, loop.state.peers.timed_out())
        torch.cuda.synchronize()
        dist.barrier()
        with open(os.path.join(out_dir, f"r{rank}"), "w") as f:
            f.write(repr((want, eager, mode, loop.graph_error, graphed, chunked, p2p)))
            f.flush()
            os.fsync(f.fileno())
        loop.state.comm.shutdown(loop)
    finally:
        faulthandler.cancel_dump_traceback_later()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp2_matches_single_gpu(tmp_path):
    import torch.multiprocessing as mp

    world = 2
    mp.spawn(_rank_main, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        want, eager, mode, err, graphed, chunked, p2p = eval((tmp_path / f"r{r}").read_text())
        assert mode == "decodev2", err
        # FP32 partials summed before the single rounding: same ids as one GPU on this model
        assert eager == want and graphed == want and chunked[:4] == want[:4]
        how, p2p_eager, p2p_mode, p2p_err, p2p_graphed, timed_out = p2p
        print(f"rank {r}: peer buffers via {how}")
        assert p2p_mode == "decodev2", p2p_err
        assert not timed_out
        assert p2p_eager == want and p2p_graphed == want
