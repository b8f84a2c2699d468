"""(batch x head) partition across ranks: two gloo ranks on CPU each run their shard through the
CPU oracle, gather, and must reproduce the single-process result bit for bit (entries are
independent recurrences, so sharding must not change a single value)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lact_b200 import parallel


def test_partition_covers_everything():
    for n in (1, 4, 12, 32, 33):
        for world in (1, 2, 3, 4, 8):
            spans = [parallel.partition(n, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (s0, e0), (s1, e1) in zip(spans, spans[1:]):
                assert e0 == s1 and e0 >= s0
            sizes = [e - s for s, e in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        parallel.partition(4, 2, 2)


def _worker(rank, world, port, n_entries, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from oracle import lact_oracle as orc
    torch.set_num_threads(1)
    inp = orc.make_inputs(n_entries, 192, 32, 32, seed=5)
    mine = parallel.shard(inp, n_entries, world, rank)
    o = orc.block_causal_lact_swiglu(mine["w0"], mine["w1"], mine["w2"], mine["q"], mine["k"], mine["v"],
                                     mine["lr0"], mine["lr1"], mine["lr2"], chunk_size=64, use_muon=True,
                                     momentum=mine["momentum"])
    full = parallel.gather_output(o, n_entries)
    if rank == 0:
        torch.save(full, out_path)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("n_entries", [4, 5])
def test_two_rank_shard_and_gather_matches_single_process(tmp_path, n_entries):
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out_path = str(tmp_path / "gathered.pt")
    mp.spawn(_worker, args=(2, port, n_entries, out_path), nprocs=2, join=True)
    from oracle import lact_oracle as orc
    torch.set_num_threads(1)
    inp = orc.make_inputs(n_entries, 192, 32, 32, seed=5)
    ref = orc.block_causal_lact_swiglu(inp["w0"], inp["w1"], inp["w2"], inp["q"], inp["k"], inp["v"], inp["lr0"],
                                       inp["lr1"], inp["lr2"], chunk_size=64, use_muon=True, momentum=inp["momentum"])
    got = torch.load(out_path)
    assert got.shape == ref.shape
    assert torch.equal(got, ref)
