"""Token-sharded recurrence, host logic on CPU: two gloo ranks, each with half of every chunk's
tokens and the oracle's sub-ops standing in for the CUDA ones, against the oracle's fused
post-norm driver on the whole sequence."""
import os
import socket
from types import SimpleNamespace

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from lact_b200 import token_sharded as ts

NAMES = ("q", "k", "v", "lr0", "lr1", "lr2", "momentum")


def oracle_sub_ops():
    from oracle import lact_oracle as orc
    return SimpleNamespace(apply=orc.apply_fused, grads=orc.grads_fused, newton_schulz=orc.newton_schulz,
                           l2_norm_add=lambda x, dx, n, eps=1e-5: orc.l2_norm_add(x, dx, n, eps=eps))


def test_shard_and_unshard_are_inverse():
    x = torch.arange(2 * 24 * 3).reshape(2, 24, 3)
    for chunk, world in ((8, 2), (12, 4), (24, 3)):
        parts = [ts.shard_tokens(x, chunk, world, r) for r in range(world)]
        assert all(p.shape == (2, 24 // world, 3) for p in parts)
        assert torch.equal(ts.unshard_tokens(parts, chunk), x)
    # rank r holds the r-th slice of every chunk
    assert ts.shard_tokens(x, 8, 2, 1)[0, :, 0].tolist() == [3 * t for t in (4, 5, 6, 7, 12, 13, 14, 15, 20, 21, 22, 23)]
    with pytest.raises(ValueError):
        ts.shard_tokens(x, 9, 2, 0)
    with pytest.raises(ValueError):
        ts.shard_tokens(x, 8, 3, 0)


def _inputs(B, L, D, H, seed):
    from oracle import lact_oracle as orc
    i = orc.make_inputs(B, L, D, H, seed=seed)
    for n in ("q", "k", "v"):
        i[n] = i[n].to(torch.bfloat16)
    return i


def _worker(rank, world, port, use_muon, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    i = _inputs(2, 256, 32, 32, seed=3)
    mine = {n: ts.shard_tokens(i[n], 64, world, rank) for n in NAMES}
    o = ts.token_sharded_block_causal_lact_swiglu(i["w0"], i["w1"], i["w2"], mine["q"], mine["k"], mine["v"],
                                                  mine["lr0"], mine["lr1"], mine["lr2"], chunk_size=64,
                                                  use_muon=use_muon, momentum=mine["momentum"],
                                                  sub_ops=oracle_sub_ops())
    torch.save(o, os.path.join(out_dir, f"o{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("use_muon", [False, True])
def test_two_ranks_reproduce_the_unsharded_recurrence(tmp_path, use_muon):
    from oracle import lact_oracle as orc
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_worker, args=(2, port, use_muon, str(tmp_path)), nprocs=2, join=True)
    torch.set_num_threads(1)
    i = _inputs(2, 256, 32, 32, seed=3)
    got = ts.unshard_tokens([torch.load(str(tmp_path / f"o{r}.pt")) for r in range(2)], 64).float()
    ref = orc.block_causal_lact_swiglu_fused(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"],
                                             i["lr2"], chunk_size=64, use_muon=use_muon,
                                             momentum=i["momentum"]).float()
    assert got.shape == ref.shape
    # chunk 0 uses the initial weights on both sides: identical
    assert torch.equal(got[:, :64], ref[:, :64])
    # later chunks: the per-rank partial gradients are rounded to bf16 before they are added, the unsharded
    # gradient once after; without Newton-Schulz that is a 2^-9 relative perturbation of the update
    if not use_muon:
        assert orc.rel_max(got, ref) <= 2e-2
        assert orc.cosine(got, ref) >= 0.9995
    else:  # the iteration amplifies the perturbation (the reference's own one-ulp response is of this size)
        assert orc.rel_max(got[:, 64:128], ref[:, 64:128]) <= 8e-2
        assert orc.cosine(got, ref) >= 0.99


def test_lock_step_instances_equal_the_process_group_path():
    """Two TokenShardedScan instances driven in lock step with a plain sum in place of the all-reduce give what the
    single-rank call on the whole sequence gives up to the rounding of the partial gradients."""
    from oracle import lact_oracle as orc
    torch.set_num_threads(1)
    i = _inputs(1, 192, 32, 32, seed=4)
    W, C = 2, 64
    scans = []
    for r in range(W):
        mine = {n: ts.shard_tokens(i[n], C, W, r) for n in NAMES}
        scans.append(ts.TokenShardedScan(i["w0"], i["w1"], i["w2"], mine["q"], mine["k"], mine["v"], mine["lr0"],
                                         mine["lr1"], mine["lr2"], C, W, use_muon=False, momentum=mine["momentum"],
                                         sub_ops=oracle_sub_ops()))
    for c in range(scans[0].n_chunks - 1):
        flats = []
        for s in scans:
            s.apply(c)
            flats.append(s.local_gradient(c))
        total = flats[0] + flats[1]
        for s in scans:
            s.update(total.clone())
    for s in scans:
        s.apply(s.n_chunks - 1)
    assert torch.equal(scans[0].w02, scans[1].w02) and torch.equal(scans[0].w1, scans[1].w1)
    got = ts.unshard_tokens([s.out for s in scans], C).float()
    one = ts.token_sharded_block_causal_lact_swiglu(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"],
                                                    i["lr1"], i["lr2"], chunk_size=C, use_muon=False,
                                                    momentum=i["momentum"], sub_ops=oracle_sub_ops()).float()
    ref = orc.block_causal_lact_swiglu_fused(i["w0"], i["w1"], i["w2"], i["q"], i["k"], i["v"], i["lr0"], i["lr1"],
                                             i["lr2"], chunk_size=C, use_muon=False, momentum=i["momentum"]).float()
    assert torch.equal(one, ref)  # one rank: the same arithmetic as the unsharded driver, bit for bit
    assert orc.rel_max(got, ref) <= 2e-2


def _loss_grads(fn, i, dO, names):
    leaves = {n: i[n].float().clone().requires_grad_(True) for n in names}
    o = fn(leaves)
    (o.float() * dO.float()).sum().backward()
    return o.detach(), {n: leaves[n].grad for n in names}


GRAD_NAMES = ("w0", "w1", "w2") + NAMES


def test_lock_step_training_gradients_match_the_unsharded_recurrence():
    """Muon off, two lock-step instances sharing the weight leaves (a plain differentiable sum in place of the
    all-reduce): the gradients of every input against autograd through the unsharded oracle driver."""
    from oracle import lact_oracle as orc
    torch.set_num_threads(1)
    i = _inputs(1, 192, 32, 32, seed=6)
    W, C = 2, 64
    dO = torch.randn(1, 192, 32, generator=torch.Generator().manual_seed(8))

    def sharded(leaves):
        scans = []
        for r in range(W):
            mine = {n: ts.shard_tokens(leaves[n], C, W, r) for n in NAMES}
            scans.append(ts.TokenShardedScan(leaves["w0"], leaves["w1"], leaves["w2"], mine["q"], mine["k"], mine["v"],
                                             mine["lr0"], mine["lr1"], mine["lr2"], C, W, use_muon=False,
                                             momentum=mine["momentum"], sub_ops=oracle_sub_ops()))
        for c in range(scans[0].n_chunks - 1):
            flats = []
            for s in scans:
                s.apply(c)
                flats.append(s.local_gradient(c))
            total = flats[0] + flats[1]
            for s in scans:
                s.update(total)
        for s in scans:
            s.apply(s.n_chunks - 1)
        return ts.unshard_tokens([s.out for s in scans], C)

    def whole(leaves):
        return orc.block_causal_lact_swiglu_fused(leaves["w0"], leaves["w1"], leaves["w2"], leaves["q"], leaves["k"],
                                                  leaves["v"], leaves["lr0"], leaves["lr1"], leaves["lr2"], chunk_size=C,
                                                  use_muon=False, momentum=leaves["momentum"])

    _, g = _loss_grads(sharded, i, dO, GRAD_NAMES)
    _, g_ref = _loss_grads(whole, i, dO, GRAD_NAMES)
    for n in GRAD_NAMES:
        assert g[n] is not None and torch.isfinite(g[n]).all(), n
        assert orc.cosine(g[n], g_ref[n]) >= 0.999, (n, orc.cosine(g[n], g_ref[n]))
        assert orc.rel_max(g[n], g_ref[n]) <= 5e-2, (n, orc.rel_max(g[n], g_ref[n]))


def _train_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(1)
    i = _inputs(2, 256, 32, 32, seed=3)
    dO = ts.shard_tokens(torch.randn(2, 256, 32, generator=torch.Generator().manual_seed(9)), 64, world, rank)
    w = {n: i[n].clone().requires_grad_(True) for n in ("w0", "w1", "w2")}
    mine = {n: ts.shard_tokens(i[n].float(), 64, world, rank).requires_grad_(True) for n in NAMES}
    o = ts.token_sharded_block_causal_lact_swiglu(w["w0"], w["w1"], w["w2"], mine["q"], mine["k"], mine["v"],
                                                  mine["lr0"], mine["lr1"], mine["lr2"], chunk_size=64, use_muon=False,
                                                  momentum=mine["momentum"], sub_ops=oracle_sub_ops())
    (o.float() * dO).sum().backward()
    for t in w.values():   # replicated parameters: the per-rank shares are summed, as a data-parallel wrapper would
        dist.all_reduce(t.grad)
    torch.save({**{n: w[n].grad for n in w}, **{n: mine[n].grad for n in NAMES}}, os.path.join(out_dir, f"g{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_training_gradients(tmp_path):
    """The process-group path with its differentiable all-reduce: two gloo ranks, gradients of the token shards
    gathered and of the replicated weights summed, against autograd through the unsharded oracle driver."""
    from oracle import lact_oracle as orc
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_train_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    torch.set_num_threads(1)
    i = _inputs(2, 256, 32, 32, seed=3)
    dO = torch.randn(2, 256, 32, generator=torch.Generator().manual_seed(9))
    parts = [torch.load(str(tmp_path / f"g{r}.pt")) for r in range(2)]
    whole = lambda leaves: orc.block_causal_lact_swiglu_fused(
        leaves["w0"], leaves["w1"], leaves["w2"], leaves["q"], leaves["k"], leaves["v"], leaves["lr0"], leaves["lr1"],
        leaves["lr2"], chunk_size=64, use_muon=False, momentum=leaves["momentum"])
    _, g_ref = _loss_grads(whole, i, dO, GRAD_NAMES)
    for n in ("w0", "w1", "w2"):
        assert torch.equal(parts[0][n], parts[1][n])   # after the sum every rank holds the same weight gradient
        assert orc.cosine(parts[0][n], g_ref[n]) >= 0.999 and orc.rel_max(parts[0][n], g_ref[n]) <= 5e-2, n
    for n in NAMES:
        got = ts.unshard_tokens([p[n] for p in parts], 64)
        assert orc.cosine(got, g_ref[n]) >= 0.999 and orc.rel_max(got, g_ref[n]) <= 5e-2, (n, orc.cosine(got, g_ref[n]))


def test_lock_step_training_with_muon():
    """With Muon the per-rank rounding of the partial gradients is amplified by Newton-Schulz (as in the forward
    test): the gradients stay close to those of the single-rank run of the same code, in direction and size."""
    from oracle import lact_oracle as orc
    torch.set_num_threads(1)
    i = _inputs(1, 192, 32, 32, seed=6)
    C = 64
    dO = torch.randn(1, 192, 32, generator=torch.Generator().manual_seed(8))

    def run(W):
        def fn(leaves):
            scans = []
            for r in range(W):
                mine = {n: ts.shard_tokens(leaves[n], C, W, r) for n in NAMES}
                scans.append(ts.TokenShardedScan(leaves["w0"], leaves["w1"], leaves["w2"], mine["q"], mine["k"],
                                                 mine["v"], mine["lr0"], mine["lr1"], mine["lr2"], C, W, use_muon=True,
                                                 momentum=mine["momentum"], sub_ops=oracle_sub_ops()))
            for c in range(scans[0].n_chunks - 1):
                flats = []
                for s_ in scans:
                    s_.apply(c)
                    flats.append(s_.local_gradient(c))
                total = flats[0] if W == 1 else flats[0] + flats[1]
                for s_ in scans:
                    s_.update(total)
            for s_ in scans:
                s_.apply(s_.n_chunks - 1)
            return ts.unshard_tokens([s_.out for s_ in scans], C)
        return _loss_grads(fn, i, dO, GRAD_NAMES)[1]

    g2, g1 = run(2), run(1)
    for n in GRAD_NAMES:
        assert g2[n] is not None and torch.isfinite(g2[n]).all(), n
        assert orc.cosine(g2[n], g1[n]) >= 0.97, (n, orc.cosine(g2[n], g1[n]))
