"""Token-sharded recurrence on the GPU: the CUDA sub-ops behind `TokenShardedScan`, (a) as two
instances in lock step on one device with a plain sum for the all-reduce, (b) as two NCCL ranks on
two devices when the machine has them, against the single-device fused post-norm driver."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
BF16 = torch.bfloat16
NAMES = ("q", "k", "v", "lr0", "lr1", "lr2", "momentum")


@pytest.fixture(scope="module")
def lb():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from lact_b200 import build
    build.build()
    import lact_b200
    return lact_b200


def _inputs(B, L, D, H, seed):
    from oracle import lact_oracle as orc
    i = orc.make_inputs(B, L, D, H, seed=seed)
    for n in ("q", "k", "v"):
        i[n] = i[n].to(BF16)
    return i


def _check(orc, got, ref, C, use_muon):
    got, ref = got.float().cpu(), ref.float().cpu()
    assert orc.rel_max(got[:, :C], ref[:, :C]) <= 5e-3  # chunk 0: the initial weights on both sides
    if not use_muon:
        assert orc.rel_max(got, ref) <= 2e-2
        assert orc.cosine(got, ref) >= 0.9995
    else:
        assert orc.rel_max(got[:, C:2 * C], ref[:, C:2 * C]) <= 8e-2
        assert orc.cosine(got, ref) >= 0.99


@pytest.mark.parametrize("use_muon", [False, True])
@pytest.mark.parametrize("B,L,D,H,C,W", [(2, 1024, 64, 128, 256, 2), (1, 2048, 192, 192, 512, 4)])
def test_lock_step_ranks_on_one_device(lb, B, L, D, H, C, W, use_muon):
    from oracle import lact_oracle as orc
    from lact_b200 import token_sharded as ts
    i = {k: v.cuda() for k, v in _inputs(B, L, D, H, seed=7).items()}
    ref = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        *[i[n] for n in ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")], chunk_size=C, use_muon=use_muon,
        momentum=i["momentum"])
    scans = []
    for r in range(W):
        mine = {n: ts.shard_tokens(i[n], C, W, r) for n in NAMES}
        scans.append(ts.TokenShardedScan(i["w0"], i["w1"], i["w2"], mine["q"], mine["k"], mine["v"], mine["lr0"],
                                         mine["lr1"], mine["lr2"], C, W, use_muon=use_muon, momentum=mine["momentum"]))
    for c in range(scans[0].n_chunks - 1):
        flats = []
        for s in scans:
            s.apply(c)
            flats.append(s.local_gradient(c))
        total = torch.stack(flats).sum(dim=0)
        for s in scans:
            s.update(total.clone())
    for s in scans:
        s.apply(s.n_chunks - 1)
    lb.synchronize_and_check()
    for s in scans[1:]:  # replicated state stays identical without any broadcast
        assert torch.equal(s.w02, scans[0].w02) and torch.equal(s.w1, scans[0].w1)
    got = ts.unshard_tokens([s.out for s in scans], C)
    _check(orc, got, ref, C, use_muon)
    # one rank, no process group: the same recurrence through the sub-ops
    one = ts.token_sharded_block_causal_lact_swiglu(*[i[n] for n in ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1",
                                                                      "lr2")], chunk_size=C, use_muon=use_muon,
                                                    momentum=i["momentum"])
    lb.synchronize_and_check()
    _check(orc, one, ref, C, use_muon)


def _nccl_worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import lact_b200
    from lact_b200 import token_sharded as ts
    B, L, D, H, C = 2, 4096, 128, 256, 1024
    i = {k: v.cuda() for k, v in _inputs(B, L, D, H, seed=9).items()}
    mine = {n: ts.shard_tokens(i[n], C, world, rank) for n in NAMES}
    o = ts.token_sharded_block_causal_lact_swiglu(i["w0"], i["w1"], i["w2"], mine["q"], mine["k"], mine["v"],
                                                  mine["lr0"], mine["lr1"], mine["lr2"], chunk_size=C, use_muon=False,
                                                  momentum=mine["momentum"])
    lact_b200.synchronize_and_check()
    torch.save(o.cpu(), os.path.join(out_dir, f"o{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_two_nccl_ranks(lb, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from oracle import lact_oracle as orc
    from lact_b200 import token_sharded as ts
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    mp.spawn(_nccl_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    B, L, D, H, C = 2, 4096, 128, 256, 1024
    i = {k: v.cuda() for k, v in _inputs(B, L, D, H, seed=9).items()}
    ref = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        *[i[n] for n in ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")], chunk_size=C, use_muon=False,
        momentum=i["momentum"])
    got = ts.unshard_tokens([torch.load(str(tmp_path / f"o{r}.pt")) for r in range(2)], C)
    _check(orc, got, ref, C, False)


@pytest.mark.parametrize("use_muon", [False, True])
def test_lock_step_training_on_one_device(lb, use_muon):
    """Two lock-step instances on the CUDA sub-ops (with their autograd formulas, the Newton-Schulz one included)
    sharing the weight leaves: gradients of every input against the fused driver's own backward on the unsharded
    sequence (with Muon the per-rank rounding of the partial gradients is amplified by the iteration: looser band)."""
    from oracle import lact_oracle as orc
    from lact_b200 import token_sharded as ts
    B, L, D, H, C, W = 2, 1024, 64, 128, 256, 2
    base = {k: v.cuda() for k, v in _inputs(B, L, D, H, seed=11).items()}
    dO = torch.randn(B, L, D, generator=torch.Generator().manual_seed(12)).to(BF16).cuda()
    names = ("w0", "w1", "w2") + NAMES

    def leaves():
        return {n: base[n].clone().requires_grad_(True) for n in names}

    a = leaves()
    ref = lb.postnorm_block_causal_lact_swiglu_fused_kernel_triton(
        *[a[n] for n in ("w0", "w1", "w2", "q", "k", "v", "lr0", "lr1", "lr2")], chunk_size=C, use_muon=use_muon,
        momentum=a["momentum"])
    (ref.float() * dO.float()).sum().backward()
    b = leaves()
    scans = []
    for r in range(W):
        mine = {n: ts.shard_tokens(b[n], C, W, r) for n in NAMES}
        scans.append(ts.TokenShardedScan(b["w0"], b["w1"], b["w2"], mine["q"], mine["k"], mine["v"], mine["lr0"],
                                         mine["lr1"], mine["lr2"], C, W, use_muon=use_muon, momentum=mine["momentum"]))
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
    out = ts.unshard_tokens([s.out for s in scans], C)
    (out.float() * dO.float()).sum().backward()
    lb.synchronize_and_check()
    for n in names:
        g, g_ref = b[n].grad, a[n].grad
        assert g is not None and torch.isfinite(g.float()).all(), n
        cs = orc.cosine(g.float().cpu(), g_ref.float().cpu())
        assert cs >= (0.97 if use_muon else 0.995), (n, cs)
