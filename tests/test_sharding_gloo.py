"""CPU, world_size 2 (gloo): the sharding logic.  The oracle stands in for the CUDA ops so that the
test exercises partition arithmetic and the two reductions, not the kernels."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from separableflowthesis_b200 import sharding
from oracle import separation_oracle as orc


def test_make_shard_partitions_cover_everything():
    for B, H1, world in ((8, 135, 8), (8, 135, 4), (1, 135, 8), (4, 55, 8), (2, 48, 2), (3, 7, 6)):
        seen = torch.zeros(B, H1, dtype=torch.int32)
        for r in range(world):
            s = sharding.make_shard(B, H1, world, r)
            assert s.g_batch * s.g_rows == world
            seen[s.b0:s.b1, s.r0:s.r1] += 1
            assert r in s.row_group_ranks and len(s.row_group_ranks) == s.g_rows
        assert (seen == 1).all(), (B, H1, world)
    s = sharding.make_shard(8, 135, 8, 3)
    assert (s.g_batch, s.g_rows, s.b0, s.b1, s.r0, s.r1) == (8, 1, 3, 4, 0, 135)
    s = sharding.make_shard(1, 135, 8, 7)
    assert (s.r0, s.r1) == (119, 135)  # 135 rows over 8 ranks = 17 x 7 + 16
    with pytest.raises(ValueError):
        sharding.make_shard(1, 3, 8, 0)
    s = sharding.make_shard(8, 135, 4, 1, prefer="rows")     # all samples, a block of rows
    assert (s.g_batch, s.g_rows, s.b0, s.b1, s.r0, s.r1) == (1, 4, 0, 8, 34, 68)
    assert sharding.halo_range(s, 135) == (33, 69, 1, 35)
    assert sharding.halo_range(sharding.make_shard(8, 135, 4, 0, prefer="rows"), 135) == (0, 35, 0, 34)
    assert sharding.halo_range(sharding.make_shard(8, 135, 8, 3), 135) == (0, 135, 0, 135)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, B, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(11)
        H1, W1, H2, W2, C, Kc = 6, 5, 6, 5, 8, 2
        F1 = torch.randn(B, H1, W1, C, generator=g, dtype=torch.float64)
        F2 = torch.randn(B, H2, W2, C, generator=g, dtype=torch.float64)
        A_u = torch.randn(B, H1, W1, Kc, W2, generator=g, dtype=torch.float64)
        A_v = torch.randn(B, H1, W1, Kc, H2, generator=g, dtype=torch.float64)
        gC_u = torch.randn(B, H1, W1, Kc, H2, generator=g, dtype=torch.float64)
        gC_v = torch.randn(B, H1, W1, Kc, W2, generator=g, dtype=torch.float64)
        full = orc.compression_backward(F1, F2, A_u, A_v, gC_u, gC_v)

        sh = sharding.make_shard(B, H1, world, rank)
        grp = sharding.new_row_groups(world, sh.g_rows)
        sl = (slice(sh.b0, sh.b1), slice(sh.r0, sh.r1))
        part = orc.compression_backward(F1[sl].contiguous(), F2[sh.b0:sh.b1].contiguous(), A_u[sl].contiguous(),
                                        A_v[sl].contiguous(), gC_u[sl].contiguous(), gC_v[sl].contiguous())
        gF2 = sharding.reduce_row_partial(part[1], grp)
        ok = torch.allclose(part[0], full[0][sl], atol=1e-12) and torch.allclose(gF2, full[1][sh.b0:sh.b1], atol=1e-12)
        ok = ok and torch.allclose(part[2], full[2][sl], atol=1e-12) and torch.allclose(part[3], full[3][sl], atol=1e-12)

        # shared-parameter gradient: every rank contributes rank+1, the sum must arrive everywhere
        conv = torch.nn.Conv3d(2, Kc, 3, padding=1).double()
        for p in conv.parameters():
            p.grad = torch.full_like(p, float(rank + 1))
        flat = sharding.reduce_parameter_grads(conv.parameters())
        expect = float(sum(range(1, world + 1)))
        ok = ok and flat.numel() == 2 * 27 * Kc + Kc and bool((flat == expect).all())
        ok = ok and all(bool((p.grad == expect).all()) for p in conv.parameters())
        # a rank without a gradient for one parameter still joins with a buffer of the full length: it contributes
        # zeros there and receives the others' sum
        for p in conv.parameters():
            p.grad = torch.full_like(p, float(rank + 1))
        if rank == 0:
            conv.bias.grad = None
        flat = sharding.reduce_parameter_grads(conv.parameters())
        ok = ok and flat.numel() == 2 * 27 * Kc + Kc and bool((conv.weight.grad == expect).all())
        ok = ok and conv.bias.grad is not None and bool((conv.bias.grad == expect - 1.0).all())
        results[rank] = ok
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("B", [1, 2])  # B=1: two row shards of one sample; B=2: two batch shards
def test_two_rank_sharded_backward_matches_unsharded(B):
    world = 2
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, B, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert all(results.get(r) for r in range(world)), dict(results)


def _halo_worker(rank, world, port, results):
    """Row-sharded call site with halo rows against the unsharded one: outputs of the shard's rows, feature
    gradients (halo rows handed to the neighbour, gF2 summed over the row group) and attention-parameter gradients."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import separableflowthesis_b200 as sfb
        from separableflowthesis_b200 import functions
        functions.MemorySaver = orc                      # the oracle stands in for the CUDA ops
        torch.manual_seed(5)
        B, C, H, W, Kc = 1, 8, 7, 6, 2
        g = torch.Generator().manual_seed(3)
        f1 = torch.randn(B, C, H, W, generator=g, dtype=torch.float64)
        f2 = torch.randn(B, C, H, W, generator=g, dtype=torch.float64)
        convs = [torch.nn.Conv3d(2, Kc, 3, padding=1).double() for _ in range(2)]
        up_u = torch.randn(B, (2 + Kc) * 2, W, H, W, generator=g, dtype=torch.float64)
        up_v = torch.randn(B, (2 + Kc) * 2, H, H, W, generator=g, dtype=torch.float64)

        def run(f1_rows, f2_all, rows):
            a = f1_rows.clone().requires_grad_(True)
            b = f2_all.clone().requires_grad_(True)
            for c in convs:
                c.zero_grad()
            blk = sfb.AlternateCorrBlockSepflow(a, b, None, num_levels=2, support_backward=True)
            su, sv = blk(None, sep=True, attention_weights=tuple(convs))
            return a, b, su, sv

        # unsharded reference
        a, b, su, sv = run(f1, f2, slice(0, H))
        ((su * up_u).sum() + (sv * up_v).sum()).backward()
        ref = dict(su=su.detach(), sv=sv.detach(), g1=a.grad.clone(), g2=b.grad.clone(),
                   gw=[c.weight.grad.clone() for c in convs])

        sh = sharding.make_shard(B, H, world, rank)
        grp = sharding.new_row_groups(world, sh.g_rows)
        e0, e1, i0, i1 = sharding.halo_range(sh, H)
        a, b, su, sv = run(f1[:, :, e0:e1].contiguous(), f2, None)
        su_own = sharding.interior(su, sh, H, 3)
        sv_own = sharding.interior(sv, sh, H, 3)
        ok = torch.allclose(su_own, ref["su"][:, :, :, sh.r0:sh.r1], atol=1e-12)
        ok = ok and torch.allclose(sv_own, ref["sv"][:, :, :, sh.r0:sh.r1], atol=1e-12)
        ((su_own * up_u[:, :, :, sh.r0:sh.r1]).sum() + (sv_own * up_v[:, :, :, sh.r0:sh.r1]).sum()).backward()
        g1 = sharding.exchange_halo_grads(a.grad, sh, H, grp, dim=2)
        g2 = sharding.reduce_row_partial(b.grad, grp)
        sharding.reduce_parameter_grads([p for c in convs for p in c.parameters()])
        ok = ok and torch.allclose(g1, ref["g1"][:, :, sh.r0:sh.r1], atol=1e-11)
        ok = ok and torch.allclose(g2, ref["g2"], atol=1e-11)
        ok = ok and all(torch.allclose(c.weight.grad, w, atol=1e-11) for c, w in zip(convs, ref["gw"]))
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_row_shards_with_halo_rows_match_the_unsharded_call_site(world):
    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = _free_port()
    procs = [ctx.Process(target=_halo_worker, args=(r, world, port, results)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(180)
        assert p.exitcode == 0
    assert all(results.get(r) for r in range(world)), dict(results)
