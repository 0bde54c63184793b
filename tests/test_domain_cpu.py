"""Domain decomposition and halo exchange on CPU ranks (gloo, world size 2 and 4)."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, world, port, grid_expect, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mace_ictc import domain as D
        from oracle import ictc_oracle as O
        rng = np.random.default_rng(0)
        box = torch.tensor([24.0, 13.0, 11.0], dtype=torch.float64)
        n, cutoff, width = 400, 4.5, 6
        pos = torch.as_tensor((rng.random((n, 3)) * box.numpy()).astype(np.float32))
        grid = D.brick_grid(world, box.tolist())
        assert grid == grid_expect
        dom = D.decompose(pos, box, grid, rank, cutoff)
        plan = D.ExchangePlan(dom, rank, world)
        # every atom has exactly one owner; owned lists partition the atoms
        counts = torch.zeros(n, dtype=torch.long)
        counts[dom.owned] += 1
        dist.all_reduce(counts)
        assert bool((counts == 1).all())
        # forward exchange delivers the owner's rows
        table = torch.as_tensor(rng.normal(size=(n, width))).float()          # "global" features, same on all ranks
        owned_rows = table[dom.owned].clone().requires_grad_(True)
        ghosts = D.exchange(owned_rows, plan)
        assert torch.equal(ghosts, table[dom.ghost_ids])
        # adjoint: d/d(owned) of <c, ghosts> accumulates the coefficients of every image of an atom
        coeff = torch.as_tensor(rng.normal(size=(n, width))).float()
        # the coefficient of a ghost row depends on (consumer rank, ghost position) to catch misrouting
        c_local = (coeff[dom.ghost_ids] * (rank + 1)).requires_grad_(True)
        (g,) = torch.autograd.grad((ghosts * c_local).sum(), owned_rows, create_graph=True)
        expect = torch.zeros(n, width)
        expect.index_add_(0, dom.ghost_ids, c_local.detach())
        dist.all_reduce(expect)
        assert torch.allclose(g, expect[dom.owned], atol=1e-6)
        # second order (force-loss training): the adjoint of the adjoint is the forward exchange
        table2 = torch.as_tensor(rng.normal(size=(n, width))).float()
        (gg,) = torch.autograd.grad((g * table2[dom.owned]).sum(), c_local)
        assert torch.equal(gg, table2[dom.ghost_ids])
        # local neighbour lists (open boundaries, ghost images as rows) reproduce the periodic global list
        local = dom.local_positions(pos, box).numpy()
        ids = dom.local_ids().numpy()
        ls, ld, _ = O.neighbor_list_bruteforce(local, dom.num_owned, box.numpy(), (0, 0, 0), cutoff)
        gs, gd, gsh = O.neighbor_list_bruteforce(pos.numpy(), n, box.numpy(), (1, 1, 1), cutoff)
        mine = np.isin(gd, dom.owned.numpy())
        assert ls.shape[0] == int(mine.sum())
        # compare as multisets of (dst global id, src global id, displacement); images of one pair differ
        # by a box length, so sorting on the displacement is robust to fp32 rounding of ghost coordinates
        def table_of(p, s, d, sh, b, gid_d, gid_s):
            v = p[d].astype(np.float64) - p[s].astype(np.float64) + sh * b
            t = np.concatenate([gid_d[:, None].astype(np.float64), gid_s[:, None].astype(np.float64), v], 1)
            return t[np.lexsort((np.round(t[:, 4]), np.round(t[:, 3]), np.round(t[:, 2]), t[:, 1], t[:, 0]))]
        lt = table_of(local, ls, ld, 0, box.numpy(), ids[ld], ids[ls])
        gt = table_of(pos.numpy(), gs[mine], gd[mine], gsh[mine], box.numpy(), gd[mine], gs[mine])
        assert np.array_equal(lt[:, :2], gt[:, :2])
        assert np.abs(lt[:, 2:] - gt[:, 2:]).max() < 1e-4
        results[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,grid,port", [(2, (2, 1, 1), 29611), (4, (2, 2, 1), 29612)])
def test_decomposition_and_exchange(world, grid, port):
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, grid, results), nprocs=world, join=True)
    assert len(results) == world


def test_brick_grid_shapes():
    from mace_ictc.domain import brick_grid
    assert brick_grid(1, (10, 10, 10)) == (1, 1, 1)
    assert brick_grid(8, (275.2, 275.2, 137.6)) == (2, 2, 2) or sorted(brick_grid(8, (275.2, 275.2, 137.6))) == [1, 2, 4]
    assert brick_grid(2, (10, 30, 10)) == (1, 2, 1)
    with pytest.raises(ValueError):
        brick_grid(3, (10, 10, 10))
