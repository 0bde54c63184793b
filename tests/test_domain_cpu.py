"""Domain decomposition with distributed state on CPU ranks (gloo): ownership, fixed-capacity halo plan and its
refresh in place, exchanges and their adjoints, local edge lists against the periodic global list, migration,
collective error decisions and the liveness check between steps."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _init(rank, world, port):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)


def _edge_table(p, s, d, sh, b, gid_d, gid_s):
    v = p[d].astype(np.float64) - p[s].astype(np.float64) + sh * b
    t = np.concatenate([gid_d[:, None].astype(np.float64), gid_s[:, None].astype(np.float64), v], 1)
    return t[np.lexsort((np.round(t[:, 4]), np.round(t[:, 3]), np.round(t[:, 2]), t[:, 1], t[:, 0]))]


def _worker(rank, world, port, grid_expect, results):
    _init(rank, world, port)
    try:
        from mace_ictc import domain as D
        from oracle import ictc_oracle as O
        rng = np.random.default_rng(0)
        box = [24.0, 13.0, 11.0]
        n, cutoff, skin, width = 400, 4.5, 1.0, 6
        pos = torch.as_tensor((rng.random((n, 3)) * np.array(box)).astype(np.float32))
        grid = D.brick_grid(world, box)
        assert grid == grid_expect
        owner = D.owner_of(pos, box, grid)
        gid = torch.nonzero(owner == rank).flatten()
        own = pos[gid].clone()
        # every atom has exactly one owner
        counts = torch.zeros(n, dtype=torch.long)
        counts[gid] += 1
        dist.all_reduce(counts)
        assert bool((counts == 1).all())
        plan = D.HaloPlan(rank, world, grid, box, cutoff + skin, gid.numel(), "cpu")
        assert plan.refresh(own)
        caps = (list(plan.send_cap), list(plan.recv_cap))
        mask = plan.ghost_mask()
        ghost_gid = plan.integers(gid)
        # forward exchange delivers the owners' rows; padding rows are never compared
        table = torch.as_tensor(rng.normal(size=(n, width))).float()          # "global" features, same on all ranks
        owned_rows = table[gid].clone().requires_grad_(True)
        ghosts = D.exchange(owned_rows, plan)
        assert ghosts.shape[0] == plan.num_ghost and int(mask.sum()) == sum(plan.recv_count)
        assert torch.equal(ghosts[mask], table[ghost_gid[mask]])
        # adjoint: d/d(owned) of <c, ghosts> accumulates the coefficients of every image of an atom; the
        # coefficient depends on (consumer rank, ghost row) to catch misrouting; padding rows carry zero
        coeff = torch.as_tensor(rng.normal(size=(n, width))).float()
        c_local = (coeff[ghost_gid] * (rank + 1) * mask.unsqueeze(1)).requires_grad_(True)
        (g,) = torch.autograd.grad((ghosts * c_local).sum(), owned_rows, create_graph=True)
        expect = torch.zeros(n, width)
        expect.index_add_(0, ghost_gid[mask], c_local.detach()[mask])
        dist.all_reduce(expect)
        assert torch.allclose(g, expect[gid], atol=1e-6)
        # second order (force-loss training): the adjoint of the adjoint is the forward exchange
        table2 = torch.as_tensor(rng.normal(size=(n, width))).float()
        (gg,) = torch.autograd.grad((g * table2[gid]).sum(), c_local)
        assert torch.equal(gg[mask], table2[ghost_gid[mask]])

        def check_edges(own_now, all_now):
            """local edge list (open boundaries, ghost images as rows) == the periodic global list of my centres"""
            local = torch.cat((own_now, plan.positions(own_now))).numpy()
            ids = torch.cat((gid, plan.integers(gid))).numpy()
            ls, ld, _ = O.neighbor_list_bruteforce(local, gid.numel(), np.array(box), (0, 0, 0), cutoff)
            gs, gd, gsh = O.neighbor_list_bruteforce(all_now, n, np.array(box), (1, 1, 1), cutoff)
            mine = np.isin(gd, gid.numpy())
            assert ls.shape[0] == int(mine.sum())
            lt = _edge_table(local, ls, ld, 0, np.array(box), ids[ld], ids[ls])
            gt = _edge_table(all_now, gs[mine], gd[mine], gsh[mine], np.array(box), gd[mine], gs[mine])
            assert np.array_equal(lt[:, :2], gt[:, :2])
            assert np.abs(lt[:, 2:] - gt[:, 2:]).max() < 1e-4
        check_edges(own, pos.numpy())
        # atoms move by less than skin/2 WITHOUT a refresh (and without wrapping): the old ghost lists still give
        # the exact edge list of the new coordinates
        step = torch.as_tensor(rng.uniform(-1, 1, size=(n, 3)).astype(np.float32))
        step = step / step.norm(dim=1, keepdim=True) * 0.49 * skin
        moved_all = pos + step
        moved_own = moved_all[gid]
        check_edges(moved_own, moved_all.numpy())
        # a refresh rewrites the lists in place: same capacities, same tensors
        rows_ptr = plan.send_rows.data_ptr()
        assert plan.refresh(moved_own)
        assert (list(plan.send_cap), list(plan.recv_cap)) == caps and plan.send_rows.data_ptr() == rows_ptr
        check_edges(moved_own, moved_all.numpy())
        # a further move of almost skin/2 after the refresh, owned atoms now up to ~skin/2 outside their bricks
        step2 = torch.as_tensor(rng.uniform(-1, 1, size=(n, 3)).astype(np.float32))
        step2 = step2 / step2.norm(dim=1, keepdim=True) * 0.24 * skin
        far_all = moved_all + step2
        check_edges(far_all[gid], far_all.numpy())
        # migration: every atom goes to the brick that holds its (wrapped) coordinates, nothing is lost
        wrapped = far_all[gid] - torch.floor(far_all[gid] / torch.tensor(box)) * torch.tensor(box)
        dest = D.owner_of(wrapped, box, grid)
        payload = torch.cat((wrapped.double(), gid.double().unsqueeze(1)), 1)
        got = D.migrate(dest, payload, world)
        assert bool((D.owner_of(got[:, :3].float(), box, grid) == rank).all())
        seen = torch.zeros(n, dtype=torch.long)
        seen[got[:, 3].long()] += 1
        dist.all_reduce(seen)
        assert bool((seen == 1).all())
        # a decision taken by one rank reaches all of them
        assert D.same_on_all_ranks(rank == world - 1) is True
        assert D.same_on_all_ranks(False) is False
        results[rank] = 1
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,grid,port", [(2, (2, 1, 1), 29611), (4, (2, 2, 1), 29612)])
def test_distributed_state_halo_plan(world, grid, port):
    results = mp.Manager().dict()
    mp.spawn(_worker, args=(world, port, grid, results), nprocs=world, join=True)
    assert len(results) == world


def _capacity_worker(rank, world, port, results):
    _init(rank, world, port)
    try:
        from mace_ictc import domain as D
        rng = np.random.default_rng(1)
        box = [20.0, 12.0, 12.0]
        pos = torch.as_tensor((rng.random((300, 3)) * np.array(box)).astype(np.float32))
        grid = D.brick_grid(world, box)
        gid = torch.nonzero(D.owner_of(pos, box, grid) == rank).flatten()
        plan = D.HaloPlan(rank, world, grid, box, 5.0, gid.numel(), "cpu", margin=1.0)
        assert plan.refresh(pos[gid])
        # only rank 0 outgrows a capacity (a wider halo selects more atoms): EVERY rank must learn that the plan
        # no longer fits, and the next refresh renegotiates the sizes on all of them
        plan.send_cap[1 - rank if world == 2 else 0] = plan.send_cap[1 - rank if world == 2 else 0] if rank else 1
        assert plan.refresh(pos[gid]) is False
        assert plan.send_cap is None
        assert plan.refresh(pos[gid]) is True
        results[rank] = 1
    finally:
        dist.destroy_process_group()


def test_capacity_overflow_is_agreed_between_ranks():
    results = mp.Manager().dict()
    mp.spawn(_capacity_worker, args=(2, 29613, results), nprocs=2, join=True)
    assert len(results) == 2


def _leaving_worker(rank, world, port, results):
    _init(rank, world, port)
    from mace_ictc import domain as D
    watch = D.PeerWatch(timeout=3.0)
    watch.check()                      # block 1: everyone is here
    if rank == world - 1:
        results[rank] = "left"         # leaves between two blocks, with nothing in flight
        return
    try:
        watch.check()                  # block 2: the others learn about it on the host
        results[rank] = "missed"
    except RuntimeError as err:
        results[rank] = "raised" if "gone or not responding" in str(err) else f"other: {err}"


def test_rank_leaving_between_steps_is_noticed_on_the_host():
    results = mp.Manager().dict()
    mp.spawn(_leaving_worker, args=(3, 29614, results), nprocs=3, join=True)
    assert dict(results) == {0: "raised", 1: "raised", 2: "left"}


def test_brick_grid_shapes():
    from mace_ictc.domain import brick_bounds, brick_grid
    assert brick_grid(1, (10, 10, 10)) == (1, 1, 1)
    assert brick_grid(8, (275.2, 275.2, 137.6)) == (2, 2, 2) or sorted(brick_grid(8, (275.2, 275.2, 137.6))) == [1, 2, 4]
    assert brick_grid(2, (10, 30, 10)) == (1, 2, 1)
    with pytest.raises(ValueError):
        brick_grid(3, (10, 10, 10))
    lo, hi = brick_bounds(3, (2, 2, 1), (20.0, 10.0, 8.0))
    assert lo == [10.0, 5.0, 0.0] and hi == [20.0, 10.0, 8.0]
