"""Domain-decomposed MD with distributed state on 2+ GPUs (NCCL) against the single-GPU evaluation: forces and
energy, a trajectory through ghost-list refreshes, the recorded step with its collectives, and a forced
re-decomposition with atom migration.

Needs at least two visible GPUs; skipped otherwise.  Ranks run as child processes, leave only between
steps, and NVLS is switched off for the test.
"""
import os

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0", NCCL_GRAPH_REGISTER="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ictc_o3 import _lib
        from mace_ictc import synthetic as S
        from mace_ictc.hp import create_model
        from mace_ictc.md import MolecularDynamics
        torch.manual_seed(11)
        pos, box, species = S.jittered_lattice(12, 10, 8, 2.15, 0.1, 4)
        z = np.array([1, 6, 8])[species]
        model = create_model(channels=64, lmax=2, cutoff=4.5, avg_num_neighbors=32.0, device=f"cuda:{rank}")
        for p in model.parameters():                       # same weights on every rank
            dist.broadcast(p.data, 0)
        single = MolecularDynamics(model, pos, z, box, dt=1.0, seed=3)
        f_ref = single.gather(single.compute_forces())
        e_ref = float(single.energy)
        multi = MolecularDynamics(model, pos, z, box, dt=1.0, seed=3, distributed=True, skin=0.6, watch_peers=True)
        assert multi.num_owned < pos.shape[0]              # a rank holds its own atoms only
        f = multi.gather(multi.compute_forces())
        assert multi.pos.shape[0] > multi.num_owned        # fixed-capacity arrays: the tail is inert padding
        assert float(multi.forces[multi.num_owned:].abs().max()) == 0.0
        scale = float(f_ref.abs().max())
        assert float((f - f_ref).abs().max()) < 2e-5 * scale, float((f - f_ref).abs().max()) / scale
        assert abs(float(multi.energy) - e_ref) < 1e-5 * abs(e_ref)
        # eager trajectory; the thin skin makes the refresh period short, so atoms migrate and ghost lists are
        # rewritten on the way
        multi.block = 2
        single.run(7)
        multi.run(7)
        assert multi.refreshes >= 2

        def wrapped(md):
            p = md.gather(md.pos)
            return p - torch.floor(p / md.box_f) * md.box_f
        d = (wrapped(multi) - single.gather(single.pos)).abs()
        d = torch.minimum(d, (d - single.box_f).abs())     # an atom sitting on the box face may wrap either way
        assert float(d.max()) < 1e-4
        assert float((multi.gather(multi.forces) - single.gather(single.forces)).abs().max()) < 5e-5 * scale
        # the recorded step (collectives inside the graph) continues the same trajectory
        multi.enable_graph()
        single.run(6)
        multi.run(6)
        d = (wrapped(multi) - single.gather(single.pos)).abs()
        d = torch.minimum(d, (d - single.box_f).abs())
        assert float(d.max()) < 2e-4
        assert float((multi.gather(multi.forces) - single.gather(single.forces)).abs().max()) < 1e-4 * scale
        # ownership re-derived from the coordinates: atoms migrate, nothing is lost, forces stay the same
        before = multi.gather(multi.forces).clone()
        multi.redecompose()
        count = torch.tensor([multi.num_owned], device=f"cuda:{rank}")
        dist.all_reduce(count)
        assert int(count) == pos.shape[0]
        assert torch.equal(multi.gather(multi.forces), before)
        f2 = multi.gather(multi.compute_forces())
        assert float((f2 - before).abs().max()) < 2e-5 * scale
        assert _lib.kernel_status() == 0
        out[rank] = multi.refreshes
        multi.close()                   # a live graph with captured collectives would block the tear-down
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decomposed_md_matches_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29650 + world, out), nprocs=world, join=True)
    assert len(out) == world
