"""Domain-decomposed MD force evaluation on 2+ GPUs (NCCL) against the single-GPU evaluation.

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
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
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
        f_ref = single.compute_forces().clone()
        e_ref = float(single.energy)
        multi = MolecularDynamics(model, pos, z, box, dt=1.0, seed=3, distributed=True)
        f = multi.compute_forces()
        scale = float(f_ref.abs().max())
        assert float((f - f_ref).abs().max()) < 2e-5 * scale, float((f - f_ref).abs().max()) / scale
        assert abs(float(multi.energy) - e_ref) < 1e-5 * abs(e_ref)
        for _ in range(3):
            single.step()
            multi.step()
        assert float((multi.pos - single.pos).abs().max()) < 1e-4
        # replicated state stays bitwise identical across ranks
        probe = multi.pos.clone()
        dist.broadcast(probe, 0)
        assert torch.equal(probe, multi.pos)
        assert _lib.kernel_status() == 0
        out[rank] = multi.num_edges
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_decomposed_forces_match_single_gpu(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    out = mp.Manager().dict()
    mp.spawn(_worker, args=(world, 29650 + world, out), nprocs=world, join=True)
    assert len(out) == world
