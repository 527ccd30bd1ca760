"""Host-side logic of the data-parallel training step on CPU with the gloo backend, world_size 2: the row sharding is a
partition, and per-rank chunk gradients (computed with the CPU oracle, loss-weighted as the GPU path does) all-reduced
over gloo equal the full-batch gradient of the reference algorithm."""
import os
import sys

import numpy as np
import pytest

from conftest import ROOT


def test_shard_ranges_partition_the_batch(lib):
    from rl_tools_b200 import parallel
    for n in (0, 1, 7, 16, 1000, 2 ** 24):
        for world in (1, 2, 3, 4, 8):
            ranges = [parallel.shard_range(n, r, world) for r in range(world)]
            assert ranges[0][0] == 0 and ranges[-1][1] == n
            assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
            sizes = [e - b for b, e in ranges]
            assert max(sizes) - min(sizes) <= 1
    assert parallel.chunk_loss_weight(256, 1024) == 0.25


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
    import torch
    import torch.distributed as dist
    import oracle
    import make_golden as mg
    import __graft_entry__ as entry
    entry.load_package()
    from rl_tools_b200 import parallel
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    orc = oracle.Oracle()
    shape = oracle.MlpShape.make(6, [16, 16, 3], ["relu", "tanh", "identity"])
    total, chunk = 192, 32
    params = mg.det_uniform(1, shape.num_params()) * np.float32(0.4)
    x = mg.det_normal(2, total * 6).reshape(total, 6)
    y = mg.det_normal(3, total * 3).reshape(total, 3)
    b, e = parallel.shard_range(total, rank, world)
    grads = np.zeros_like(params)
    for c in range(b, e, chunk):
        xc, yc = np.ascontiguousarray(x[c:c + chunk]), np.ascontiguousarray(y[c:c + chunk])
        pre, out = orc.mlp_forward(shape, params, xc)
        d = orc.mse_gradient(np.ascontiguousarray(out[-chunk * 3:].reshape(chunk, 3)), yc, parallel.chunk_loss_weight(chunk, total))
        grads, _ = orc.mlp_backward(shape, params, grads, xc, pre, out, d)
    t = torch.from_numpy(grads)
    parallel.allreduce_sum_(t, dist)
    np.save(os.path.join(out_dir, f"grads_{rank}.npy"), t.numpy())
    dist.destroy_process_group()


def test_gloo_world2_sharded_gradients_equal_full_batch(orc, tmp_path, lib):
    import torch.multiprocessing as mp
    import make_golden as mg
    import oracle
    port = 29600 + os.getpid() % 300
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    g0, g1 = np.load(tmp_path / "grads_0.npy"), np.load(tmp_path / "grads_1.npy")
    assert np.array_equal(g0, g1)                                    # replicas see the same reduced arena
    shape = oracle.MlpShape.make(6, [16, 16, 3], ["relu", "tanh", "identity"])
    params = mg.det_uniform(1, shape.num_params()) * np.float32(0.4)
    x = mg.det_normal(2, 192 * 6).reshape(192, 6)
    y = mg.det_normal(3, 192 * 3).reshape(192, 3)
    pre, out = orc.mlp_forward(shape, params, x)
    d = orc.mse_gradient(np.ascontiguousarray(out[-192 * 3:].reshape(192, 3)), y, 1.0)
    full, _ = orc.mlp_backward(shape, params, np.zeros_like(params), x, pre, out, d)
    assert np.all(np.abs(g0 - full) <= 1e-6 + 1e-5 * np.abs(full))
