"""The library against the reference's OWN CUDA device (oracle/_ref/libref_cuda.so: the unmodified reference headers compiled with nvcc, cuBLAS
SGEMM per layer) on the same GPU, same inputs: the training step of the benchmark network, chunked as bench.py's mlp_train line chunks it.
Skipped where that library was not built (it needs the reference tree at build time)."""
import os

import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch


@pytest.fixture(scope="module")
def lib():
    from __graft_entry__ import load_package
    return load_package()


@pytest.fixture(scope="module")
def ref_cuda():
    if not os.path.exists(oracle.REF_CUDA_SO):
        pytest.skip("oracle/_ref/libref_cuda.so was not built (needs the reference tree and nvcc at build time)")
    return oracle.ReferenceCuda()


@pytest.mark.parametrize("case,dims,chunk,rows", [("c5_b1024", (64, [256, 256, 256, 16]), 1024, 4096), ("c3_b256", (4, [256, 256, 1]), 256, 256),
                                                  ("c5_b65536", (64, [256, 256, 256, 16]), 65536, 131072)])
def test_training_step_matches_the_reference_cuda_device(lib, torch, ref_cuda, case, dims, chunk, rows):
    """One step (zero_gradient; per chunk forward, MSE gradient weighted chunk / rows, backward; Adam) from the same parameters on the same
    device-resident rows. Gradients: |g - ref| <= 1e-6 + 1e-5 |ref| + 1e-5 max|ref| of the tensor -- both sides sum `rows` products per
    weight in their own order (cuBLAS's split-k there, fixed-order batch splits here), so a gradient is compared relative to the scale
    of its tensor as well as to itself. Parameters after the Adam step: 1e-6 + 1e-5 |ref|, except where a gradient is so close to zero that
    its sign or size is rounding noise (Adam moves those by up to alpha = 1e-3 either way): fewer than 0.1 % of the entries, each within
    2 alpha."""
    from rl_tools_b200 import parallel                       # importable once load_package() has run (the `lib` fixture)
    input_dim, layer_dims = dims
    acts = ["relu"] * (len(layer_dims) - 1) + ["identity"]
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    x = torch.randn((rows, input_dim), device="cuda", generator=g)
    y = torch.randn((rows, layer_dims[-1]), device="cuda", generator=g)
    net = lib.Mlp(input_dim, layer_dims, acts, chunk)
    off, fan_in = 0, input_dim
    for d in layer_dims:
        n = d * fan_in + d
        net.params[off:off + n] = (torch.rand(n, device="cuda", generator=g) * 2 - 1) / fan_in ** 0.5
        off += n; fan_in = d
    params0 = net.params.cpu().numpy().copy()
    torch.cuda.synchronize()
    _, want_params, want_grads = ref_cuda.mlp_train(case, params0, x.data_ptr(), y.data_ptr(), rows, steps=1)
    net.reset_optimizer_state()
    parallel.sharded_train_step(lib, net, x, y, rows)
    got_grads, got_params = net.grads.cpu().numpy(), net.params.cpu().numpy()
    off, fan_in = 0, input_dim
    for d in layer_dims:                                        # per tensor: weights, then biases of each layer
        for n in (d * fan_in, d):
            ref_t, got_t = want_grads[off:off + n], got_grads[off:off + n]
            assert np.all(np.abs(got_t - ref_t) <= 1e-6 + 1e-5 * np.abs(ref_t) + 1e-5 * np.abs(ref_t).max()), (case, off)
            off += n
        fan_in = d
    err = np.abs(got_params - want_params)
    loose = err > 1e-6 + 1e-5 * np.abs(want_params)
    assert loose.mean() < 1e-3 and err.max() <= 2e-3, (case, int(loose.sum()), float(err.max()))


def test_reference_cuda_runner_steps_the_environments(ref_cuda):
    """The second baseline of the headline line: the reference's own off-policy runner on its CUDA device rolls 512 Pendulum environments for
    200 steps and reports a time and a (negative) mean episode return."""
    rs = np.random.RandomState(0)
    ms, mean_return = ref_cuda.rollout("512env", (rs.uniform(-1, 1, 4481) * 0.3).astype(np.float32), steps=1, warmup=1)
    assert ms > 0 and -16.3 * 200 <= mean_return < 0
