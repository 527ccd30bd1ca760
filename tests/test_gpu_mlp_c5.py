"""Whole-network parity of the sharded training configuration (64 -> 256 -> 256 -> 256 -> 16, ReLU, identity) at the chunk size the
benchmark runs: 65,536 rows per chunk, two chunks accumulated into one gradient, one Adam step -- the sequence of
rl_tools_b200.parallel.sharded_train_step. At this size the 256-wide contractions take the tensor-core kernel (forward, input gradient on the
transposed weights, split-batch weight gradient) and the 16-wide output layer the one-pass kernels for few outputs (forward; d_pre, both
gradients and the input gradient in one pass).

Checked against the fixture written from the real reference's zero_gradient / forward / mse::gradient / backward / step
(tests/golden/c5_chunked_b65536.npz, make_golden.py `c5`):
  activations (255 sampled rows of the last chunk, every layer): |x - ref| <= 1e-6 + 1e-5 |ref|   (fp32 path tolerance)
  gradients: |g - ref| <= 1e-6 + 1e-5 * sum|terms|  -- a sum of 131,072 products taken in another order than the reference's loop
  Adam moments and parameters: bit-exact GIVEN the gradient (checked by feeding the GPU's own gradient to the oracle's update), and
  against the fixture within alpha (the first Adam step moves every parameter by at most alpha = 1e-3 times a factor that depends
  smoothly on the gradient: |dp| <= alpha * |dg| / (|g| + eps)).
"""
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-6
DIMS = [256, 256, 256, 16]


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


@pytest.fixture(scope="module")
def fix():
    return np.load(os.path.join(GOLDEN, "c5_chunked_b65536.npz"))


@pytest.fixture(scope="module")
def stepped(lib, torch):
    """Runs the chunked step once on the GPU and returns host copies of everything the tests look at."""
    from rl_tools_b200 import parallel
    params, x, target = mg.c5_inputs()
    net = lib.Mlp(64, DIMS, ["relu", "relu", "relu", "identity"], mg.C5_CHUNK)
    net.params.copy_(torch.from_numpy(params))
    xd, yd = torch.from_numpy(x).cuda(), torch.from_numpy(target).cuda()
    rows = x.shape[0]
    # sharded_train_step without its final step(), so that the gradient can be read before Adam consumes it
    net.zero_gradient()
    w = parallel.chunk_loss_weight(net.batch, rows)
    for c in range(0, rows, net.batch):
        out = net.forward(xd[c:c + net.batch])
        d_out = lib.mse_gradient(out, yd[c:c + net.batch], w, d_a=net.d_out_buffer())
        net.backward(xd[c:c + net.batch], d_out)
    torch.cuda.synchronize()
    res = dict(grads=net.grads.cpu().numpy().copy(), pre=net.pre.cpu().numpy().copy(), out=net.out.cpu().numpy().copy(), params0=params)
    net.step()
    torch.cuda.synchronize()
    res.update(params=net.params.cpu().numpy().copy(), m=net.m.cpu().numpy().copy(), v=net.v.cpu().numpy().copy())
    state = np.zeros(1, np.int32)
    assert lib.lib().b200rl_device_error_state(state.ctypes.data) == 0 and state[0] == 0
    return res


def test_activations_of_the_last_chunk(stepped, fix):
    off = 0
    rows = fix["act_rows"]
    for l, d in enumerate(DIMS):
        for k in ("pre", "out"):
            got = stepped[k][off:off + mg.C5_CHUNK * d].reshape(mg.C5_CHUNK, d)[rows]
            want = fix[f"{k}_{l}"]
            err = np.abs(got.astype(np.float64) - want)
            assert np.all(err <= ATOL + RTOL * np.abs(want)), (k, l, err.max())
        off += mg.C5_CHUNK * d


def test_activations_against_the_oracle_on_sampled_rows(stepped, orc):
    """Rows are independent in the forward pass, so the oracle's forward on a sample of rows of the last chunk is the full-size answer."""
    params, x, _ = mg.c5_inputs()
    rows = np.arange(7, mg.C5_CHUNK, 509)
    xs = np.ascontiguousarray(x[mg.C5_CHUNK * (mg.C5_CHUNKS - 1):][rows])
    pre, out = orc.mlp_forward(oracle.C5_SHAPE(), params, xs)
    off_s = off = 0
    for d in DIMS:
        for got_all, want_all in ((stepped["pre"], pre), (stepped["out"], out)):
            got = got_all[off:off + mg.C5_CHUNK * d].reshape(mg.C5_CHUNK, d)[rows]
            want = want_all[off_s:off_s + rows.size * d].reshape(rows.size, d)
            assert np.all(np.abs(got.astype(np.float64) - want) <= ATOL + RTOL * np.abs(want))
        off += mg.C5_CHUNK * d; off_s += rows.size * d


def test_accumulated_gradient(stepped, fix):
    got = stepped["grads"][::mg.C5_STRIDE].astype(np.float64)
    want, scale = fix["grads"].astype(np.float64), fix["grad_scale"].astype(np.float64)
    excess = np.abs(got - want) - (ATOL + RTOL * scale)
    assert np.all(excess <= 0), f"worst excess {excess.max():.3e} at sampled element {int(np.argmax(excess))}"
    # the whole arena through its sum: bounded by the sum of the per-element bounds (taken from the sampled scale, times the stride)
    total = stepped["grads"].astype(np.float64).sum()
    assert abs(total - float(fix["grads_sum"])) <= mg.C5_STRIDE * (ATOL * want.size + RTOL * scale.sum())


def test_adam_step_is_bit_exact_given_the_gradient(stepped, orc):
    g = stepped["grads"]
    c1, c2, _ = orc.adam_bias_correction(0.9, 0.999, 1)
    p, m, v = orc.adam_update(stepped["params0"], g, np.zeros_like(g), np.zeros_like(g), 1e-3, 0.9, 0.999, 1e-7, 1e-7, c1, c2)
    assert np.array_equal(stepped["m"], m) and np.array_equal(stepped["v"], v) and np.array_equal(stepped["params"], p)


def test_parameters_and_moments_against_the_reference(stepped, fix):
    s = mg.C5_STRIDE
    scale = fix["grad_scale"].astype(np.float64)
    g_bound = ATOL + RTOL * scale
    # m = (1 - beta_1) g: the gradient's bound scaled by 0.1 (+ one rounding)
    assert np.all(np.abs(stepped["m"][::s].astype(np.float64) - fix["m"]) <= 0.1 * g_bound + 1e-12)
    # v = (1 - beta_2) g^2 with 1 - beta_2 = 1e-3: d(g^2) = (2 |g| + dg) dg
    g = np.abs(fix["grads"].astype(np.float64))
    assert np.all(np.abs(stepped["v"][::s].astype(np.float64) - fix["v"]) <= 1e-3 * (2 * g + g_bound) * g_bound + 1e-20)
    # first step (alpha = 1e-3): p -= alpha * g / (|g| + eps') with eps' >= eps = 1e-7, so |dp| <= alpha * dg / (|g| + eps) + one rounding of p
    dp = np.abs(stepped["params"][::s].astype(np.float64) - fix["params"])
    assert np.all(dp <= 1e-3 * g_bound / (g + 1e-7) + 1.2e-7 * np.abs(fix["params"]) + 1e-9)


@pytest.mark.gpu
def test_c5_gradients_do_not_depend_on_the_chunk_size():
    """The training step accumulates gradients over chunks of the rank's rows; the benchmark's chunk is 2^20 rows, the reference fixtures of this
    file pin chunks of 65,536. One million rows of the C5 network, same parameters and data: the gradient arena accumulated over sixteen
    65,536-row chunks against the one accumulated in a single 2^20-row chunk (every kernel of the step at sixteen times the batch: tile
    counts, split ranges, byte offsets beyond 2^31 in the activation arenas) -- equal up to the order of fp32 sums over the batch."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    from rl_tools_b200 import parallel
    rows, dims, acts = 1 << 20, [256, 256, 256, 16], ["relu", "relu", "relu", "identity"]
    g = torch.Generator(device="cuda"); g.manual_seed(5)
    x, y = torch.randn((rows, 64), device="cuda", generator=g), torch.randn((rows, 16), device="cuda", generator=g)
    grads = []
    for chunk in (65536, rows):
        net = pkg.Mlp(64, dims, acts, chunk)
        gp = torch.Generator(device="cuda"); gp.manual_seed(7)
        off, fan_in = 0, 64
        for d in dims:
            n = d * fan_in + d
            net.params[off:off + n] = (torch.rand(n, device="cuda", generator=gp) * 2 - 1) / fan_in ** 0.5
            off += n; fan_in = d
        net.zero_gradient()
        w = parallel.chunk_loss_weight(chunk, rows)
        for c in range(0, rows, chunk):
            out = net.forward(x[c:c + chunk])
            net.backward(x[c:c + chunk], pkg.mse_gradient(out, y[c:c + chunk], w, d_a=net.d_out_buffer()))
        grads.append(net.grads.double().cpu().numpy())
        del net
    a, b = grads
    scale = np.abs(a).max()
    assert scale > 1e-4 and np.isfinite(b).all()
    assert np.abs(a - b).max() <= 2e-5 * scale, (float(np.abs(a - b).max()), float(scale))

