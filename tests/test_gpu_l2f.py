"""GPU parity of the L2F quadrotor step (b200rl_l2f_steps) through the C ABI: the kernel keeps the reference's association of every expression
and is compiled without multiply-add contraction, so its states equal the reference's CPU step() BIT FOR BIT -- against the fixture written
from the real reference (1 and 50 steps) and against the oracle on a large ragged batch."""
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


@pytest.fixture(scope="module")
def fix():
    return np.load(os.path.join(GOLDEN, "l2f.npz"))


def test_l2f_step_vs_reference_golden(lib, torch, fix):
    states, actions = mg.l2f_inputs()
    params = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    d_actions = torch.from_numpy(actions).cuda()
    for n_steps, key in ((1, "next_1"), (50, "next_50")):
        d_states = torch.from_numpy(states).cuda()
        lib.l2f_steps(params, d_states, d_actions, n_steps)
        assert np.array_equal(d_states.cpu().numpy(), fix[key]), key
    # 50 single-step calls are the same as one call of 50 steps
    d_states = torch.from_numpy(states).cuda()
    for _ in range(50):
        lib.l2f_steps(params, d_states, d_actions, 1)
    assert np.array_equal(d_states.cpu().numpy(), fix["next_50"])


def test_l2f_step_large_ragged_batch_vs_oracle(lib, orc, torch, fix):
    """100,003 quadrotors x 20 steps (the last block partly filled) against the oracle, bit for bit; zero steps and an empty batch change nothing."""
    states, actions = mg.l2f_inputs(100003, seed=3)
    params = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    d_states, d_actions = torch.from_numpy(states).cuda(), torch.from_numpy(actions).cuda()
    lib.l2f_steps(params, d_states, d_actions, 0)
    assert np.array_equal(d_states.cpu().numpy(), states)
    lib.l2f_steps(params, d_states[:0].contiguous(), d_actions[:0].contiguous(), 5)
    lib.l2f_steps(params, d_states, d_actions, 20)
    assert np.array_equal(d_states.cpu().numpy(), orc.l2f_steps(fix["dynamics"], float(fix["dt"]), states, actions, 20))


def test_l2f_state_limits_and_action_clamp(lib, orc, torch, fix):
    """Tight state limits (post_integration clamps position and velocities) and actions far outside [-1, 1] (clamped before the rotor map)."""
    states, actions = mg.l2f_inputs(2048, seed=9)
    actions *= np.float32(10)
    limits = (0.5, 1.0, 3.0)
    params = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]), limits)
    d_states = torch.from_numpy(states).cuda()
    lib.l2f_steps(params, d_states, torch.from_numpy(actions).cuda(), 10)
    got = d_states.cpu().numpy()
    assert np.array_equal(got, orc.l2f_steps(fix["dynamics"], float(fix["dt"]), states, actions, 10, state_limits=np.array(limits, np.float32)))
    assert np.abs(got[:, :3]).max() <= 0.5 and np.abs(got[:, 7:10]).max() <= 1.0 and np.abs(got[:, 10:13]).max() <= 3.0
