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


@pytest.mark.parametrize("hidden", [16, 32, 64])
def test_l2f_rollout_vs_oracle(lib, orc, torch, fix, hidden):
    """The fused runner loop on the quadrotor, 600 environments x 40 steps from the reference sampler's initial states with an episode limit of
    25 (every environment is reset from the table inside the call; environments that drift off terminate earlier): observations, counters and
    flags against the oracle's loop; per step, teacher-forced on the kernel's own trajectory, the action against the oracle's MLP on the
    kernel's observation (fp32 tolerance), the next observation's state part bit for bit and the reward within the GPU's acosf."""
    import oracle
    N, T, limit = 600, 40, 25
    rs = np.random.RandomState(hidden)
    acts = ["tanh", "tanh", "tanh"]
    shape, oshape = lib.MlpShape.make(18, [hidden, hidden, 4], acts), oracle.MlpShape.make(18, [hidden, hidden, 4], acts)
    params = (rs.uniform(-1, 1, oshape.num_params()) * (1.0 / np.sqrt(hidden))).astype(np.float32)
    init = fix["initial_states"]
    p = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    st, es, er = dev(np.zeros((N, 23), np.float32)), torch.zeros(N, dtype=torch.int32, device="cuda"), torch.zeros(N, device="cuda")
    tr = torch.ones(N, dtype=torch.uint8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew, term = lib.l2f_rollout(p, fix["mdp"], shape, dev(params), st, es, tr, er, dev(init), T, limit, error_flag=flag)
    assert int(flag.item()) == 0
    obs, act, rew, term = (x.cpu().numpy() for x in (obs, act, rew, term))
    want = orc.l2f_rollout(oshape, params, fix["dynamics"], float(fix["dt"]), fix["mdp"], np.zeros((N, 23), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8),
                           np.zeros(N, np.float32), init, T, limit)
    assert np.array_equal(obs[:N], want["obs"][:N])                                     # first step: the table's states, bit for bit
    tol = lambda got, ref, rtol=1e-5, atol=1e-6: np.all(np.abs(got.astype(np.float64) - ref.astype(np.float64)) <= atol + rtol * np.abs(ref))
    assert tol(act.reshape(-1), orc.mlp_evaluate(oshape, params, obs).reshape(-1))      # every step's action on the kernel's own observation
    # teacher forcing: rebuild each step's state from the kernel's outputs is not possible from 18 observation values alone (rotor speeds and
    # disturbances are hidden), so the trajectories are compared directly: the dynamics are bit-exact, only the action's last bits differ
    assert tol(obs, want["obs"], rtol=1e-4, atol=1e-5)
    assert np.array_equal(term, want["terminated"]) and np.array_equal(es.cpu().numpy(), want["episode_step"]) and np.array_equal(tr.cpu().numpy(), want["truncated"])
    assert tol(rew, want["rew"], rtol=1e-4, atol=1e-5)
    assert tol(st.cpu().numpy(), want["states"], rtol=1e-4, atol=1e-5) and tol(er.cpu().numpy(), want["episode_return"], rtol=1e-4, atol=1e-4)
    assert term.sum() > 0 and (want["episode_step"] < T).all()


@pytest.mark.parametrize("N", [1, 31, 449])
def test_l2f_rollout_ragged_environment_counts(lib, orc, torch, fix, N):
    """Environment counts that leave most of a warp, or of the second CTA, idle: the idle lanes take part in their warp's tiles without
    touching memory. Same checks as the full-size case, 8 steps with an episode limit of 5."""
    import oracle
    T, limit, hidden = 8, 5, 16
    rs = np.random.RandomState(N)
    acts = ["relu", "tanh", "tanh"]
    shape, oshape = lib.MlpShape.make(18, [hidden, hidden, 4], acts), oracle.MlpShape.make(18, [hidden, hidden, 4], acts)
    params = (rs.uniform(-1, 1, oshape.num_params()) * 0.25).astype(np.float32)
    init = np.ascontiguousarray(fix["initial_states"][:2, :N])
    p = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    guard = 64                                                    # rows behind the outputs must stay untouched
    obs = torch.full((T * N + guard, 18), 7.0, device="cuda"); act = torch.full((T * N + guard, 4), 7.0, device="cuda")
    rew = torch.full((T * N + guard,), 7.0, device="cuda"); term = torch.full((T * N + guard,), 7, dtype=torch.uint8, device="cuda")
    st, es, er = torch.zeros((N, 23), device="cuda"), torch.zeros(N, dtype=torch.int32, device="cuda"), torch.zeros(N, device="cuda")
    tr = torch.ones(N, dtype=torch.uint8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.l2f_rollout(p, fix["mdp"], shape, torch.from_numpy(params).cuda(), st, es, tr, er, torch.from_numpy(init).cuda(), T, limit, obs=obs, act=act, rew=rew, terminated=term,
                    error_flag=flag)
    assert int(flag.item()) == 0
    assert bool((obs[T * N:] == 7).all()) and bool((act[T * N:] == 7).all()) and bool((rew[T * N:] == 7).all()) and bool((term[T * N:] == 7).all())
    want = orc.l2f_rollout(oshape, params, fix["dynamics"], float(fix["dt"]), fix["mdp"], np.zeros((N, 23), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8),
                           np.zeros(N, np.float32), init, T, limit)
    o, a_ = obs[:T * N].cpu().numpy(), act[:T * N].cpu().numpy()
    assert np.array_equal(o[:N], want["obs"][:N])
    ref_act = orc.mlp_evaluate(oshape, params, o)
    assert np.all(np.abs(a_.astype(np.float64) - ref_act) <= 1e-6 + 1e-5 * np.abs(ref_act))
    assert np.all(np.abs(o.astype(np.float64) - want["obs"]) <= 1e-5 + 1e-4 * np.abs(want["obs"]))
    assert np.array_equal(term[:T * N].cpu().numpy(), want["terminated"]) and np.array_equal(es.cpu().numpy(), want["episode_step"])


def test_l2f_rollout_argument_checks(lib, torch, fix):
    p = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    st, es, er = torch.zeros((4, 23), device="cuda"), torch.zeros(4, dtype=torch.int32, device="cuda"), torch.zeros(4, device="cuda")
    tr = torch.ones(4, dtype=torch.uint8, device="cuda")
    bad = lib.MlpShape.make(18, [48, 48, 4], ["relu", "relu", "tanh"])
    with pytest.raises(lib.B200RLError):
        lib.l2f_rollout(p, fix["mdp"], bad, torch.zeros(8000, device="cuda"), st, es, tr, er, None, 3)
    shape = lib.MlpShape.make(18, [16, 16, 4], ["relu", "relu", "tanh"])
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.l2f_rollout(p, fix["mdp"], shape, torch.zeros(18 * 16 + 16 + 16 * 16 + 16 + 64 + 4, device="cuda"), st, es, tr, er, None, 3, error_flag=flag)
    assert int(flag.item()) == 1                                                        # a reset without a table entry raises the flag


def test_l2f_initial_states_from_draws_vs_oracle(lib, orc, torch, fix):
    """sample_initial_state as a function of its draws on the device against the oracle (which equals the reference bit for bit): everything
    but the orientation bit for bit, the orientation within the GPU's sinf / cosf; the default distribution, one whose disturbances have a
    spread, and absolute rotor-speed bounds."""
    rs = np.random.RandomState(12)
    n = 5000
    u, nrm = rs.uniform(0, 1, (n, 17)).astype(np.float32), rs.randn(n, 6).astype(np.float32)
    p = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    spread = fix["init"].copy(); spread[8:12] = (0.01, 0.02, -0.001, 0.003)
    absolute = spread.copy(); absolute[5:8] = (0.0, 0.2, 3.0); absolute[2] = 0.0        # rpm 0.2 .. min(3, action max), no orientation draw
    for init in (fix["init"], spread, absolute):
        want = orc.l2f_initial_states_from_draws(init, fix["dynamics"], u, nrm)
        got = lib.l2f_initial_states_from_draws(p, init, torch.from_numpy(u).cuda(), torch.from_numpy(nrm).cuda()).cpu().numpy()
        rest = [c for c in range(23) if not 3 <= c < 7]
        assert np.array_equal(got[:, rest], want[:, rest])
        assert np.abs(got[:, 3:7] - want[:, 3:7]).max() <= 1e-6


def test_l2f_rollout_with_device_side_resets(lib, torch, fix):
    """Resets drawn in the kernel: the first observations follow the reference's initial-state distribution (a tenth of the quadrotors start
    at the origin at rest, the others inside the position / velocity bounds with a proper rotation matrix, moments of a uniform
    distribution); the draws are a function of (seed, environment, first_step + step) only: the same seed repeats, another seed differs,
    and a call starting at step 10 resets to the states the first call drew at its step 10."""
    N, T, limit, H = 8192, 12, 10, 32
    rs = np.random.RandomState(5)
    shape = lib.MlpShape.make(18, [H, H, 4], ["relu", "relu", "tanh"])
    params = torch.from_numpy((rs.uniform(-1, 1, shape.num_params()) * 0.02).astype(np.float32)).cuda()
    p = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    init = fix["init"]

    def run(seed, first_step, steps):
        st, es, er = torch.zeros((N, 23), device="cuda"), torch.zeros(N, dtype=torch.int32, device="cuda"), torch.zeros(N, device="cuda")
        tr = torch.ones(N, dtype=torch.uint8, device="cuda")
        obs, act, rew, term = lib.l2f_rollout_device_rng(p, fix["mdp"], init, shape, params, st, es, tr, er, seed, first_step, steps, limit)
        return obs.cpu().numpy().reshape(steps, N, 18), term.cpu().numpy().reshape(steps, N)

    obs, term = run(77, 0, T)
    first = obs[0]
    guided = np.all(first[:, :3] == 0, axis=1)
    assert 0.08 < guided.mean() < 0.12
    assert np.all(first[guided, 12:] == 0) and np.all(first[guided, 3:12] == np.eye(3, dtype=np.float32).reshape(-1))
    free = first[~guided]
    assert np.all(np.abs(free[:, :3]) <= init[1]) and np.all(np.abs(free[:, 12:15]) <= init[3]) and np.all(np.abs(free[:, 15:]) <= init[4])
    R = free[:, 3:12].reshape(-1, 3, 3).astype(np.float64)
    assert np.abs(R @ R.transpose(0, 2, 1) - np.eye(3)).max() < 1e-5
    assert np.abs(free[:, :3].mean(axis=0)).max() < 0.02 and np.abs(free[:, :3].var(axis=0) - init[1] ** 2 / 3).max() < 0.01
    # rotation angle uniform in [0, 1) rad about a uniform axis: trace = 1 + 2 cos(angle)
    angle = np.arccos(np.clip((np.trace(R, axis1=1, axis2=2) - 1) / 2, -1, 1))
    assert angle.max() <= 1.0 + 1e-3 and abs(angle.mean() - 0.5) < 0.02
    again, _ = run(77, 0, T)
    other, _ = run(78, 0, T)
    assert np.array_equal(obs, again) and not np.array_equal(obs[0], other[0])
    whole = ~term[:limit].any(axis=0)                     # no termination in the first episode: these reset exactly at step 10
    assert whole.sum() > N // 2
    shifted, _ = run(77, limit, 1)
    assert np.array_equal(shifted[0][whole], obs[limit][whole])


def test_l2f_offpolicy_step_halves_with_replay_buffers(lib, orc, torch, fix):
    """The off-policy runner step on the quadrotor in two halves around given actions, 40 steps of 200 environments with an episode limit of
    7, replay buffers of 16 rows (they wrap) and some initial states pushed beyond the termination threshold: per step the observations
    and next observations bit for bit against the oracle's functions under the runner's bookkeeping (restated here in numpy); at the end
    every replay row (reward column within the GPU's acosf), episode starts, positions, full flags and the runner counters."""
    N, T, limit, cap = 200, 40, 7, 16
    rs = np.random.RandomState(3)
    dyn, dt, mdp = fix["dynamics"], float(fix["dt"]), fix["mdp"]
    pool = fix["initial_states"].reshape(-1, 23).copy()
    pool[::5, :3] *= np.float32(4.0)                                   # a fifth of the resets start far out: many of them beyond the position threshold of 1 after one step
    p = lib.L2fParameters.make(dyn, dt)
    layout = lib.ReplayLayout.packed(cap, 18, 4)
    assert layout.ld_data == 43
    replay = torch.zeros(N * layout.env_stride, dtype=torch.uint8, device="cuda")
    st, es, er = torch.zeros((N, 23), device="cuda"), torch.zeros(N, dtype=torch.int32, device="cuda"), torch.zeros(N, device="cuda")
    tr, was = torch.ones(N, dtype=torch.uint8, device="cuda"), torch.zeros(N, dtype=torch.uint8, device="cuda")
    obs_d, nobs_d = torch.zeros((N, 18), device="cuda"), torch.zeros((N, 18), device="cuda")
    # the runner's bookkeeping in numpy
    h_st, h_es, h_er, h_tr = np.zeros((N, 23), np.float32), np.zeros(N, np.int32), np.zeros(N, np.float32), np.ones(N, bool)
    data, ep_start = np.zeros((N, cap, 43), np.float32), np.zeros((N, cap), np.uint32)
    pos, ces, full = np.zeros(N, np.int64), np.zeros(N, np.int64), np.zeros(N, bool)
    terminations = 0
    for t in range(T):
        table = pool[(t * N + np.arange(N)) % pool.shape[0]]
        actions = rs.uniform(-1, 1, (N, 4)).astype(np.float32)
        lib.l2f_offpolicy_prologue(p, st, es, tr, er, obs_d, was, reset_states=torch.from_numpy(table).cuda())
        lib.l2f_offpolicy_epilogue(p, mdp, st, es, tr, er, limit, torch.from_numpy(actions).cuda(), nobs_d, replay, layout, was)
        h_was = h_tr.copy()
        h_st[h_tr] = table[h_tr]; h_es[h_tr] = 0; h_er[h_tr] = 0
        nxt = orc.l2f_steps(dyn, dt, h_st, actions, 1)
        obs, rew, term = orc.l2f_functions(dyn, dt, mdp, h_st, actions, nxt)
        nobs = orc.l2f_functions(dyn, dt, mdp, nxt, actions, nxt)[0]
        h_es += 1; h_er += rew
        term = term.astype(bool); trunc = term | (h_es == limit)
        terminations += int(term.sum())
        for e in range(N):
            if h_was[e] and (full[e] or pos[e] > 0):
                data[e, (pos[e] - 1) % cap, 42] = 1.0
                ces[e] = pos[e]
            data[e, pos[e]] = np.concatenate([obs[e], actions[e], [rew[e]], nobs[e], [float(term[e])], [float(trunc[e])]])
            ep_start[e, pos[e]] = ces[e]
            pos[e] = (pos[e] + 1) % cap
            if trunc[e]: ces[e] = pos[e]
            if pos[e] == 0 and not full[e]: full[e] = True
        h_st, h_tr = nxt, trunc
        assert np.array_equal(obs_d.cpu().numpy(), obs) and np.array_equal(nobs_d.cpu().numpy(), nobs), t
        assert np.array_equal(tr.cpu().numpy().astype(bool), trunc) and np.array_equal(es.cpu().numpy(), h_es), t
    assert terminations > 50 and full.all()
    raw = replay.cpu().numpy().reshape(N, layout.env_stride)
    g_data = raw[:, layout.off_data:layout.off_data + 4 * 43 * cap].copy().view(np.float32).reshape(N, cap, 43)
    g_start = raw[:, layout.off_episode_start:layout.off_episode_start + 4 * cap].copy().view(np.uint32).reshape(N, cap)
    g_pos = raw[:, layout.off_position:layout.off_position + 4].copy().view(np.uint32).reshape(N)
    g_ces = raw[:, layout.off_current_episode_start:layout.off_current_episode_start + 4].copy().view(np.uint32).reshape(N)
    exact = [c for c in range(43) if c != 22]
    assert np.array_equal(g_data[:, :, exact], data[:, :, exact])
    assert np.abs(g_data[:, :, 22] - data[:, :, 22]).max() <= 1e-5
    assert np.array_equal(g_start, ep_start) and np.array_equal(g_pos, pos) and np.array_equal(g_ces, ces) and np.all(raw[:, layout.off_full] == 1)
    assert np.array_equal(st.cpu().numpy(), h_st) and np.abs(er.cpu().numpy() - h_er).max() <= 1e-4

