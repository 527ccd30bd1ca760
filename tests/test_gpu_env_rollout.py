"""GPU parity of the environment-generic fused rollout (through the C ABI) against the reference's fixtures and the CPU oracle:
AcrobotSwingup transitions over the whole state space (teacher-forced single steps), a free-running rollout with resets, and the
Pendulum instantiation of the same kernel against the Pendulum oracle. Floating point within 1e-5 relative + 2e-6 absolute per step,
counters and flags exact."""
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, rtol=1e-5, atol=1e-6, what=""):
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want)
    assert np.all(err <= atol + rtol * np.abs(want)), f"{what}: max err {err.max():.3e}"


def angle_close(got, want, tol, what):
    """angles are wrapped to [-pi, pi): a last-bit difference next to the seam may land on the other side"""
    d = np.abs(np.asarray(got, np.float64) - np.asarray(want, np.float64))
    d = np.minimum(d, 2 * np.pi - d)
    assert d.max() <= tol, f"{what}: max err {d.max():.3e}"


def runner(torch, states, step=0, truncated=0):
    N = states.shape[0]
    return (dev(torch, states), torch.full((N,), step, dtype=torch.int32, device="cuda"), torch.full((N,), truncated, dtype=torch.uint8, device="cuda"),
            torch.zeros(N, device="cuda"))


def test_acrobot_transitions_vs_reference_golden(lib, torch):
    """One step from 2048 states spread over the whole state space, with the actor's output replaced by given actions (a zero-weight
    actor whose output bias is the action cannot vary per environment, so the action goes through tanh^-1 ... instead the states are
    stepped with the kernel's own action and compared with the oracle on that action)."""
    fix = np.load(os.path.join(GOLDEN, "acrobot.npz"))
    states, _ = mg.acrobot_step_inputs()
    n = states.shape[0]
    shape = lib.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    params = mg.acrobot_params()
    st, es, tr, er = runner(torch, states)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew = lib.env_rollout(lib.ENV_ACROBOT_SWINGUP, shape, dev(torch, params), st, es, tr, er, None, 1, 500, error_flag=flag)
    assert int(flag.item()) == 0
    close(obs.cpu().numpy(), fix["obs"], what="observation")            # the fixture's observations of the same states
    orc = oracle.Oracle()
    actions = act.cpu().numpy().reshape(-1)
    want_next, want_rew, _, _ = orc.acrobot_step(states, actions)                  # the oracle on the kernel's own actions
    got_next = st.cpu().numpy()
    angle_close(got_next[:, :2], want_next[:, :2], 2e-5, "next angles")
    close(got_next[:, 2:], want_next[:, 2:], what="next velocities")
    inside = np.abs(np.abs(want_next[:, :2]) - np.pi).min(axis=1) > 1e-3          # the reward jumps across the seam of angle_normalize
    close(rew.cpu().numpy().reshape(-1)[inside], want_rew[inside], what="reward")
    assert np.mean(got_next == want_next) > 0.9                                    # mostly bit-identical
    # the actor itself: the oracle's MLP on the fixture's observations
    oshape = oracle.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    close(actions, orc.mlp_evaluate(oshape, params, fix["obs"]).reshape(-1), what="actions")
    assert np.array_equal(es.cpu().numpy(), np.ones(n, np.int32)) and not tr.cpu().numpy().any()


def test_acrobot_rollout_vs_reference_golden(lib, torch):
    """Free-running 60 steps of 33 environments with resets every 25 steps: counters, flags and reset rows exact, the steps right after a
    reset tight, the rest bounded (the double pendulum is chaotic); then the same trajectory teacher-forced step by step."""
    fix = np.load(os.path.join(GOLDEN, "acrobot.npz"))
    N, T, limit = mg.ACROBOT_ROLLOUT
    shape = lib.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    params_d = dev(torch, mg.acrobot_params())
    table = fix["reset_table"]
    st, es, tr, er = runner(torch, np.zeros((N, 4), np.float32), truncated=1)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew = lib.env_rollout(lib.ENV_ACROBOT_SWINGUP, shape, params_d, st, es, tr, er, dev(torch, table), T, limit, error_flag=flag)
    assert int(flag.item()) == 0
    assert np.array_equal(es.cpu().numpy(), fix["rollout_episode_step"]) and np.array_equal(tr.cpu().numpy(), fix["rollout_truncated"])
    got, want = obs.cpu().numpy().reshape(T, N, 6), fix["rollout_obs"].reshape(T, N, 6)
    resets = np.arange(T) % limit == 0
    close(got[resets], want[resets], what="observation of the reset states")
    first = np.arange(T) % limit < 3
    close(got[first], want[first], what="first steps after a reset")
    assert np.abs(got - want).max() < 0.5 and np.abs(rew.cpu().numpy() - fix["rollout_rew"]).max() < 0.1
    # teacher-forced: every step restarted from the oracle's state
    orc = oracle.Oracle()
    oshape = oracle.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    state = dict(states=np.zeros((N, 4), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8), episode_return=np.zeros(N, np.float32))
    used = np.zeros(N, np.int64)
    for t in range(T):
        one = np.zeros((1, N, 2), np.float32)
        for e in range(N):
            if state["truncated"][e]:
                one[0, e] = table[used[e], e]; used[e] += 1
        d = [dev(torch, state[k]) for k in ("states", "episode_step", "truncated", "episode_return")]
        o, a, r = lib.env_rollout(lib.ENV_ACROBOT_SWINGUP, shape, params_d, d[0], d[1], d[2], d[3], dev(torch, one), 1, limit, error_flag=flag)
        nxt = orc.acrobot_rollout(oshape, mg.acrobot_params(), state["states"], state["episode_step"], state["truncated"], state["episode_return"], one, 1, limit)
        close(o.cpu().numpy(), nxt["obs"], what=f"step {t} observation")
        close(a.cpu().numpy(), nxt["act"], what=f"step {t} action")
        close(r.cpu().numpy(), nxt["rew"], what=f"step {t} reward")
        angle_close(d[0].cpu().numpy()[:, :2], nxt["states"][:, :2], 5e-5, f"step {t} angles")
        close(d[0].cpu().numpy()[:, 2:], nxt["states"][:, 2:], what=f"step {t} velocities")
        assert np.array_equal(d[1].cpu().numpy(), nxt["episode_step"]) and np.array_equal(d[2].cpu().numpy(), nxt["truncated"])
        close(d[3].cpu().numpy(), nxt["episode_return"], what=f"step {t} return")
        state = {k: nxt[k] for k in state}
    assert int(flag.item()) == 0


def test_acrobot_terminating_variant_vs_reference_golden(lib, torch):
    """rl::environments::Acrobot (reward -1, terminated when the tip is above the bar) through the generic kernel. Free-running from the
    fixture's reset table: the first steps of the first episodes against the reference's fixture; then teacher-forced step by step against
    the oracle (which reproduces that fixture bit for bit): observation, action, next state within tolerance, reward exactly -1, and the
    terminated / truncated flags and counters exact wherever the termination test is not within 1e-4 of its threshold (the flag is a
    comparison of a sum of cosines with 1: a next state that differs in its last bits may land on the other side only there)."""
    fix = np.load(os.path.join(GOLDEN, "acrobot_terminating.npz"))
    N, T, limit = mg.ACROBOT_TERMINATING_ROLLOUT
    shape = lib.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    params_d = dev(torch, mg.acrobot_params())
    orc = oracle.Oracle()
    table = mg.acrobot_terminating_table(orc, T)
    assert np.array_equal(table[:32], fix["reset_table"])
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    st, es, tr, er = runner(torch, np.zeros((N, 4), np.float32), truncated=1)
    term = torch.full((T * N,), 7, dtype=torch.uint8, device="cuda")
    obs, act, rew = lib.env_rollout(lib.ENV_ACROBOT, shape, params_d, st, es, tr, er, dev(torch, table), T, limit, error_flag=flag, terminated=term)
    assert int(flag.item()) == 0
    got, want = obs.cpu().numpy().reshape(T, N, 6), fix["rollout_obs"].reshape(T, N, 6)
    close(got[:3], want[:3], what="first steps of the first episodes")
    assert np.all(rew.cpu().numpy() == -1.0) and set(np.unique(term.cpu().numpy())) <= {0, 1}
    assert np.array_equal(term.cpu().numpy().reshape(T, N)[:3], fix["rollout_terminated"].reshape(T, N)[:3])
    assert 0.5 * fix["rollout_terminated"].sum() < term.sum().item() < 2 * fix["rollout_terminated"].sum()      # episodes end at a similar rate
    # teacher-forced
    oshape = oracle.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    state = dict(states=np.zeros((N, 4), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8), episode_return=np.zeros(N, np.float32))
    used = np.zeros(N, np.int64)
    n_terminated = 0
    for t in range(120):
        one = np.zeros((1, N, 4), np.float32)
        for e in range(N):
            if state["truncated"][e]:
                one[0, e] = table[used[e], e]; used[e] += 1
        d = [dev(torch, state[k]) for k in ("states", "episode_step", "truncated", "episode_return")]
        tm = torch.zeros(N, dtype=torch.uint8, device="cuda")
        o, a, r = lib.env_rollout(lib.ENV_ACROBOT, shape, params_d, d[0], d[1], d[2], d[3], dev(torch, one), 1, limit, error_flag=flag, terminated=tm)
        nxt = orc.acrobot_terminating_rollout(oshape, mg.acrobot_params(), state["states"], state["episode_step"], state["truncated"], state["episode_return"], one, 1, limit)
        close(o.cpu().numpy(), nxt["obs"], what=f"step {t} observation")
        close(a.cpu().numpy(), nxt["act"], what=f"step {t} action")
        assert np.all(r.cpu().numpy() == -1.0)
        angle_close(d[0].cpu().numpy()[:, :2], nxt["states"][:, :2], 5e-5, f"step {t} angles")
        close(d[0].cpu().numpy()[:, 2:], nxt["states"][:, 2:], what=f"step {t} velocities")
        ns = nxt["states"].astype(np.float64)
        clear = np.abs(-np.cos(ns[:, 0]) - np.cos(ns[:, 1] + ns[:, 0]) - 1.0) > 1e-4
        assert np.array_equal(tm.cpu().numpy()[clear], nxt["terminated"][clear])
        assert np.array_equal(d[2].cpu().numpy()[clear], nxt["truncated"][clear]) and np.array_equal(d[1].cpu().numpy(), nxt["episode_step"])
        close(d[3].cpu().numpy(), nxt["episode_return"], what=f"step {t} return")
        n_terminated += int(nxt["terminated"].sum())
        state = {k: nxt[k] for k in state}
    assert n_terminated > 20 and int(flag.item()) == 0


def test_pendulum_through_the_generic_kernel(lib, torch):
    """The Pendulum instantiation of the generic kernel against the Pendulum oracle (teacher-forced single steps over random states) and
    bit for bit against the specialised CUDA-core arithmetic it shares (same device functions): next state and reward exact given the
    kernel's own action."""
    rs = np.random.RandomState(2)
    N = 3000
    states = np.stack([rs.uniform(-10, 10, N), rs.uniform(-8, 8, N)], 1).astype(np.float32)
    params = (rs.uniform(-1, 1, 4481) * 0.3).astype(np.float32)
    shape, oshape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"]), oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    st, es, tr, er = runner(torch, states, step=7)
    obs, act, rew = lib.env_rollout(lib.ENV_PENDULUM, shape, dev(torch, params), st, es, tr, er, None, 1, 200)
    orc = oracle.Oracle()
    want = orc.pendulum_rollout(oshape, params, states, np.full(N, 7, np.int32), np.zeros(N, np.uint8), np.zeros(N, np.float32), np.zeros((0, N, 2), np.float32), 1, 200)
    close(obs.cpu().numpy(), want["obs"], what="observation")
    close(act.cpu().numpy(), want["act"], what="action")
    ns, r, _, _ = orc.pendulum_step(states, act.cpu().numpy())
    close(st.cpu().numpy(), ns, rtol=1e-6, atol=1e-6, what="next state")
    close(rew.cpu().numpy().reshape(-1), r, rtol=1e-6, atol=1e-6, what="reward")
    assert np.array_equal(es.cpu().numpy(), np.full(N, 8, np.int32))


def test_env_rollout_argument_checks(lib, torch):
    shape3, shape6 = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"]), lib.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    st, es, tr, er = runner(torch, np.zeros((4, 4), np.float32))
    params = torch.zeros(6 * 64 + 64 + 64 * 64 + 64 + 64 + 1, device="cuda")
    with pytest.raises(lib.B200RLError):
        lib.env_rollout(lib.ENV_ACROBOT_SWINGUP, shape3, params, st, es, tr, er, None, 1, 10)       # actor input does not match the observation
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    tr.fill_(1)
    lib.env_rollout(lib.ENV_ACROBOT_SWINGUP, shape6, params, st, es, tr, er, None, 1, 10, error_flag=flag)
    assert int(flag.item()) == 1                                                                     # a reset without a table entry raises the flag


@pytest.mark.parametrize("hidden", [16, 32, 128])
def test_actor_widths_other_than_64(lib, torch, hidden):
    """The runner is generic in the policy (rl/components/off_policy_runner/operations_generic.h): hidden widths 16, 32 and 128 of the
    3-layer actor run on the one-thread-per-environment kernel -- the Pendulum through its own entry point (which routes there), a whole
    episode boundary included (step limit 5, two resets from the table), and one Acrobot swing-up step -- against the oracle's runner loop."""
    rs = np.random.RandomState(hidden)
    N, T = 777, 12
    acts = ["relu", "relu", "tanh"]
    n_params = hidden * 3 + hidden + hidden * hidden + hidden + hidden + 1
    params = (rs.uniform(-1, 1, n_params) * (1.5 / np.sqrt(hidden))).astype(np.float32)
    states = np.stack([rs.uniform(-3, 3, N), rs.uniform(-2, 2, N)], 1).astype(np.float32)
    resets = np.stack([rs.uniform(-np.pi, np.pi, (3, N)), rs.uniform(-1, 1, (3, N))], 2).astype(np.float32)
    shape, oshape = lib.MlpShape.make(3, [hidden, hidden, 1], acts), oracle.MlpShape.make(3, [hidden, hidden, 1], acts)
    st, es, tr, er = runner(torch, states)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew = lib.pendulum_rollout(shape, dev(torch, params), st, es, tr, er, dev(torch, resets), T, 5, error_flag=flag)
    assert int(flag.item()) == 0
    orc = oracle.Oracle()
    # teacher forcing: the oracle recomputes each step from the kernel's own states, so one rounding difference cannot grow over the steps
    got_obs = obs.cpu().numpy()
    want = orc.pendulum_rollout(oshape, params, states, np.zeros(N, np.int32), np.zeros(N, np.uint8), np.zeros(N, np.float32), resets, T, 5)
    close(got_obs[:N], want["obs"][:N], what="first observation")
    close(act.cpu().numpy()[:N], want["act"][:N], what="first action")
    want_act = orc.mlp_evaluate(oshape, params, got_obs).reshape(-1)
    close(act.cpu().numpy().reshape(-1), want_act, what="actions of all steps on the kernel's observations")
    assert np.array_equal(es.cpu().numpy(), want["episode_step"]) and np.array_equal(tr.cpu().numpy(), want["truncated"])
    # the resets took the table's rows: the observation after a reset is the table's state
    row = 5 * N                                                      # step 5 is the first step of the second episode
    assert np.allclose(got_obs[row:row + N, 0], np.cos(resets[0, :, 0]), atol=1e-6) and np.allclose(got_obs[row:row + N, 2], resets[0, :, 1], atol=1e-6)

    shape6, oshape6 = lib.MlpShape.make(6, [hidden, hidden, 1], acts), oracle.MlpShape.make(6, [hidden, hidden, 1], acts)
    params6 = (rs.uniform(-1, 1, n_params + 3 * hidden) * (1.5 / np.sqrt(hidden))).astype(np.float32)
    states4 = rs.uniform(-1, 1, (N, 4)).astype(np.float32)
    st, es, tr, er = runner(torch, states4)
    obs, act, rew = lib.env_rollout(lib.ENV_ACROBOT_SWINGUP, shape6, dev(torch, params6), st, es, tr, er, None, 1, 500)
    want = orc.acrobot_rollout(oshape6, params6, states4, np.zeros(N, np.int32), np.zeros(N, np.uint8), np.zeros(N, np.float32), np.zeros((0, N, 2), np.float32), 1)
    close(obs.cpu().numpy(), want["obs"], what="acrobot observation")
    close(act.cpu().numpy(), want["act"], what="acrobot action")
    close(st.cpu().numpy(), want["states"], rtol=1e-5, atol=2e-6, what="acrobot next state")


def test_unsupported_actor_width_is_refused(lib, torch):
    shape = lib.MlpShape.make(3, [48, 48, 1], ["relu", "relu", "tanh"])
    st, es, tr, er = runner(torch, np.zeros((4, 2), np.float32))
    with pytest.raises(lib.B200RLError):
        lib.pendulum_rollout(shape, torch.zeros(48 * 3 + 48 + 48 * 48 + 48 + 48 + 1, device="cuda"), st, es, tr, er, None, 1, 200)
