"""GPU parity of the SAC update pieces through the C ABI: the sample-and-squash policy head against the golden outputs of the
reference's layer (forward with external noise, backward_full), the critic target and the min-value gradient selection against
float32 restatements of the reference's lines. Tolerance for floating point: 1e-5 relative + 1e-6 absolute."""
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


@pytest.mark.parametrize("case", range(len(oracle.Reference.SAS_CASES)))
def test_sample_and_squash_vs_reference_golden(lib, torch, case):
    fix = np.load(os.path.join(GOLDEN, "sample_and_squash.npz"))
    inp, noise, d_output = mg.sas_inputs(case)
    B, A = noise.shape
    inp_d, noise_d = dev(torch, inp), dev(torch, noise)
    output, pre, logp = lib.sample_and_squash_forward(inp_d, noise_d)
    close(pre.cpu().numpy(), fix[f"pre_squashing_{case}"], what="pre_squashing")
    close(output.cpu().numpy(), fix[f"output_{case}"], what="output")
    close(logp.cpu().numpy(), fix[f"log_probs_{case}"], what="log_probs")
    exact = np.mean(output.cpu().numpy() == fix[f"output_{case}"])
    assert exact > 0.5, exact                      # the host libm's tanhf is within one ulp of the correctly rounded value the kernel produces
    log_alpha = dev(torch, np.array([mg.SAS_LOG_ALPHA], np.float32))
    grad = torch.full((1,), 0.25, device="cuda")                # the gradient accumulates
    d_input, per_sample = lib.sample_and_squash_backward(inp_d, noise_d, pre, output, dev(torch, d_output), log_alpha, log_alpha_gradient=grad)
    close(d_input.cpu().numpy(), fix[f"d_input_{case}"], what="d_input")
    close(per_sample.cpu().numpy(), fix[f"d_log_alpha_per_sample_{case}"], what="d_log_alpha_per_sample")
    close(grad.item() - 0.25, fix[f"log_alpha_gradient_{case}"], what="log_alpha gradient")
    # clamped rows: no log_std gradient
    assert d_input.cpu().numpy()[0, A] == 0 and d_input.cpu().numpy()[1 % B, 2 * A - 1] == 0
    # strided views: input inside a wider matrix, output into a column block
    wide_in = torch.zeros((B, 2 * A + 5), device="cuda"); wide_in[:, 2:2 + 2 * A] = inp_d
    wide_out = torch.full((B, A + 3), 9.0, device="cuda")
    lib.sample_and_squash_forward(wide_in[:, 2:2 + 2 * A], noise_d, output=wide_out[:, 3:])
    assert torch.equal(wide_out[:, 3:], output) and bool((wide_out[:, :3] == 9).all())


@pytest.mark.parametrize("bonus,next_step,ignore", [(True, True, False), (True, False, False), (False, True, True), (True, True, True)])
def test_target_action_values(lib, torch, bonus, next_step, ignore):
    """rl/algorithms/sac/operations_generic.h:133-163 in float32."""
    rs = np.random.RandomState(3)
    B = 300
    q1, q2 = rs.randn(B, 1).astype(np.float32) * 10, rs.randn(B, 1).astype(np.float32) * 10
    rew, logp = rs.randn(B).astype(np.float32), rs.randn(B).astype(np.float32) * 3
    term = (rs.rand(B) < 0.3).astype(np.uint8)
    log_alpha, gamma = np.float32(-0.7), np.float32(0.99)
    got = lib.sac_target_action_values(dev(torch, q1), dev(torch, q2), dev(torch, rew), dev(torch, term), dev(torch, logp), dev(torch, np.array([log_alpha])),
                                       gamma=float(gamma), ignore_termination=ignore, entropy_bonus=bonus, entropy_bonus_next_step=next_step).cpu().numpy()[:, 0]
    alpha = np.float32(np.exp(np.float64(log_alpha)))
    m = np.minimum(q1[:, 0], q2[:, 0])
    entropy_bonus = -alpha * logp
    if bonus and next_step:
        m = m + entropy_bonus
    future = np.where(ignore | (term == 0), gamma * m, np.float32(0)).astype(np.float32)
    want = rew + future
    if bonus and not next_step:
        want = want + entropy_bonus
    assert np.array_equal(got, want.astype(np.float32))


def test_min_value_d_output(lib, torch):
    rs = np.random.RandomState(4)
    B, O, A = 257, 5, 3
    q1, q2 = rs.randn(B, 1).astype(np.float32), rs.randn(B, 1).astype(np.float32)
    q2[:7] = q1[:7]                                            # ties take critic 2 (strict <)
    d1, d2 = rs.randn(B, O + A).astype(np.float32), rs.randn(B, O + A).astype(np.float32)
    got = lib.sac_min_value_d_output(dev(torch, q1), dev(torch, q2), dev(torch, d1), dev(torch, d2), A).cpu().numpy()
    want = np.where(q1 < q2, d1[:, O:], d2[:, O:])
    assert np.array_equal(got, want)


def build_agent(lib, torch, case, updates):
    from rl_tools_b200 import sac
    B, H = oracle.Reference.SAC_CASES[case]
    actor_p, log_alpha, critic_p, target_p, oa, rew, term, noise_c, noise_a = mg.sac_inputs(case, updates)
    agent = sac.ActorCritic(3, 1, H, B)
    agent.actor.params.copy_(dev(torch, actor_p))
    agent.log_alpha.fill_(float(log_alpha))
    for c in range(2):
        agent.critics[c].params.copy_(dev(torch, critic_p[c]))
        agent.critics_target[c].params.copy_(dev(torch, target_p[c]))
    batches = [dict(oa_base=dev(torch, oa[u]), rewards=dev(torch, rew[u]), terminated=dev(torch, term[u])) for u in range(updates)]
    return agent, batches, dev(torch, noise_c), dev(torch, noise_a)


def scale_close(got, want, tol=2e-5, what=""):
    """within tol of the tensor's scale (gradients of a 256-row batch summed in another order than the reference's loops)"""
    got, want = np.asarray(got, np.float64), np.asarray(want, np.float64)
    err = np.abs(got - want).max()
    assert err <= tol * max(np.abs(want).max(), 1e-6), f"{what}: max err {err:.3e} against scale {np.abs(want).max():.3e}"


@pytest.mark.parametrize("case", range(len(oracle.Reference.SAC_CASES)))
def test_sac_first_update_vs_reference_golden(lib, torch, case):
    """train_critic (both critics), update_critic_targets, train_actor of rl_tools_b200.sac against what the real reference's functions left
    behind after one update on the same batch and noise: critic target values, every gradient, the Adam moments and the stepped parameters."""
    fix = np.load(os.path.join(GOLDEN, "sac.npz"))
    agent, batches, noise_c, noise_a = build_agent(lib, torch, case, 1)
    agent.update(batches[0], noise_c[0, 0], noise_c[0, 1], noise_a[0])
    f = lambda k: fix[f"{k}_{case}_u1"]
    close(agent.target_action_value.cpu().numpy()[:, 0], f("target_values"), what="target values")
    for c in range(2):
        scale_close(agent.critics[c].grads.cpu().numpy(), f(f"critic{c}_grads"), what=f"critic {c} gradient")
        scale_close(agent.critics[c].m.cpu().numpy(), f(f"critic{c}_m"), what=f"critic {c} first moment")
        close(agent.critics_target[c].params.cpu().numpy(), f(f"target{c}"), what=f"target {c}")
    scale_close(agent.actor.grads.cpu().numpy(), f("actor_grads"), what="actor gradient")
    close(agent.log_alpha_grad.item(), f("log_alpha_grads"), what="log_alpha gradient")
    # first Adam step: |update| = alpha for every element whose gradient is not ~0, sign decided by the gradient
    for name, got, want, grad in (("actor", agent.actor.params, f("actor_params"), f("actor_grads")), ("critic 0", agent.critics[0].params, f("critic0_params"), f("critic0_grads")),
                                  ("critic 1", agent.critics[1].params, f("critic1_params"), f("critic1_grads"))):
        solid = np.abs(grad) > 1e-4 * np.abs(grad).max()
        close(got.cpu().numpy()[solid], want[solid], what=name + " parameters")
    close(agent.log_alpha.item(), f("log_alpha_params"), what="log_alpha")


@pytest.mark.parametrize("case", range(len(oracle.Reference.SAC_CASES)))
def test_sac_updates_vs_reference_golden(lib, torch, case):
    """Three consecutive updates (new batch and noise each) against the reference: parameters within the drift-aware bound of the PPO tests."""
    from test_gpu_ppo import assert_params_close
    fix = np.load(os.path.join(GOLDEN, "sac.npz"))
    U = mg.SAC_UPDATES
    agent, batches, noise_c, noise_a = build_agent(lib, torch, case, U)
    for u in range(U):
        agent.update(batches[u], noise_c[u, 0], noise_c[u, 1], noise_a[u])
    f = lambda k: fix[f"{k}_{case}_u{U}"]
    assert_params_close("actor", agent.actor.params.cpu().numpy(), f("actor_params"), U)
    for c in range(2):
        assert_params_close(f"critic {c}", agent.critics[c].params.cpu().numpy(), f(f"critic{c}_params"), 2 * U)
        assert_params_close(f"target {c}", agent.critics_target[c].params.cpu().numpy(), f(f"target{c}"), 2 * U)
    assert abs(agent.log_alpha.item() - float(f("log_alpha_params"))) < 2e-6
    close(agent.target_action_value.cpu().numpy()[:, 0], f("target_values"), what="last target values")


@pytest.mark.parametrize("case", range(len(oracle.Reference.NORMALIZER_CASES)))
def test_running_normalizer_and_standardize_vs_reference_golden(lib, torch, case):
    """Observation normalisation against the reference's fixture: running mean / std after each of three updates, the layer statistics, the
    standardized batch (1e-5 relative + 1e-6 absolute; the column sums are taken in double instead of the reference's fp32 row order); the
    constant column gives standard deviation and precision exactly 0. Data read through a row pitch."""
    fix = np.load(os.path.join(GOLDEN, "normalizer.npz"))
    data = mg.normalizer_inputs(case)
    U, R, D = data.shape
    normalizer = lib.RunningNormalizer(D)
    wide = torch.zeros((R, D + 7), device="cuda")
    for u in range(U):
        wide[:, 3:3 + D] = dev(torch, data[u])
        normalizer.update(wide[:, 3:3 + D])
        close(normalizer.mean.cpu().numpy(), fix[f"mean_{case}"][u], what=f"mean after update {u}")
        close(normalizer.std.cpu().numpy(), fix[f"std_{case}"][u], what=f"std after update {u}")
    assert normalizer.std.cpu().numpy()[-1] == 0
    normalizer.set_statistics()
    close(normalizer.layer_mean.cpu().numpy(), fix[f"layer_mean_{case}"], what="layer mean")
    close(normalizer.layer_precision.cpu().numpy(), fix[f"layer_precision_{case}"], what="layer precision")
    assert normalizer.layer_precision.cpu().numpy()[-1] == 0
    out = torch.full((R, D + 2), 5.0, device="cuda")
    normalizer.standardize(wide[:, 3:3 + D], y=out[:, 1:1 + D])
    # (x - mean) * precision with statistics that agree to 1e-5 relative: the difference of the means enters scaled by the precision
    got_out, want_out = out[:, 1:1 + D].cpu().numpy().astype(np.float64), fix[f"output_{case}"].astype(np.float64)
    bound = 2e-6 + 1e-5 * (np.abs(data[-1]) + np.abs(fix[f"layer_mean_{case}"])) * fix[f"layer_precision_{case}"] + 1e-5 * np.abs(want_out)
    assert np.all(np.abs(got_out - want_out) <= bound), f"standardized batch: max err {np.abs(got_out - want_out).max():.3e}"
    assert bool((out[:, 0] == 5).all()) and bool((out[:, -1] == 5).all())
    # given the reference's statistics the layer itself is exact
    normalizer.layer_mean.copy_(dev(torch, fix[f"layer_mean_{case}"])); normalizer.layer_precision.copy_(dev(torch, fix[f"layer_precision_{case}"]))
    assert np.array_equal(normalizer.standardize(wide[:, 3:3 + D]).cpu().numpy(), fix[f"output_{case}"])


def test_off_policy_training_step_end_to_end_as_one_graph(lib, torch):
    """Runner step with replay buffers -> gather_batch -> SAC update, 40 eager loop steps to fill the buffers, then the sampling + update
    captured once and replayed: the device-resident call counter advances, consecutive replays sample different batches, no error flag
    is raised, every parameter stays finite and the critics move."""
    from rl_tools_b200 import sac
    N, cap, limit, B = 64, 128, 50, 256
    rs = np.random.RandomState(6)
    shape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    policy = dev(torch, (rs.uniform(-1, 1, 4481) * 0.3).astype(np.float32))
    L = lib.ReplayLayout.packed(cap)
    replay = torch.zeros(N * L.env_stride, dtype=torch.uint8, device="cuda")
    states, es, tr, er = torch.zeros((N, 2), device="cuda"), torch.zeros(N, dtype=torch.int32, device="cuda"), torch.ones(N, dtype=torch.uint8, device="cuda"), torch.zeros(N, device="cuda")
    obs, act, nobs = torch.zeros((N, 3), device="cuda"), torch.zeros((N, 1), device="cuda"), torch.zeros((N, 3), device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    rng = lib.rng_init_host(3)
    import ctypes as C
    for _ in range(40):
        table = np.zeros((1, N, 2), np.float32)
        e_h, t_h = es.cpu().numpy(), tr.cpu().numpy()
        lib.check(lib.lib().b200rl_reset_table_host(C.c_void_p(rng.ctypes.data), N, 1, C.c_void_p(e_h.ctypes.data), C.c_void_p(t_h.ctypes.data), limit,
                                                    C.c_void_p(table.ctypes.data), 1, None), "b200rl_reset_table_host")
        lib.pendulum_offpolicy_step(shape, policy, states, es, tr, er, dev(torch, table), limit, obs, act, nobs, replay, L, error_flag=flag)
    position, full = lib.replay_counters(replay, L, N)
    assert int(flag.item()) == 0 and bool((position == 40).all()) and not bool(full.any())

    agent = sac.ActorCritic(3, 1, 64, B)
    for net in [agent.actor] + agent.critics:
        net.params.copy_(dev(torch, (rs.uniform(-1, 1, net.params.numel()) * 0.2).astype(np.float32)))
    agent.copy_critics_to_targets()
    before = [c.params.clone() for c in agent.critics]
    batch, noise = lib.new_batch(B), torch.empty((3, B, 1), device="cuda")
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")

    def step():
        lib.gather_batch(replay, L, N, batch, seed=9, call_counter=counter, error_flag=flag)
        lib.randn_device_rng(noise, 9, stream_id=1, call_counter=counter)
        agent.update(batch, noise[0], noise[1], noise[2])
        lib.counter_advance(counter, 1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                                       # warm-up outside the capture
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    seen = []
    for _ in range(5):
        graph.replay()
        torch.cuda.synchronize()
        seen.append(batch["oa_base"].clone())
    assert int(counter.item()) == 6 and int(flag.item()) == 0          # one eager warm-up step + five replays (capturing executes nothing)
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[3], seen[4])
    for net in [agent.actor] + agent.critics + agent.critics_target:
        assert bool(torch.isfinite(net.params).all())
    assert bool(torch.isfinite(agent.log_alpha).all())
    for c in range(2):
        assert not torch.equal(agent.critics[c].params, before[c])


def test_runner_step_in_two_halves_equals_the_fused_step(lib, torch):
    """prologue + (the fused step's own actions) + epilogue leaves the runner state and the replay buffers bit for bit as
    b200rl_pendulum_offpolicy_step does (which the reference fixture pins): 25 steps over an episode limit of 10, i.e. with resets from
    the table, truncation marks and the episode-start bookkeeping."""
    N, cap, limit = 48, 16, 10
    rs = np.random.RandomState(11)
    shape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    policy = dev(torch, (rs.uniform(-1, 1, 4481) * 0.3).astype(np.float32))
    L = lib.ReplayLayout.packed(cap)

    def fresh():
        return dict(replay=torch.zeros(N * L.env_stride, dtype=torch.uint8, device="cuda"), states=torch.zeros((N, 2), device="cuda"),
                    es=torch.zeros(N, dtype=torch.int32, device="cuda"), tr=torch.ones(N, dtype=torch.uint8, device="cuda"), er=torch.zeros(N, device="cuda"),
                    obs=torch.zeros((N, 3), device="cuda"), act=torch.zeros((N, 1), device="cuda"), nobs=torch.zeros((N, 3), device="cuda"))
    a, b = fresh(), fresh()
    was = torch.zeros(N, dtype=torch.uint8, device="cuda")
    for step in range(25):
        table = dev(torch, np.stack([rs.uniform(-np.pi, np.pi, N), rs.uniform(-1, 1, N)], 1).astype(np.float32).reshape(1, N, 2))
        lib.pendulum_offpolicy_step(shape, policy, a["states"], a["es"], a["tr"], a["er"], table, limit, a["obs"], a["act"], a["nobs"], a["replay"], L)
        lib.pendulum_offpolicy_prologue(b["states"], b["es"], b["tr"], b["er"], b["obs"], was, reset_states=table[0])
        assert torch.equal(b["obs"], a["obs"])
        lib.pendulum_offpolicy_epilogue(b["states"], b["es"], b["tr"], b["er"], limit, b["obs"], a["act"], b["nobs"], b["replay"], L, was)
        for k in ("states", "es", "tr", "er", "nobs", "replay"):
            assert torch.equal(a[k], b[k]), (step, k)
    position, full = lib.replay_counters(b["replay"], L, N)
    assert bool((position == 25 % cap).all()) and bool(full.all())


def test_prologue_draws_initial_states_on_the_device(lib, torch):
    """Without a table the prologue draws theta ~ U(-pi, pi), theta_dot ~ U(-1, 1) per (environment, call): inside the bounds, different per
    environment and per call, reproducible, and only for the truncated environments."""
    N = 4096
    st = torch.full((N, 2), 9.0, device="cuda")
    es, er = torch.full((N,), 5, dtype=torch.int32, device="cuda"), torch.ones(N, device="cuda")
    tr = torch.ones(N, dtype=torch.uint8, device="cuda"); tr[::2] = 0
    obs, was = torch.zeros((N, 3), device="cuda"), torch.zeros(N, dtype=torch.uint8, device="cuda")
    counter = torch.full((1,), 3, dtype=torch.int64, device="cuda")
    lib.pendulum_offpolicy_prologue(st, es, tr, er, obs, was, seed=5, call_counter=counter)
    s = st.cpu().numpy()
    assert np.all(s[::2] == 9.0) and np.all(es.cpu().numpy()[::2] == 5) and np.all(er.cpu().numpy()[::2] == 1.0)
    drawn = s[1::2]
    assert np.all(np.abs(drawn[:, 0]) <= np.pi) and np.all(np.abs(drawn[:, 1]) <= 1.0) and len(np.unique(drawn[:, 0])) > 2000
    assert abs(drawn[:, 0].mean()) < 0.15 and abs(drawn[:, 1].mean()) < 0.05
    assert np.all(es.cpu().numpy()[1::2] == 0) and np.all(er.cpu().numpy()[1::2] == 0.0) and torch.equal(was, tr)
    close(obs.cpu().numpy(), np.stack([np.cos(s[:, 0].astype(np.float64)), np.sin(s[:, 0].astype(np.float64)), s[:, 1]], 1), what="observation")
    st2 = torch.full((N, 2), 9.0, device="cuda")
    lib.pendulum_offpolicy_prologue(st2, es, tr, er, obs, was, seed=5, call_index=3)              # the same call index given on the host
    assert torch.equal(st2, st)
    lib.pendulum_offpolicy_prologue(st2, es, tr, er, obs, was, seed=5, call_index=4)
    assert not torch.equal(st2[1::2], st[1::2])


def test_sac_loop_learns_the_pendulum(lib, torch):
    """The off-policy training loop with the reference example's configuration (one environment, 64-wide networks, batch 100, 10,000 steps):
    the deterministic evaluation policy goes from a random policy's return (below -900) to swinging up (above -400; the reference's
    example reports about -200 to -150 after the same number of steps)."""
    from rl_tools_b200.loops import PendulumSacLoop
    torch.manual_seed(0)
    loop = PendulumSacLoop(seed=0)
    before = loop.evaluate()
    while not loop.step():
        pass
    torch.cuda.synchronize()
    assert int(loop.error_flag.item()) == 0 and int(loop.counter.item()) == 10000
    after = loop.evaluate()
    print(f"SAC Pendulum: evaluation return {before:.0f} -> {after:.0f}, alpha {float(loop.agent.log_alpha.exp().item()):.3f}")
    assert before < -900 and after > -400, (before, after)
    for net in [loop.agent.actor] + loop.agent.critics + loop.agent.critics_target:
        assert bool(torch.isfinite(net.params).all())


def test_sac_loop_on_the_quadrotor(lib, torch):
    """The same loop on the L2F quadrotor (16 environments, resets drawn in the kernel, 64-wide networks, batch 256): warm-up with uniformly
    random actions, then captured training steps. Checked: the loop's counters, the replay buffers fill with rows of 43 floats whose
    observations carry proper rotation matrices, every parameter stays finite, and 6,000 steps move the deterministic evaluation policy
    (256 evaluation episodes) from leaving the termination bounds after ~30 steps to staying inside them several times longer, at a better
    reward per step (measured: episode length 29 -> 88, return per step -3.4 -> -1.4)."""
    import os
    import numpy as np
    from rl_tools_b200.loops import L2fSacLoop
    fix = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "l2f.npz"))
    torch.manual_seed(0)
    p = lib.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    loop = L2fSacLoop(p, fix["mdp"], fix["init"], n_envs=16, batch_size=256, step_limit=6000, n_warmup_steps=200, replay_capacity=8192, seed=3)
    ret0, len0 = loop.evaluate()
    while not loop.step():
        pass
    torch.cuda.synchronize()
    assert int(loop.error_flag.item()) == 0 and int(loop.counter.item()) == 6000
    ret1, len1 = loop.evaluate()
    print(f"SAC L2F: evaluation return {ret0:.1f} -> {ret1:.1f}, episode length {len0:.0f} -> {len1:.0f}, alpha {float(loop.agent.log_alpha.exp().item()):.3f}")
    for net in [loop.agent.actor] + loop.agent.critics + loop.agent.critics_target:
        assert bool(torch.isfinite(net.params).all())
    position, full = lib.replay_counters(loop.replay, loop.layout, 16)
    assert bool((position == 6000).all()) and not bool(full.any())
    L = loop.layout
    raw = loop.replay.cpu().numpy().reshape(16, L.env_stride)
    rows = raw[:, L.off_data:L.off_data + 4 * 43 * 6000].copy().view(np.float32).reshape(16, 6000, 43)
    R = rows[:, :, 3:12].reshape(-1, 3, 3).astype(np.float64)
    assert np.abs(R @ R.transpose(0, 2, 1) - np.eye(3)).max() < 1e-4 and np.abs(rows[:, :, 18:22]).max() <= 1.0
    assert np.isfinite(rows).all() and (rows[:, :, 41].sum() > 0)            # terminations occurred and were recorded
    assert len1 > 1.5 * len0 and ret1 / len1 > ret0 / len0, (ret0, ret1, len0, len1)        # it stays inside the bounds longer, at a better reward per step

