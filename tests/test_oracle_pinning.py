"""The CPU oracle against the REAL reference run live (oracle/_ref, built from the unmodified RLtools headers).
Skipped where the reference build is absent; the committed golden fixtures cover those machines."""
import numpy as np
import pytest

import make_golden as mg
import oracle


def test_rng_streams_live(orc, ref_strict):
    for seed in (3, 99):
        assert np.array_equal(orc.uniform_stream(seed, 4000, -2.5, 0.75), ref_strict.uniform_stream(seed, 4000, -2.5, 0.75))
        assert np.array_equal(orc.normal_stream(seed, 4000, -1.0, 0.3), ref_strict.normal_stream(seed, 4000, -1.0, 0.3))
        assert np.array_equal(orc.pendulum_initial_states(seed, 3000), ref_strict.pendulum_initial_states(seed, 3000))
    # std == 0 returns the mean and consumes nothing (random/operations_cpu.h:41-43)
    kinds = np.array([1, 0, 1, 0], np.uint8)
    a = np.array([5.0, -1.0, 0.0, -1.0], np.float32)
    b = np.array([0.0, 1.0, 1.0, 1.0], np.float32)
    assert np.array_equal(orc.mixed_stream(4, kinds, a, b), ref_strict.mixed_stream(4, kinds, a, b))


def test_pendulum_live(orc, ref_strict):
    st = np.stack([mg.det_uniform(11, 50000, -40, 40), mg.det_uniform(11, 50000, -9, 9, stream=1)], 1).astype(np.float32)
    ac = mg.det_uniform(11, 50000, -3, 3, stream=2)
    for a, b in zip(orc.pendulum_step(st, ac), ref_strict.pendulum_step(st, ac)):
        assert np.array_equal(a, b)


@pytest.mark.parametrize("name", ["c1_actor_eval", "c3_critic", "c4_actor_b2048", "tanh_b17", "fast_tanh_b33", "sweep_b9", "sweep_b200"])
def test_mlp_live(orc, ref_strict, name):
    c = ref_strict.cases()[name]
    shape = ref_strict.case_shape(c)
    params, x, target = mg.mlp_inputs(c, seed=4242)
    ref = ref_strict.mlp_run(name, params, x, target, 2, 4)
    p, g, m, v, pre, out = orc.mlp_train_steps(shape, params, x, target, 4)
    for k, arr in (("params", p), ("grads", g), ("m", m), ("v", v), ("pre", pre), ("out", out)):
        assert np.array_equal(arr, ref[k]), k
    full = ref_strict.mlp_run(name, params, x, target, 3)
    pre, out = orc.mlp_forward(shape, params, x)
    grads, d_in = orc.mlp_backward(shape, params, np.zeros_like(params), x, pre, out, target, want_d_input=True)
    assert np.array_equal(grads, full["grads"])
    assert np.array_equal(d_in, full["d_input"])


def test_chunked_training_step_live(orc, ref_strict):
    """The data-parallel replica's step (gradients accumulated over chunks, each weighted chunk / rows, then Adam) through the reference's own
    verbs equals the oracle's composition bit for bit (chunks of 1024 rows; the 65,536-row chunk is pinned through its fixture)."""
    import oracle
    params, x, target = mg.c5_inputs(3 * 1024)
    ref = ref_strict.mlp_c5_chunked(1024, params, x, target)
    mine = orc.mlp_chunked_step(oracle.C5_SHAPE(), params, x, target, 1024)
    for k in ("params", "grads", "m", "v", "pre", "out"):
        assert np.array_equal(ref[k], mine[k]), k


def test_rollout_live_chunked_evaluate(orc, ref_strict):
    """Reference evaluate() on 256-env batches (the way the runner calls it) equals the per-env oracle bit for bit
    on the generic device, because each output element is the same left-to-right sum."""
    N, T = 512, 230
    actor = ref_strict.mlp_run("c2_actor_b256", None, None, None, 0, init_seed=3)["params"]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    table = orc.reset_table(8, N, T, np.zeros(N, np.int32), np.ones(N, np.uint8), 200, 2)
    a = orc.pendulum_rollout(shape, actor, np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32), table, T)
    b = ref_strict.pendulum_rollout(actor, np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32), table, T, chunk=256)
    for k in a:
        assert np.array_equal(a[k], b[k]), k


def test_collect_live(orc, ref_strict):
    """collect() of the real reference, compiled here, against the oracle on parameters the fixtures do not cover."""
    for i, (N, T, limit, hact) in enumerate(oracle.Reference.COLLECT_CASES):
        params = (np.random.RandomState(100 + i).randn(4482) * 0.4).astype(np.float32)
        params[-1] = 0.3 - 0.4 * i
        want, runner_ref = ref_strict.collect(N, T, limit, hact, params, 5 + i, 2)
        shape = oracle.MlpShape.make(3, [64, 64, 1], [hact, hact, 0])
        rng = orc.new_rng(5 + i)
        runner = dict(states=np.zeros((N, 2), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8),
                      episode_return=np.zeros(N, np.float32))
        ds = np.zeros(((T + 1) * N, 13), np.float32)
        for c in range(2):
            orc.pendulum_collect(shape, params, runner, T, limit, rng=rng, dataset=ds)
            assert np.array_equal(ds, want[c])
        for k in ("states", "episode_step", "truncated", "episode_return"):
            assert np.array_equal(runner[k], runner_ref[k]), k


def test_ppo_train_live(orc, ref_strict):
    """train() of the real reference, compiled here, against the oracle on inputs the fixtures do not cover."""
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"])
    rs = np.random.RandomState(4)
    for (N, T, B, E) in oracle.Reference.PPO_TRAIN_CASES:
        ap = (rs.randn(4482) * 0.3).astype(np.float32)
        ap[-1] = -0.4
        cp = (rs.randn(4481) * 0.3).astype(np.float32)
        runner = dict(states=np.zeros((N, 2), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8),
                      episode_return=np.zeros(N, np.float32))
        ds = orc.pendulum_collect(shape, ap, runner, T, 20, rng=orc.new_rng(3))
        ds[:, 10] = orc.mlp_evaluate(shape, cp, np.ascontiguousarray(ds[:, 0:3]))[:, 0]
        n = N * T
        adv, tgt = orc.gae(np.ascontiguousarray(ds[:n, 6]), np.ascontiguousarray(ds[:, 10]), np.ascontiguousarray(ds[:n, 7]).astype(np.uint8),
                           np.ascontiguousarray(ds[:n, 8]).astype(np.uint8), N, T)
        ds[:n, 11], ds[:n, 12] = adv, tgt
        want = ref_strict.ppo_train(N, T, B, E, ap, cp, ds)
        got = orc.ppo_train(shape, shape, ap, cp, ds, n, B, E)
        for name, g, w in zip(("actor", "actor_grad", "actor_m", "critic", "critic_grad", "critic_m"), got, want):
            assert np.array_equal(g, w), (N, T, B, E, name)


def test_uniform_int_and_shuffled_train_live(orc, ref_strict):
    rs = np.random.RandomState(9)
    lo = rs.randint(0, 5000, 30000).astype(np.uint64)
    hi = lo + rs.choice([0, 1, 6, 7, 8, 1000, 2 ** 20 + 1, 2 ** 32 - 1], 30000).astype(np.uint64)
    assert np.array_equal(orc.uniform_int_stream(3, lo, hi), ref_strict.uniform_int_stream(3, lo, hi))
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"])
    for (N, T, B, E) in oracle.Reference.PPO_TRAIN_SHUFFLE_CASES:
        ap = (rs.randn(4482) * 0.3).astype(np.float32)
        cp = (rs.randn(4481) * 0.3).astype(np.float32)
        ds = (rs.randn((T + 1) * N, 13) * 0.5).astype(np.float32)           # train() consumes any matrix
        want = ref_strict.ppo_train(N, T, B, E, ap, cp, ds, shuffle_seed=77)
        mine = ds.copy()
        got = orc.ppo_train(shape, shape, ap, cp, mine, N * T, B, E, shuffle_rng=orc.new_rng(77))
        assert np.array_equal(mine, want[6])
        for g, w in zip(got, want[:6]):
            assert np.array_equal(g, w)


def test_offpolicy_runner_live(orc, ref_strict):
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rs = np.random.RandomState(12)
    for (N, cap, lim) in oracle.Reference.OFFPOLICY_CASES:
        params = (rs.randn(4481) * 0.3).astype(np.float32)
        for n_steps in (1, cap - 1, cap, 3 * cap + 5):
            want = ref_strict.offpolicy_steps(N, cap, lim, params, 4, n_steps)
            got = orc.offpolicy_steps(shape, params, orc.new_offpolicy_state(N, cap), lim, n_steps, orc.new_rng(4))
            w = min(n_steps, cap)
            for k in want:
                if k in ("replay_states", "replay_next_states"):
                    continue
                a, b = (want[k][:, :w], got[k][:, :w]) if k in ("replay_data", "episode_start") else (want[k], got[k])
                assert np.array_equal(a, b), (N, cap, lim, n_steps, k)


def test_gather_batch_live(orc, ref_strict):
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rs = np.random.RandomState(13)
    for (N, cap, lim, batch) in oracle.Reference.GATHER_CASES:
        params = (rs.randn(4481) * 0.3).astype(np.float32)
        for n_steps in (1, 2, cap - 1, cap, cap + 13, 3 * cap + 5):
            want, next_draw = ref_strict.offpolicy_gather(N, cap, lim, batch, params, 6, n_steps, 2)
            rng = orc.new_rng(6)
            st = orc.offpolicy_steps(shape, params, orc.new_offpolicy_state(N, cap), lim, n_steps, rng)
            for g in range(2):
                got = orc.gather_batch(st, batch, rng)
                for k in want[g]:
                    assert np.array_equal(got[k], want[g][k]), (N, cap, n_steps, g, k)
            assert (orc.lib.orc_rng_next(rng) & 0xFFFFFFFF) == next_draw


def test_gather_batch_sequences_live(orc, ref_strict):
    """Sequence lengths 5 and 8, every combination of the sampling parameters the driver instantiates, replay buffers from barely eligible to
    wrapped three times: batch tensors and the engine's position, bit for bit."""
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rs = np.random.RandomState(17)
    for which, (N, cap, lim, batch, L) in enumerate(ref_strict.GATHER_SEQUENCE_CASES):
        params = (rs.randn(4481) * 0.3).astype(np.float32)
        for mode in ref_strict.GATHER_SEQUENCE_MODES:
            for n_steps in (201 + lim, cap - 1, cap, cap + 13, 3 * cap + 5):
                want, next_draw = ref_strict.offpolicy_gather_sequences(which, mode, params, 6, n_steps, 2)
                rng = orc.new_rng(6)
                st = orc.offpolicy_steps(shape, params, orc.new_offpolicy_state(N, cap), lim, n_steps, rng)
                flags = (mode & 3) | orc.GATHER_FIRST_STEP_TARGET | (orc.GATHER_DETERMINISTIC if mode & 8 else 0)
                for g in range(2):
                    got = orc.gather_batch_sequences(st, batch, L, flags, rng)
                    for k in want[g]:
                        assert np.array_equal(got[k], want[g][k]), (which, mode, n_steps, g, k)
                assert (orc.lib.orc_rng_next(rng) & 0xFFFFFFFF) == next_draw


def test_l2f_step_live(orc, ref_strict):
    """4,000 other random quadrotor states and actions through 1, 7 and 120 steps: the restatement equals the reference's step() bit for bit."""
    import make_golden as mg
    dynamics, dt, noise = ref_strict.l2f_parameters()
    assert noise == 0.0
    states, actions = mg.l2f_inputs(4000, seed=5)
    for n_steps in (1, 7, 120):
        assert np.array_equal(orc.l2f_steps(dynamics, dt, states, actions, n_steps), ref_strict.l2f_steps(states, actions, n_steps)), n_steps


def test_l2f_environment_functions_live(orc, ref_strict):
    import make_golden as mg
    dynamics, dt, _ = ref_strict.l2f_parameters()
    mdp = ref_strict.l2f_mdp()
    states, actions = mg.l2f_inputs(5000, seed=8)
    states[::2, :3] *= 2.5
    nxt = ref_strict.l2f_steps(states, actions, 1)
    want, got = ref_strict.l2f_functions(states, actions, nxt), orc.l2f_functions(dynamics, dt, mdp, states, actions, nxt)
    for w, g in zip(want, got):
        assert np.array_equal(w, g)


def test_sac_updates_live(orc, ref_strict):
    import make_golden as mg
    for case, (B, H) in enumerate(oracle.Reference.SAC_CASES):
        args = list(mg.sac_inputs(case, 2))
        args[1] = np.float32(0.3)                                      # another log_alpha than the fixture's
        want, got = mg.flatten_sac(ref_strict.sac_updates(B, H, *args)), mg.flatten_sac(orc.sac_updates(H, *args))
        for k in want:
            assert np.array_equal(want[k], got[k]), (case, k)


def test_sample_and_squash_live(orc, ref_strict):
    rs = np.random.RandomState(8)
    for (B, A) in oracle.Reference.SAS_CASES:
        inp = (rs.randn(B, 2 * A) * 2).astype(np.float32)
        inp[0, A], inp[B - 1, 2 * A - 1] = 2.5, -30
        noise, dout = rs.randn(B, A).astype(np.float32), (rs.randn(B, A) / B).astype(np.float32)
        for log_alpha in (0.0, -2.0):
            want, got = ref_strict.sample_and_squash(inp, noise, dout, log_alpha), orc.sample_and_squash(inp, noise, dout, log_alpha)
            for k in want:
                assert np.array_equal(want[k], got[k]), (B, A, log_alpha, k)


def test_running_normalizer_live(orc, ref_strict):
    rs = np.random.RandomState(21)
    for (R, D) in oracle.Reference.NORMALIZER_CASES:
        data = (rs.randn(4, R, D) * rs.uniform(0.05, 8, D) + rs.uniform(-5, 5, D)).astype(np.float32)
        data[:, :, 0] = -1.5
        want, got = ref_strict.normalizer(data), orc.normalizer(data)
        for k in want:
            assert np.array_equal(want[k], got[k]), (R, D, k)


def test_acrobot_live(orc, ref_strict):
    rs = np.random.RandomState(33)
    n = 5000
    states = (rs.uniform(-1, 1, (n, 4)) * [np.pi, np.pi, 4 * np.pi, 9 * np.pi]).astype(np.float32)
    actions = rs.uniform(-2, 2, n).astype(np.float32)
    for a, b in zip(ref_strict.acrobot_step(states, actions), orc.acrobot_step(states, actions)):
        assert np.array_equal(a, b)
    assert np.array_equal(ref_strict.acrobot_initial_states(9, 300), orc.acrobot_initial_states(9, 300))
    # the terminating variant: double-bounded initial draws, terminated flags, reward -1, episodes cut by termination
    assert np.array_equal(ref_strict.acrobot_terminating_initial_states(9, 300), orc.acrobot_terminating_initial_states(9, 300))
    N, T, limit = 16, 150, 60
    table = ref_strict.acrobot_terminating_initial_states(4, T * N).reshape(T, N, 4)
    shape = oracle.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    params = (rs.uniform(-1, 1, 6 * 64 + 64 + 64 * 64 + 64 + 64 + 1) * 0.3).astype(np.float32)
    zero = lambda: (np.zeros((N, 4), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32))
    want, got = ref_strict.acrobot_terminating_rollout(params, *zero(), table, T, limit), orc.acrobot_terminating_rollout(shape, params, *zero(), table, T, limit)
    for k in want:
        assert np.array_equal(want[k], got[k]), k


def test_l2f_initial_state_sampler_live(orc, ref_strict):
    """sample_initial_state of the L2F environment: the oracle's restatement with the engine's draws against the reference for several seeds,
    3,000 consecutive states each, bit for bit."""
    dynamics, _, _ = ref_strict.l2f_parameters()
    init = ref_strict.l2f_init()
    for seed in (0, 7, 1234567):
        assert np.array_equal(orc.l2f_sample_initial_states(seed, 3000, init, dynamics), ref_strict.l2f_initial_states(seed, 3000)), seed

