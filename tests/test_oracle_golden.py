"""The CPU oracle (oracle/oracle.c) against the golden fixtures produced by the REAL reference
(tests/golden/make_golden.py). Everything here is bit-exact: the oracle restates the reference's generic-device
loop order with the same strict floating-point flags."""
import glob
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle


def test_rng_streams_match_reference(orc):
    fix = np.load(os.path.join(GOLDEN, "rng.npz"))
    for seed in (0, 1, 12345):
        assert np.array_equal(orc.uniform_stream(seed, 1024, -np.float32(np.pi), np.float32(np.pi)), fix[f"uniform_{seed}"])
        assert np.array_equal(orc.normal_stream(seed, 1024, 0.25, 1.5), fix[f"normal_{seed}"])
        kinds = (np.arange(1024) % 3 == 0).astype(np.uint8)
        a = np.where(kinds == 0, -1.0, 0.0).astype(np.float32)
        b = np.where(kinds == 0, 1.0, 0.5).astype(np.float32)
        assert np.array_equal(orc.mixed_stream(seed, kinds, a, b), fix[f"mixed_{seed}"])
        assert np.array_equal(orc.pendulum_initial_states(seed, 1024), fix[f"initial_states_{seed}"])


def test_pendulum_step_reward_observe(orc):
    fix = np.load(os.path.join(GOLDEN, "pendulum_step.npz"))
    ns, r, obs, nobs = orc.pendulum_step(fix["states"], fix["actions"])
    assert np.array_equal(ns, fix["next_states"])
    assert np.array_equal(r, fix["rewards"])
    assert np.array_equal(obs, fix["obs"])
    assert np.array_equal(nobs, fix["next_obs"])


def _case_from_dims(d):
    return dict(batch=int(d[0]), input_dim=int(d[1]), hidden_dim=int(d[2]), output_dim=int(d[3]), num_layers=int(d[4]),
                hidden_act=int(d[5]), output_act=int(d[6]))


MLP_FIXTURES = sorted(glob.glob(os.path.join(GOLDEN, "mlp_*.npz")))


@pytest.mark.parametrize("path", MLP_FIXTURES, ids=[os.path.basename(p)[4:-4] for p in MLP_FIXTURES])
def test_mlp_forward_backward_adam(orc, path):
    fix = np.load(path)
    name = os.path.basename(path)[4:-4]
    c = _case_from_dims(fix["dims"])
    shape = oracle.Reference.case_shape(c)
    params, x, target = mg.mlp_inputs(c, mg.case_seed(name))
    B, O = c["batch"], c["output_dim"]

    def check(key, arr):
        s, tot = mg.sample(arr)
        assert np.array_equal(s, fix[key]), key
        assert tot == fix[key + "_sum"], key

    check("eval_out", orc.mlp_evaluate(shape, params, x))
    pre, out = orc.mlp_forward(shape, params, x)
    check("fwd_pre", pre)
    check("fwd_out", out)
    y = np.ascontiguousarray(out[-B * O:].reshape(B, O))
    d = orc.mse_gradient(y, target, 1.0)
    grads, _ = orc.mlp_backward(shape, params, np.zeros_like(params), x, pre, out, d)
    check("bwd_grads", grads)
    p, g, m, v, _, _ = orc.mlp_train_steps(shape, params, x, target, mg.MLP_STEPS)
    check("train_params", p)
    check("train_grads", g)
    check("train_m", m)
    check("train_v", v)
    grads_full, d_in = orc.mlp_backward(shape, params, np.zeros_like(params), x, pre, out, target, want_d_input=True)
    check("full_grads", grads_full)
    check("full_d_input", d_in)


def test_rollout_with_resets(orc):
    fix = np.load(os.path.join(GOLDEN, "rollout.npz"))
    N, T, limit = int(fix["N"]), int(fix["T"]), int(fix["step_limit"])
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    ro = orc.pendulum_rollout(shape, fix["actor_params"], np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8),
                              np.zeros(N, np.float32), fix["reset_table"], T, limit)
    for k in ("obs", "act", "rew", "states", "episode_step", "truncated", "episode_return"):
        assert np.array_equal(ro[k], fix[k]), k
    # the reset table in the fixture is the reference engine's stream in the runner's draw order
    table = orc.reset_table(int(fix["reset_seed"]), N, T, np.zeros(N, np.int32), np.ones(N, np.uint8), limit, 3)
    assert np.array_equal(table, fix["reset_table"])


def test_rollout_staggered_counters(orc):
    fix = np.load(os.path.join(GOLDEN, "rollout_staggered.npz"))
    base = np.load(os.path.join(GOLDEN, "rollout.npz"))
    N = int(base["N"])
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    ro = orc.pendulum_rollout(shape, base["actor_params"], fix["states0"], fix["episode_step0"], fix["truncated0"], np.zeros(N, np.float32),
                              base["reset_table"], int(fix["T"]), 200)
    for k in ("obs", "act", "rew"):
        assert np.array_equal(ro[k][::7], fix[k]), k
    for k in ("states", "episode_step", "truncated", "episode_return"):
        assert np.array_equal(ro[k], fix[k]), k


def test_kaiming_init_bounds_from_reference_engine():
    """The fixture's actor came from the reference's init_weights (legacy Kaiming-uniform): every layer is bounded
    by 1/sqrt(fan_in) and the first values are the reference engine's uniform stream (bias first, then the row)."""
    fix = np.load(os.path.join(GOLDEN, "rollout.npz"))
    p = fix["actor_params"]
    assert p.size == 3 * 64 + 64 + 64 * 64 + 64 + 64 + 1
    assert np.abs(p[:256]).max() <= 1 / np.sqrt(3) + 1e-7
    assert np.abs(p[256:256 + 64 * 64 + 64]).max() <= 1 / 8 + 1e-7


def test_gae_and_gaussian_head_match_reference(orc):
    """orc_gae against the reference's estimate_generalized_advantages on its own Dataset type; the Gaussian log-prob
    and its derivatives against random/operations_generic.h (all bit-exact)."""
    fix = np.load(os.path.join(GOLDEN, "ppo.npz"))
    for N, steps in ((64, 1024), (5, 37)):
        n = N * steps
        rewards = mg.det_normal(31, n, stream=N)
        all_values = mg.det_normal(32, n + N, stream=N)
        truncated = (mg._hash_u64(33, n, N) % np.uint64(97) == 0).astype(np.uint8)
        terminated = (truncated & (mg._hash_u64(34, n, N) % np.uint64(2) == 0)).astype(np.uint8)
        adv, tgt = orc.gae(rewards, all_values, terminated, truncated, N, steps)
        assert np.array_equal(adv, fix[f"gae_{N}x{steps}_adv"]) and np.array_equal(tgt, fix[f"gae_{N}x{steps}_tgt"])
    mean, log_std, value = mg.det_normal(35, 4096), mg.det_uniform(36, 4096, -2.0, 0.5), mg.det_normal(37, 4096) * np.float32(1.5)
    lp, dm, dl = orc.normal_functions(mean, log_std, value)
    assert np.array_equal(lp, fix["normal_log_prob"]) and np.array_equal(dm, fix["normal_d_mean"]) and np.array_equal(dl, fix["normal_d_log_std"])


def fresh_runner(N):
    """Runner state right after init(): every environment flagged truncated (on_policy_runner/operations_generic.h:69-82)."""
    return dict(states=np.zeros((N, 2), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8),
                episode_return=np.zeros(N, np.float32))


@pytest.mark.parametrize("case", range(len(mg.COLLECT_CASES)))
def test_on_policy_collect_matches_reference(orc, case):
    """Consecutive collect() calls of the reference's OnPolicyRunner (one engine, resets and action noise interleaved) against the
    oracle, once drawing inline from the engine and once through the draw tables the GPU path consumes. Bit-exact."""
    fix = np.load(os.path.join(GOLDEN, "collect.npz"))
    N, T, limit, hact, n_collects = mg.COLLECT_CASES[case]
    params = mg.collect_params(case)
    shape = oracle.MlpShape.make(3, [64, 64, 1], [hact, hact, 0])
    for mode in ("inline", "tables"):
        rng = orc.new_rng(mg.COLLECT_SEED)
        runner = fresh_runner(N)
        ds = np.zeros(((T + 1) * N, 13), np.float32)
        for c in range(n_collects):
            if mode == "inline":
                orc.pendulum_collect(shape, params, runner, T, limit, rng=rng, dataset=ds)
            else:
                table, noise = orc.collect_tables(rng, N, T, runner["episode_step"], runner["truncated"], limit, 8)
                orc.pendulum_collect(shape, params, runner, T, limit, reset_states=table, noise=noise, dataset=ds)
            assert np.array_equal(ds, fix[f"dataset_{case}"][c]), (mode, c)
        for k in ("states", "episode_step", "truncated", "episode_return"):
            assert np.array_equal(runner[k], fix[f"{k}_{case}"]), (mode, k)
        assert int(fix[f"runner_step_{case}"]) == n_collects * N * T


@pytest.mark.parametrize("case", range(len(mg.PPO_TRAIN_CASES)))
def test_ppo_train_matches_reference(orc, case):
    """The reference's train() (epochs x minibatches of clipped-surrogate actor update + critic regression, Adam) on a stored dataset
    matrix against the oracle's composition of its dense / PPO-gradient / Adam pieces: parameters, last gradients and first moments of
    both networks, bit for bit. This pins the PPO policy-gradient restatement."""
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    N, steps, batch, epochs = mg.PPO_TRAIN_CASES[case]
    actor, critic = mg.ppo_train_params(case)
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"])
    got = orc.ppo_train(shape, shape, actor, critic, fix[f"dataset_{case}"], N * steps, batch, epochs)
    for name, g in zip(("actor", "actor_grad", "actor_m", "critic", "critic_grad", "critic_m"), got):
        assert np.array_equal(g, fix[f"{name}_{case}"]), name


def test_uniform_int_distribution_matches_reference(orc):
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    lo, hi = mg.uniform_int_ranges()
    assert np.array_equal(orc.uniform_int_stream(mg.PPO_SHUFFLE_SEED, lo, hi), fix["uniform_int"])


@pytest.mark.parametrize("case", [1, 2])
def test_ppo_train_with_epoch_shuffle_matches_reference(orc, case):
    """SHUFFLE_EPOCH = true: the in-place Fisher-Yates row swaps of the observation / action / log-prob / advantage / target columns
    driven by std::uniform_int_distribution, then the same minibatch updates. Dataset after train() and all parameters bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    N, steps, batch, epochs = mg.PPO_TRAIN_CASES[case]
    actor, critic = mg.ppo_train_params(case)
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"])
    ds = fix[f"dataset_{case}"].copy()
    got = orc.ppo_train(shape, shape, actor, critic, ds, N * steps, batch, epochs, shuffle_rng=orc.new_rng(mg.PPO_SHUFFLE_SEED))
    assert np.array_equal(ds, fix[f"shuffled_dataset_{case}"])
    assert not np.array_equal(ds, fix[f"dataset_{case}"])
    for name, g in zip(("actor", "actor_grad", "actor_m", "critic", "critic_grad", "critic_m"), got):
        assert np.array_equal(g, fix[f"shuffled_{name}_{case}"]), name


@pytest.mark.parametrize("tag", ["plain", "shuffled"])
def test_ppo_train_on_ant_shapes_matches_reference(orc, tag):
    """One epoch (32 minibatches of 2048) of the reference's train() on the Ant shapes of the PPO configuration: observation 27, actor
    27 -> 64 -> 64 -> 8 tanh + log_std[8], critic 27 -> 64 -> 64 -> 1, 64 envs x 1024 steps. Bit for bit on the machine that generated the
    fixture (tanhf comes from the C library on both sides); 1e-6 elsewhere."""
    fix = np.load(os.path.join(GOLDEN, "ppo_train_ant.npz"))
    actor, critic, ds = mg.ppo_ant_inputs()
    sa, sc = oracle.MlpShape.make(27, [64, 64, 8], ["tanh", "tanh", "identity"]), oracle.MlpShape.make(27, [64, 64, 1], ["tanh", "tanh", "identity"])
    rng = orc.new_rng(mg.PPO_SHUFFLE_SEED) if tag == "shuffled" else None
    got = orc.ppo_train(sa, sc, actor, critic, ds, 64 * 1024, 2048, 1, shuffle_rng=rng)
    s, tot = mg.sample(ds)
    assert np.array_equal(s, fix[f"{tag}_dataset_sample"]) and tot == fix[f"{tag}_dataset_sum"]        # data movement only: exact everywhere
    for name, g in zip(("actor", "actor_grad", "actor_m", "critic", "critic_grad", "critic_m"), got):
        want = fix[f"{tag}_{name}"]
        assert np.array_equal(g, want) or np.all(np.abs(g - want) <= 1e-6 + 1e-5 * np.abs(want)), name


@pytest.mark.parametrize("case", range(len(mg.OFFPOLICY_CASES)))
def test_offpolicy_runner_with_replay_buffers_matches_reference(orc, case):
    """n x step<0>() of the reference's OffPolicyRunner: replay rows, episode_start, position / full / current_episode_start (wrap-around
    and the truncation mark on the previous transition included), runner state and step buffers, bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "offpolicy.npz"))
    N, cap, limit, steps = mg.OFFPOLICY_CASES[case]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    st = orc.offpolicy_steps(shape, mg.offpolicy_params(case), orc.new_offpolicy_state(N, cap), limit, steps, orc.new_rng(mg.OFFPOLICY_SEED))
    w = min(steps, cap)
    for k, v in st.items():
        if k in ("replay_states", "replay_next_states"):
            assert not v.any()                                  # not stored, like the reference
            continue
        got = v[:, :w] if k in ("replay_data", "episode_start") else v
        assert np.array_equal(got, fix[f"{k}_{case}"]), k


@pytest.mark.parametrize("case", range(len(mg.GATHER_CASES)))
def test_gather_batch_matches_reference(orc, case):
    """gather_batch (sequence length 1) after n runner steps, three consecutive batches on one engine: every batch tensor and the engine's
    position afterwards, bit for bit (full and partly filled replay buffers, a buffer holding a single transition)."""
    fix = np.load(os.path.join(GOLDEN, "gather.npz"))
    N, cap, limit, batch, steps = mg.GATHER_CASES[case]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rng = orc.new_rng(mg.GATHER_SEED)
    st = orc.offpolicy_steps(shape, mg.gather_params(case), orc.new_offpolicy_state(N, cap), limit, steps, rng)
    for g in range(mg.N_GATHERS):
        got = orc.gather_batch(st, batch, rng)
        for k in ("oa_base", "rewards", "terminated", "reset", "next_reset_base", "final_step_mask", "next_final_step_mask_base"):
            assert np.array_equal(got[k], fix[f"{k}_{case}"][g]), (g, k)
        # the sampled transition really is the row the indices name
        rows = st["replay_data"][got["env_index"], got["sample_index"]]
        assert np.array_equal(got["oa_base"][0], rows[:, :4]) and np.array_equal(got["oa_base"][1, :, :3], rows[:, 5:8])
    assert (orc.lib.orc_rng_next(rng) & 0xFFFFFFFF) == int(fix[f"next_draw_{case}"])


@pytest.mark.parametrize("run", range(len(mg.GATHER_SEQ_RUNS)))
def test_gather_batch_sequences_match_reference(orc, run):
    """gather_batch with sequence lengths 5 and 8 after n runner steps, two consecutive batches on one engine: every batch tensor and the
    engine's position afterwards, bit for bit -- the reference's default sampling parameters (sequences from their episode's first step,
    random lengths), each of them alone, neither, and the DETERMINISTIC flag; partly filled and wrapped replay buffers."""
    fix = np.load(os.path.join(GOLDEN, "gather_sequences.npz"))
    which, mode, steps = mg.GATHER_SEQ_RUNS[run]
    N, cap, limit, batch, L = oracle.Reference.GATHER_SEQUENCE_CASES[which]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rng = orc.new_rng(mg.GATHER_SEQ_SEED)
    st = orc.offpolicy_steps(shape, mg.gather_sequence_params(which), orc.new_offpolicy_state(N, cap), limit, steps, rng)
    flags = (mode & 3) | orc.GATHER_FIRST_STEP_TARGET | (orc.GATHER_DETERMINISTIC if mode & 8 else 0)
    for g in range(2):
        got = orc.gather_batch_sequences(st, batch, L, flags, rng)
        for k in mg.GATHER_SEQ_KEYS:
            assert np.array_equal(got[k], fix[f"{k}_{run}"][g]), (g, k)
    assert (orc.lib.orc_rng_next(rng) & 0xFFFFFFFF) == int(fix[f"next_draw_{run}"])


@pytest.mark.parametrize("which,steps,flags", [(0, 230, 7), (1, 950, 6), (0, 600, 4), (1, 299, 5)])
def test_sequence_batch_checker_accepts_the_oracle(orc, which, steps, flags):
    """The structural checker that the GPU tests apply to batches drawn by the kernel's own generator, applied to 2,048-element batches of the
    (reference-pinned) oracle: it has to accept them."""
    N, cap, limit, batch, L = oracle.Reference.GATHER_SEQUENCE_CASES[which]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rng = orc.new_rng(mg.GATHER_SEQ_SEED)
    st = orc.offpolicy_steps(shape, mg.gather_sequence_params(which), orc.new_offpolicy_state(N, cap), limit, steps, rng)
    mg.check_sequence_batch(orc.gather_batch_sequences(st, 2048, L, flags, rng), st, L, flags)


def test_l2f_step_matches_reference(orc):
    """The L2F quadrotor step (the reference's GPU-harness configuration, default parameter set) from 768 random states with random
    actions, 1 and 50 steps: bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "l2f.npz"))
    states, actions = mg.l2f_inputs()
    assert np.array_equal(orc.l2f_steps(fix["dynamics"], float(fix["dt"]), states, actions, 1), fix["next_1"])
    assert np.array_equal(orc.l2f_steps(fix["dynamics"], float(fix["dt"]), states, actions, 50), fix["next_50"])
    assert not np.isnan(fix["next_50"]).any() and np.abs(np.linalg.norm(fix["next_50"][:, 3:7], axis=1) - 1).max() < 1e-6


def test_l2f_environment_functions_match_reference(orc):
    """observe, reward (with transitions that terminate) and terminated of the L2F environment: bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "l2f.npz"))
    states, actions = mg.l2f_inputs()
    far = states.copy(); far[::3, :3] *= 3
    assert np.array_equal(orc.l2f_steps(fix["dynamics"], float(fix["dt"]), far, actions, 1), fix["next_far"])
    obs, rew, term = orc.l2f_functions(fix["dynamics"], float(fix["dt"]), fix["mdp"], far, actions, fix["next_far"])
    assert np.array_equal(obs, fix["observations"]) and np.array_equal(rew, fix["rewards"]) and np.array_equal(term, fix["terminated"])
    assert 0.2 < term.mean() < 0.6


@pytest.mark.parametrize("case", range(len(mg.POLYAK_CASES)))
def test_polyak_update_matches_reference(orc, case):
    """utils::polyak::update / update_squared, repeated: bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "polyak.npz"))
    polyak, square, n = mg.POLYAK_CASES[case]
    source, target = mg.polyak_inputs()
    target = target.copy()
    for _ in range(n):
        orc.polyak_update(source, target, np.float32(polyak), square)
    assert np.array_equal(target, fix[f"target_{case}"])


@pytest.mark.parametrize("case", range(len(oracle.Reference.SAS_CASES)))
def test_sample_and_squash_matches_reference(orc, case):
    """The SAC policy head: forward with external noise and backward_full of the reference's LayerGradient, every output bit for bit
    (clamped log_std rows included)."""
    fix = np.load(os.path.join(GOLDEN, "sample_and_squash.npz"))
    got = orc.sample_and_squash(*mg.sas_inputs(case), mg.SAS_LOG_ALPHA)
    for k, v in got.items():
        assert np.array_equal(v, fix[f"{k}_{case}"]), k


@pytest.mark.parametrize("case", range(len(oracle.Reference.SAC_CASES)))
@pytest.mark.parametrize("updates", [1, mg.SAC_UPDATES])
def test_sac_updates_match_reference(orc, case, updates):
    """train_critic (both critics), update_critic_targets, train_actor incl. the log_alpha step: parameters, gradients, first moments, target
    networks and the last critic target values, bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "sac.npz"))
    B, H = oracle.Reference.SAC_CASES[case]
    got = mg.flatten_sac(orc.sac_updates(H, *mg.sac_inputs(case, updates)))
    for k, v in got.items():
        assert np.array_equal(v, fix[f"{k}_{case}_u{updates}"]), k


@pytest.mark.parametrize("case", range(len(oracle.Reference.NORMALIZER_CASES)))
def test_running_normalizer_and_standardize_match_reference(orc, case):
    """RunningNormalizer::update over three batches (running mean / std after each), set_statistics and the standardize layer's evaluate,
    bit for bit, a constant column (standard deviation and precision 0) included."""
    fix = np.load(os.path.join(GOLDEN, "normalizer.npz"))
    got = orc.normalizer(mg.normalizer_inputs(case))
    for k, v in got.items():
        assert np.array_equal(v, fix[f"{k}_{case}"]), k
    assert got["layer_precision"][-1] == 0 and np.all(got["output"][:, -1] == np.float32(0.25) - got["layer_mean"][-1])


def test_acrobot_swingup_matches_reference(orc):
    """AcrobotSwingup: 2048 single transitions over the whole state space (next state, reward, both observations) and a free-running
    60-step rollout of 33 environments with resets every 25 steps, bit for bit; the initial-state draws too."""
    fix = np.load(os.path.join(GOLDEN, "acrobot.npz"))
    states, actions = mg.acrobot_step_inputs()
    ns, r, obs, nobs = orc.acrobot_step(states, actions)
    assert np.array_equal(ns, fix["next_states"]) and np.array_equal(r, fix["rewards"]) and np.array_equal(obs, fix["obs"]) and np.array_equal(nobs, fix["next_obs"])
    N, T, limit = mg.ACROBOT_ROLLOUT
    table = mg.acrobot_reset_table(orc, T // limit + 1)
    assert np.array_equal(table, fix["reset_table"])
    shape = oracle.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    out = orc.acrobot_rollout(shape, mg.acrobot_params(), np.zeros((N, 4), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32), table, T, limit)
    for k, v in out.items():
        assert np.array_equal(v, fix[f"rollout_{k}"]), k


def test_acrobot_terminating_matches_reference(orc):
    """rl::environments::Acrobot, the variant that terminates: the initial-state draws (double-bounded uniforms: two engine words each) and a
    free-running 200-step rollout of 64 environments whose episodes end by termination or at the step limit, every array bit for bit --
    observations, actions, rewards, the terminated flags and the runner's counters."""
    fix = np.load(os.path.join(GOLDEN, "acrobot_terminating.npz"))
    N, T, limit = mg.ACROBOT_TERMINATING_ROLLOUT
    table = mg.acrobot_terminating_table(orc, T)
    assert np.array_equal(table[:32], fix["reset_table"])
    shape = oracle.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    out = orc.acrobot_terminating_rollout(shape, mg.acrobot_params(), np.zeros((N, 4), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32), table, T, limit)
    for k, v in out.items():
        assert np.array_equal(v, fix[f"rollout_{k}"]), k
    assert out["terminated"].sum() > 50


def test_c5_chunk_65536_forward_rows_match_reference(orc):
    """The fixture of the 65,536-row chunk (the reference's own forward through its scalar loops): rows are independent in the forward pass,
    so the oracle's forward on the sampled rows of the last chunk must reproduce the stored activations bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "c5_chunked_b65536.npz"))
    params, x, _ = mg.c5_inputs()
    rows = fix["act_rows"]
    xs = np.ascontiguousarray(x[mg.C5_CHUNK * (mg.C5_CHUNKS - 1):][rows])
    pre, out = orc.mlp_forward(oracle.C5_SHAPE(), params, xs)
    off = 0
    for l, d in enumerate([256, 256, 256, 16]):
        assert np.array_equal(pre[off:off + rows.size * d].reshape(rows.size, d), fix[f"pre_{l}"])
        assert np.array_equal(out[off:off + rows.size * d].reshape(rows.size, d), fix[f"out_{l}"])
        off += rows.size * d


def test_l2f_initial_state_sampler_matches_reference(orc):
    """sample_initial_state restated with the engine's draws: 1,800 consecutive calls on one engine equal the fixture written by the reference
    bit for bit (position, orientation, velocities, rotor speeds; the default disturbances have no spread and draw nothing), and the state
    as a function of explicit draws agrees with it where the draw decides nothing else (guidance off: positions inside +-max_position ...)."""
    fix = np.load(os.path.join(GOLDEN, "l2f.npz"))
    got = orc.l2f_sample_initial_states(mg.L2F_INIT_SEED, 1800, fix["init"], fix["dynamics"])
    assert np.array_equal(got.reshape(3, 600, 23), fix["initial_states"])
    rs = np.random.RandomState(2)
    u, nrm = rs.uniform(0, 1, (500, 17)).astype(np.float32), rs.randn(500, 6).astype(np.float32)
    init = fix["init"].copy(); init[8:12] = (0.01, 0.02, -0.001, 0.003)       # disturbances with a spread
    st = orc.l2f_initial_states_from_draws(init, fix["dynamics"], u, nrm)
    guided = u[:, 0] < init[0]
    assert 20 < guided.sum() < 90 and np.all(st[guided, :3] == 0) and np.all(st[guided, 3] == 1) and np.all(st[guided, 7:13] == 0)
    free = ~guided
    assert np.all(np.abs(st[free, :3]) <= init[1]) and np.all(np.abs(st[free, 7:10]) <= init[3]) and np.all(np.abs(st[free, 10:13]) <= init[4])
    assert np.allclose(np.linalg.norm(st[:, 3:7], axis=1), 1.0, atol=1e-6)
    assert np.array_equal(st[:, 13:16], nrm[:, :3] * np.float32(0.02) + np.float32(0.01))
    assert np.array_equal(st[:, 18], nrm[:, 5] * (np.float32(0.003) / np.float32(100)) + np.float32(-0.001))
    assert np.all(st[:, 19:] >= 0) and np.all(st[:, 19:] <= 0.5)             # relative rotor speeds -1 .. 0 of the action range 0 .. 1

