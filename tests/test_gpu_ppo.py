"""GPU parity of the PPO update pieces (through the C ABI): GAE against the REAL reference's golden output (bit-exact),
the minibatch policy gradient against the CPU oracle, and one full minibatch update on the Ant-like shapes of the PPO
configuration (obs 27, actions 8, minibatch 2048; synthetic N(0,1) data -- MuJoCo is not part of this path)."""
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


def gae_inputs(N, steps):
    n = N * steps
    rewards = mg.det_normal(31, n, stream=N)
    all_values = mg.det_normal(32, n + N, stream=N)
    truncated = (mg._hash_u64(33, n, N) % np.uint64(97) == 0).astype(np.uint8)
    terminated = (truncated & (mg._hash_u64(34, n, N) % np.uint64(2) == 0)).astype(np.uint8)
    return rewards, all_values, terminated, truncated


@pytest.mark.parametrize("N,steps", [(64, 1024), (5, 37)])
def test_gae_bit_exact_vs_reference_golden(lib, torch, N, steps):
    fix = np.load(os.path.join(GOLDEN, "ppo.npz"))
    rewards, all_values, terminated, truncated = gae_inputs(N, steps)
    adv, tgt = lib.gae(dev(torch, rewards), dev(torch, all_values), dev(torch, terminated.astype(np.float32)), dev(torch, truncated.astype(np.float32)), N, steps)
    assert np.array_equal(adv.cpu().numpy(), fix[f"gae_{N}x{steps}_adv"])
    assert np.array_equal(tgt.cpu().numpy(), fix[f"gae_{N}x{steps}_tgt"])


def test_gae_on_column_views_of_the_dataset_matrix(lib, torch):
    """Same result when the columns live inside the reference's row-major dataset matrix (pitch = DATA_DIM = 51 for Ant)."""
    N, steps, D = 64, 1024, 51
    fix = np.load(os.path.join(GOLDEN, "ppo.npz"))
    rewards, all_values, terminated, truncated = gae_inputs(N, steps)
    data = torch.zeros(((steps + 1) * N, D), device="cuda")
    data[:steps * N, 44] = dev(torch, rewards); data[:steps * N, 45] = dev(torch, terminated.astype(np.float32))
    data[:steps * N, 46] = dev(torch, truncated.astype(np.float32)); data[:, 48] = dev(torch, all_values)
    adv, tgt = lib.gae(data[:, 44], data[:, 48], data[:, 45], data[:, 46], N, steps)
    assert np.array_equal(adv.cpu().numpy(), fix[f"gae_{N}x{steps}_adv"]) and np.array_equal(tgt.cpu().numpy(), fix[f"gae_{N}x{steps}_tgt"])


@pytest.mark.parametrize("B,A,normalize,learn", [(2048, 8, True, True), (300, 1, True, True), (64, 3, False, True), (1000, 8, True, False)])
def test_ppo_policy_gradient_vs_oracle(lib, orc, torch, B, A, normalize, learn):
    cur = mg.det_normal(B, B * A).reshape(B, A) * np.float32(0.5)
    roll = cur + mg.det_normal(B + 1, B * A).reshape(B, A) * np.float32(0.4)
    log_std = mg.det_uniform(B + 2, A, -1.2, -0.2)
    old_lp = mg.det_normal(B + 3, B) * np.float32(0.3) - np.float32(0.5 * A)
    adv = mg.det_normal(B + 4, B) * np.float32(2.0) + np.float32(0.3)
    g0 = mg.det_normal(B + 5, A)
    d_ref, dls_ref = orc.ppo_policy_gradient(cur, roll, log_std, old_lp, adv, d_log_std=g0, normalize_advantage=normalize, learn_action_std=learn)
    dls = dev(torch, g0)
    d = lib.ppo_policy_gradient(dev(torch, cur), dev(torch, roll), dev(torch, log_std), dev(torch, old_lp), dev(torch, adv), dls,
                                normalize_advantage=normalize, learn_action_std=learn)
    # the advantage statistics are sums over the minibatch in a different order: relative 1e-5 of each value's scale
    scale = np.abs(d_ref).max()
    assert np.all(np.abs(d.cpu().numpy() - d_ref) <= 2e-6 * scale + 1e-5 * np.abs(d_ref) + 1e-9)
    if learn:
        # the reference adds 2 * B small increments to log_std.gradient one after the other in fp32: its own rounding error
        # is up to B half-ulps of the running sum (observed: ~9e-6 at B = 2048), which bounds the comparison
        bound = 1e-6 + B * 3e-8 * np.maximum(np.abs(dls_ref), np.abs(g0)) + 1e-5 * np.abs(d_ref).sum(0).max()
        assert np.all(np.abs(dls.cpu().numpy() - dls_ref) <= bound)
    else:
        assert np.array_equal(dls.cpu().numpy(), g0)


def test_ppo_minibatch_update_on_ant_shapes(lib, orc, torch):
    """One minibatch of the PPO update (actor 27-64-64-8 tanh + log_std, critic 27-64-64-1, batch 2048): actor forward,
    policy gradient, backward, critic forward / 0.5-weighted MSE / backward, one Adam step each -- against the oracle."""
    B, OBS, A = 2048, 27, 8
    dims_a, dims_c, acts = [64, 64, A], [64, 64, 1], ["tanh", "tanh", "identity"]
    sa, sc = oracle.MlpShape.make(OBS, dims_a, acts), oracle.MlpShape.make(OBS, dims_c, acts)
    pa = np.concatenate([mg.mlp_inputs(dict(batch=1, input_dim=OBS, hidden_dim=64, output_dim=A, num_layers=3), 5)[0], np.full(A, np.log(0.5), np.float32)])
    pc = mg.mlp_inputs(dict(batch=1, input_dim=OBS, hidden_dim=64, output_dim=1, num_layers=3), 6)[0]
    obs = mg.det_normal(7, B * OBS).reshape(B, OBS)
    n_a = sa.num_params()
    mean0 = orc.mlp_evaluate(sa, pa[:n_a].copy(), obs)
    roll = (mean0 + np.float32(0.5) * mg.det_normal(8, B * A).reshape(B, A)).astype(np.float32)
    lp, _, _ = orc.normal_functions(mean0.reshape(-1), np.tile(pa[n_a:], B), roll.reshape(-1))
    old_lp = lp.reshape(B, A).sum(1).astype(np.float32) + mg.det_normal(9, B) * np.float32(0.05)     # a slightly different old policy
    adv, targets = mg.det_normal(10, B), mg.det_normal(11, B).reshape(B, 1)
    # --- oracle ---
    pre, out = orc.mlp_forward(sa, pa[:n_a].copy(), obs)
    cur = np.ascontiguousarray(out[-B * A:].reshape(B, A))
    d_act, d_ls = orc.ppo_policy_gradient(cur, roll, pa[n_a:].copy(), old_lp, adv)
    ga, _ = orc.mlp_backward(sa, pa[:n_a].copy(), np.zeros(n_a, np.float32), obs, pre, out, d_act)
    ga = np.concatenate([ga, d_ls])
    c1, c2, _ = orc.adam_bias_correction(0.9, 0.999, 1)
    pa_ref, _, _ = orc.adam_update(pa, ga, np.zeros_like(pa), np.zeros_like(pa), 1e-3, 0.9, 0.999, 1e-7, 1e-7, c1, c2)
    prec, outc = orc.mlp_forward(sc, pc, obs)
    d_c = orc.mse_gradient(np.ascontiguousarray(outc[-B:].reshape(B, 1)), targets, 0.5)
    gc, _ = orc.mlp_backward(sc, pc, np.zeros_like(pc), obs, prec, outc, d_c)
    pc_ref, _, _ = orc.adam_update(pc, gc, np.zeros_like(pc), np.zeros_like(pc), 1e-3, 0.9, 0.999, 1e-7, 1e-7, c1, c2)
    # --- library ---
    actor, critic = lib.Mlp(OBS, dims_a, acts, B, extra_params=A), lib.Mlp(OBS, dims_c, acts, B)
    actor.params.copy_(dev(torch, pa)); critic.params.copy_(dev(torch, pc))
    od = dev(torch, obs)
    actor.zero_gradient(); critic.zero_gradient()
    cur_d = actor.forward(od)
    d_act_d = lib.ppo_policy_gradient(cur_d, dev(torch, roll), actor.extra("params"), dev(torch, old_lp), dev(torch, adv), actor.extra("grads"))
    actor.backward(od, d_act_d)
    actor.step()
    val = critic.forward(od)
    critic.backward(od, lib.mse_gradient(val, dev(torch, targets), 0.5))
    critic.step()
    ga_d = actor.grads.cpu().numpy()
    assert np.all(np.abs(ga_d - ga) <= 1e-6 + 1e-5 * np.abs(ga) + 2e-6 * np.abs(ga).max())
    assert np.all(np.abs(actor.params.cpu().numpy() - pa_ref) <= 1e-6 + 1e-5 * np.abs(pa_ref))
    assert np.all(np.abs(critic.params.cpu().numpy() - pc_ref) <= 1e-6 + 1e-5 * np.abs(pc_ref))


def assert_params_close(name, got, want, n_updates, alpha=1e-3):
    """Parameters after n_updates Adam steps: within 1e-6 + 1e-5 |ref| everywhere, except that Adam divides by sqrt(v): where a gradient
    is ~0 a last-bit difference of the gradient moves the parameter by a visible fraction of alpha, and a sample whose probability ratio
    sits on the clipping boundary can take the other branch of the clipped surrogate (a discontinuous gradient), so up to 1 % of the
    elements may deviate, by at most 5 % of the distance Adam can move a parameter in n_updates steps (the drift is printed)."""
    err = np.abs(got - want)
    loose = err > 1e-6 + 1e-5 * np.abs(want)
    print(f"{name}: max err {err.max():.3e} after {n_updates} updates, {int(loose.sum())} of {err.size} elements beyond 1e-5")
    assert loose.mean() <= 1e-2 and err.max() <= 0.05 * alpha * n_updates, f"{name}: max err {err.max():.3e}, {int(loose.sum())} elements beyond tolerance"


@pytest.mark.parametrize("case", range(len(mg.PPO_TRAIN_CASES)))
def test_ppo_train_vs_reference_golden(lib, torch, case):
    """The whole PPO update (rl_tools_b200.ppo.train: epochs x minibatches over the dataset matrix, column views with the matrix's row
    pitch) against what the REAL reference's train() left behind on the same stored dataset: parameters of both networks within
    1e-5 |ref| + 2e-6 after up to 16 Adam steps, last-minibatch gradients within 1e-5 of the tensor's scale."""
    from rl_tools_b200 import ppo
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    N, steps, batch, epochs = mg.PPO_TRAIN_CASES[case]
    pa, pc = mg.ppo_train_params(case)
    dims, acts = [64, 64, 1], ["relu", "relu", "identity"]
    actor, critic = lib.Mlp(3, dims, acts, batch, extra_params=1), lib.Mlp(3, dims, acts, batch)
    actor.params.copy_(dev(torch, pa)); critic.params.copy_(dev(torch, pc))
    dataset = dev(torch, fix[f"dataset_{case}"])
    layout = ppo.DatasetLayout(3, 1)
    assert layout.data_dim == 13 and layout.target_values == 12
    ppo.train(actor, critic, dataset, layout, N * steps, batch, n_epochs=epochs)
    for name, got in (("actor", actor.params), ("critic", critic.params)):
        assert_params_close(name, got.cpu().numpy(), fix[f"{name}_{case}"], epochs * (N * steps // batch))
    for name, got in (("actor_grad", actor.grads), ("critic_grad", critic.grads), ("actor_m", actor.m), ("critic_m", critic.m)):
        want = fix[f"{name}_{case}"]
        err = np.abs(got.cpu().numpy() - want)
        tol = 1e-5 * np.abs(want).max() + 1e-5 * np.abs(want) + 1e-8
        if name.startswith("actor"):
            # log_std: the reference adds 2 * batch increments of mixed sign to the gradient one after the other in fp32, so its own
            # rounding error is a multiple of the running sum's ulp (observed 4e-4 relative at batch 4096); the kernel sums pairwise
            tol[-1] = 1e-3 * np.abs(want[-1]) + 1e-6
        assert np.all(err <= tol), f"{name}: max err {err.max():.3e} of scale {np.abs(want).max():.3e} at {int(np.argmax(err - tol))}"


def test_gae_and_values_in_place_on_the_dataset_matrix(lib, orc, torch):
    """evaluate_values + estimate_generalized_advantages write the value / advantage / target columns of the dataset matrix in place;
    advantage and target are bit-exact against the oracle given the same value column."""
    from rl_tools_b200 import ppo
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    N, steps = 64, 64
    ds = fix["dataset_0"].copy()
    _, pc = mg.ppo_train_params(0)
    critic = lib.Mlp(3, [64, 64, 1], ["relu", "relu", "identity"], 1024)
    critic.params.copy_(dev(torch, pc))
    d = dev(torch, ds)
    d[:, 10:13] = 0
    layout = ppo.DatasetLayout(3, 1)
    ppo.evaluate_values(critic, d, layout)
    values = d[:, 10].cpu().numpy()
    assert np.all(np.abs(values - ds[:, 10]) <= 1e-6 + 1e-5 * np.abs(ds[:, 10]))
    ppo.estimate_generalized_advantages(d, layout, N, steps)
    n = N * steps
    adv, tgt = orc.gae(np.ascontiguousarray(ds[:n, 6]), values, ds[:n, 7].astype(np.uint8), ds[:n, 8].astype(np.uint8), N, steps)
    got = d.cpu().numpy()
    assert np.array_equal(got[:n, 11], adv) and np.array_equal(got[:n, 12], tgt)
    assert np.array_equal(got[:, :10], ds[:, :10])


@pytest.mark.parametrize("case", [1, 2])
def test_ppo_train_with_epoch_shuffle_vs_reference_golden(lib, torch, case):
    """SHUFFLE_EPOCH = true through rl_tools_b200.ppo.train: the dataset matrix after the call equals the reference's bit for bit (the
    permutation comes from the reference-compatible host engine, the device only moves rows), parameters within 1e-5 |ref| + 2e-6."""
    from rl_tools_b200 import ppo
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    N, steps, batch, epochs = mg.PPO_TRAIN_CASES[case]
    pa, pc = mg.ppo_train_params(case)
    dims, acts = [64, 64, 1], ["relu", "relu", "identity"]
    actor, critic = lib.Mlp(3, dims, acts, batch, extra_params=1), lib.Mlp(3, dims, acts, batch)
    actor.params.copy_(dev(torch, pa)); critic.params.copy_(dev(torch, pc))
    dataset = dev(torch, fix[f"dataset_{case}"])
    ppo.train(actor, critic, dataset, ppo.DatasetLayout(3, 1), N * steps, batch, n_epochs=epochs, shuffle_rng_state=lib.rng_init_host(mg.PPO_SHUFFLE_SEED))
    assert np.array_equal(dataset.cpu().numpy(), fix[f"shuffled_dataset_{case}"])
    for name, got in (("actor", actor.params), ("critic", critic.params)):
        assert_params_close(name, got.cpu().numpy(), fix[f"shuffled_{name}_{case}"], epochs * (N * steps // batch))


def test_permute_rows_on_a_wide_matrix(lib, torch):
    """Row gather on selected columns of a 51-column matrix (the Ant dataset's width), other columns untouched."""
    rows, D = 5000, 51
    g = torch.Generator(device="cuda"); g.manual_seed(1)
    data = torch.randn((rows + 64, D), device="cuda", generator=g)
    before = data.clone()
    perm = torch.randperm(rows, device="cuda", generator=g).to(torch.int32)
    cols = list(range(0, 27)) + list(range(35, 43)) + [43, 49, 50]
    lib.permute_rows(data, rows, perm, cols)
    rest = [c for c in range(D) if c not in cols]
    assert torch.equal(data[:rows][:, cols], before[perm.long()][:, cols])
    assert torch.equal(data[:rows][:, rest], before[:rows][:, rest]) and torch.equal(data[rows:], before[rows:])


@pytest.mark.parametrize("tag", ["plain", "shuffled"])
def test_ppo_train_on_ant_shapes_vs_reference_golden(lib, torch, tag):
    """The PPO configuration's shapes (observation 27, actions 8, 64 envs x 1024 steps, minibatch 2048, tanh) through
    rl_tools_b200.ppo.train against the REAL reference's train(): one epoch = 32 updates; the shuffled dataset is exact."""
    from rl_tools_b200 import ppo
    fix = np.load(os.path.join(GOLDEN, "ppo_train_ant.npz"))
    pa, pc, ds = mg.ppo_ant_inputs()
    acts = ["tanh", "tanh", "identity"]
    actor, critic = lib.Mlp(27, [64, 64, 8], acts, 2048, extra_params=8), lib.Mlp(27, [64, 64, 1], acts, 2048)
    actor.params.copy_(dev(torch, pa)); critic.params.copy_(dev(torch, pc))
    dataset = dev(torch, ds)
    layout = ppo.DatasetLayout(27, 8)
    assert layout.data_dim == 51
    state = lib.rng_init_host(mg.PPO_SHUFFLE_SEED) if tag == "shuffled" else None
    ppo.train(actor, critic, dataset, layout, 64 * 1024, 2048, n_epochs=1, shuffle_rng_state=state)
    s, tot = mg.sample(dataset.cpu().numpy())
    assert np.array_equal(s, fix[f"{tag}_dataset_sample"]) and tot == fix[f"{tag}_dataset_sum"]
    for name, got in (("actor", actor.params), ("critic", critic.params)):
        assert_params_close(name, got.cpu().numpy(), fix[f"{tag}_{name}"], 32)


def test_ppo_train_graph_replay_equals_eager_launches(lib, torch):
    """MinibatchGraphs replays the same kernels as the eager path: parameters, moments and the shuffled dataset are bit-identical."""
    from rl_tools_b200 import ppo
    fix = np.load(os.path.join(GOLDEN, "ppo_train.npz"))
    N, steps, batch, epochs = mg.PPO_TRAIN_CASES[1]
    pa, pc = mg.ppo_train_params(1)
    dims, acts = [64, 64, 1], ["relu", "relu", "identity"]
    layout = ppo.DatasetLayout(3, 1)
    results = []
    for use_graphs in (False, True):
        actor, critic = lib.Mlp(3, dims, acts, batch, extra_params=1), lib.Mlp(3, dims, acts, batch)
        actor.params.copy_(dev(torch, pa)); critic.params.copy_(dev(torch, pc))
        dataset = dev(torch, fix["dataset_1"])
        graphs = ppo.MinibatchGraphs(actor, critic, dataset, layout, N * steps, batch) if use_graphs else None
        ppo.train(actor, critic, dataset, layout, N * steps, batch, n_epochs=epochs, shuffle_rng_state=lib.rng_init_host(5), graphs=graphs)
        results.append([t.clone() for t in (actor.params, actor.m, actor.v, critic.params, critic.m, critic.v, dataset)])
    for a, b in zip(*results):
        assert torch.equal(a, b)


@pytest.mark.gpu
def test_ppo_loop_learns_the_pendulum(lib, torch):
    """The whole on-policy loop (collect -> critic values -> GAE -> train) with the hyper-parameters of the reference's Pendulum PPO example
    (src/rl/environments/pendulum/ppo/cpu/config.h: 4 environments x 1024 steps per iteration, minibatch 256, 2 epochs, gamma 0.9, initial
    action std 2.0, no entropy bonus, PyTorch Adam defaults, 300,000 environment steps = 74 iterations): the return of the collected episodes,
    exploration noise included, must rise from the random policy's (about -1,300 per 200-step episode) to above -700, as the reference's
    example does on its way to about -200 with noise-free evaluation episodes. Every piece of the loop is held against the reference on its own
    elsewhere; this is the composition."""
    from rl_tools_b200 import loops
    loop = loops.PendulumPpoLoop(n_envs=4, steps_per_env=1024, batch_size=256, n_epochs=2, gamma=0.9, entropy_coefficient=0.0, initial_action_std=2.0,
                                 adam=dict(alpha=1e-3, epsilon=1e-8, epsilon_sqrt=1e-8), seed=3)
    returns = []
    for _ in range(74):
        loop.step()
        returns.append(loop.mean_episode_return())
    assert int(loop.error_flag.item()) == 0
    first, last = float(np.mean(returns[:3])), float(np.mean(returns[-5:]))
    print(f"PPO loop: mean episode return {first:.0f} -> {last:.0f} over {len(returns)} iterations; log_std {loop.actor.extra('params').item():.3f}")
    assert first < -900 and last > -700 and last > first + 400
