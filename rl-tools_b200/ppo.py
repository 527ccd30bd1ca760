"""Host-side mirror of the reference's PPO update on the on-policy dataset matrix, driving the C ABI.

`DatasetLayout` gives the column views of rl/components/on_policy_runner/on_policy_runner.h:38-72 (symmetric observations);
`estimate_generalized_advantages` and `train` follow rl/algorithms/ppo/operations_generic.h:59-95 and :96-336 with the default
parameters of rl/algorithms/ppo/ppo.h:13-38. Everything runs on the GPU on torch CUDA tensors; there is no CPU path.
"""
from . import gae as _gae, mse_gradient as _mse_gradient, ppo_policy_gradient as _ppo_policy_gradient, permute_rows as _permute_rows, shuffle_permutation_host as _shuffle_permutation_host


class DatasetLayout:
    """Column offsets of the dataset matrix [(steps + 1) * n_envs, data_dim], row = step * n_envs + env."""

    def __init__(self, observation_dim, action_dim):
        o, a = observation_dim, action_dim
        self.observation_dim, self.action_dim = o, a
        self.observations = slice(0, o)
        self.actions_mean = slice(o, o + a)
        self.actions = slice(o + a, o + 2 * a)
        self.action_log_probs = o + 2 * a
        self.rewards = o + 2 * a + 1
        self.terminated = o + 2 * a + 2
        self.truncated = o + 2 * a + 3
        self.reset = o + 2 * a + 4
        self.values = o + 2 * a + 5
        self.advantages = o + 2 * a + 6
        self.target_values = o + 2 * a + 7
        self.data_dim = o + 2 * a + 8


def estimate_generalized_advantages(dataset, layout, n_envs, steps, gamma=0.99, lam=0.95, ignore_termination=False):
    """Fills the advantage and target-value columns from rewards / values / flags, in place (one backward scan per environment).
    The value column must hold the critic's values of all (steps + 1) * n_envs observations."""
    rows = steps * n_envs
    adv, tgt = _gae(dataset[:, layout.rewards], dataset[:, layout.values], dataset[:, layout.terminated], dataset[:, layout.truncated],
                    n_envs, steps, gamma, lam, ignore_termination)
    dataset[:rows, layout.advantages] = adv
    dataset[:rows, layout.target_values] = tgt
    return dataset


def evaluate_values(critic, dataset, layout):
    """critic(all observations) -> value column, as the PPO loop does before the advantage estimate
    (rl/algorithms/ppo/loop/core/operations_generic.h: evaluate(critic, all_observations_privileged, all_values))."""
    for begin in range(0, dataset.shape[0], critic.batch):           # the Mlp's ping-pong buffers hold critic.batch rows
        rows = dataset[begin:begin + critic.batch]
        critic.evaluate(rows[:, layout.observations], y=rows[:, layout.values:layout.values + 1])
    return dataset


def _minibatch_update(actor, critic, rows, layout, epsilon_clip=0.2, entropy_coefficient=0.01, advantage_epsilon=1e-8, normalize_advantage=True, learn_action_std=True):
    import torch
    obs = rows[:, layout.observations]
    # the critic's update does not depend on the actor's: it runs on a second stream (a parallel branch once captured in a CUDA graph)
    side = critic.__dict__.get("_side_stream") or critic.__dict__.setdefault("_side_stream", torch.cuda.Stream(device=obs.device))
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        critic.zero_gradient()
        values = critic.forward(obs)
        critic.backward(obs, _mse_gradient(values, rows[:, layout.target_values:layout.target_values + 1], 0.5, d_a=critic.d_out_buffer()))
        critic.step()
    actor.zero_gradient()
    current = actor.forward(obs)
    d_actions = _ppo_policy_gradient(current, rows[:, layout.actions], actor.extra("params"), rows[:, layout.action_log_probs], rows[:, layout.advantages],
                                     actor.extra("grads"), epsilon_clip, entropy_coefficient, advantage_epsilon, normalize_advantage, learn_action_std,
                                     d_actions=actor.d_out_buffer(), scratch=actor.__dict__.setdefault("_ppo_scratch", {}))
    actor.backward(obs, d_actions)
    actor.step()
    torch.cuda.current_stream().wait_stream(side)


class MinibatchGraphs:
    """One captured CUDA graph per minibatch position of a dataset matrix: the ~24 launches of a minibatch update replayed with a
    single launch. Valid for one (actor, critic, dataset, batch_size) combination; every pointer is baked into the graphs."""

    def __init__(self, actor, critic, dataset, layout, n_rows, batch_size, **hyper):
        import torch
        self.key = (dataset.data_ptr(), n_rows, batch_size)
        self.graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        saved = [t.clone() for t in (actor.params, actor.m, actor.v, actor.adam_state, critic.params, critic.m, critic.v, critic.adam_state)]
        with torch.cuda.stream(side):
            _minibatch_update(actor, critic, dataset[:batch_size], layout, **hyper)             # warm-up outside capture (lazy module loading)
        torch.cuda.current_stream().wait_stream(side)
        for b in range(n_rows // batch_size):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                _minibatch_update(actor, critic, dataset[b * batch_size:(b + 1) * batch_size], layout, **hyper)
            self.graphs.append(g)
        for t, s in zip((actor.params, actor.m, actor.v, actor.adam_state, critic.params, critic.m, critic.v, critic.adam_state), saved):
            t.copy_(s)                                                                          # the warm-up update is undone


def train(actor, critic, dataset, layout, n_rows, batch_size, n_epochs=10, epsilon_clip=0.2, entropy_coefficient=0.01, advantage_epsilon=1e-8,
          normalize_advantage=True, learn_action_std=True, shuffle_rng_state=None, graphs=None):
    """n_epochs x (n_rows // batch_size) minibatch updates. shuffle_rng_state (from rng_init_host) switches the reference's SHUFFLE_EPOCH
    on: before every epoch the observation / action / log-prob / advantage / target-value columns of the dataset matrix are permuted in
    place with the permutation the reference's engine would produce (:127-158); None keeps dataset order. Per minibatch: zero_gradient,
    actor forward, clipped-surrogate gradient (+ log_std gradient), actor backward, critic forward, 0.5-weighted MSE gradient against
    the target values, critic backward, one Adam step each. `actor` is an Mlp with extra_params = action_dim (the log_std behind the
    layers), `critic` an Mlp with one output; both built for batch_size rows. graphs = a MinibatchGraphs built for these arguments
    replays each minibatch update as one CUDA graph launch instead of ~24 kernel launches (same kernels, same results)."""
    import torch
    assert actor.batch == batch_size and critic.batch == batch_size and actor.n_extra == layout.action_dim
    hyper = dict(epsilon_clip=epsilon_clip, entropy_coefficient=entropy_coefficient, advantage_epsilon=advantage_epsilon,
                 normalize_advantage=normalize_advantage, learn_action_std=learn_action_std)
    if graphs is not None:
        assert graphs.key == (dataset.data_ptr(), n_rows, batch_size), "graphs were captured for another dataset matrix"
    shuffled = list(range(layout.observations.start, layout.observations.stop)) + list(range(layout.actions.start, layout.actions.stop)) + \
        [layout.action_log_probs, layout.advantages, layout.target_values]
    for _ in range(n_epochs):
        if shuffle_rng_state is not None:
            perm = torch.from_numpy(_shuffle_permutation_host(shuffle_rng_state, n_rows)).to(dataset.device)
            _permute_rows(dataset, n_rows, perm, shuffled)
        for b in range(n_rows // batch_size):
            if graphs is not None:
                graphs.graphs[b].replay()
            else:
                _minibatch_update(actor, critic, dataset[b * batch_size:(b + 1) * batch_size], layout, **hyper)
