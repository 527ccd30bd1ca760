"""The on-policy training loop around the path: state, init and step of rl/algorithms/ppo/loop/core (operations_generic.h:20-58 malloc,
:66-85 init, :88-131 step) for the Pendulum, composed of the library's pieces -- nothing in a step leaves the GPU except the statistics the
caller asks for. One `step()` = collect (fused actor inference + environment steps into the dataset matrix), the critic's values of all
observations, generalized advantage estimation, `train` (epochs x minibatches of the clipped-surrogate update, each minibatch one CUDA-graph
replay). Observation normalisation (NORMALIZE_OBSERVATIONS) is off, as in the loop's default parameters (config.h:42-43); the
RunningNormalizer / standardize pieces exist separately (rl_tools_b200.RunningNormalizer).

Randomness: initial weights and the epoch shuffles come from the reference-compatible host engine (so a loop seeded like the reference's
starts from the reference's weights); resets and action noise are drawn inside the collect kernel (Philox), because host draw tables for
every collect would put a host round trip into every step.
"""
import math

from . import MlpShape, Mlp, AdamHyper, dense_init_weights, rng_init_host, pendulum_collect_device_rng
from . import ppo as _ppo


class PendulumPpoLoop:
    """ppo::loop::core::State for rl::environments::Pendulum with MLP actor (unconditional log_std) and critic, 3 -> H -> H -> 1 each."""

    def __init__(self, n_envs=64, steps_per_env=64, batch_size=512, hidden_dim=64, episode_step_limit=200, seed=0, n_epochs=10, gamma=0.99, lam=0.95,
                 epsilon_clip=0.2, entropy_coefficient=0.01, initial_action_std=0.5, adam=None, use_graphs=True, device="cuda"):
        import torch
        assert (n_envs * steps_per_env) % batch_size == 0, "the dataset must be a whole number of minibatches (ppo.h:41)"
        self.n_envs, self.steps_per_env, self.batch_size, self.step_limit = n_envs, steps_per_env, batch_size, episode_step_limit
        self.hyper = dict(n_epochs=n_epochs, epsilon_clip=epsilon_clip, entropy_coefficient=entropy_coefficient)
        self.gamma, self.lam = gamma, lam
        self.layout = _ppo.DatasetLayout(3, 1)
        acts = ["relu", "relu", "identity"]
        self.shape = MlpShape.make(3, [hidden_dim, hidden_dim, 1], acts)
        self.actor = Mlp(3, [hidden_dim, hidden_dim, 1], acts, batch_size, device=device, extra_params=1)
        self.critic = Mlp(3, [hidden_dim, hidden_dim, 1], acts, batch_size, device=device)
        if adam is not None:
            self.actor.hyper, self.critic.hyper = AdamHyper(**adam), AdamHyper(**adam)
        # init(device, ppo, ...) (rl/algorithms/ppo/operations_generic.h:40-57): init_weights of the actor, then of the critic, on one engine;
        # log_std = log(INITIAL_ACTION_STD)
        self.rng = rng_init_host(seed)
        for net in (self.actor, self.critic):
            off, fan_in = 0, 3
            for d in (hidden_dim, hidden_dim, 1):
                dense_init_weights(self.rng, net.params[off:off + d * fan_in].view(d, fan_in), net.params[off + d * fan_in:off + d * fan_in + d])
                off += d * fan_in + d; fan_in = d
            net.reset_optimizer_state()
        self.actor.extra("params").fill_(math.log(initial_action_std))
        z = lambda *s, dtype=torch.float32: torch.zeros(*s, device=device, dtype=dtype)
        # init(device, on_policy_runner, ...): every environment starts truncated, i.e. is reset by the first collect
        self.states, self.episode_step, self.episode_return = z(n_envs, 2), z(n_envs, dtype=torch.int32), z(n_envs)
        self.truncated = torch.ones(n_envs, device=device, dtype=torch.uint8)
        self.dataset = z((steps_per_env + 1) * n_envs, self.layout.data_dim)
        self.error_flag = z(1, dtype=torch.int32)
        self.seed, self.step_index = seed, 0
        self.graphs = _ppo.MinibatchGraphs(self.actor, self.critic, self.dataset, self.layout, n_envs * steps_per_env, batch_size,
                                           epsilon_clip=epsilon_clip, entropy_coefficient=entropy_coefficient) if use_graphs else None

    def step(self):
        """One loop step (operations_generic.h:88-131). Returns the mean reward per environment step of the collected data (a device tensor)."""
        L, n, T = self.layout, self.n_envs, self.steps_per_env
        pendulum_collect_device_rng(self.shape, self.actor.params, self.actor.extra("params"), self.states, self.episode_step, self.truncated, self.episode_return,
                                    self.seed, self.step_index * T, T, self.step_limit, dataset=self.dataset, error_flag=self.error_flag)
        _ppo.evaluate_values(self.critic, self.dataset, L)
        _ppo.estimate_generalized_advantages(self.dataset, L, n, T, self.gamma, self.lam)
        _ppo.train(self.actor, self.critic, self.dataset, L, n * T, self.batch_size, shuffle_rng_state=self.rng, graphs=self.graphs, **self.hyper)
        self.step_index += 1
        return self.dataset[:n * T, L.rewards].mean()

    def mean_episode_return(self):
        """Mean reward per step of the last collect scaled to a whole episode: what the reference's evaluation step reports, up to the
        exploration noise that the collected actions carry."""
        L = self.layout
        return float(self.dataset[:self.n_envs * self.steps_per_env, L.rewards].mean().item()) * self.step_limit
