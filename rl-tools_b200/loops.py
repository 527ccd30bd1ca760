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


class PendulumSacLoop:
    """sac::loop::core::State for rl::environments::Pendulum (rl/algorithms/sac/loop/core: config.h:19-49 parameters, operations_generic.h:71-87
    init, :110-152 step) with the configuration of the reference's Pendulum example (src/rl/environments/pendulum/sac/cpu/training.h:44-54):
    one environment, actor 3 -> 64 -> 64 -> 2 with the sample-and-squash head, two critics 4 -> 64 -> 64 -> 1, batch 100, replay capacity =
    step limit = 10,000, 100 warm-up steps with uniformly random actions, every interval 1, shared batch.

    One `step()` = the runner step in two halves around the stochastic actor (prologue: reset / observe; actor evaluate; head sample;
    epilogue: environment step, reward, replay append), then -- past the warm-up -- gather_batch, the three noise tensors, train_critic x 2,
    update_critic_targets, train_actor (incl. log_alpha). Past the warm-up the whole step is ONE CUDA-graph replay: every random draw inside it
    (reset states, exploration noise, batch indices, update noise) comes from the counter-based generator keyed by a device-resident step counter
    that the graph's last node advances, so nothing returns to the host between steps."""

    OBS_DIM, ACTION_DIM, STATE_DIM = 3, 1, 2

    def __init__(self, n_envs=1, batch_size=100, hidden_dim=64, step_limit=10000, n_warmup_steps=100, episode_step_limit=200, replay_capacity=None, seed=0,
                 use_graph=True, device="cuda"):
        import torch
        from . import sac, ReplayLayout, new_batch
        O, A, S = self.OBS_DIM, self.ACTION_DIM, self.STATE_DIM
        assert n_warmup_steps * n_envs >= batch_size, "config.h:25"
        self.n_envs, self.batch_size, self.step_limit, self.n_warmup_steps, self.episode_step_limit = n_envs, batch_size, step_limit, n_warmup_steps, episode_step_limit
        self.seed, self.step_index, self.use_graph, self.device = seed, 0, use_graph, device
        self.agent = sac.ActorCritic(O, A, hidden_dim, batch_size, device=device)
        self.hidden_dim = hidden_dim
        # init(device, actor_critic, rng) (rl/algorithms/sac/operations_generic.h:112-131): init_weights of the actor and the two critics on one engine
        self.rng = rng_init_host(seed)
        for net, fan_in0, out in ((self.agent.actor, O, 2 * A), (self.agent.critics[0], O + A, 1), (self.agent.critics[1], O + A, 1)):
            off, fan_in = 0, fan_in0
            for d in (hidden_dim, hidden_dim, out):
                dense_init_weights(self.rng, net.params[off:off + d * fan_in].view(d, fan_in), net.params[off + d * fan_in:off + d * fan_in + d])
                off += d * fan_in + d; fan_in = d
            net.zero_gradient(); net.reset_optimizer_state()
        self.agent.copy_critics_to_targets()
        z = lambda *s, dtype=torch.float32: torch.zeros(*s, device=device, dtype=dtype)
        # init(device, off_policy_runner): every environment starts truncated (reset by the first step), empty replay buffers
        N = n_envs
        self.layout = ReplayLayout.packed(step_limit if replay_capacity is None else replay_capacity, O, A)
        self.replay = z(N * self.layout.env_stride, dtype=torch.uint8)
        self.states, self.episode_step, self.episode_return = z(N, S), z(N, dtype=torch.int32), z(N)
        self.truncated, self.was_truncated = torch.ones(N, device=device, dtype=torch.uint8), z(N, dtype=torch.uint8)
        self.observations, self.actions, self.next_observations = z(N, O), z(N, A), z(N, O)
        self.head_input, self.explore_noise = z(N, 2 * A), z(N, A)
        self.explore_pre, self.explore_log_prob = z(N, A), z(N)
        self.batch, self.update_noise = new_batch(batch_size, O, A, device=device), z(3, batch_size, A)
        self.counter = z(1, dtype=torch.int64)                      # the loop's step index on the device
        self.error_flag = z(1, dtype=torch.int32)
        self.graph = None

    # ---- the two halves of the runner step -------------------------------------------------------------------------------------------
    def _prologue(self):
        from . import pendulum_offpolicy_prologue
        pendulum_offpolicy_prologue(self.states, self.episode_step, self.truncated, self.episode_return, self.observations, self.was_truncated, seed=self.seed,
                                    call_counter=self.counter)

    def _epilogue(self):
        from . import pendulum_offpolicy_epilogue
        pendulum_offpolicy_epilogue(self.states, self.episode_step, self.truncated, self.episode_return, self.episode_step_limit, self.observations, self.actions,
                                    self.next_observations, self.replay, self.layout, self.was_truncated)

    def _warmup_step(self):
        """step<0> with the uniform random exploration policy (operations_generic.h:117-121)."""
        import torch
        from . import counter_advance
        self._prologue()
        self.actions.copy_(torch.rand_like(self.actions) * 2 - 1)
        self._epilogue()
        counter_advance(self.counter, 1)

    def _train_step(self):
        """step<1> with the actor, then the update (operations_generic.h:114-148), all draws keyed by the device-resident step counter."""
        from . import sample_and_squash_forward, randn_device_rng, gather_batch, counter_advance
        a = self.agent
        self._prologue()
        a.actor.evaluate(self.observations, y=self.head_input)
        randn_device_rng(self.explore_noise, self.seed, stream_id=2, call_counter=self.counter)
        sample_and_squash_forward(self.head_input, self.explore_noise, output=self.actions, pre_squashing=self.explore_pre, log_probs=self.explore_log_prob)
        self._epilogue()
        gather_batch(self.replay, self.layout, self.n_envs, self.batch, seed=self.seed, call_counter=self.counter, max_episode_length=self.episode_step_limit,
                     obs_dim=self.OBS_DIM, action_dim=self.ACTION_DIM, error_flag=self.error_flag)
        randn_device_rng(self.update_noise, self.seed, stream_id=1, call_counter=self.counter)
        a.update(self.batch, self.update_noise[0], self.update_noise[1], self.update_noise[2])
        counter_advance(self.counter, 1)

    def step(self):
        """One loop step; returns True once the step limit is reached (operations_generic.h:111-113)."""
        import torch
        if self.step_index >= self.step_limit:
            return True
        if self.step_index < self.n_warmup_steps:
            self._warmup_step()
        elif not self.use_graph:
            self._train_step()
        else:
            if self.graph is None:
                side = torch.cuda.Stream(device=self.device)
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self._train_step()                             # this loop step, eagerly (also warms every kernel up before the capture)
                torch.cuda.current_stream().wait_stream(side)
                self.graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.graph, stream=side):
                    self._train_step()
            else:
                self.graph.replay()
        self.step_index += 1
        return False

    def evaluation_actor(self):
        """The deterministic evaluation policy (the head in evaluation mode: action = tanh(mean)) as a 3 -> H -> H -> 1 actor with tanh output:
        the mean row of the actor's output layer. Returns (shape, parameter arena)."""
        import torch
        H = self.hidden_dim
        p = self.agent.actor.params
        body = H * 3 + H + H * H + H
        arena = torch.cat([p[:body], p[body:body + H], p[body + 2 * H:body + 2 * H + 1]])
        return MlpShape.make(3, [H, H, 1], ["relu", "relu", "tanh"]), arena

    def evaluate(self, n_episodes=100, seed=12345):
        """Mean return of n_episodes evaluation episodes (one fused rollout launch of n_episodes environments x the episode step limit)."""
        import torch
        from . import pendulum_rollout_device_rng
        shape, arena = self.evaluation_actor()
        z = lambda *s, dtype=torch.float32: torch.zeros(*s, device=self.device, dtype=dtype)
        st, es, er = z(n_episodes, 2), z(n_episodes, dtype=torch.int32), z(n_episodes)
        tr = torch.ones(n_episodes, device=self.device, dtype=torch.uint8)
        _, _, rew = pendulum_rollout_device_rng(shape, arena, st, es, tr, er, seed, 0, self.episode_step_limit, self.episode_step_limit)
        return float(rew.view(self.episode_step_limit, n_episodes).sum(0).mean().item())


class L2fSacLoop(PendulumSacLoop):
    """The same loop on the L2F quadrotor (rl::environments::Multirotor in the configuration of the reference's GPU harness: 18 observations,
    4 rotor commands, episodes of at most 500 steps that end early when the quadrotor leaves the termination bounds): the runner's halves are
    b200rl_l2f_offpolicy_prologue / _epilogue with every reset drawn in the kernel from the environment's own initial-state distribution;
    actor 18 -> H -> H -> 8 with the sample-and-squash head, critics 22 -> H -> H -> 1. `parameters` is an L2fParameters, `mdp` the 18 floats of
    the reward function and termination thresholds, `init` the 12 floats of the initial-state distribution (all read out of the reference's
    structs when the fixtures are written)."""
    OBS_DIM, ACTION_DIM, STATE_DIM = 18, 4, 23

    def __init__(self, parameters, mdp, init, n_envs=16, batch_size=256, hidden_dim=64, step_limit=100000, n_warmup_steps=None, episode_step_limit=500,
                 replay_capacity=None, seed=0, use_graph=True, device="cuda"):
        self.parameters, self.mdp, self.init = parameters, [float(v) for v in mdp], [float(v) for v in init]
        warm = n_warmup_steps if n_warmup_steps is not None else max(100, -(-batch_size // n_envs))
        super().__init__(n_envs=n_envs, batch_size=batch_size, hidden_dim=hidden_dim, step_limit=step_limit, n_warmup_steps=warm, episode_step_limit=episode_step_limit,
                         replay_capacity=replay_capacity, seed=seed, use_graph=use_graph, device=device)

    def _prologue(self):
        from . import l2f_offpolicy_prologue
        l2f_offpolicy_prologue(self.parameters, self.states, self.episode_step, self.truncated, self.episode_return, self.observations, self.was_truncated,
                               init=self.init, seed=self.seed, call_counter=self.counter)

    def _epilogue(self):
        from . import l2f_offpolicy_epilogue
        l2f_offpolicy_epilogue(self.parameters, self.mdp, self.states, self.episode_step, self.truncated, self.episode_return, self.episode_step_limit, self.actions,
                               self.next_observations, self.replay, self.layout, self.was_truncated)

    def evaluation_actor(self):
        """The deterministic evaluation policy, action = tanh(mean): the four mean rows of the actor's output layer as an 18 -> H -> H -> 4 actor."""
        import torch
        H, O, A = self.hidden_dim, self.OBS_DIM, self.ACTION_DIM
        p = self.agent.actor.params
        body = H * O + H + H * H + H
        arena = torch.cat([p[:body], p[body:body + A * H], p[body + 2 * A * H:body + 2 * A * H + A]])
        return MlpShape.make(O, [H, H, A], ["relu", "relu", "tanh"]), arena

    def evaluate(self, n_episodes=256, seed=12345):
        """(mean return, mean length) of n_episodes evaluation episodes: one fused rollout launch, each environment's first episode."""
        import torch
        from . import l2f_rollout_device_rng
        shape, arena = self.evaluation_actor()
        T = self.episode_step_limit
        z = lambda *s, dtype=torch.float32: torch.zeros(*s, device=self.device, dtype=dtype)
        st, es, er = z(n_episodes, 23), z(n_episodes, dtype=torch.int32), z(n_episodes)
        tr = torch.ones(n_episodes, device=self.device, dtype=torch.uint8)
        _, _, rew, term = l2f_rollout_device_rng(self.parameters, self.mdp, self.init, shape, arena, st, es, tr, er, seed, 0, T, T)
        rew, term = rew.view(T, n_episodes), term.view(T, n_episodes)
        alive = (term.cumsum(0) - term) == 0                          # steps up to and including the first termination
        return float((rew * alive).sum(0).mean().item()), float(alive.sum(0).float().mean().item())

