"""Host-side mirror of the reference's SAC update, driving the C ABI (rl/algorithms/sac/operations_generic.h).

`ActorCritic` holds what rl::algorithms::sac::ActorCritic holds (sac.h:131-146): the actor (an MLP whose 2 * action_dim outputs feed the
sample-and-squash head, plus the head's log_alpha parameter), two critics, their two target networks and four Adam states. Its verbs
are the reference's: `train_critic` (:223-336), `update_critic_targets` (:486-522), `train_actor` (:378-456), for sequence length 1 with
the default parameters of sac.h:9-35 (entropy bonus inside the discounted term, non-terminal masking — a no-op at sequence length 1 —
termination honoured). Batches are the tensors `gather_batch` fills. Everything runs on the GPU on torch CUDA tensors; there is no CPU path.
"""
import math

from . import (Mlp, AdamHyper, lib, check, fill, _ptr, _stream, mse_gradient as _mse_gradient, polyak_update as _polyak_update,
               sample_and_squash_forward as _head_forward, sample_and_squash_backward as _head_backward,
               sac_target_action_values as _target_action_values, sac_min_value_d_output as _min_value_d_output)


class ActorCritic:
    def __init__(self, observation_dim, action_dim, hidden_dim, batch, hidden_activation="relu", device="cuda", gamma=0.99, critic_polyak=1.0 - 0.005,
                 alpha=0.5, target_entropy=None):
        import torch
        O, A, H = observation_dim, action_dim, hidden_dim
        self.observation_dim, self.action_dim, self.batch, self.device = O, A, batch, device
        acts = [hidden_activation, hidden_activation, "identity"]
        self.actor = Mlp(O, [H, H, 2 * A], acts, batch, device=device)
        self.critics = [Mlp(O + A, [H, H, 1], acts, batch, device=device) for _ in range(2)]
        self.critics_target = [Mlp(O + A, [H, H, 1], acts, 2 * batch, device=device) for _ in range(2)]     # evaluated on both critics' next inputs at once
        self.gamma, self.critic_polyak = gamma, critic_polyak
        import numpy as np
        self._minus_one_over_batch = float(np.float32(-1) / np.float32(batch))                  # the reference divides in fp32
        self.target_entropy = -float(A) if target_entropy is None else target_entropy           # sac.h:28
        z = lambda *s: torch.zeros(*s, device=device, dtype=torch.float32)
        # log_alpha: a one-element parameter with its own optimizer (alpha_optimizer, sac.h:145)
        self.log_alpha, self.log_alpha_grad, self.log_alpha_m, self.log_alpha_v = z(1), z(1), z(1), z(1)
        self.log_alpha.fill_(math.log(alpha))                                                    # nn/layers/sample_and_squash/operations_generic.h:76-80
        self.log_alpha_adam_state = torch.zeros(4, device=device, dtype=torch.int32)
        self.alpha_hyper = AdamHyper()
        check(lib().b200rl_adam_reset(_ptr(self.log_alpha_adam_state), _stream()), "b200rl_adam_reset")
        # training buffers (CriticTrainingBuffers / ActorTrainingBuffers, sac.h:58-129)
        self.next_input, self.actor_input = z(batch, O + A), z(batch, O + A)
        self.next_head_input = z(batch, 2 * A)
        self.next_log_probs, self.target_action_value = z(batch), z(batch, 1)
        self.q_next = [z(batch, 1), z(batch, 1)]
        self.pre_squashing, self.actions, self.log_probs = z(batch, A), z(batch, A), z(batch)
        self.d_critic_input = [z(batch, O + A), z(batch, O + A)]
        self.d_actor_output, self.d_head_input, self.d_output = z(batch, A), z(batch, 2 * A), z(batch, 1)
        # update(): both critics' next inputs stacked [2B, O + A], per-critic targets and loss gradients, and a second stream for the
        # work of critic 1 (the two critics' chains are independent; captured in a CUDA graph they become parallel branches)
        self.next_input_2, self.q_next_2 = z(2 * batch, O + A), [z(2 * batch, 1), z(2 * batch, 1)]
        self.next_log_probs_2, self.target_2 = z(2 * batch), z(2 * batch, 1)
        self.d_output_2 = [z(batch, 1), z(batch, 1)]
        self.side_stream = torch.cuda.Stream(device=device)

    def copy_critics_to_targets(self):
        """init(): the target networks start as copies of the critics (:126-131)."""
        for c in range(2):
            self.critics_target[c].params.copy_(self.critics[c].params)

    def train_critic(self, critic_index, batch, action_noise):
        """One critic update on `batch` (dict of gather_batch tensors) with the external noise [B, A] of the next-state action sample."""
        O = self.observation_dim
        critic = self.critics[critic_index]
        critic.zero_gradient()
        self.next_input.copy_(batch["oa_base"][1])                                               # next observation | (action columns overwritten below)
        self.actor.evaluate(self.next_input[:, :O], y=self.next_head_input)
        _head_forward(self.next_head_input, action_noise, output=self.next_input[:, O:], pre_squashing=self.pre_squashing, log_probs=self.next_log_probs)
        for c in range(2):
            self.critics_target[c].evaluate(self.next_input, y=self.q_next[c])
        _target_action_values(self.q_next[0], self.q_next[1], batch["rewards"], batch["terminated"], self.next_log_probs, self.log_alpha, gamma=self.gamma,
                              target=self.target_action_value)
        values = critic.forward(batch["oa_base"][0])
        critic.backward(batch["oa_base"][0], _mse_gradient(values, self.target_action_value, 0.5, d_a=critic.d_out_buffer()))
        critic.step()

    def update_critic_targets(self):
        for c in range(2):
            _polyak_update(self.critics[c].params.view(1, -1), self.critics_target[c].params.view(1, -1), self.critic_polyak)

    def train_actor(self, batch, action_noise):
        """One actor update (and one log_alpha update) on `batch` with the external noise [B, A] of the action sample."""
        O, A, B = self.observation_dim, self.action_dim, self.batch
        self.actor.zero_gradient()
        fill(self.log_alpha_grad, 0.0)
        self.actor_input.copy_(batch["oa_base"][0])
        observations = self.actor_input[:, :O]
        head_input = self.actor.forward(observations)
        _head_forward(head_input, action_noise, output=self.actor_input[:, O:], pre_squashing=self.pre_squashing, log_probs=self.log_probs)
        self.actions.copy_(self.actor_input[:, O:])
        def through_critic(c):
            value = self.critics[c].forward(self.actor_input)
            fill(self.d_output_2[c], self._minus_one_over_batch)                                 # the mean over the (all final) steps, negated (:424-431)
            self.critics[c].backward(self.actor_input, self.d_output_2[c], d_input=self.d_critic_input[c], accumulate_gradients=False)     # backward_input (:433-434)
            return value
        with self._fork():                                                                       # the two critics are independent: two streams
            q1 = through_critic(1)
        q = [through_critic(0), q1]
        self._join()
        _min_value_d_output(q[0], q[1], self.d_critic_input[0], self.d_critic_input[1], A, d_actor_output=self.d_actor_output)
        _head_backward(head_input, action_noise, self.pre_squashing, self.actions, self.d_actor_output, self.log_alpha, log_alpha_gradient=self.log_alpha_grad,
                       target_entropy=self.target_entropy, d_input=self.d_head_input)
        self.actor.backward(observations, self.d_head_input)
        self.actor.step()
        check(lib().b200rl_adam_step(_ptr(self.log_alpha), _ptr(self.log_alpha_grad), _ptr(self.log_alpha_m), _ptr(self.log_alpha_v), 1, self.alpha_hyper,
                                     _ptr(self.log_alpha_adam_state), _stream()), "b200rl_adam_step")

    def _fork(self):
        import torch
        self.side_stream.wait_stream(torch.cuda.current_stream())
        return torch.cuda.stream(self.side_stream)

    def _join(self):
        import torch
        torch.cuda.current_stream().wait_stream(self.side_stream)

    def train_critics(self, batch, noise_0, noise_1):
        """train_critic for both critics on one shared batch, with the same results as two train_critic calls: the actor's pass over the
        next observations is shared (it does not depend on the noise), each target network runs once over both critics' next inputs, and
        the two critics' forward / backward / Adam chains run on two streams."""
        O, B = self.observation_dim, self.batch
        self.next_input_2[:B].copy_(batch["oa_base"][1]); self.next_input_2[B:].copy_(batch["oa_base"][1])
        self.actor.evaluate(self.next_input_2[:B, :O], y=self.next_head_input)
        for c, noise in enumerate((noise_0, noise_1)):
            rows = slice(c * B, (c + 1) * B)
            _head_forward(self.next_head_input, noise, output=self.next_input_2[rows, O:], pre_squashing=self.pre_squashing, log_probs=self.next_log_probs_2[rows])
        with self._fork():                                               # the two target networks are independent
            self.critics_target[1].evaluate(self.next_input_2, y=self.q_next_2[1])
        self.critics_target[0].evaluate(self.next_input_2, y=self.q_next_2[0])
        self._join()
        for c in range(2):
            rows = slice(c * B, (c + 1) * B)
            _target_action_values(self.q_next_2[0][rows], self.q_next_2[1][rows], batch["rewards"], batch["terminated"], self.next_log_probs_2[rows], self.log_alpha,
                                  gamma=self.gamma, target=self.target_2[rows])
        self.target_action_value = self.target_2[B:]                     # what the second train_critic call would have left behind

        def chain(c):
            critic = self.critics[c]
            critic.zero_gradient()
            values = critic.forward(batch["oa_base"][0])
            critic.backward(batch["oa_base"][0], _mse_gradient(values, self.target_2[c * B:(c + 1) * B], 0.5, d_a=critic.d_out_buffer()))
            critic.step()
        with self._fork():
            chain(1)
        chain(0)
        self._join()

    def update(self, batch, noise_critic_0, noise_critic_1, noise_actor):
        """One step of the reference's training loop on a shared batch (rl/algorithms/sac/loop/core/operations_generic.h:124-152)."""
        self.train_critics(batch, noise_critic_0, noise_critic_1)
        # the target update reads the critics and writes the targets; train_actor reads the critics only: independent of each other.
        # (train_actor forks onto the same side stream itself, after this work in stream order.)
        with self._fork():
            self.update_critic_targets()
        self.train_actor(batch, noise_actor)
        self._join()
