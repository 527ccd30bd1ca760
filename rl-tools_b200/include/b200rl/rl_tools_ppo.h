// Header-only adapter, part 4: the PPO update on `devices::B200`.
//
// Include after <b200rl/rl_tools_on_policy_runner.h> and <rl_tools/rl/algorithms/ppo/operations_generic.h>.
//
// The reference's estimate_generalized_advantages and train (rl/algorithms/ppo/operations_generic.h:59-95, 96-336) are host loops
// over single matrix elements, which cannot touch device memory; these overloads keep their signatures and run the same update on the
// dataset matrix in device memory: GAE as one scan per environment, the per-sample clipped-surrogate loop as three kernels between the
// actor's forward and backward pass (which go through the reference's own generic network code on this device tag), the critic
// regression, one Adam step each. The epoch shuffle draws its swap targets on the host from the caller's engine with the reference's own
// uniform_int_distribution, in the reference's order, and applies the resulting row permutation on the device.
//
// Not supported (static_assert): ADAPTIVE_LEARNING_RATE, STATEFUL_ACTOR_AND_CRITIC, asymmetric observations, multi-agent environments.
#pragma once
#include "rl_tools_operations.h"
#include <vector>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    template <typename DEV_SPEC, typename DATASET_SPEC, typename PPO_PARAMETERS>
    void estimate_generalized_advantages(devices::B200<DEV_SPEC>& device, rl::components::on_policy_runner::Dataset<DATASET_SPEC>& dataset, PPO_PARAMETERS){
        using OPR_SPEC = typename DATASET_SPEC::SPEC;
        static_assert(utils::typing::is_same_v<typename OPR_SPEC::TYPE_POLICY::DEFAULT, float>, "fp32 only");
        const int ld = (int)rl_tools::b200::ld(dataset.data);
        b200::note(device, b200rl_gae(dataset.rewards._data, ld, dataset.all_values._data, ld, dataset.terminated._data, ld, dataset.truncated._data, ld,
                                      dataset.advantages._data, ld, dataset.target_values._data, ld, (int)OPR_SPEC::N_ENVIRONMENTS, (int)DATASET_SPEC::STEPS_PER_ENV,
                                      (float)PPO_PARAMETERS::GAMMA, (float)PPO_PARAMETERS::LAMBDA, PPO_PARAMETERS::IGNORE_TERMINATION ? 1 : 0, device.stream));
    }

    template <typename DEV_SPEC, typename PPO_SPEC, typename DATASET_SPEC, typename ACTOR_OPTIMIZER, typename CRITIC_OPTIMIZER, typename BUFFERS_SPEC, typename ACTOR_BUFFER, typename CRITIC_BUFFER, typename RNG>
    void train(devices::B200<DEV_SPEC>& device, rl::algorithms::PPO<PPO_SPEC>& ppo, rl::components::on_policy_runner::Dataset<DATASET_SPEC>& dataset,
               ACTOR_OPTIMIZER& actor_optimizer, CRITIC_OPTIMIZER& critic_optimizer, rl::algorithms::ppo::Buffers<BUFFERS_SPEC>& ppo_buffers,
               ACTOR_BUFFER& actor_buffers, CRITIC_BUFFER& critic_buffers, RNG& rng){
        using T = typename PPO_SPEC::TYPE_POLICY::DEFAULT;
        using TI = typename PPO_SPEC::TI;
        using ENVIRONMENT = typename PPO_SPEC::ENVIRONMENT;
        using PARAMETERS = typename PPO_SPEC::PARAMETERS;
        using DATASET = rl::components::on_policy_runner::Dataset<DATASET_SPEC>;
        static_assert(utils::typing::is_same_v<T, float>, "fp32 only");
        static_assert(!PARAMETERS::ADAPTIVE_LEARNING_RATE && !PARAMETERS::STATEFUL_ACTOR_AND_CRITIC, "not implemented on this device");
        static_assert(!PPO_SPEC::ASYMMETRIC_OBSERVATIONS && ENVIRONMENT::N_AGENTS == 1, "not implemented on this device");
        constexpr TI N_EPOCHS = PARAMETERS::N_EPOCHS, BATCH_SIZE = PARAMETERS::BATCH_SIZE, N_BATCHES = DATASET::STEPS_TOTAL / BATCH_SIZE;
        constexpr TI ACTION_DIM = ENVIRONMENT::ACTION_DIM, OBSERVATION_DIM = ENVIRONMENT::Observation::DIM;
        static_assert(N_BATCHES > 0 && DATASET::DATA_DIM <= 64, "the row permutation takes a 64-bit column mask");
        const int ld = (int)rl_tools::b200::ld(dataset.data);

        void *d_perm = nullptr, *d_scratch = nullptr, *d_shuffle_scratch = nullptr;
        const size_t ppo_scratch_bytes = b200rl_ppo_scratch_bytes((int)BATCH_SIZE, (int)ACTION_DIM);
        unsigned long long shuffled_columns = 0;
        {   // observation, action, log-prob, advantage, target value: the columns the reference swaps (:127-158)
            const TI o = 0, a = OBSERVATION_DIM + ACTION_DIM;
            for(TI c = 0; c < OBSERVATION_DIM; c++) shuffled_columns |= 1ull << (o + c);
            for(TI c = 0; c < ACTION_DIM; c++) shuffled_columns |= 1ull << (a + c);
            const TI log_prob = OBSERVATION_DIM + 2 * ACTION_DIM;
            shuffled_columns |= (1ull << log_prob) | (1ull << (log_prob + 6)) | (1ull << (log_prob + 7));
        }
        const size_t shuffle_scratch_bytes = b200rl_permute_rows_scratch_bytes((int)DATASET::STEPS_TOTAL, shuffled_columns);
        b200::note(device, b200rl_device_malloc(&d_scratch, ppo_scratch_bytes));
        if constexpr(PARAMETERS::SHUFFLE_EPOCH){
            b200::note(device, b200rl_device_malloc(&d_perm, sizeof(int32_t) * DATASET::STEPS_TOTAL));
            b200::note(device, b200rl_device_malloc(&d_shuffle_scratch, shuffle_scratch_bytes));
        }
        auto& last_layer = get_last_layer(ppo.actor);
        for(TI epoch_i = 0; epoch_i < N_EPOCHS; epoch_i++){
            if constexpr(PARAMETERS::SHUFFLE_EPOCH){
                std::vector<int32_t> perm(DATASET::STEPS_TOTAL);
                for(TI i = 0; i < DATASET::STEPS_TOTAL; i++) perm[i] = (int32_t)i;
                for(TI dataset_i = 0; dataset_i < DATASET::STEPS_TOTAL; dataset_i++){
                    const TI sample_index = random::uniform_int_distribution(device.random, dataset_i, (TI)(DATASET::STEPS_TOTAL - 1), rng);
                    const int32_t tmp = perm[dataset_i]; perm[dataset_i] = perm[sample_index]; perm[sample_index] = tmp;
                }
                b200::note(device, b200rl_memcpy(d_perm, perm.data(), sizeof(int32_t) * perm.size(), 0, device.stream));
                b200::note(device, b200rl_permute_rows(dataset.data._data, ld, (int)DATASET::STEPS_TOTAL, static_cast<const int32_t*>(d_perm), shuffled_columns,
                                                       d_shuffle_scratch, shuffle_scratch_bytes, device.stream));
            }
            for(TI batch_i = 0; batch_i < N_BATCHES; batch_i++){
                zero_gradient(device, ppo.critic);
                zero_gradient(device, ppo.actor);
                const TI batch_offset = batch_i * BATCH_SIZE;
                auto batch_observations     = view(device, dataset.observations    , matrix::ViewSpec<BATCH_SIZE, OBSERVATION_DIM>(), batch_offset, 0);
                auto batch_actions          = view(device, dataset.actions         , matrix::ViewSpec<BATCH_SIZE, ACTION_DIM     >(), batch_offset, 0);
                auto batch_action_log_probs = view(device, dataset.action_log_probs, matrix::ViewSpec<BATCH_SIZE, 1              >(), batch_offset, 0);
                auto batch_advantages       = view(device, dataset.advantages      , matrix::ViewSpec<BATCH_SIZE, 1              >(), batch_offset, 0);
                auto batch_target_values    = view(device, dataset.target_values   , matrix::ViewSpec<BATCH_SIZE, 1              >(), batch_offset, 0);

                auto batch_observations_tensor = to_tensor(device, batch_observations);
                auto batch_observations_tensor_reshaped = reshape_row_major(device, batch_observations_tensor, tensor::Shape<TI, 1, BATCH_SIZE, OBSERVATION_DIM>{});
                auto current_batch_actions_tensor = to_tensor(device, ppo_buffers.current_batch_actions);
                auto current_batch_actions_tensor_reshaped = reshape_row_major(device, current_batch_actions_tensor, tensor::Shape<TI, 1, BATCH_SIZE, ACTION_DIM>{});
                forward(device, ppo.actor, batch_observations_tensor_reshaped, current_batch_actions_tensor_reshaped, actor_buffers, rng);

                b200::note(device, b200rl_ppo_policy_gradient(ppo_buffers.current_batch_actions._data, (int)rl_tools::b200::ld(ppo_buffers.current_batch_actions),
                                                              batch_actions._data, ld, last_layer.log_std.parameters._data, batch_action_log_probs._data, ld,
                                                              batch_advantages._data, ld, ppo_buffers.d_action_log_prob_d_action._data,
                                                              (int)rl_tools::b200::ld(ppo_buffers.d_action_log_prob_d_action), last_layer.log_std.gradient._data,
                                                              (int)BATCH_SIZE, (int)ACTION_DIM, (float)PARAMETERS::EPSILON_CLIP, (float)PARAMETERS::ACTION_ENTROPY_COEFFICIENT,
                                                              (float)PARAMETERS::ADVANTAGE_EPSILON, PARAMETERS::NORMALIZE_ADVANTAGE ? 1 : 0, PARAMETERS::LEARN_ACTION_STD ? 1 : 0,
                                                              d_scratch, ppo_scratch_bytes, device.stream));
                auto d_actions_tensor = to_tensor(device, ppo_buffers.d_action_log_prob_d_action);
                auto d_actions_tensor_reshaped = reshape_row_major(device, d_actions_tensor, tensor::Shape<TI, 1, BATCH_SIZE, ACTION_DIM>{});
                backward(device, ppo.actor, batch_observations_tensor_reshaped, d_actions_tensor_reshaped, actor_buffers);

                forward(device, ppo.critic, batch_observations_tensor_reshaped, critic_buffers, rng);
                auto output_tensor = output(device, ppo.critic);
                auto output_matrix_view = matrix_view(device, output_tensor);
                nn::loss_functions::mse::gradient(device, output_matrix_view, batch_target_values, ppo_buffers.d_critic_output, (T)0.5);
                auto d_critic_output_tensor = to_tensor(device, ppo_buffers.d_critic_output);
                auto d_critic_output_tensor_reshaped = reshape_row_major(device, d_critic_output_tensor, tensor::Shape<TI, 1, BATCH_SIZE, 1>{});
                backward(device, ppo.critic, batch_observations_tensor_reshaped, d_critic_output_tensor_reshaped, critic_buffers);

                step(device, actor_optimizer, ppo.actor);
                step(device, critic_optimizer, ppo.critic);
            }
        }
        b200::note(device, b200rl_stream_synchronize(device.stream));
        b200::note(device, b200rl_device_free(d_scratch));
        if(d_perm) b200::note(device, b200rl_device_free(d_perm));
        if(d_shuffle_scratch) b200::note(device, b200rl_device_free(d_shuffle_scratch));
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
