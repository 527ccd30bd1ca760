// Header-only adapter, part 5: the off-policy runner on `devices::B200`.
//
// Include after <b200rl/rl_tools_on_policy_runner.h> and <rl_tools/rl/components/off_policy_runner/operations_generic.h>.
//
// Mirrors malloc / free / init / step<POLICY_INDEX> / gather_batch of the reference's CUDA runner (rl/components/off_policy_runner/operations_cuda.h:
// 117-204): the runner's matrices, including the statically allocated per-environment replay-buffer structs, live in device memory,
// and one step is the fused rollout kernel (T = 1) into the runner's step buffers followed by the replay-buffer append kernel, which
// writes the reference's struct layout in place (byte offsets taken from the struct type on the host). Reset draws are made on the host
// with the reference's own sample_initial_state on the caller's engine, in environment order, like the reference's CPU runner.
//
// Supported: rl::environments::Pendulum, symmetric observations, fp32. The policy sequential< mlp 3 -> 64 -> 64 -> 1 > (or that mlp itself)
// takes the fused kernel; ANY other policy that evaluates on this device runs as the reference's CUDA runner does -- prologue kernel, the
// reference's own interlude (evaluate_step of the policy on the runner's observation / action buffers), epilogue kernel.
// gather_batch: SequentialBatch with sequence length 1 draws on the caller's host engine in the reference's order (same batch as the reference);
// longer sequences and the DETERMINISTIC flag go to the kernel with in-kernel draws. Not provided: episode statistics. The view members
// inside the device-resident replay-buffer structs are not initialised: only the data matrix, episode_start and the position / full /
// current_episode_start counters are maintained, and the kernels address rows through byte offsets.
#pragma once
#include "rl_tools_on_policy_runner.h"
#include <memory>
#include <vector>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    namespace b200{
        template <typename SPEC>
        b200rl_replay_layout replay_layout(){
            using RUNNER = rl::components::OffPolicyRunner<SPEC>;
            using RB = typename RUNNER::REPLAY_BUFFER_TYPE;
            static_assert(!SPEC::DYNAMIC_ALLOCATION_REPLAY_BUFFER, "the replay buffers must be statically allocated inside the runner (as for the reference's CUDA runner)");
            static std::unique_ptr<RB> probe(new RB());                       // only its member addresses are used
            const char* base = reinterpret_cast<const char*>(probe.get());
            b200rl_replay_layout L{};
            L.env_stride = sizeof(RB);
            L.off_data = reinterpret_cast<const char*>(probe->data._data) - base;
            L.off_episode_start = reinterpret_cast<const char*>(probe->episode_start._data) - base;
            L.off_position = reinterpret_cast<const char*>(&probe->position) - base;
            L.off_full = reinterpret_cast<const char*>(&probe->full) - base;
            L.off_current_episode_start = reinterpret_cast<const char*>(&probe->current_episode_start) - base;
            L.capacity = (int)SPEC::PARAMETERS::REPLAY_BUFFER_CAPACITY;
            L.ld_data = (int)rl_tools::b200::ld(probe->data);
            L.index_bytes = (int)sizeof(typename SPEC::TI);
            return L;
        }
        // whether a policy is the shape the fused runner kernel takes (overloads on the forward base classes, so that every capability of a
        // model matches; anything else falls to the last overload)
        template <typename MLP_SPEC>
        constexpr bool fused_actor(const nn_models::mlp::NeuralNetworkForward<MLP_SPEC>*){
            return MLP_SPEC::INPUT_DIM == 3 && MLP_SPEC::CONFIG::HIDDEN_DIM == 64 && MLP_SPEC::CONFIG::NUM_LAYERS == 3 && MLP_SPEC::CONFIG::OUTPUT_DIM == 1;
        }
        template <typename MODULE_SPEC>
        constexpr bool fused_actor(const nn_models::sequential::ModuleForward<MODULE_SPEC>*){
            using CONTENT = decltype(nn_models::sequential::ModuleForward<MODULE_SPEC>::content);
            return utils::typing::is_same_v<typename MODULE_SPEC::NEXT_MODULE, nn_models::sequential::OutputModule> && fused_actor(static_cast<const CONTENT*>(nullptr));
        }
        constexpr bool fused_actor(const void*){ return false; }
        // the six parameter tensors of a 3-layer MLP, for a bare mlp or a one-module sequential model around it
        template <typename MLP_SPEC>
        void actor_layers(nn_models::mlp::NeuralNetworkForward<MLP_SPEC>& mlp, const float* (&layers)[6], int (&acts)[3]){
            static_assert(MLP_SPEC::INPUT_DIM == 3 && MLP_SPEC::CONFIG::HIDDEN_DIM == 64 && MLP_SPEC::CONFIG::NUM_LAYERS == 3 && MLP_SPEC::CONFIG::OUTPUT_DIM == 1, "actor 3 -> 64 -> 64 -> 1");
            layers[0] = mlp.input_layer.weights.parameters._data; layers[1] = mlp.input_layer.biases.parameters._data;
            layers[2] = mlp.hidden_layers[0].weights.parameters._data; layers[3] = mlp.hidden_layers[0].biases.parameters._data;
            layers[4] = mlp.output_layer.weights.parameters._data; layers[5] = mlp.output_layer.biases.parameters._data;
            acts[0] = acts[1] = activation_id<MLP_SPEC::CONFIG::HIDDEN_ACTIVATION_FUNCTION>();
            acts[2] = activation_id<MLP_SPEC::CONFIG::OUTPUT_ACTIVATION_FUNCTION>();
        }
        template <typename MODULE_SPEC>
        void actor_layers(nn_models::sequential::ModuleForward<MODULE_SPEC>& model, const float* (&layers)[6], int (&acts)[3]){
            static_assert(utils::typing::is_same_v<typename MODULE_SPEC::NEXT_MODULE, nn_models::sequential::OutputModule>, "the policy must be the bare MLP module");
            actor_layers(model.content, layers, acts);
        }
    }
    // rl/components/off_policy_runner/operations_cuda.h:117-134
    template<typename DEV_SPEC, typename SPEC>
    void malloc(devices::B200<DEV_SPEC>& device, rl::components::OffPolicyRunner<SPEC>& runner){
        static_assert(!SPEC::DYNAMIC_ALLOCATION_REPLAY_BUFFER && !SPEC::DYNAMIC_ALLOCATION_EPISODE_STATS, "static allocation inside the runner, as for the reference's CUDA runner");
        malloc(device, runner.buffers.observations); malloc(device, runner.buffers.actions); malloc(device, runner.buffers.next_observations);
        malloc(device, runner.envs); malloc(device, runner.states); malloc(device, runner.env_parameters);
        malloc(device, runner.episode_return); malloc(device, runner.episode_step); malloc(device, runner.truncated);
        malloc(device, runner.replay_buffers); malloc(device, runner.episode_stats);
    }
    template<typename DEV_SPEC, typename SPEC>
    void free(devices::B200<DEV_SPEC>& device, rl::components::OffPolicyRunner<SPEC>& runner){
        free(device, runner.buffers.observations); free(device, runner.buffers.actions); free(device, runner.buffers.next_observations);
        free(device, runner.envs); free(device, runner.states); free(device, runner.env_parameters);
        free(device, runner.episode_return); free(device, runner.episode_step); free(device, runner.truncated);
        free(device, runner.replay_buffers); free(device, runner.episode_stats);
    }
    // rl/components/off_policy_runner/operations_generic.h:162-183: every environment truncated, empty replay buffers
    template<typename DEV_SPEC, typename SPEC>
    void init(devices::B200<DEV_SPEC>& device, rl::components::OffPolicyRunner<SPEC>& runner){
        using RUNNER = rl::components::OffPolicyRunner<SPEC>;
        static_assert(b200::is_pendulum<typename SPEC::ENVIRONMENT>::value, "only rl::environments::Pendulum is implemented on this device");
        static_assert(sizeof(typename RUNNER::REPLAY_BUFFER_TYPE) % 4 == 0);
        b200::note(device, b200rl_fill(reinterpret_cast<float*>(runner.replay_buffers._data), sizeof(typename RUNNER::REPLAY_BUFFER_TYPE) / 4 * (size_t)RUNNER::N_ENVIRONMENTS, 0.0f, device.stream));
        b200::fill_any(device, runner.truncated, true);
        b200::fill_any(device, runner.episode_step, 0);
        b200::fill_any(device, runner.episode_return, 0);
        runner.previous_policy_set = false;
        runner.previous_policy = 0;
#ifdef RL_TOOLS_DEBUG_RL_COMPONENTS_OFF_POLICY_RUNNER_CHECK_INIT
        runner.initialized = true;
#endif
    }
    // rl/components/off_policy_runner/operations_cuda.h:184-204
    template<auto POLICY_INDEX, typename DEV_SPEC, typename SPEC, typename POLICY, typename POLICY_BUFFERS, typename RNG>
    void step(devices::B200<DEV_SPEC>& device, rl::components::OffPolicyRunner<SPEC>& runner, POLICY& policy, POLICY_BUFFERS& policy_eval_buffers, RNG& rng){
        using RUNNER = rl::components::OffPolicyRunner<SPEC>;
        using ENVIRONMENT = typename SPEC::ENVIRONMENT;
        using T = typename SPEC::TYPE_POLICY::DEFAULT;
        using TI = typename SPEC::TI;
        constexpr TI N = RUNNER::N_ENVIRONMENTS;
        static_assert(b200::is_pendulum<ENVIRONMENT>::value, "only rl::environments::Pendulum is implemented on this device");
        static_assert(utils::typing::is_same_v<T, float> && sizeof(TI) == 4 && sizeof(bool) == 1 && sizeof(typename ENVIRONMENT::State) == 2 * sizeof(float));
        static_assert(!SPEC::PARAMETERS::ASYMMETRIC_OBSERVATIONS && !SPEC::PARAMETERS::COLLECT_EPISODE_STATS, "not implemented on this device");
        const bool policy_switch = runner.previous_policy_set && (POLICY_INDEX != runner.previous_policy);
        if(policy_switch) b200::fill_any(device, runner.truncated, true);

        // reset draws on the host, environments ascending (operations_generic_per_env.h:37-40)
        std::vector<uint8_t> truncated(N);
        b200::note(device, b200rl_memcpy(truncated.data(), runner.truncated._data, N, 1, device.stream));
        std::vector<float> reset_states((size_t)N * 2, 0.0f);
        ENVIRONMENT env; typename ENVIRONMENT::Parameters parameters; typename ENVIRONMENT::State state;
        for(TI env_i = 0; env_i < N; env_i++){
            if(truncated[env_i]){
                if(SPEC::PARAMETERS::SAMPLE_PARAMETERS) sample_initial_parameters(device, env, parameters, rng);
                sample_initial_state(device, env, parameters, state, rng);
                reset_states[2 * env_i] = state.theta; reset_states[2 * env_i + 1] = state.theta_dot;
            }
        }
        // work area kept for the life of the process: reset states [N, 2], rewards [N], previous flags [N], error flag
        static void* scratch = nullptr;
        constexpr size_t RESET_BYTES = sizeof(float) * 2 * N, REWARD_BYTES = sizeof(float) * N, FLAG_OFFSET = RESET_BYTES + REWARD_BYTES + ((N + 15) / 16) * 16;
        if(!scratch) b200::note(device, b200rl_device_malloc(&scratch, FLAG_OFFSET + 16));
        if(!scratch) return;
        char* sc = static_cast<char*>(scratch);
        int flag = 0;
        b200::note(device, b200rl_memcpy(sc, reset_states.data(), RESET_BYTES, 0, device.stream));
        b200::note(device, b200rl_memcpy(sc + FLAG_OFFSET, &flag, sizeof(int), 0, device.stream));
        static const b200rl_replay_layout layout = b200::replay_layout<SPEC>();
        static_assert(decltype(runner.buffers.observations)::SPEC::COLS == 3 && decltype(runner.buffers.actions)::SPEC::COLS == 1);
        if constexpr(b200::fused_actor(static_cast<const POLICY*>(nullptr))){
            const float* layers[6]; int acts[3];
            b200::actor_layers(policy, layers, acts);
            b200rl_mlp_shape shape{};
            shape.n_layers = 3; shape.input_dim = 3; shape.dims[0] = 64; shape.dims[1] = 64; shape.dims[2] = 1;
            for(int l = 0; l < 3; l++) shape.acts[l] = acts[l];
            b200::note(device, b200rl_pendulum_offpolicy_step(&shape, nullptr, layers, reinterpret_cast<float*>(runner.states._data), reinterpret_cast<int32_t*>(runner.episode_step._data),
                                                              reinterpret_cast<uint8_t*>(runner.truncated._data), runner.episode_return._data, reinterpret_cast<const float*>(sc), (int)N,
                                                              (int)SPEC::PARAMETERS::EPISODE_STEP_LIMIT, runner.buffers.observations._data, runner.buffers.actions._data,
                                                              runner.buffers.next_observations._data, runner.replay_buffers._data, &layout, reinterpret_cast<float*>(sc + RESET_BYTES),
                                                              reinterpret_cast<uint8_t*>(sc + RESET_BYTES + REWARD_BYTES), reinterpret_cast<int*>(sc + FLAG_OFFSET), device.stream));
        }
        else{
            // any other policy: the reference's three phases (operations_cuda.h:199-201) with the runner's buffers in device memory
            uint8_t* was_truncated = reinterpret_cast<uint8_t*>(sc + RESET_BYTES + REWARD_BYTES);
            b200::note(device, b200rl_pendulum_offpolicy_prologue(reinterpret_cast<float*>(runner.states._data), reinterpret_cast<int32_t*>(runner.episode_step._data),
                                                                  reinterpret_cast<const uint8_t*>(runner.truncated._data), runner.episode_return._data, reinterpret_cast<const float*>(sc), 0, 0,
                                                                  nullptr, (int)N, runner.buffers.observations._data, was_truncated, device.stream));
            rl::components::off_policy_runner::interlude<POLICY_INDEX>(device, runner, policy, policy_eval_buffers, rng);
            b200::note(device, b200rl_pendulum_offpolicy_epilogue(reinterpret_cast<float*>(runner.states._data), reinterpret_cast<int32_t*>(runner.episode_step._data),
                                                                  reinterpret_cast<uint8_t*>(runner.truncated._data), runner.episode_return._data, (int)N,
                                                                  (int)SPEC::PARAMETERS::EPISODE_STEP_LIMIT, runner.buffers.observations._data, runner.buffers.actions._data,
                                                                  runner.buffers.next_observations._data, runner.replay_buffers._data, &layout, was_truncated, device.stream));
        }
        b200::note(device, b200rl_memcpy(&flag, sc + FLAG_OFFSET, sizeof(int), 1, device.stream));
        if(flag != 0) b200::note(device, B200RL_ERR_DEVICE_FLAG);
        runner.previous_policy = POLICY_INDEX;
        runner.previous_policy_set = true;
    }
    // rl/components/off_policy_runner/operations_generic.h:413-423 (per batch element: environment index, then gather_batch_step :239-411), CUDA
    // form operations_cuda.h:166-182. Sequence length 1 with its default sampling parameters: the two indices of every element are drawn on the
    // host from the caller's engine with the reference's own uniform_int_distribution, in the reference's order (the ranges depend on each
    // buffer's position / full, read back from the device first); one kernel then fills the batch tensors.
    template <typename DEV_SPEC, typename SPEC, typename BATCH_SPEC, typename RNG, bool DETERMINISTIC = false>
    void gather_batch(devices::B200<DEV_SPEC>& device, rl::components::OffPolicyRunner<SPEC>& runner, rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>& batch, RNG& rng){
        using RUNNER = rl::components::OffPolicyRunner<SPEC>;
        using BATCH = rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>;
        using TI = typename SPEC::TI;
        using BP = typename BATCH_SPEC::PARAMETERS;
        static_assert(utils::typing::is_same_v<SPEC, typename BATCH_SPEC::SPEC>);
        static_assert(!SPEC::PARAMETERS::ASYMMETRIC_OBSERVATIONS && utils::typing::is_same_v<typename BATCH::T_INPUT, float> && sizeof(bool) == 1, "not implemented on this device");
        constexpr TI N = RUNNER::N_ENVIRONMENTS, B = BATCH::BATCH_SIZE, CAPACITY = SPEC::PARAMETERS::REPLAY_BUFFER_CAPACITY;
        static const b200rl_replay_layout layout = b200::replay_layout<SPEC>();
        if constexpr(BATCH_SPEC::SEQUENCE_LENGTHH != 1 || BP::RANDOM_SEQ_LENGTH || BP::ALWAYS_SAMPLE_FROM_INITIAL_STATE || DETERMINISTIC){
            // Sequences (or any non-default sampling parameter): how many draws an element takes depends on the flags stored in the replay
            // buffer, so they cannot be made ahead on the host engine; the kernel draws from its counter-based generator, seeded per call with
            // two words of the caller's engine (none with DETERMINISTIC, where nothing is drawn). The batch then follows the reference's
            // distribution, not its engine's sequence.
            static_assert(BP::ENABLE_NOMINAL_SEQUENCE_LENGTH_PROBABILITY || !BP::RANDOM_SEQ_LENGTH, "random lengths without the nominal-length probability are not implemented");
            constexpr int FLAGS = (BP::ALWAYS_SAMPLE_FROM_INITIAL_STATE ? B200RL_GATHER_FROM_INITIAL_STATE : 0) | (BP::RANDOM_SEQ_LENGTH ? B200RL_GATHER_RANDOM_LENGTH : 0) |
                                  (BP::INCLUDE_FIRST_STEP_IN_TARGETS ? B200RL_GATHER_FIRST_STEP_TARGET : 0) | (DETERMINISTIC ? B200RL_GATHER_DETERMINISTIC : 0);
            unsigned long long seed = 0;
            if constexpr(!DETERMINISTIC){
                const unsigned long long lo = random::uniform_int_distribution(device.random, (TI)0, (TI)0xFFFFFFFFu, rng), hi = random::uniform_int_distribution(device.random, (TI)0, (TI)0xFFFFFFFFu, rng);
                seed = lo | (hi << 32);
            }
            static void* flag_slot = nullptr;
            if(!flag_slot) b200::note(device, b200rl_device_malloc(&flag_slot, 16));
            if(!flag_slot) return;
            int flag = 0;
            b200::note(device, b200rl_memcpy(flag_slot, &flag, sizeof(int), 0, device.stream));
            b200::note(device, b200rl_gather_batch_sequences(runner.replay_buffers._data, &layout, (int)N, (int)SPEC::MAX_EPISODE_LENGTH, (int)BATCH::OBSERVATION_DIM, (int)BATCH::ACTION_DIM,
                                                             (int)BATCH_SPEC::SEQUENCE_LENGTHH, FLAGS, (float)BP::NOMINAL_SEQUENCE_LENGTH_PROBABILITY, seed, 0, nullptr, (int)B,
                                                             batch.observations_actions_base._data, (int)BATCH::DATA_DIM, batch.rewards._data,
                                                             reinterpret_cast<uint8_t*>(batch.terminated._data), reinterpret_cast<uint8_t*>(batch.reset._data),
                                                             reinterpret_cast<uint8_t*>(batch.next_reset_base._data), reinterpret_cast<uint8_t*>(batch.final_step_mask._data),
                                                             reinterpret_cast<uint8_t*>(batch.next_final_step_mask_base._data), static_cast<int*>(flag_slot), device.stream));
            b200::note(device, b200rl_memcpy(&flag, flag_slot, sizeof(int), 1, device.stream));
            if(flag != 0) b200::note(device, B200RL_ERR_DEVICE_FLAG);
            return;
        }
        // work area kept for the life of the process: position [N], env_index [B], sample_offset [B] (int32), full [N] bytes, error flag
        constexpr size_t OFF_ENV = sizeof(int32_t) * N, OFF_OFFSET = OFF_ENV + sizeof(int32_t) * B, OFF_FULL = OFF_OFFSET + sizeof(int32_t) * B, OFF_FLAG = OFF_FULL + ((N + 15) / 16) * 16;
        static void* scratch = nullptr;
        if(!scratch) b200::note(device, b200rl_device_malloc(&scratch, OFF_FLAG + 16));
        if(!scratch) return;
        char* sc = static_cast<char*>(scratch);
        b200::note(device, b200rl_replay_counters(runner.replay_buffers._data, &layout, (int)N, reinterpret_cast<int32_t*>(sc), reinterpret_cast<uint8_t*>(sc + OFF_FULL), device.stream));
        std::vector<int32_t> position(N), env_index(B), sample_offset(B);
        std::vector<uint8_t> full(N);
        b200::note(device, b200rl_memcpy(position.data(), sc, sizeof(int32_t) * N, 1, device.stream));
        b200::note(device, b200rl_memcpy(full.data(), sc + OFF_FULL, N, 1, device.stream));
        for(TI batch_step_i = 0; batch_step_i < B; batch_step_i++){
            const TI env_i = random::uniform_int_distribution(device.random, (TI)0, (TI)(N - 1), rng);
            const TI eligible = full[env_i] ? CAPACITY : (TI)position[env_i];
            if(eligible == 0){ b200::note(device, B200RL_ERR_INVALID_ARGUMENT); return; }       // the reference requires a non-empty replay buffer (:241)
            env_index[batch_step_i] = (int32_t)env_i;
            sample_offset[batch_step_i] = (int32_t)random::uniform_int_distribution(device.random, (TI)0, (TI)(eligible - 1), rng);
        }
        int flag = 0;
        b200::note(device, b200rl_memcpy(sc + OFF_ENV, env_index.data(), sizeof(int32_t) * B, 0, device.stream));
        b200::note(device, b200rl_memcpy(sc + OFF_OFFSET, sample_offset.data(), sizeof(int32_t) * B, 0, device.stream));
        b200::note(device, b200rl_memcpy(sc + OFF_FLAG, &flag, sizeof(int), 0, device.stream));
        b200::note(device, b200rl_gather_batch(runner.replay_buffers._data, &layout, (int)N, (int)SPEC::MAX_EPISODE_LENGTH, (int)BATCH::OBSERVATION_DIM, (int)BATCH::ACTION_DIM,
                                               reinterpret_cast<const int32_t*>(sc + OFF_ENV), reinterpret_cast<const int32_t*>(sc + OFF_OFFSET), (int)B,
                                               batch.observations_actions_base._data, (int)BATCH::DATA_DIM, batch.rewards._data,
                                               reinterpret_cast<uint8_t*>(batch.terminated._data), reinterpret_cast<uint8_t*>(batch.reset._data),
                                               reinterpret_cast<uint8_t*>(batch.next_reset_base._data), reinterpret_cast<uint8_t*>(batch.final_step_mask._data),
                                               reinterpret_cast<uint8_t*>(batch.next_final_step_mask_base._data), reinterpret_cast<int*>(sc + OFF_FLAG), device.stream));
        b200::note(device, b200rl_memcpy(&flag, sc + OFF_FLAG, sizeof(int), 1, device.stream));
        if(flag != 0) b200::note(device, B200RL_ERR_DEVICE_FLAG);
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
