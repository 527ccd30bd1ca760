// Header-only adapter, part 3: the on-policy runner on `devices::B200`.
//
// Include after <b200rl/rl_tools_operations.h>, <rl_tools/rl/environments/pendulum/operations_generic.h>,
// <rl_tools/nn_models/mlp_unconditional_stddev/operations_generic.h>, <rl_tools/nn_models/sequential/operations_generic.h> and
// <rl_tools/rl/components/on_policy_runner/operations_generic.h>.
//
// The reference has no device-resident on-policy runner (its hybrid collect keeps the environments on the host,
// rl/components/on_policy_runner/operations_generic_extensions.h:37-77). Here the runner's per-environment state (states,
// episode_step, truncated, episode_return) and the dataset matrix live in device memory and one kernel launch does all steps of a
// collect call. Randomness stays on the host engine passed by the caller: its draws are made with the reference's own
// distribution functions in the reference's order (per step: initial states of the truncated environments, then one normal draw per
// action) and handed to the kernel as tables, so the engine ends a call in the same state as after the reference's collect.
//
// Supported: rl::environments::Pendulum, actor = sequential< mlp_unconditional_stddev 3 -> 64 -> 64 -> 1 >, fp32.
#pragma once
#include "rl_tools_operations.h"
#include <vector>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    namespace b200{
        template <typename ENVIRONMENT> struct is_pendulum{ static constexpr bool value = false; };
        template <typename SPEC> struct is_pendulum<rl::environments::Pendulum<SPEC>>{ static constexpr bool value = true; };
        // containers of non-float element types (counters, flags): filled through a host staging vector
        template <typename DEVICE, typename SPEC, typename VALUE_T>
        void fill_any(DEVICE& device, Matrix<SPEC>& m, VALUE_T value){
            static_assert(SPEC::COL_PITCH == 1);
            using ELEMENT = typename SPEC::T;
            constexpr size_t COUNT = (size_t)SPEC::ROWS * SPEC::COLS;
            std::vector<unsigned char> host(COUNT * sizeof(ELEMENT));          // raw bytes: std::vector<bool> has no data()
            ELEMENT* typed = reinterpret_cast<ELEMENT*>(host.data());
            for(size_t i = 0; i < COUNT; i++) typed[i] = (ELEMENT)value;
            if(rl_tools::b200::ld(m) == SPEC::COLS) note(device, b200rl_memcpy(m._data, typed, COUNT * sizeof(ELEMENT), 0, device.stream));
            else note(device, b200rl_memcpy_2d(m._data, rl_tools::b200::ld(m) * sizeof(ELEMENT), typed, SPEC::COLS * sizeof(ELEMENT),
                                               SPEC::COLS * sizeof(ELEMENT), SPEC::ROWS, 0, device.stream));
        }
    }
    // rl/components/on_policy_runner/operations_generic.h:69-82. Pendulum's environment and parameter structs carry no data
    // (rl/environments/pendulum/pendulum.h), so nothing per environment is copied.
    template <typename DEV_SPEC, typename SPEC, typename ENV_SPEC, typename PARAM_SPEC, typename ACTOR, typename RNG>
    void init(devices::B200<DEV_SPEC>& device, rl::components::OnPolicyRunner<SPEC>& runner, Tensor<ENV_SPEC>, Tensor<PARAM_SPEC>, ACTOR&, RNG&){
        static_assert(b200::is_pendulum<typename SPEC::ENVIRONMENT>::value, "only rl::environments::Pendulum is implemented on this device");
        b200::fill_any(device, runner.episode_step, 0);
        b200::fill_any(device, runner.episode_return, 0);
        b200::fill_any(device, runner.truncated, true);
        runner.step = 0;
#ifdef RL_TOOLS_DEBUG_RL_COMPONENTS_ON_POLICY_RUNNER_CHECK_INIT
        runner.initialized = true;
#endif
    }
    // rl/components/on_policy_runner/operations_generic.h:105-146
    template <typename DEV_SPEC, typename DATASET_SPEC, typename ACTOR, typename ACTOR_BUFFER, typename RNG>
    void collect(devices::B200<DEV_SPEC>& device, rl::components::on_policy_runner::Dataset<DATASET_SPEC>& dataset,
                 rl::components::OnPolicyRunner<typename DATASET_SPEC::SPEC>& runner, ACTOR& actor, ACTOR_BUFFER&, RNG& rng){
        using SPEC = typename DATASET_SPEC::SPEC;
        using ENVIRONMENT = typename SPEC::ENVIRONMENT;
        using T = typename SPEC::TYPE_POLICY::DEFAULT;
        using TI = typename SPEC::TI;
        constexpr TI N = SPEC::N_ENVIRONMENTS, STEPS = DATASET_SPEC::STEPS_PER_ENV, STEP_LIMIT = SPEC::STEP_LIMIT;
        using DATASET = rl::components::on_policy_runner::Dataset<DATASET_SPEC>;
        static_assert(b200::is_pendulum<ENVIRONMENT>::value, "only rl::environments::Pendulum is implemented on this device");
        static_assert(utils::typing::is_same_v<T, float> && sizeof(TI) == 4 && sizeof(bool) == 1, "fp32 data, 32-bit counters");
        static_assert(!SPEC::ASYMMETRIC_OBSERVATIONS && ENVIRONMENT::Observation::DIM == 3 && ENVIRONMENT::ACTION_DIM == 1 && DATASET::DATA_DIM == B200RL_COLLECT_DATA_DIM);
        static_assert(sizeof(typename ENVIRONMENT::State) == 2 * sizeof(float), "state = (theta, theta_dot)");
        static_assert(utils::typing::is_same_v<typename ACTOR::NEXT_MODULE, nn_models::sequential::OutputModule>, "the actor must be the bare MLP module");
        auto& mlp = get_last_layer(actor);
        using MLP_SPEC = typename utils::typing::remove_reference_t<decltype(mlp)>::SPEC;
        static_assert(MLP_SPEC::INPUT_DIM == 3 && MLP_SPEC::CONFIG::HIDDEN_DIM == 64 && MLP_SPEC::CONFIG::NUM_LAYERS == 3 && MLP_SPEC::CONFIG::OUTPUT_DIM == 1, "actor 3 -> 64 -> 64 -> 1");

        // 1. the integer part of the runner state decides which draws happen: bring it to the host
        std::vector<TI> episode_step(N);
        std::vector<uint8_t> truncated(N);
        if constexpr(SPEC::TRUNCATE_ON_EACH_ITERATION) b200::fill_any(device, runner.truncated, true);
        b200::note(device, b200rl_memcpy(episode_step.data(), runner.episode_step._data, N * sizeof(TI), 1, device.stream));
        b200::note(device, b200rl_memcpy(truncated.data(), runner.truncated._data, N, 1, device.stream));
        // 2. draws in the reference's order with the reference's own functions on the caller's engine
        constexpr TI ROUNDS = STEP_LIMIT > 0 ? (STEPS + STEP_LIMIT - 1) / STEP_LIMIT + 1 : 1;
        std::vector<float> reset_states((size_t)ROUNDS * N * 2, 0.0f), noise((size_t)STEPS * N);
        std::vector<TI> rounds(N, 0);
        ENVIRONMENT env; typename ENVIRONMENT::Parameters parameters; typename ENVIRONMENT::State state;
        for(TI step_i = 0; step_i < STEPS; step_i++){
            for(TI env_i = 0; env_i < N; env_i++){
                if(truncated[env_i]){
                    sample_initial_parameters(device, env, parameters, rng);
                    sample_initial_state(device, env, parameters, state, rng);
                    float* dst = reset_states.data() + ((size_t)rounds[env_i] * N + env_i) * 2;
                    dst[0] = state.theta; dst[1] = state.theta_dot;
                    rounds[env_i]++; episode_step[env_i] = 0;
                }
            }
            for(TI env_i = 0; env_i < N; env_i++){
                noise[(size_t)step_i * N + env_i] = random::normal_distribution::sample(device.random, (T)0, (T)1, rng);
                episode_step[env_i] += 1;
                truncated[env_i] = STEP_LIMIT > 0 && episode_step[env_i] >= STEP_LIMIT;
            }
        }
        // 3. tables to the device, one launch for the whole call
        void *d_reset = nullptr, *d_noise = nullptr, *d_flag = nullptr;
        b200::note(device, b200rl_device_malloc(&d_reset, reset_states.size() * sizeof(float)));
        b200::note(device, b200rl_device_malloc(&d_noise, noise.size() * sizeof(float)));
        b200::note(device, b200rl_device_malloc(&d_flag, sizeof(int)));
        int flag = 0;
        if(d_reset && d_noise && d_flag){
            b200::note(device, b200rl_memcpy(d_reset, reset_states.data(), reset_states.size() * sizeof(float), 0, device.stream));
            b200::note(device, b200rl_memcpy(d_noise, noise.data(), noise.size() * sizeof(float), 0, device.stream));
            b200::note(device, b200rl_memcpy(d_flag, &flag, sizeof(int), 0, device.stream));
            b200rl_mlp_shape shape{};
            shape.n_layers = 3; shape.input_dim = 3; shape.dims[0] = 64; shape.dims[1] = 64; shape.dims[2] = 1;
            shape.acts[0] = shape.acts[1] = b200::activation_id<MLP_SPEC::CONFIG::HIDDEN_ACTIVATION_FUNCTION>();
            shape.acts[2] = b200::activation_id<MLP_SPEC::CONFIG::OUTPUT_ACTIVATION_FUNCTION>();
            const float* layers[6] = {mlp.input_layer.weights.parameters._data, mlp.input_layer.biases.parameters._data,
                                      mlp.hidden_layers[0].weights.parameters._data, mlp.hidden_layers[0].biases.parameters._data,
                                      mlp.output_layer.weights.parameters._data, mlp.output_layer.biases.parameters._data};
            b200::note(device, b200rl_pendulum_collect_layers(&shape, layers, mlp.log_std.parameters._data, reinterpret_cast<float*>(runner.states._data),
                                                              reinterpret_cast<int32_t*>(runner.episode_step._data), reinterpret_cast<uint8_t*>(runner.truncated._data),
                                                              runner.episode_return._data, static_cast<const float*>(d_reset), ROUNDS, static_cast<const float*>(d_noise),
                                                              N, STEPS, STEP_LIMIT, dataset.data._data, rl_tools::b200::ld(dataset.data), static_cast<int*>(d_flag), device.stream));
            b200::note(device, b200rl_memcpy(&flag, d_flag, sizeof(int), 1, device.stream));
            if(flag != 0) b200::note(device, B200RL_ERR_DEVICE_FLAG);
        }
        b200::note(device, b200rl_device_free(d_reset)); b200::note(device, b200rl_device_free(d_noise)); b200::note(device, b200rl_device_free(d_flag));
        runner.step += N * STEPS;
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
