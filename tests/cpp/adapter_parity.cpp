// Parity test of the header-only adapter: the reference's OWN generic code (nn_models::mlp forward / backward, the
// Adam step, mse::gradient) instantiated once on the reference CPU device and once on devices::B200, on the same
// CPU-initialised weights and inputs -- the pattern and thresholds of the reference's CPU<->CUDA tests
// (tests/src/nn/cuda/cuda_basics.cu:828-972: abs_diff / (BATCH * OUTPUT) < 1e-6 for float).
// Built with the host compiler only: g++ -std=c++17 -I<reference>/include -I<repo>/include -I<repo>/rl-tools_b200/include
//                                    adapter_parity.cpp -L<repo>/rl-tools_b200 -lb200rl
#include <rl_tools/operations/cpu.h>
#include <b200rl/rl_tools_device.h>
#include <rl_tools/nn/optimizers/adam/instance/operations_generic.h>
#include <rl_tools/nn/operations_generic.h>
#include <rl_tools/nn/layers/dense/operations_cpu.h>
#include <rl_tools/nn/loss_functions/mse/operations_generic.h>
#include <rl_tools/nn/layers/sample_and_squash/operations_generic.h>     // before the model headers that recurse into it
#include <rl_tools/nn/layers/standardize/operations_generic.h>
#include <rl_tools/rl/components/running_normalizer/operations_generic.h>
#include <b200rl/rl_tools_standardize.h>                          // before the model headers that recurse into the layer
#include <b200rl/rl_tools_mlp.h>                                  // whole-model overloads: before the generic MLP operations
#include <rl_tools/nn_models/mlp/operations_generic.h>
#include <rl_tools/nn_models/mlp_unconditional_stddev/operations_generic.h>
#include <rl_tools/nn_models/sequential/operations_generic.h>
#include <rl_tools/nn/optimizers/adam/operations_generic.h>      // after every model type it steps (same rule as for the reference's own devices)
#include <rl_tools/rl/environments/pendulum/operations_generic.h>
#include <rl_tools/rl/components/on_policy_runner/operations_generic.h>
#include <rl_tools/rl/components/off_policy_runner/operations_generic.h>
#include <b200rl/rl_tools_sac.h>                                  // before the SAC operations: min_value_d_output and the MSE gradient are looked up at their definition
#include <rl_tools/rl/algorithms/sac/operations_generic.h>
#include <rl_tools/rl/algorithms/ppo/ppo.h>
#include <rl_tools/rl/algorithms/ppo/operations_generic.h>
#include <b200rl/rl_tools_operations.h>
#include <b200rl/rl_tools_on_policy_runner.h>
#include <b200rl/rl_tools_ppo.h>
#include <b200rl/rl_tools_off_policy_runner.h>

#include <cstdio>
#include <cmath>
#include <vector>
#include <memory>

namespace rlt = rl_tools;
using DEVICE_CPU = rlt::devices::DefaultCPU;
using DEVICE_GPU = rlt::devices::DefaultB200;
using T = float;
using TI = typename DEVICE_GPU::index_t;
using TYPE_POLICY = rlt::numeric_types::Policy<T>;
namespace act = rlt::nn::activation_functions;

static int failures = 0;

template <TI BATCH, TI INPUT_DIM, TI HIDDEN_DIM, TI OUTPUT_DIM, TI NUM_LAYERS, act::ActivationFunction HIDDEN_ACT, act::ActivationFunction OUTPUT_ACT, int STEPS>
void train_steps(const char* name){
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, OUTPUT_DIM, NUM_LAYERS, HIDDEN_DIM, HIDDEN_ACT, OUTPUT_ACT>;
    using INPUT_SHAPE = rlt::tensor::Shape<TI, 1, BATCH, INPUT_DIM>;
    using CAPABILITY = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, CAPABILITY, INPUT_SHAPE>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    NET net_cpu, net_gpu, net_back;
    typename NET::template Buffer<> buf_cpu, buf_gpu;
    OPTIMIZER opt_cpu, opt_gpu;
    rlt::malloc(cpu, net_cpu); rlt::malloc(cpu, net_back); rlt::malloc(cpu, buf_cpu); rlt::malloc(cpu, opt_cpu);
    rlt::malloc(gpu, net_gpu); rlt::malloc(gpu, buf_gpu); rlt::malloc(gpu, opt_gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng;
    rlt::malloc(cpu, rng); rlt::init(cpu, rng, 7);
    rlt::init(cpu, opt_cpu); rlt::init(gpu, opt_gpu);
    rlt::init_weights(cpu, net_cpu, rng);
    rlt::zero_gradient(cpu, net_cpu);
    rlt::reset_optimizer_state(cpu, opt_cpu, net_cpu);
    rlt::copy(cpu, gpu, net_cpu, net_gpu);
    rlt::reset_optimizer_state(gpu, opt_gpu, net_gpu);

    rlt::Matrix<rlt::matrix::Specification<T, TI, BATCH, INPUT_DIM>> x_cpu, x_gpu;
    rlt::Matrix<rlt::matrix::Specification<T, TI, BATCH, OUTPUT_DIM>> y_cpu, y_gpu, d_cpu, d_gpu, out_gpu_on_cpu;
    rlt::malloc(cpu, x_cpu); rlt::malloc(cpu, y_cpu); rlt::malloc(cpu, d_cpu); rlt::malloc(cpu, out_gpu_on_cpu);
    rlt::malloc(gpu, x_gpu); rlt::malloc(gpu, y_gpu); rlt::malloc(gpu, d_gpu);
    rlt::randn(cpu, x_cpu, rng); rlt::randn(cpu, y_cpu, rng);
    rlt::copy(cpu, gpu, x_cpu, x_gpu); rlt::copy(cpu, gpu, y_cpu, y_gpu);

    for(int s = 0; s < STEPS; s++){
        rlt::zero_gradient(cpu, net_cpu);
        rlt::forward(cpu, net_cpu, x_cpu, buf_cpu, rng);
        { auto out = rlt::output(cpu, net_cpu); auto out_m = rlt::matrix_view(cpu, out); rlt::nn::loss_functions::mse::gradient(cpu, out_m, y_cpu, d_cpu, (T)1); }
        rlt::backward(cpu, net_cpu, x_cpu, d_cpu, buf_cpu);
        rlt::step(cpu, opt_cpu, net_cpu);

        rlt::zero_gradient(gpu, net_gpu);
        rlt::forward(gpu, net_gpu, x_gpu, buf_gpu, rng);
        { auto out = rlt::output(gpu, net_gpu); auto out_m = rlt::matrix_view(gpu, out); rlt::nn::loss_functions::mse::gradient(gpu, out_m, y_gpu, d_gpu, (T)1); }
        rlt::backward(gpu, net_gpu, x_gpu, d_gpu, buf_gpu);
        rlt::step(gpu, opt_gpu, net_gpu);
    }
    int status = rlt::check_status(gpu);
    rlt::copy(gpu, cpu, net_gpu, net_back);
    // forward outputs of the last step
    { auto out = rlt::output(gpu, net_gpu); auto out_m = rlt::matrix_view(gpu, out); rlt::copy(gpu, cpu, out_m, out_gpu_on_cpu); }
    auto out_cpu = rlt::output(cpu, net_cpu); auto out_cpu_m = rlt::matrix_view(cpu, out_cpu);
    T out_diff = rlt::abs_diff(cpu, out_cpu_m, out_gpu_on_cpu) / (BATCH * OUTPUT_DIM);
    // abs_diff(network) sums over parameters, gradients, both Adam moments and the stored pre-activations / outputs of every
    // layer; the reference divides by BATCH * OUTPUT (cuda_basics.cu:945), which only normalises well for its 100..256-wide
    // outputs, so the mean over the compared elements is used here (and a tighter bound)
    constexpr double HIDDEN_SUM = (double)HIDDEN_DIM * (NUM_LAYERS - 1) + OUTPUT_DIM;
    constexpr double N_PARAMS = (double)INPUT_DIM * HIDDEN_DIM + HIDDEN_DIM + (NUM_LAYERS - 2) * ((double)HIDDEN_DIM * HIDDEN_DIM + HIDDEN_DIM) + (double)HIDDEN_DIM * OUTPUT_DIM + OUTPUT_DIM;
    T net_diff = (T)(rlt::abs_diff(cpu, net_back, net_cpu) / (4 * N_PARAMS + 2 * BATCH * HIDDEN_SUM));
    bool ok = status == 0 && out_diff < 1e-6 && net_diff < 1e-7 && !std::isnan(out_diff) && !std::isnan(net_diff);
    std::printf("%-28s batch %4u  %u->%u x%u->%u  steps %d  status %d  output diff %.3e  network mean diff %.3e  %s\n",
                name, BATCH, INPUT_DIM, HIDDEN_DIM, NUM_LAYERS - 1, OUTPUT_DIM, STEPS, status, out_diff, net_diff, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, net_cpu); rlt::free(cpu, net_back); rlt::free(cpu, buf_cpu); rlt::free(cpu, opt_cpu);
    rlt::free(gpu, net_gpu); rlt::free(gpu, buf_gpu); rlt::free(gpu, opt_gpu);
    rlt::free(cpu, x_cpu); rlt::free(cpu, y_cpu); rlt::free(cpu, d_cpu); rlt::free(cpu, out_gpu_on_cpu);
    rlt::free(gpu, x_gpu); rlt::free(gpu, y_gpu); rlt::free(gpu, d_gpu);
}

// On-policy collect: the reference's OnPolicyRunner on the CPU device against the same runner type on devices::B200, same engine
// seed, consecutive collect calls. Flags, counters and the engine's final state must be identical; float columns agree to the first
// steps' rounding and stay within a small drift over the horizon (the trajectories are free-running).
template <TI N, TI STEPS, TI STEP_LIMIT, act::ActivationFunction HACT, int COLLECTS>
void collect_parity(const char* name){
    using PENDULUM = rlt::rl::environments::Pendulum<rlt::rl::environments::pendulum::Specification<T, TI, rlt::rl::environments::pendulum::DefaultParameters<T>>>;
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, HACT, act::IDENTITY>;
    using ACTOR_MLP = rlt::nn_models::mlp_unconditional_stddev::BindConfiguration<ACTOR_CONFIG>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<ACTOR_MLP>, rlt::tensor::Shape<TI, 1, N, 3>>;
    using RUNNER_SPEC = rlt::rl::components::on_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, typename ACTOR::template State<>, N, STEP_LIMIT>;
    using RUNNER = rlt::rl::components::OnPolicyRunner<RUNNER_SPEC>;
    using DATASET = rlt::rl::components::on_policy_runner::Dataset<rlt::rl::components::on_policy_runner::DatasetSpecification<RUNNER_SPEC, STEPS>>;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng_cpu, rng_gpu;
    rlt::malloc(cpu, rng_cpu); rlt::malloc(cpu, rng_gpu);
    rlt::init(cpu, rng_cpu, 3); rlt::init(cpu, rng_gpu, 3);
    ACTOR actor_cpu, actor_gpu; typename ACTOR::template Buffer<> buf_cpu, buf_gpu;
    RUNNER runner_cpu, runner_gpu; DATASET ds_cpu, ds_gpu, ds_back;
    rlt::malloc(cpu, actor_cpu); rlt::malloc(cpu, buf_cpu); rlt::malloc(cpu, runner_cpu); rlt::malloc(cpu, ds_cpu); rlt::malloc(cpu, ds_back);
    rlt::malloc(gpu, actor_gpu); rlt::malloc(gpu, buf_gpu); rlt::malloc(gpu, runner_gpu); rlt::malloc(gpu, ds_gpu);
    rlt::init_weights(cpu, actor_cpu, rng_cpu); rlt::init_weights(cpu, actor_cpu, rng_gpu);          // both engines advance alike
    rlt::set(cpu, actor_cpu.content.log_std.parameters, (T)-0.7, 0);
    rlt::copy(cpu, gpu, actor_cpu, actor_gpu);
    rlt::Tensor<rlt::tensor::Specification<PENDULUM, TI, rlt::tensor::Shape<TI, N>>> envs;
    rlt::Tensor<rlt::tensor::Specification<typename PENDULUM::Parameters, TI, rlt::tensor::Shape<TI, N>>> env_parameters;
    rlt::malloc(cpu, envs); rlt::malloc(cpu, env_parameters);
    rlt::set_all(cpu, ds_cpu.data, 0); rlt::set_all(gpu, ds_gpu.data, 0);
    rlt::init(cpu, runner_cpu, envs, env_parameters, actor_cpu, rng_cpu);
    rlt::init(gpu, runner_gpu, envs, env_parameters, actor_gpu, rng_gpu);
    double worst_flag = 0, worst_first = 0, worst_drift = 0;
    for(int c = 0; c < COLLECTS; c++){
        rlt::collect(cpu, ds_cpu, runner_cpu, actor_cpu, buf_cpu, rng_cpu);
        rlt::collect(gpu, ds_gpu, runner_gpu, actor_gpu, buf_gpu, rng_gpu);
        rlt::copy(gpu, cpu, ds_gpu.data, ds_back.data);
        for(TI r = 0; r < (STEPS + 1) * N; r++){
            for(TI k = 0; k < 10; k++){
                if(r >= STEPS * N && k >= 3 && k != 9) continue;          // final-observation rows carry only the observation and reset
                double d = std::fabs((double)rlt::get(ds_cpu.data, r, k) - (double)rlt::get(ds_back.data, r, k));
                if(k >= 7) worst_flag = std::fmax(worst_flag, d);
                else{
                    worst_drift = std::fmax(worst_drift, d);
                    if(c == 0 && r < N) worst_first = std::fmax(worst_first, d);
                }
            }
        }
    }
    int status = rlt::check_status(gpu);
    std::vector<TI> es(N); std::vector<uint8_t> tr(N);
    b200rl_memcpy(es.data(), runner_gpu.episode_step._data, N * sizeof(TI), 1, gpu.stream);
    b200rl_memcpy(tr.data(), runner_gpu.truncated._data, N, 1, gpu.stream);
    bool counters = runner_cpu.step == runner_gpu.step;
    for(TI e = 0; e < N; e++) counters = counters && es[e] == rlt::get(runner_cpu.episode_step, 0, e) && (tr[e] != 0) == rlt::get(runner_cpu.truncated, 0, e);
    bool engines = rlt::random::uniform_real_distribution(cpu.random, (T)0, (T)1, rng_cpu) == rlt::random::uniform_real_distribution(cpu.random, (T)0, (T)1, rng_gpu);
    bool ok = status == 0 && counters && engines && worst_flag == 0 && worst_first < 2e-5 && worst_drift < 5e-3;
    std::printf("%-28s envs %4u steps %3u limit %3u collects %d  status %d  counters %d  engine %d  flags diff %.1e  first step diff %.2e  drift %.2e  %s\n",
                name, N, STEPS, STEP_LIMIT, COLLECTS, status, (int)counters, (int)engines, worst_flag, worst_first, worst_drift, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, actor_cpu); rlt::free(cpu, buf_cpu); rlt::free(cpu, runner_cpu); rlt::free(cpu, ds_cpu); rlt::free(cpu, ds_back);
    rlt::free(gpu, actor_gpu); rlt::free(gpu, buf_gpu); rlt::free(gpu, runner_gpu); rlt::free(gpu, ds_gpu);
    rlt::free(cpu, envs); rlt::free(cpu, env_parameters);
}

// PPO update: the reference's train() + estimate_generalized_advantages on the CPU device against the overloads on devices::B200, on the same
// randomly filled dataset matrix, same initial networks, same engine seed (epoch shuffle on). The shuffled dataset must be identical (data
// movement only), advantages / target values bit-identical (same arithmetic per element), network parameters within the drift of
// EPOCHS x BATCHES Adam steps.
template <TI BATCH, TI EPOCHS>
struct PpoParityParameters: rlt::rl::algorithms::ppo::DefaultParameters<TYPE_POLICY, TI, BATCH>{
    static constexpr TI N_EPOCHS = EPOCHS;
};
template <TI N, TI STEPS, TI BATCH, TI EPOCHS>
void ppo_parity(const char* name){
    using PENDULUM = rlt::rl::environments::Pendulum<rlt::rl::environments::pendulum::Specification<T, TI, rlt::rl::environments::pendulum::DefaultParameters<T>>>;
    using CAPABILITY = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using INPUT_SHAPE = rlt::tensor::Shape<TI, 1, BATCH, 3>;
    using MLP_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::IDENTITY>;
    using ACTOR = rlt::nn_models::sequential::Build<CAPABILITY, rlt::nn_models::sequential::Module<rlt::nn_models::mlp_unconditional_stddev::BindConfiguration<MLP_CONFIG>>, INPUT_SHAPE>;
    using CRITIC = rlt::nn_models::sequential::Build<CAPABILITY, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<MLP_CONFIG>>, INPUT_SHAPE>;
    using PARAMETERS = PpoParityParameters<BATCH, EPOCHS>;
    using PPO_SPEC = rlt::rl::algorithms::ppo::Specification<TYPE_POLICY, TI, PENDULUM, ACTOR, CRITIC, PARAMETERS>;
    using PPO = rlt::rl::algorithms::PPO<PPO_SPEC>;
    using PPO_BUFFERS = rlt::rl::algorithms::ppo::Buffers<rlt::rl::algorithms::ppo::BufferSpecification<PPO_SPEC>>;
    using RUNNER_SPEC = rlt::rl::components::on_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, typename ACTOR::template State<>, N, 100>;
    using DATASET = rlt::rl::components::on_policy_runner::Dataset<rlt::rl::components::on_policy_runner::DatasetSpecification<RUNNER_SPEC, STEPS>>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng_init, rng_cpu, rng_gpu;
    rlt::malloc(cpu, rng_init); rlt::malloc(cpu, rng_cpu); rlt::malloc(cpu, rng_gpu);
    rlt::init(cpu, rng_init, 11); rlt::init(cpu, rng_cpu, 5); rlt::init(cpu, rng_gpu, 5);
    PPO ppo_cpu, ppo_gpu, ppo_back; PPO_BUFFERS pb_cpu, pb_gpu; DATASET ds_cpu, ds_gpu, ds_back;
    OPTIMIZER ao_cpu, co_cpu, ao_gpu, co_gpu;
    typename ACTOR::template Buffer<> ab_cpu, ab_gpu; typename CRITIC::template Buffer<> cb_cpu, cb_gpu;
    rlt::malloc(cpu, ppo_cpu); rlt::malloc(cpu, ppo_back); rlt::malloc(cpu, pb_cpu); rlt::malloc(cpu, ds_cpu); rlt::malloc(cpu, ds_back);
    rlt::malloc(cpu, ao_cpu); rlt::malloc(cpu, co_cpu); rlt::malloc(cpu, ab_cpu); rlt::malloc(cpu, cb_cpu);
    rlt::malloc(gpu, ppo_gpu); rlt::malloc(gpu, pb_gpu); rlt::malloc(gpu, ds_gpu);
    rlt::malloc(gpu, ao_gpu); rlt::malloc(gpu, co_gpu); rlt::malloc(gpu, ab_gpu); rlt::malloc(gpu, cb_gpu);
    rlt::init(cpu, ppo_cpu, ao_cpu, co_cpu, rng_init);
    rlt::init(gpu, ao_gpu); rlt::init(gpu, co_gpu);
    rlt::copy(cpu, gpu, ppo_cpu.actor, ppo_gpu.actor); rlt::copy(cpu, gpu, ppo_cpu.critic, ppo_gpu.critic);
    rlt::reset_optimizer_state(gpu, ao_gpu, ppo_gpu.actor); rlt::reset_optimizer_state(gpu, co_gpu, ppo_gpu.critic);
    // a synthetic dataset matrix: train() and the advantage estimate consume any values; flags are 0 / 1
    rlt::randn(cpu, ds_cpu.data, rng_init);
    for(TI r = 0; r < (STEPS + 1) * N; r++){
        rlt::set(ds_cpu.data, r, 5, rlt::get(ds_cpu.data, r, 5) * (T)0.3 - (T)1.2);                 // rollout log-probabilities
        rlt::set(ds_cpu.data, r, 7, (T)0); rlt::set(ds_cpu.data, r, 8, (T)((r / N) % 20 == 19)); rlt::set(ds_cpu.data, r, 9, (T)0);
    }
    rlt::copy(cpu, gpu, ds_cpu.data, ds_gpu.data);
    rlt::estimate_generalized_advantages(cpu, ds_cpu, PARAMETERS{});
    rlt::estimate_generalized_advantages(gpu, ds_gpu, PARAMETERS{});
    rlt::copy(gpu, cpu, ds_gpu.data, ds_back.data);
    T gae_diff = rlt::abs_diff(cpu, ds_cpu.data, ds_back.data);
    rlt::train(cpu, ppo_cpu, ds_cpu, ao_cpu, co_cpu, pb_cpu, ab_cpu, cb_cpu, rng_cpu);
    rlt::train(gpu, ppo_gpu, ds_gpu, ao_gpu, co_gpu, pb_gpu, ab_gpu, cb_gpu, rng_gpu);
    int status = rlt::check_status(gpu);
    rlt::copy(gpu, cpu, ds_gpu.data, ds_back.data);
    T shuffle_diff = rlt::abs_diff(cpu, ds_cpu.data, ds_back.data);
    rlt::copy(gpu, cpu, ppo_gpu.actor, ppo_back.actor); rlt::copy(gpu, cpu, ppo_gpu.critic, ppo_back.critic);
    // mean absolute parameter difference (weights + biases of the three layers + log_std); Adam moves a parameter by ~1e-3 per step
    double actor_diff = 0, critic_diff = 0, count = 0;
    auto layer_diff = [&](auto& a, auto& b){
        double d = rlt::abs_diff(cpu, a.weights.parameters, b.weights.parameters) + rlt::abs_diff(cpu, a.biases.parameters, b.biases.parameters);
        return d;
    };
    { auto& a = ppo_cpu.actor.content; auto& b = ppo_back.actor.content;
      actor_diff = layer_diff(a.input_layer, b.input_layer) + layer_diff(a.hidden_layers[0], b.hidden_layers[0]) + layer_diff(a.output_layer, b.output_layer)
                   + std::fabs((double)rlt::get(cpu, a.log_std.parameters, 0) - (double)rlt::get(cpu, b.log_std.parameters, 0)); }
    { auto& a = ppo_cpu.critic.content; auto& b = ppo_back.critic.content;
      critic_diff = layer_diff(a.input_layer, b.input_layer) + layer_diff(a.hidden_layers[0], b.hidden_layers[0]) + layer_diff(a.output_layer, b.output_layer); }
    count = 3 * 64 + 64 + 64 * 64 + 64 + 64 + 1;
    actor_diff /= count + 1; critic_diff /= count;
    bool engines = rlt::random::uniform_real_distribution(cpu.random, (T)0, (T)1, rng_cpu) == rlt::random::uniform_real_distribution(cpu.random, (T)0, (T)1, rng_gpu);
    bool ok = status == 0 && gae_diff == 0 && shuffle_diff == 0 && engines && actor_diff < 2e-6 && critic_diff < 2e-6;
    std::printf("%-28s envs %3u steps %3u batch %4u epochs %u  status %d  gae diff %.1e  shuffled dataset diff %.1e  engine %d  mean actor diff %.2e  mean critic diff %.2e  %s\n",
                name, N, STEPS, BATCH, EPOCHS, status, gae_diff, shuffle_diff, (int)engines, actor_diff, critic_diff, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, ppo_cpu); rlt::free(cpu, ppo_back); rlt::free(cpu, pb_cpu); rlt::free(cpu, ds_cpu); rlt::free(cpu, ds_back);
    rlt::free(cpu, ao_cpu); rlt::free(cpu, co_cpu); rlt::free(cpu, ab_cpu); rlt::free(cpu, cb_cpu);
    rlt::free(gpu, ppo_gpu); rlt::free(gpu, pb_gpu); rlt::free(gpu, ds_gpu);
    rlt::free(gpu, ao_gpu); rlt::free(gpu, co_gpu); rlt::free(gpu, ab_gpu); rlt::free(gpu, cb_gpu);
}

// Off-policy runner: the reference's OffPolicyRunner (per-environment replay buffers) on the CPU device against the same runner type on
// devices::B200, same actor, same engine seed, STEPS x step<0>(). Counters, flags, episode_start and the engine's final state must be
// identical; replay rows agree within the drift of the free-running trajectories.
template <TI T_N, TI T_CAPACITY, TI T_LIMIT>
struct OffPolicyParityParameters: rlt::rl::components::off_policy_runner::ParametersDefault<TYPE_POLICY, TI>{
    static constexpr TI N_ENVIRONMENTS = T_N;
    static constexpr TI REPLAY_BUFFER_CAPACITY = T_CAPACITY;
    static constexpr TI EPISODE_STEP_LIMIT = T_LIMIT;
};
// sampling parameters of the sequence check: fixed lengths, starts anywhere (what the DETERMINISTIC flag then leaves is a walk without draws)
struct AdapterSequenceParameters: rlt::rl::components::off_policy_runner::SequentialBatchParameters<TYPE_POLICY, TI, 4>{
    static constexpr bool ALWAYS_SAMPLE_FROM_INITIAL_STATE = false;
    static constexpr bool RANDOM_SEQ_LENGTH = false;
};
// HIDDEN = 64 takes the fused runner kernel; any other width takes the reference's three phases (prologue kernel, the reference's own
// interlude with the policy's evaluate on the device tag, epilogue kernel).
template <TI N, TI CAPACITY, TI LIMIT, int STEPS, TI HIDDEN = 64>
void offpolicy_parity(const char* name){
    using PENDULUM = rlt::rl::environments::Pendulum<rlt::rl::environments::pendulum::Specification<T, TI, rlt::rl::environments::pendulum::DefaultParameters<T>>>;
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, HIDDEN, act::RELU, act::TANH>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<ACTOR_CONFIG>>, rlt::tensor::Shape<TI, 1, N, 3>>;
    using POLICIES = rlt::utils::Tuple<TI, ACTOR>;
    using SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, POLICIES, OffPolicyParityParameters<N, CAPACITY, LIMIT>>;
    using RUNNER = rlt::rl::components::OffPolicyRunner<SPEC>;
    using RB = typename RUNNER::REPLAY_BUFFER_TYPE;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng_init, rng_cpu, rng_gpu;
    rlt::malloc(cpu, rng_init); rlt::malloc(cpu, rng_cpu); rlt::malloc(cpu, rng_gpu);
    rlt::init(cpu, rng_init, 2); rlt::init(cpu, rng_cpu, 8); rlt::init(cpu, rng_gpu, 8);
    ACTOR actor_cpu, actor_gpu; typename ACTOR::template Buffer<> buf_cpu, buf_gpu;
    rlt::malloc(cpu, actor_cpu); rlt::malloc(cpu, buf_cpu); rlt::malloc(gpu, actor_gpu); rlt::malloc(gpu, buf_gpu);
    rlt::init_weights(cpu, actor_cpu, rng_init);
    rlt::copy(cpu, gpu, actor_cpu, actor_gpu);
    std::unique_ptr<RUNNER> runner_cpu(new RUNNER()), runner_gpu(new RUNNER());
    rlt::malloc(cpu, *runner_cpu); rlt::malloc(gpu, *runner_gpu);
    rlt::init(cpu, *runner_cpu); rlt::init(gpu, *runner_gpu);
    for(int s = 0; s < STEPS; s++){
        rlt::step<0>(cpu, *runner_cpu, actor_cpu, buf_cpu, rng_cpu);
        rlt::step<0>(gpu, *runner_gpu, actor_gpu, buf_gpu, rng_gpu);
    }
    int status = rlt::check_status(gpu);
    // raw copy of the device-resident replay-buffer structs (their view members hold no host-valid pointers: only data members are read)
    std::vector<unsigned char> raw(sizeof(RB) * (size_t)N);
    b200rl_memcpy(raw.data(), runner_gpu->replay_buffers._data, raw.size(), 1, gpu.stream);
    std::vector<TI> es(N); std::vector<uint8_t> tr(N);
    b200rl_memcpy(es.data(), runner_gpu->episode_step._data, N * sizeof(TI), 1, gpu.stream);
    b200rl_memcpy(tr.data(), runner_gpu->truncated._data, N, 1, gpu.stream);
    bool counters = true; double flags_diff = 0, rows_diff = 0;
    const TI written = STEPS < (int)CAPACITY ? (TI)STEPS : CAPACITY;
    for(TI e = 0; e < N; e++){
        const RB& g = *reinterpret_cast<const RB*>(raw.data() + sizeof(RB) * (size_t)e);
        const RB& c = rlt::get(runner_cpu->replay_buffers, 0, e);
        counters = counters && g.position == c.position && g.full == c.full && g.current_episode_start == c.current_episode_start;
        counters = counters && es[e] == rlt::get(runner_cpu->episode_step, 0, e) && (tr[e] != 0) == rlt::get(runner_cpu->truncated, 0, e);
        for(TI r = 0; r < written; r++){
            counters = counters && g.episode_start._data[r] == c.episode_start._data[r];
            for(TI k = 0; k < 10; k++){
                const double d = std::fabs((double)g.data._data[r * 10 + k] - (double)c.data._data[r * 10 + k]);
                if(k >= 8) flags_diff = std::fmax(flags_diff, d); else rows_diff = std::fmax(rows_diff, d);
            }
        }
    }
    // replay-buffer sampling on both devices from the same engine position: same indices (so the rows differ only by the replay rows' own
    // drift), identical masks
    using BATCH_SPEC = rlt::rl::components::off_policy_runner::SequentialBatchSpecification<SPEC, 1, 48>;
    using BATCH = rlt::rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>;
    BATCH batch_cpu, batch_gpu, batch_back;
    rlt::malloc(cpu, batch_cpu); rlt::malloc(gpu, batch_gpu); rlt::malloc(cpu, batch_back);
    double gather_diff = 0; bool masks = true;
    for(int g = 0; g < 3; g++){
        rlt::gather_batch(cpu, *runner_cpu, batch_cpu, rng_cpu);
        rlt::gather_batch(gpu, *runner_gpu, batch_gpu, rng_gpu);
        rlt::copy(gpu, cpu, batch_gpu, batch_back);
        for(TI q = 0; q < 2; q++) for(TI b = 0; b < 48; b++){
            for(TI k = 0; k < 4; k++) gather_diff = std::fmax(gather_diff, std::fabs((double)rlt::get(cpu, batch_cpu.observations_actions_base, q, b, k) - (double)rlt::get(cpu, batch_back.observations_actions_base, q, b, k)));
            masks = masks && rlt::get(cpu, batch_cpu.next_reset_base, q, b, 0) == rlt::get(cpu, batch_back.next_reset_base, q, b, 0);
            masks = masks && rlt::get(cpu, batch_cpu.next_final_step_mask_base, q, b, 0) == rlt::get(cpu, batch_back.next_final_step_mask_base, q, b, 0);
        }
        for(TI b = 0; b < 48; b++){
            gather_diff = std::fmax(gather_diff, std::fabs((double)rlt::get(cpu, batch_cpu.rewards, 0, b, 0) - (double)rlt::get(cpu, batch_back.rewards, 0, b, 0)));
            masks = masks && rlt::get(cpu, batch_cpu.terminated, 0, b, 0) == rlt::get(cpu, batch_back.terminated, 0, b, 0);
            masks = masks && rlt::get(cpu, batch_cpu.reset, 0, b, 0) == rlt::get(cpu, batch_back.reset, 0, b, 0);
            masks = masks && rlt::get(cpu, batch_cpu.final_step_mask, 0, b, 0) == rlt::get(cpu, batch_back.final_step_mask, 0, b, 0);
        }
    }
    // sequences of length 4 through gather_batch<..., DETERMINISTIC = true> (environment 0, offset = batch element: no draws on either device):
    // the kernel's walk through the device-resident replay-buffer structs against the reference's -- identical masks, rows within the drift
    {
        using SEQ_SPEC = rlt::rl::components::off_policy_runner::SequentialBatchSpecification<SPEC, 4, 8, AdapterSequenceParameters>;
        using SEQ_BATCH = rlt::rl::components::off_policy_runner::SequentialBatch<SEQ_SPEC>;
        SEQ_BATCH seq_cpu, seq_gpu, seq_back;
        rlt::malloc(cpu, seq_cpu); rlt::malloc(gpu, seq_gpu); rlt::malloc(cpu, seq_back);
        rlt::set_all(cpu, seq_cpu.observations_actions_base, 0); rlt::set_all(cpu, seq_cpu.rewards, 0); rlt::set_all(cpu, seq_cpu.terminated, false);
        rlt::copy(cpu, gpu, seq_cpu, seq_gpu);
        rlt::gather_batch<DEVICE_CPU, SPEC, SEQ_SPEC, decltype(rng_cpu), true>(cpu, *runner_cpu, seq_cpu, rng_cpu);
        rlt::gather_batch<DEVICE_GPU::SPEC, SPEC, SEQ_SPEC, decltype(rng_gpu), true>(gpu, *runner_gpu, seq_gpu, rng_gpu);
        rlt::copy(gpu, cpu, seq_gpu, seq_back);
        for(TI q = 0; q < 5; q++) for(TI b = 0; b < 8; b++){
            for(TI k = 0; k < 4; k++) gather_diff = std::fmax(gather_diff, std::fabs((double)rlt::get(cpu, seq_cpu.observations_actions_base, q, b, k) - (double)rlt::get(cpu, seq_back.observations_actions_base, q, b, k)));
            masks = masks && rlt::get(cpu, seq_cpu.next_reset_base, q, b, 0) == rlt::get(cpu, seq_back.next_reset_base, q, b, 0);
            masks = masks && rlt::get(cpu, seq_cpu.next_final_step_mask_base, q, b, 0) == rlt::get(cpu, seq_back.next_final_step_mask_base, q, b, 0);
            if(q < 4){
                gather_diff = std::fmax(gather_diff, std::fabs((double)rlt::get(cpu, seq_cpu.rewards, q, b, 0) - (double)rlt::get(cpu, seq_back.rewards, q, b, 0)));
                masks = masks && rlt::get(cpu, seq_cpu.terminated, q, b, 0) == rlt::get(cpu, seq_back.terminated, q, b, 0);
                masks = masks && rlt::get(cpu, seq_cpu.reset, q, b, 0) == rlt::get(cpu, seq_back.reset, q, b, 0);
                masks = masks && rlt::get(cpu, seq_cpu.final_step_mask, q, b, 0) == rlt::get(cpu, seq_back.final_step_mask, q, b, 0);
            }
        }
        rlt::free(cpu, seq_cpu); rlt::free(gpu, seq_gpu); rlt::free(cpu, seq_back);
    }
    status = status ? status : rlt::check_status(gpu);
    bool engines = rlt::random::uniform_real_distribution(cpu.random, (T)0, (T)1, rng_cpu) == rlt::random::uniform_real_distribution(cpu.random, (T)0, (T)1, rng_gpu);
    bool ok = status == 0 && counters && engines && flags_diff == 0 && rows_diff < 5e-3 && masks && gather_diff < 5e-3;
    std::printf("%-28s envs %3u capacity %3u limit %3u steps %d  status %d  counters %d  engine %d  flags diff %.1e  replay rows drift %.2e  gather masks %d rows %.2e  %s\n",
                name, N, CAPACITY, LIMIT, STEPS, status, (int)counters, (int)engines, flags_diff, rows_diff, (int)masks, gather_diff, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, batch_cpu); rlt::free(gpu, batch_gpu); rlt::free(cpu, batch_back);
    rlt::free(cpu, *runner_cpu); rlt::free(gpu, *runner_gpu);
    rlt::free(cpu, actor_cpu); rlt::free(cpu, buf_cpu); rlt::free(gpu, actor_gpu); rlt::free(gpu, buf_gpu);
}

// utils::polyak::update / update_squared on both devices from the same inputs: the CPU build here may contract a * b + c, so the bound is
// one rounding of the result rather than zero
void polyak_parity(const char* name){
    constexpr TI ROWS = 67, COLS = 45;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng; rlt::malloc(cpu, rng); rlt::init(cpu, rng, 3);
    rlt::Matrix<rlt::matrix::Specification<T, TI, ROWS, COLS>> src_cpu, dst_cpu, src_gpu, dst_gpu, back;
    rlt::malloc(cpu, src_cpu); rlt::malloc(cpu, dst_cpu); rlt::malloc(cpu, back); rlt::malloc(gpu, src_gpu); rlt::malloc(gpu, dst_gpu);
    rlt::randn(cpu, src_cpu, rng); rlt::randn(cpu, dst_cpu, rng);
    rlt::copy(cpu, gpu, src_cpu, src_gpu); rlt::copy(cpu, gpu, dst_cpu, dst_gpu);
    for(int i = 0; i < 4; i++){
        rlt::utils::polyak::update(cpu, src_cpu, dst_cpu, (T)0.995); rlt::utils::polyak::update(gpu, src_gpu, dst_gpu, (T)0.995);
        rlt::utils::polyak::update_squared(cpu, src_cpu, dst_cpu, (T)0.9); rlt::utils::polyak::update_squared(gpu, src_gpu, dst_gpu, (T)0.9);
    }
    rlt::copy(gpu, cpu, dst_gpu, back);
    const int status = rlt::check_status(gpu);
    const double diff = rlt::abs_diff(cpu, dst_cpu, back) / (ROWS * COLS);
    const bool ok = status == 0 && diff < 1e-7;
    std::printf("%-28s %u x %u  status %d  mean diff %.2e  %s\n", name, ROWS, COLS, status, diff, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, src_cpu); rlt::free(cpu, dst_cpu); rlt::free(cpu, back); rlt::free(gpu, src_gpu); rlt::free(gpu, dst_gpu);
}

// The PPO loop's observation normalisation on both devices: three normalizer updates, set_statistics, then a sequential model
// <standardize, mlp> evaluated on the last batch (the reference's generic sequential recursion, dispatched on the device tag).
void normalizer_parity(const char* name){
    constexpr TI ROWS = 2048, DIM = 27;
    using NORMALIZER = rlt::rl::components::RunningNormalizer<rlt::rl::components::running_normalizer::Specification<TYPE_POLICY, TI, DIM>>;
    using STANDARDIZE = rlt::nn::layers::standardize::BindConfiguration<rlt::nn::layers::standardize::Configuration<TYPE_POLICY, TI>>;
    using MLP = rlt::nn_models::mlp::BindConfiguration<rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 8, 3, 64, act::TANH, act::IDENTITY>>;
    using MODEL = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<STANDARDIZE, rlt::nn_models::sequential::Module<MLP>>, rlt::tensor::Shape<TI, 1, ROWS, DIM>>;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng; rlt::malloc(cpu, rng); rlt::init(cpu, rng, 5);
    NORMALIZER norm_cpu, norm_gpu, norm_back;
    MODEL model_cpu, model_gpu; typename MODEL::template Buffer<> buf_cpu, buf_gpu;
    rlt::Matrix<rlt::matrix::Specification<T, TI, ROWS, DIM>> data_cpu, data_gpu;
    rlt::Matrix<rlt::matrix::Specification<T, TI, ROWS, 8>> out_cpu, out_gpu, out_back;
    rlt::malloc(cpu, norm_cpu); rlt::malloc(gpu, norm_gpu); rlt::malloc(cpu, norm_back); rlt::malloc(cpu, model_cpu); rlt::malloc(gpu, model_gpu);
    rlt::malloc(cpu, buf_cpu); rlt::malloc(gpu, buf_gpu); rlt::malloc(cpu, data_cpu); rlt::malloc(gpu, data_gpu);
    rlt::malloc(cpu, out_cpu); rlt::malloc(gpu, out_gpu); rlt::malloc(cpu, out_back);
    rlt::init_weights(cpu, model_cpu, rng);
    rlt::copy(cpu, gpu, model_cpu, model_gpu);
    rlt::init(cpu, norm_cpu); rlt::init(gpu, norm_gpu);
    for(int u = 0; u < 3; u++){
        rlt::randn(cpu, data_cpu, rng);
        for(TI r = 0; r < ROWS; r++) for(TI c = 0; c < DIM; c++) rlt::set(data_cpu, r, c, rlt::get(data_cpu, r, c) * (T)(0.2 + c) + (T)c - 9);
        rlt::copy(cpu, gpu, data_cpu, data_gpu);
        rlt::update(cpu, norm_cpu, data_cpu); rlt::update(gpu, norm_gpu, data_gpu);
    }
    rlt::set_statistics(cpu, model_cpu.content, norm_cpu.mean, norm_cpu.std);
    rlt::set_statistics(gpu, model_gpu.content, norm_gpu.mean, norm_gpu.std);
    auto in_cpu = rlt::to_tensor(cpu, data_cpu); auto in_gpu = rlt::to_tensor(gpu, data_gpu);
    auto o_cpu = rlt::to_tensor(cpu, out_cpu); auto o_gpu = rlt::to_tensor(gpu, out_gpu);
    auto in_cpu_r = rlt::reshape_row_major(cpu, in_cpu, rlt::tensor::Shape<TI, 1, ROWS, DIM>{}); auto in_gpu_r = rlt::reshape_row_major(gpu, in_gpu, rlt::tensor::Shape<TI, 1, ROWS, DIM>{});
    auto o_cpu_r = rlt::reshape_row_major(cpu, o_cpu, rlt::tensor::Shape<TI, 1, ROWS, 8>{}); auto o_gpu_r = rlt::reshape_row_major(gpu, o_gpu, rlt::tensor::Shape<TI, 1, ROWS, 8>{});
    rlt::evaluate(cpu, model_cpu, in_cpu_r, o_cpu_r, buf_cpu, rng);
    rlt::evaluate(gpu, model_gpu, in_gpu_r, o_gpu_r, buf_gpu, rng);
    rlt::copy(gpu, cpu, out_gpu, out_back);
    rlt::copy(gpu, cpu, norm_gpu.mean, norm_back.mean); rlt::copy(gpu, cpu, norm_gpu.std, norm_back.std);
    const int status = rlt::check_status(gpu);
    const double stats = (rlt::abs_diff(cpu, norm_cpu.mean, norm_back.mean) + rlt::abs_diff(cpu, norm_cpu.std, norm_back.std)) / (2 * DIM);
    const double out = rlt::abs_diff(cpu, out_cpu, out_back) / (ROWS * 8);
    // columns reach |x| ~ 80 (scale 0.2 .. 26, offset -9 .. 17): 1e-5 absolute is ~1e-6 of the data's scale
    const bool ok = status == 0 && norm_cpu.age == norm_gpu.age && stats < 1e-5 && out < 1e-5;
    std::printf("%-28s rows %u dim %u  status %d  age %u/%u  mean statistics diff %.2e  mean output diff %.2e  %s\n", name, ROWS, DIM, status, (unsigned)norm_cpu.age, (unsigned)norm_gpu.age,
                stats, out, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, norm_cpu); rlt::free(gpu, norm_gpu); rlt::free(cpu, norm_back); rlt::free(cpu, model_cpu); rlt::free(gpu, model_gpu);
    rlt::free(cpu, buf_cpu); rlt::free(gpu, buf_gpu); rlt::free(cpu, data_cpu); rlt::free(gpu, data_gpu); rlt::free(cpu, out_cpu); rlt::free(gpu, out_gpu); rlt::free(cpu, out_back);
}

// init_weights, randn and mse::evaluate on the device tag against the CPU device from the same engine state: the draws are made by the
// reference's own distributions on the host, so parameters, matrices and the engine's final state are identical; the loss value agrees to
// the float sum's rounding. Also: the network lives in ONE arena (whole-model path), and a network allocated layer by layer (the
// per-layer path of the same verbs) trains to the same parameters.
template <TI BATCH, TI INPUT_DIM, TI HIDDEN_DIM, TI OUTPUT_DIM>
void boundary_extras(const char* name){
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, OUTPUT_DIM, 3, HIDDEN_DIM, act::RELU, act::IDENTITY>;
    using INPUT_SHAPE = rlt::tensor::Shape<TI, 1, BATCH, INPUT_DIM>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>, INPUT_SHAPE>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    NET net_cpu, net_gpu, net_layers, net_back, net_back2;
    typename NET::template Buffer<> buf_gpu, buf_layers;
    OPTIMIZER opt_gpu, opt_layers;
    rlt::malloc(cpu, net_cpu); rlt::malloc(cpu, net_back); rlt::malloc(cpu, net_back2);
    rlt::malloc(gpu, net_gpu); rlt::malloc(gpu, buf_gpu); rlt::malloc(gpu, opt_gpu); rlt::malloc(gpu, buf_layers); rlt::malloc(gpu, opt_layers);
    // layer by layer: the reference's per-tensor allocation, which the whole-model verbs must detect and serve through the per-layer path
    rlt::malloc(gpu, net_layers.input_layer); rlt::malloc(gpu, net_layers.hidden_layers[0]); rlt::malloc(gpu, net_layers.output_layer);
    const bool arena = (bool)rlt::b200::mlp::arena_of(net_gpu), no_arena = !(bool)rlt::b200::mlp::arena_of(net_layers);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng_cpu, rng_gpu;
    rlt::malloc(cpu, rng_cpu); rlt::malloc(cpu, rng_gpu);
    rlt::init(cpu, rng_cpu, 11); rlt::init(cpu, rng_gpu, 11);
    rlt::init_weights(cpu, net_cpu, rng_cpu);
    rlt::init_weights(gpu, net_gpu, rng_gpu);
    rlt::zero_gradient(cpu, net_cpu); rlt::zero_gradient(gpu, net_gpu);
    rlt::init(gpu, opt_gpu); rlt::init(gpu, opt_layers);
    rlt::reset_optimizer_state(gpu, opt_gpu, net_gpu);
    rlt::copy(gpu, cpu, net_gpu, net_back);
    rlt::Matrix<rlt::matrix::Specification<T, TI, BATCH, INPUT_DIM>> x_cpu, x_gpu, x_back;
    rlt::Matrix<rlt::matrix::Specification<T, TI, BATCH, OUTPUT_DIM>> y_cpu, y_gpu, d_gpu, d_layers, out_cpu;
    rlt::malloc(cpu, x_cpu); rlt::malloc(cpu, x_back); rlt::malloc(cpu, y_cpu); rlt::malloc(cpu, out_cpu);
    rlt::malloc(gpu, x_gpu); rlt::malloc(gpu, y_gpu); rlt::malloc(gpu, d_gpu); rlt::malloc(gpu, d_layers);
    rlt::randn(cpu, x_cpu, rng_cpu); rlt::randn(gpu, x_gpu, rng_gpu);
    rlt::randn(cpu, y_cpu, rng_cpu); rlt::randn(gpu, y_gpu, rng_gpu);
    rlt::copy(gpu, cpu, x_gpu, x_back);
    const T init_diff = rlt::abs_diff(cpu, net_back.input_layer.weights.parameters, net_cpu.input_layer.weights.parameters) + rlt::abs_diff(cpu, net_back.input_layer.biases.parameters, net_cpu.input_layer.biases.parameters)
                      + rlt::abs_diff(cpu, net_back.hidden_layers[0].weights.parameters, net_cpu.hidden_layers[0].weights.parameters) + rlt::abs_diff(cpu, net_back.output_layer.biases.parameters, net_cpu.output_layer.biases.parameters)
                      + rlt::abs_diff(cpu, net_back.output_layer.weights.parameters, net_cpu.output_layer.weights.parameters);
    const T randn_diff = rlt::abs_diff(cpu, x_back, x_cpu);
    const bool engine_equal = rlt::abs_diff(cpu, rng_cpu, rng_gpu) == 0;
    // loss of y against a shifted copy, on both devices
    for(TI b = 0; b < BATCH; b++) for(TI o = 0; o < OUTPUT_DIM; o++) rlt::set(out_cpu, b, o, rlt::get(y_cpu, b, o) * (T)0.75 + (T)0.1);
    rlt::copy(cpu, gpu, out_cpu, d_gpu);
    const T l_cpu = rlt::nn::loss_functions::mse::evaluate(cpu, y_cpu, out_cpu, (T)1.5), l_gpu = rlt::nn::loss_functions::mse::evaluate(gpu, y_gpu, d_gpu, (T)1.5);
    // the CPU device adds BATCH * OUTPUT_DIM squares in float, one after the other: its own rounding error grows like sqrt(n) * 2^-24 (the device
    // sums in double and rounds once); four standard deviations of that random walk bound the difference
    const double loss_tolerance = 4.0 * std::sqrt((double)BATCH * OUTPUT_DIM) * 5.96e-8 + 1e-7;
    // the same two training steps through the arena path and through the layer-by-layer path
    rlt::copy(cpu, gpu, net_cpu, net_layers);
    rlt::zero_gradient(gpu, net_layers);
    rlt::reset_optimizer_state(gpu, opt_layers, net_layers);
    for(int s = 0; s < 2; s++){
        rlt::zero_gradient(gpu, net_gpu);
        rlt::forward(gpu, net_gpu, x_gpu, buf_gpu, rng_gpu);
        { auto out = rlt::output(gpu, net_gpu); auto out_m = rlt::matrix_view(gpu, out); rlt::nn::loss_functions::mse::gradient(gpu, out_m, y_gpu, d_gpu, (T)1); }
        rlt::backward(gpu, net_gpu, x_gpu, d_gpu, buf_gpu);
        rlt::step(gpu, opt_gpu, net_gpu);
        rlt::zero_gradient(gpu, net_layers);
        rlt::forward(gpu, net_layers, x_gpu, buf_layers, rng_gpu);
        { auto out = rlt::output(gpu, net_layers); auto out_m = rlt::matrix_view(gpu, out); rlt::nn::loss_functions::mse::gradient(gpu, out_m, y_gpu, d_layers, (T)1); }
        rlt::backward(gpu, net_layers, x_gpu, d_layers, buf_layers);
        rlt::step(gpu, opt_layers, net_layers);
    }
    const int status = rlt::check_status(gpu);
    rlt::copy(gpu, cpu, net_gpu, net_back); rlt::copy(gpu, cpu, net_layers, net_back2);
    const double n_all = 4.0 * (INPUT_DIM * HIDDEN_DIM + HIDDEN_DIM + HIDDEN_DIM * HIDDEN_DIM + HIDDEN_DIM + HIDDEN_DIM * OUTPUT_DIM + OUTPUT_DIM) + 2.0 * BATCH * (2 * HIDDEN_DIM + OUTPUT_DIM);
    const T path_diff = (T)(rlt::abs_diff(cpu, net_back, net_back2) / n_all);
    const bool ok = status == 0 && arena && no_arena && init_diff == 0 && randn_diff == 0 && engine_equal && std::fabs(l_cpu - l_gpu) <= loss_tolerance * std::fabs(l_cpu) && path_diff < 1e-7;
    std::printf("%-28s batch %4u  status %d  arena %d/%d  init_weights diff %.1e  randn diff %.1e  engine %d  mse loss %.7f vs %.7f  arena vs per-layer mean diff %.2e  %s\n",
                name, BATCH, status, (int)arena, (int)no_arena, init_diff, randn_diff, (int)engine_equal, l_cpu, l_gpu, path_diff, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, net_cpu); rlt::free(cpu, net_back); rlt::free(cpu, net_back2);
    rlt::free(gpu, net_gpu); rlt::free(gpu, buf_gpu); rlt::free(gpu, opt_gpu); rlt::free(gpu, buf_layers); rlt::free(gpu, opt_layers);
    rlt::free(gpu, net_layers.input_layer); rlt::free(gpu, net_layers.hidden_layers[0]); rlt::free(gpu, net_layers.output_layer);
    rlt::free(cpu, x_cpu); rlt::free(cpu, x_back); rlt::free(cpu, y_cpu); rlt::free(cpu, out_cpu);
    rlt::free(gpu, x_gpu); rlt::free(gpu, y_gpu); rlt::free(gpu, d_gpu); rlt::free(gpu, d_layers);
}

// SAC update: the reference's OWN generic train_critic / update_critic_targets / train_actor (rl/algorithms/sac/operations_generic.h) instantiated on
// devices::B200 next to the CPU device: same initial networks (initialised on the CPU, copied over), same hand-filled SequentialBatch of sequence
// length 1, same action noise; per update critic 0, critic 1, target update, actor. Compared: every network with gradients and Adam moments,
// log_alpha, the target critics, the last target values.
template <TI T_BATCH>
struct SacParityParameters: rlt::rl::algorithms::sac::DefaultParameters<TYPE_POLICY, TI, 1>{
    static constexpr TI ACTOR_BATCH_SIZE = T_BATCH;
    static constexpr TI CRITIC_BATCH_SIZE = T_BATCH;
};
template <typename SAC_PARAMETERS>
struct SacParityHeadParameters{
    static constexpr T LOG_STD_LOWER_BOUND = SAC_PARAMETERS::LOG_STD_LOWER_BOUND, LOG_STD_UPPER_BOUND = SAC_PARAMETERS::LOG_STD_UPPER_BOUND;
    static constexpr T LOG_PROBABILITY_EPSILON = SAC_PARAMETERS::LOG_PROBABILITY_EPSILON, ALPHA = SAC_PARAMETERS::ALPHA, TARGET_ENTROPY = SAC_PARAMETERS::TARGET_ENTROPY;
    static constexpr bool ADAPTIVE_ALPHA = SAC_PARAMETERS::ADAPTIVE_ALPHA, UPDATE_ALPHA_WITH_ACTOR = false;
};
template <TI BATCH, TI HIDDEN, int UPDATES>
void sac_parity(const char* name){
    using PENDULUM = rlt::rl::environments::Pendulum<rlt::rl::environments::pendulum::Specification<TYPE_POLICY, TI, rlt::rl::environments::pendulum::DefaultParameters<T>>>;
    using SAC_PARAMETERS = SacParityParameters<BATCH>;
    using ACTOR_MLP = rlt::nn_models::mlp::BindConfiguration<rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 2, 3, HIDDEN, act::RELU, act::IDENTITY>>;
    using SAS = rlt::nn::layers::sample_and_squash::BindConfiguration<rlt::nn::layers::sample_and_squash::Configuration<TYPE_POLICY, TI, SacParityHeadParameters<SAC_PARAMETERS>>>;
    using CAP_GRADIENT = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using ACTOR = rlt::nn_models::sequential::Build<CAP_GRADIENT, rlt::nn_models::sequential::Module<ACTOR_MLP, rlt::nn_models::sequential::Module<SAS>>, rlt::tensor::Shape<TI, 1, BATCH, 3>>;
    using CRITIC_MLP = rlt::nn_models::mlp::BindConfiguration<rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, HIDDEN, act::RELU, act::IDENTITY>>;
    using CRITIC = rlt::nn_models::sequential::Build<CAP_GRADIENT, rlt::nn_models::sequential::Module<CRITIC_MLP>, rlt::tensor::Shape<TI, 1, BATCH, 4>>;
    using CRITIC_TARGET = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<CRITIC_MLP>, rlt::tensor::Shape<TI, 1, BATCH, 4>>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    using AC_SPEC = rlt::rl::algorithms::sac::Specification<TYPE_POLICY, TI, PENDULUM, ACTOR, CRITIC, CRITIC_TARGET, rlt::nn::parameters::Adam, OPTIMIZER, OPTIMIZER, OPTIMIZER, SAC_PARAMETERS, false>;
    using ACTOR_CRITIC = rlt::rl::algorithms::sac::ActorCritic<AC_SPEC>;
    using EVAL_ACTOR = typename ACTOR::template CHANGE_BATCH_SIZE<TI, 4>;
    using RUNNER_SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, rlt::utils::Tuple<TI, EVAL_ACTOR>, OffPolicyParityParameters<4, 16, 200>>;
    using BATCH_TYPE = rlt::rl::components::off_policy_runner::SequentialBatch<rlt::rl::components::off_policy_runner::SequentialBatchSpecification<RUNNER_SPEC, 1, BATCH>>;
    using CRITIC_TRAINING_BUFFERS = rlt::rl::algorithms::sac::CriticTrainingBuffers<rlt::rl::algorithms::sac::CriticTrainingBuffersSpecification<AC_SPEC, true>>;
    using ACTOR_TRAINING_BUFFERS = rlt::rl::algorithms::sac::ActorTrainingBuffers<rlt::rl::algorithms::sac::ActorTrainingBuffersSpecification<AC_SPEC, true>>;
    using NOISE = rlt::Matrix<rlt::matrix::Specification<T, TI, BATCH, 1>>;
    DEVICE_CPU cpu; DEVICE_GPU gpu;
    rlt::init(gpu);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng;
    rlt::malloc(cpu, rng); rlt::init(cpu, rng, 11);
    auto ac_cpu = std::make_unique<ACTOR_CRITIC>(); auto ac_gpu = std::make_unique<ACTOR_CRITIC>(); auto ac_back = std::make_unique<ACTOR_CRITIC>();
    BATCH_TYPE batch_cpu, batch_gpu; CRITIC_TRAINING_BUFFERS ctb_cpu, ctb_gpu, ctb_back; ACTOR_TRAINING_BUFFERS atb_cpu, atb_gpu;
    typename ACTOR::template Buffer<> ab_cpu, atgt_cpu, ab_gpu, atgt_gpu; typename CRITIC::template Buffer<> cb_cpu, cb_gpu; typename CRITIC_TARGET::template Buffer<> ctgt_cpu, ctgt_gpu;
    NOISE noise_cpu, noise_gpu;
    rlt::malloc(cpu, *ac_cpu); rlt::malloc(cpu, *ac_back); rlt::malloc(cpu, batch_cpu); rlt::malloc(cpu, ctb_cpu); rlt::malloc(cpu, ctb_back); rlt::malloc(cpu, atb_cpu);
    rlt::malloc(cpu, ab_cpu); rlt::malloc(cpu, atgt_cpu); rlt::malloc(cpu, cb_cpu); rlt::malloc(cpu, ctgt_cpu); rlt::malloc(cpu, noise_cpu);
    rlt::malloc(gpu, *ac_gpu); rlt::malloc(gpu, batch_gpu); rlt::malloc(gpu, ctb_gpu); rlt::malloc(gpu, atb_gpu);
    rlt::malloc(gpu, ab_gpu); rlt::malloc(gpu, atgt_gpu); rlt::malloc(gpu, cb_gpu); rlt::malloc(gpu, ctgt_gpu); rlt::malloc(gpu, noise_gpu);
    rlt::init(cpu, *ac_cpu, rng);
    rlt::init(gpu, *ac_gpu, rng);                              // allocates nothing new; every value is overwritten by the copy below
    rlt::copy(cpu, gpu, *ac_cpu, *ac_gpu);
    std::normal_distribution<T> normal(0, 1); std::uniform_real_distribution<T> uniform(0, 1);
    std::mt19937 fill(3);
    const char* first_failure = "";
    auto probe = [&](const char* what){ if(gpu.status != B200RL_OK && !first_failure[0]) first_failure = what; };
    probe("setup");
    for(int u = 0; u < UPDATES; u++){
        for(TI q = 0; q < 2; q++) for(TI b = 0; b < BATCH; b++){
            T theta = (uniform(fill) * 2 - 1) * (T)3.14159265, theta_dot = (uniform(fill) * 2 - 1) * 8;
            rlt::set(cpu, batch_cpu.observations_actions_base, std::cos(theta), q, b, 0);
            rlt::set(cpu, batch_cpu.observations_actions_base, std::sin(theta), q, b, 1);
            rlt::set(cpu, batch_cpu.observations_actions_base, theta_dot, q, b, 2);
            rlt::set(cpu, batch_cpu.observations_actions_base, uniform(fill) * 2 - 1, q, b, 3);
            rlt::set(cpu, batch_cpu.next_reset_base, true, q, b, 0);
            rlt::set(cpu, batch_cpu.next_final_step_mask_base, q == 1, q, b, 0);
        }
        for(TI b = 0; b < BATCH; b++){
            rlt::set(cpu, batch_cpu.rewards, -uniform(fill) * 16, 0, b, 0);
            rlt::set(cpu, batch_cpu.terminated, uniform(fill) < (T)0.1, 0, b, 0);
            rlt::set(cpu, batch_cpu.reset, true, 0, b, 0);
            rlt::set(cpu, batch_cpu.final_step_mask, true, 0, b, 0);
        }
        rlt::copy(cpu, gpu, batch_cpu, batch_gpu);
        for(int c = 0; c < 2; c++){
            for(TI b = 0; b < BATCH; b++) rlt::set(noise_cpu, b, 0, normal(fill));
            rlt::copy(cpu, gpu, noise_cpu, noise_gpu);
            rlt::train_critic(cpu, *ac_cpu, ac_cpu->critics[c], batch_cpu, ac_cpu->critic_optimizers[c], atgt_cpu, cb_cpu, ctgt_cpu, ctb_cpu, noise_cpu, rng);
            rlt::train_critic(gpu, *ac_gpu, ac_gpu->critics[c], batch_gpu, ac_gpu->critic_optimizers[c], atgt_gpu, cb_gpu, ctgt_gpu, ctb_gpu, noise_gpu, rng);
            probe("train_critic");
        }
        rlt::update_critic_targets(cpu, *ac_cpu);
        rlt::update_critic_targets(gpu, *ac_gpu);
        probe("update_critic_targets");
        for(TI b = 0; b < BATCH; b++) rlt::set(noise_cpu, b, 0, normal(fill));
        rlt::copy(cpu, gpu, noise_cpu, noise_gpu);
        rlt::train_actor(cpu, *ac_cpu, batch_cpu, ac_cpu->actor_optimizer, ab_cpu, cb_cpu, atb_cpu, noise_cpu, rng);
        rlt::train_actor(gpu, *ac_gpu, batch_gpu, ac_gpu->actor_optimizer, ab_gpu, cb_gpu, atb_gpu, noise_gpu, rng);
        probe("train_actor");
    }
    int status = rlt::check_status(gpu);
    rlt::copy(gpu, cpu, *ac_gpu, *ac_back);
    rlt::copy(gpu, cpu, ctb_gpu.target_action_value, ctb_back.target_action_value);
    constexpr double N_ACTOR = 3.0 * HIDDEN + HIDDEN + (double)HIDDEN * HIDDEN + HIDDEN + HIDDEN * 2.0 + 2, N_CRITIC = 4.0 * HIDDEN + HIDDEN + (double)HIDDEN * HIDDEN + HIDDEN + HIDDEN + 1;
    // abs_diff of a network sums over parameters, gradients, both Adam moments and the saved activations of every layer
    T actor_diff = (T)(rlt::abs_diff(cpu, ac_back->actor.content, ac_cpu->actor.content) / (4 * N_ACTOR + 2.0 * BATCH * (2 * HIDDEN + 2)));
    T critic_diff = 0, target_diff = 0;
    for(int c = 0; c < 2; c++){
        critic_diff += (T)(rlt::abs_diff(cpu, ac_back->critics[c].content, ac_cpu->critics[c].content) / (4 * N_CRITIC + 2.0 * BATCH * (2 * HIDDEN + 1)) / 2);
        target_diff += (T)(rlt::abs_diff(cpu, ac_back->critics_target[c].content, ac_cpu->critics_target[c].content) / N_CRITIC / 2);
    }
    auto& la_cpu = rlt::get_last_layer(ac_cpu->actor).log_alpha; auto& la_back = rlt::get_last_layer(ac_back->actor).log_alpha;
    T log_alpha_diff = std::abs(rlt::get(cpu, la_cpu.parameters, 0) - rlt::get(cpu, la_back.parameters, 0));
    T log_alpha_grad_diff = std::abs(rlt::get(cpu, la_cpu.gradient, 0) - rlt::get(cpu, la_back.gradient, 0));
    T target_value_diff = 0, target_value_scale = 0;
    for(TI b = 0; b < BATCH; b++){
        T want = rlt::get(cpu, ctb_cpu.target_action_value, 0, b, 0), got = rlt::get(cpu, ctb_back.target_action_value, 0, b, 0);
        target_value_diff = std::max(target_value_diff, std::abs(want - got)); target_value_scale = std::max(target_value_scale, std::abs(want));
    }
    // bounds: means of absolute differences over fp32 tensors whose entries are O(1e-1) (the MLP cases above use 1e-7 for one network); the
    // target values are single fp32 numbers of magnitude target_value_scale compared at 1e-5 relative + 1e-6
    bool ok = status == 0 && actor_diff < 2e-7 && critic_diff < 2e-7 && target_diff < 1e-7 && log_alpha_diff < 1e-7 && log_alpha_grad_diff < 1e-5 &&
              target_value_diff <= 1e-6 + 1e-5 * target_value_scale && !std::isnan(actor_diff) && !std::isnan(critic_diff);
    std::printf("%-28s batch %4u hidden %3u updates %d  status %d  mean diff actor %.2e critics %.2e targets %.2e  log_alpha %.1e (grad %.1e)  target values %.2e of %.1f  %s%s  %s\n",
                name, BATCH, HIDDEN, UPDATES, status, actor_diff, critic_diff, target_diff, log_alpha_diff, log_alpha_grad_diff, target_value_diff, target_value_scale, first_failure[0] ? "first failing verb: " : "", first_failure, ok ? "OK" : "FAIL");
    if(!ok) failures++;
    rlt::free(cpu, *ac_cpu); rlt::free(cpu, *ac_back); rlt::free(cpu, batch_cpu); rlt::free(cpu, ctb_cpu); rlt::free(cpu, ctb_back); rlt::free(cpu, atb_cpu);
    rlt::free(cpu, ab_cpu); rlt::free(cpu, atgt_cpu); rlt::free(cpu, cb_cpu); rlt::free(cpu, ctgt_cpu); rlt::free(cpu, noise_cpu);
    rlt::free(gpu, *ac_gpu); rlt::free(gpu, batch_gpu); rlt::free(gpu, ctb_gpu); rlt::free(gpu, atb_gpu);
    rlt::free(gpu, ab_gpu); rlt::free(gpu, atgt_gpu); rlt::free(gpu, cb_gpu); rlt::free(gpu, ctgt_gpu); rlt::free(gpu, noise_gpu);
}

int main(){
    std::setvbuf(stdout, nullptr, _IOLBF, 0);                          // a crash must not swallow the lines already printed
    // the reference's CUDA sweep (cuda_basics.cu:961-972) plus the BASELINE shapes
    train_steps<   1, 256,  10, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b1");
    train_steps<   2, 256,  10, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b2");
    train_steps<  32, 256,  10, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b32");
    train_steps<1024, 256,  10, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b1024");
    train_steps<  10, 256, 200, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b10");
    train_steps<   9, 256,  60, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b9");
    train_steps< 200, 256,  11, 100, 3, act::RELU, act::IDENTITY, 1>("sweep_b200");
    train_steps<  64, 256,  50, 101, 3, act::RELU, act::IDENTITY, 3>("sweep_b64_3steps");
    train_steps< 256, 256, 256, 256, 3, act::RELU, act::IDENTITY, 3>("sweep_b256_3steps");
    train_steps< 256,   3,  64,   2, 3, act::RELU, act::IDENTITY, 2>("c1_actor");
    train_steps< 256,   4, 256,   1, 3, act::RELU, act::IDENTITY, 5>("c3_sac_critic_5steps");
    train_steps<2048,  27,  64,   8, 3, act::TANH, act::IDENTITY, 2>("c4_ppo_actor");
    train_steps<1024,  64, 256,  16, 4, act::RELU, act::IDENTITY, 2>("c5_b1024");
    boundary_extras<256, 4, 64, 2>("init_randn_mse_arena");
    boundary_extras<2048, 27, 64, 8>("init_randn_mse_arena_b2048");
    collect_parity<  64, 64, 100, act::RELU, 3>("collect_ppo_default");
    collect_parity<1000, 40,  15, act::TANH, 2>("collect_tanh_1000");
    offpolicy_parity<8, 64, 50, 137>("off_policy_runner_step");
    offpolicy_parity<33, 40, 17, 90>("off_policy_runner_wraps");
    offpolicy_parity<5, 300, 60, 47>("off_policy_runner_part_full");
    offpolicy_parity<9, 48, 20, 70, 32>("off_policy_runner_generic_policy");
    polyak_parity("polyak_target_update");
    normalizer_parity("observation_normalisation");
    ppo_parity<64, 64, 512, 2>("ppo_train_shuffled");
    ppo_parity<16, 128, 2048, 1>("ppo_train_one_batch");
    sac_parity<256, 64, 3>("sac_update_verbs");
    sac_parity<100, 256, 2>("sac_update_verbs_h256");
    std::printf("%s\n", failures ? "ADAPTER PARITY FAILED" : "ADAPTER PARITY OK");
    return failures ? 1 : 0;
}
