// TEST INFRASTRUCTURE -- not part of the shipped library.
//
// Thin extern "C" driver around the UNMODIFIED RLtools headers (header-only C++17). It instantiates the
// reference's own templates for the shapes the parity suite needs and exposes them as a flat C interface so
// that (a) the plain-C restatement in oracle.c can be pinned against the real reference, bit for bit, and
// (b) golden fixtures can be generated, and (c) the reference CPU path can be timed as the CPU baseline.
//
// Nothing from the reference is copied here: the headers are included from where they lie
// (-I<reference>/include). Build recipe: oracle/Makefile (targets _ref/libref_strict.so, _ref/libref_fast.so).
//
//   strict : generic CPU device, -O2 -fno-fast-math -ffp-contract=off  -> fixed summation order, parity anchor
//   fast   : CPU_OPENBLAS device (-DREF_USE_OPENBLAS), project default flags -> the timed CPU baseline
//
// Reference entry points exercised (paths inside the reference's include/rl_tools):
//   nn_models/mlp/operations_generic.h   evaluate / forward / backward / zero_gradient / update
//   nn/layers/dense/operations_generic.h (strict)  nn/layers/dense/operations_cpu_blas.h (fast)
//   nn/optimizers/adam/operations_generic.h   init / reset_optimizer_state / step
//   nn/loss_functions/mse/operations_generic.h   gradient
//   rl/environments/pendulum/operations_generic.h   sample_initial_state / step / reward / observe
//   random/operations_cpu.h   init(device, rng, seed), uniform_real_distribution, normal_distribution::sample
//   rl/components/off_policy_runner/operations_generic.h  malloc / init / step<0> (per-environment replay buffers)
//   rl/components/on_policy_runner/operations_generic.h   init / collect (actor: sequential<mlp_unconditional_stddev>)
//   rl/algorithms/ppo/operations_generic.h   estimate_generalized_advantages
#ifdef REF_USE_OPENBLAS
#include <rl_tools/operations/cpu_mux.h>
#else
#include <rl_tools/operations/cpu.h>
#endif
#include <rl_tools/nn/optimizers/adam/instance/operations_generic.h>
#ifdef REF_USE_OPENBLAS
#include <rl_tools/nn/operations_cpu_mux.h>
#else
#include <rl_tools/nn/operations_generic.h>
#endif
#include <rl_tools/nn/layers/dense/operations_cpu.h>
#include <rl_tools/nn/loss_functions/mse/operations_generic.h>
#include <rl_tools/nn/layers/sample_and_squash/operations_generic.h>     // before the model headers that recurse into it
#include <rl_tools/nn/layers/standardize/operations_generic.h>
#include <rl_tools/rl/components/running_normalizer/operations_generic.h>
#include <rl_tools/nn_models/mlp/operations_generic.h>
#include <rl_tools/nn_models/mlp_unconditional_stddev/operations_generic.h>
#include <rl_tools/nn_models/sequential/operations_generic.h>
#include <rl_tools/nn/optimizers/adam/operations_generic.h>
#include <rl_tools/rl/environments/pendulum/operations_generic.h>
#include <rl_tools/rl/environments/acrobot/operations_generic.h>
#include <rl_tools/rl/environments/l2f/operations_generic.h>
#include <rl_tools/rl/components/on_policy_runner/operations_generic.h>
#include <rl_tools/rl/components/off_policy_runner/operations_generic.h>
#include <rl_tools/rl/algorithms/sac/operations_generic.h>
#include <rl_tools/rl/algorithms/ppo/ppo.h>
#include <rl_tools/rl/algorithms/ppo/operations_generic.h>

#include <cstdint>
#include <cstring>
#include <string>
#include <map>
#include <vector>
#include <thread>
#include <chrono>

namespace rlt = rl_tools;

#ifdef REF_USE_OPENBLAS
using DEVICE = rlt::devices::DEVICE_FACTORY<>;
#else
using DEVICE = rlt::devices::DefaultCPU;
#endif
using TI = typename DEVICE::index_t;
using T = float;
using TYPE_POLICY = rlt::numeric_types::Policy<T>;
using RNG = DEVICE::SPEC::RANDOM::ENGINE<>;
namespace act = rlt::nn::activation_functions;

using PENDULUM_SPEC = rlt::rl::environments::pendulum::Specification<T, TI, rlt::rl::environments::pendulum::DefaultParameters<T>>;
using PENDULUM = rlt::rl::environments::Pendulum<PENDULUM_SPEC>;

static act::ActivationFunction act_from_int(int a){
    switch(a){
        case 0: return act::IDENTITY; case 1: return act::RELU; case 2: return act::TANH; case 3: return act::FAST_TANH; case 4: return act::SIGMOID;
        default: return act::IDENTITY;
    }
}

// ---------------------------------------------------------------------------------------------------------
// MLP cases: the reference fixes every shape at compile time, so each (batch, dims, activations) tuple the
// parity suite sweeps is one template instantiation, looked up by name at run time.
// ---------------------------------------------------------------------------------------------------------
struct MlpVTable{
    int batch, input_dim, hidden_dim, output_dim, num_layers, hidden_act, output_act;
    // params layout (flat): per layer W[O,I] row-major then b[O]
    void (*run)(const float* params_in, uint32_t init_seed, const float* x, const float* target, int mode, int n_steps,
                float* params_out, float* grads_out, float* m_out, float* v_out, float* pre_out, float* act_out, float* d_input_out, double* seconds);
};

template <typename LAYER>
static void load_layer(DEVICE& device, LAYER& layer, const float*& p){
    constexpr TI O = LAYER::OUTPUT_DIM, I = LAYER::INPUT_DIM;
    for(TI o = 0; o < O; o++) for(TI i = 0; i < I; i++) rlt::set(device, layer.weights.parameters, p[o * I + i], o, i);
    p += O * I;
    for(TI o = 0; o < O; o++) rlt::set(device, layer.biases.parameters, p[o], o);
    p += O;
}
enum Which{PARAMS, GRADS, MOM1, MOM2};
template <typename LAYER>
static void store_layer(DEVICE& device, LAYER& layer, float*& p, Which which){
    constexpr TI O = LAYER::OUTPUT_DIM, I = LAYER::INPUT_DIM;
    if(!p) return;
    auto& w = which == PARAMS ? layer.weights.parameters : (which == GRADS ? layer.weights.gradient : (which == MOM1 ? layer.weights.gradient_first_order_moment : layer.weights.gradient_second_order_moment));
    auto& b = which == PARAMS ? layer.biases.parameters : (which == GRADS ? layer.biases.gradient : (which == MOM1 ? layer.biases.gradient_first_order_moment : layer.biases.gradient_second_order_moment));
    for(TI o = 0; o < O; o++) for(TI i = 0; i < I; i++) p[o * I + i] = rlt::get(device, w, o, i);
    p += O * I;
    for(TI o = 0; o < O; o++) p[o] = rlt::get(device, b, o);
    p += O;
}
template <typename LAYER>
static void store_acts(DEVICE& device, LAYER& layer, float*& pre, float*& out){
    constexpr TI O = LAYER::OUTPUT_DIM, B = LAYER::INTERNAL_BATCH_SIZE;
    for(TI b = 0; b < B; b++) for(TI o = 0; o < O; o++){
        if(pre) pre[b * O + o] = rlt::get(layer.pre_activations, b, o);
        if(out) out[b * O + o] = rlt::get(layer.output, b, o);
    }
    if(pre) pre += B * O;
    if(out) out += B * O;
}

template <TI B, TI I, TI H, TI O, TI NL, act::ActivationFunction HACT, act::ActivationFunction OACT>
struct MlpCase{
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, O, NL, H, HACT, OACT>;
    using INPUT_SHAPE = rlt::tensor::Shape<TI, 1, B, I>;
    using CAPABILITY = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, CAPABILITY, INPUT_SHAPE>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;

    template <typename F>
    static void for_each_layer(NET& net, F f){
        f(net.input_layer);
        for(TI l = 0; l < NET::NUM_HIDDEN_LAYERS; l++) f(net.hidden_layers[l]);
        f(net.output_layer);
    }
    // mode 0: evaluate only (act_out receives the network output [B,O])
    // mode 1: zero_gradient, forward, mse::gradient(weight 1), backward            (n_steps ignored)
    // mode 2: n_steps x { zero_gradient, forward, mse::gradient, backward, step }  (Adam, TF defaults)
    // mode 3: like 1 but d_output := target (no loss) and the FULL backward incl. d_input (backward_full)
    static void run(const float* params_in, uint32_t init_seed, const float* x, const float* target, int mode, int n_steps,
                    float* params_out, float* grads_out, float* m_out, float* v_out, float* pre_out, float* act_out, float* d_input_out, double* seconds){
        DEVICE device;
        RNG rng;
        rlt::malloc(device, rng);
        rlt::init(device, rng, init_seed);
        NET net;
        typename NET::template Buffer<> buffers;
        OPTIMIZER optimizer;
        rlt::malloc(device, net);
        rlt::malloc(device, buffers);
        rlt::malloc(device, optimizer);
        rlt::init(device, optimizer);
        if(params_in){
            const float* p = params_in;
            for_each_layer(net, [&](auto& layer){ load_layer(device, layer, p); });
        }
        else{
            rlt::init_weights(device, net, rng);
        }
        rlt::zero_gradient(device, net);
        rlt::reset_optimizer_state(device, optimizer, net);
        rlt::Matrix<rlt::matrix::Specification<T, TI, B, I>> input, d_input;
        rlt::Matrix<rlt::matrix::Specification<T, TI, B, O>> output, tgt, d_output;
        rlt::malloc(device, input); rlt::malloc(device, d_input); rlt::malloc(device, output); rlt::malloc(device, tgt); rlt::malloc(device, d_output);
        if(x) for(TI b = 0; b < B; b++) for(TI i = 0; i < I; i++) rlt::set(input, b, i, x[b * I + i]);
        if(target) for(TI b = 0; b < B; b++) for(TI o = 0; o < O; o++) rlt::set(tgt, b, o, target[b * O + o]);
        auto t0 = std::chrono::steady_clock::now();
        if(mode == 0){
            int reps = n_steps > 0 ? n_steps : 1;
            for(int r = 0; r < reps; r++) rlt::evaluate(device, net, input, output, buffers, rng);
        }
        else if(mode == 1){
            rlt::forward(device, net, input, buffers, rng);
            auto out = rlt::output(device, net);
            auto out_m = rlt::matrix_view(device, out);
            rlt::nn::loss_functions::mse::gradient(device, out_m, tgt, d_output, (T)1);
            rlt::backward(device, net, input, d_output, buffers);
        }
        else if(mode == 2){
            for(int s = 0; s < n_steps; s++){
                rlt::zero_gradient(device, net);
                rlt::forward(device, net, input, buffers, rng);
                auto out = rlt::output(device, net);
                auto out_m = rlt::matrix_view(device, out);
                rlt::nn::loss_functions::mse::gradient(device, out_m, tgt, d_output, (T)1);
                rlt::backward(device, net, input, d_output, buffers);
                rlt::step(device, optimizer, net);
            }
        }
        else if(mode == 3){
            rlt::forward(device, net, input, buffers, rng);
            rlt::copy(device, device, tgt, d_output);
            rlt::backward_full(device, net, input, d_output, d_input, buffers);
        }
        auto t1 = std::chrono::steady_clock::now();
        if(seconds) *seconds = std::chrono::duration<double>(t1 - t0).count();
        if(mode == 0){
            if(act_out) for(TI b = 0; b < B; b++) for(TI o = 0; o < O; o++) act_out[b * O + o] = rlt::get(output, b, o);
        }
        else{
            float* pre = pre_out; float* ao = act_out;
            for_each_layer(net, [&](auto& layer){ store_acts(device, layer, pre, ao); });
        }
        if(d_input_out && mode == 3) for(TI b = 0; b < B; b++) for(TI i = 0; i < I; i++) d_input_out[b * I + i] = rlt::get(d_input, b, i);
        float* p;
        p = params_out; for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, PARAMS); });
        p = grads_out;  for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, GRADS); });
        p = m_out;      for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, MOM1); });
        p = v_out;      for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, MOM2); });
        rlt::free(device, input); rlt::free(device, d_input); rlt::free(device, output); rlt::free(device, tgt); rlt::free(device, d_output);
        rlt::free(device, net); rlt::free(device, buffers); rlt::free(device, optimizer);
    }
    // One optimizer step over n_chunks chunks of B rows, the way a data-parallel replica runs it: zero_gradient, then per chunk forward,
    // mse::gradient with weight B / total_rows (so that the chunk gradients add up to the gradient of the whole batch) and backward --
    // gradients accumulate over the chunks -- then, if do_step, one Adam step. pre / act: the LAST chunk's activations.
    static void run_chunked(const float* params_in, const float* x, const float* target, int n_chunks, int total_rows, int do_step,
                            float* params_out, float* grads_out, float* m_out, float* v_out, float* pre_out, float* act_out){
        DEVICE device;
        RNG rng;
        rlt::malloc(device, rng);
        rlt::init(device, rng, 0);
        NET net;
        typename NET::template Buffer<> buffers;
        OPTIMIZER optimizer;
        rlt::malloc(device, net); rlt::malloc(device, buffers); rlt::malloc(device, optimizer);
        rlt::init(device, optimizer);
        { const float* p = params_in; for_each_layer(net, [&](auto& layer){ load_layer(device, layer, p); }); }
        rlt::reset_optimizer_state(device, optimizer, net);
        rlt::Matrix<rlt::matrix::Specification<T, TI, B, I>> input;
        rlt::Matrix<rlt::matrix::Specification<T, TI, B, O>> tgt, d_output;
        rlt::malloc(device, input); rlt::malloc(device, tgt); rlt::malloc(device, d_output);
        rlt::zero_gradient(device, net);
        const T weight = (T)B / (T)total_rows;
        for(int c = 0; c < n_chunks; c++){
            const float* xc = x + (size_t)c * B * I; const float* tc = target + (size_t)c * B * O;
            for(TI b = 0; b < B; b++) for(TI i = 0; i < I; i++) rlt::set(input, b, i, xc[b * I + i]);
            for(TI b = 0; b < B; b++) for(TI o = 0; o < O; o++) rlt::set(tgt, b, o, tc[b * O + o]);
            rlt::forward(device, net, input, buffers, rng);
            auto out = rlt::output(device, net);
            auto out_m = rlt::matrix_view(device, out);
            rlt::nn::loss_functions::mse::gradient(device, out_m, tgt, d_output, weight);
            rlt::backward(device, net, input, d_output, buffers);
        }
        if(do_step) rlt::step(device, optimizer, net);
        { float* pre = pre_out; float* ao = act_out; for_each_layer(net, [&](auto& layer){ store_acts(device, layer, pre, ao); }); }
        float* p;
        p = params_out; for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, PARAMS); });
        p = grads_out;  for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, GRADS); });
        p = m_out;      for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, MOM1); });
        p = v_out;      for_each_layer(net, [&](auto& layer){ store_layer(device, layer, p, MOM2); });
        rlt::free(device, input); rlt::free(device, tgt); rlt::free(device, d_output);
        rlt::free(device, net); rlt::free(device, buffers); rlt::free(device, optimizer);
    }
    static MlpVTable vtable(){
        return MlpVTable{(int)B, (int)I, (int)H, (int)O, (int)NL, (int)HACT, (int)OACT, &run};
    }
};

static int act_to_int(act::ActivationFunction a){
    switch(a){ case act::IDENTITY: return 0; case act::RELU: return 1; case act::TANH: return 2; case act::FAST_TANH: return 3; case act::SIGMOID: return 4; default: return -1; }
}

#define MLP_CASES(X) \
    X(c1_actor_eval,   256,  3,  64,   2, 3, act::RELU, act::IDENTITY) \
    X(c2_actor_b256,   256,  3,  64,   1, 3, act::RELU, act::TANH) \
    X(c3_critic,       256,  4, 256,   1, 3, act::RELU, act::IDENTITY) \
    X(c4_actor_b2048, 2048, 27,  64,   8, 3, act::TANH, act::IDENTITY) \
    X(c4_critic_b2048,2048, 27,  64,   1, 3, act::TANH, act::IDENTITY) \
    X(c5_b1024,       1024, 64, 256,  16, 4, act::RELU, act::IDENTITY) \
    X(sweep_b1,          1, 256, 10, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b2,          2, 256, 10, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b32,        32, 256, 10, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b1024,    1024, 256, 10, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b10,        10, 256,200, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b9,          9, 256, 60, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b200,      200, 256, 11, 100, 3, act::RELU, act::IDENTITY) \
    X(sweep_b64,        64, 256, 50, 101, 3, act::RELU, act::IDENTITY) \
    X(sweep_b256,      256, 256,256, 256, 3, act::RELU, act::IDENTITY) \
    X(tanh_b17,         17,   5, 33,   7, 4, act::TANH, act::TANH) \
    X(fast_tanh_b33,    33,  13, 20,   3, 3, act::FAST_TANH, act::SIGMOID)

static std::map<std::string, MlpVTable>& registry(){
    static std::map<std::string, MlpVTable> r;
    if(r.empty()){
#define X(name, B, I, H, O, NL, HACT, OACT) r[#name] = MlpCase<B, I, H, O, NL, HACT, OACT>::vtable();
        MLP_CASES(X)
#undef X
    }
    return r;
}

// ---------------------------------------------------------------------------------------------------------
// Pendulum + actor rollout with the reference functions (semantics of the off-policy runner's
// prologue / interlude / epilogue for deterministic actions: observe -> evaluate -> step + reward).
// ---------------------------------------------------------------------------------------------------------
template <TI CHUNK>
struct Rollout{
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::TANH>;
    using INPUT_SHAPE = rlt::tensor::Shape<TI, 1, CHUNK, 3>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, rlt::nn::capability::Forward<>, INPUT_SHAPE>;

    // states [N,2] (theta, theta_dot) in/out; episode_step [N] in/out; truncated [N] in/out (uint8);
    // reset_states [R,N,2]: the k-th reset of env e during this call takes reset_states[k][e] (k counts per env).
    // outputs obs [T*N,3], act [T*N,1], rew [T*N,1], row t*N+e.
    static int run(const float* params, TI N, TI Tsteps, float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                   const float* reset_states, TI R, TI step_limit, float* obs, float* actions, float* rew, int num_threads){
        if(N % CHUNK != 0) return -1;
        DEVICE device;
        RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
        NET net; typename NET::template Buffer<> buffers;
        rlt::malloc(device, net); rlt::malloc(device, buffers);
        { const float* p = params;
          load_layer(device, net.input_layer, p); load_layer(device, net.hidden_layers[0], p); load_layer(device, net.output_layer, p); }
        PENDULUM env; typename PENDULUM::Parameters env_params;
        std::vector<TI> reset_count(N, 0);
        int rc = 0;
        for(TI t = 0; t < Tsteps; t++){
            float* obs_t = obs + (size_t)t * N * 3;
            float* act_t = actions + (size_t)t * N;
            float* rew_t = rew + (size_t)t * N;
            auto prologue = [&](TI begin, TI end){
                for(TI e = begin; e < end; e++){
                    if(truncated[e]){
                        if(reset_count[e] >= R){ rc = -2; continue; }
                        states[2 * e + 0] = reset_states[((size_t)reset_count[e] * N + e) * 2 + 0];
                        states[2 * e + 1] = reset_states[((size_t)reset_count[e] * N + e) * 2 + 1];
                        reset_count[e]++;
                        episode_step[e] = 0;
                        episode_return[e] = 0;
                    }
                    typename PENDULUM::State s; s.theta = states[2 * e]; s.theta_dot = states[2 * e + 1];
                    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 3, false>> o;
                    rlt::observe(device, env, env_params, s, typename PENDULUM::Observation{}, o, rng);
                    for(TI k = 0; k < 3; k++) obs_t[3 * e + k] = rlt::get(o, 0, k);
                }
            };
            auto epilogue = [&](TI begin, TI end){
                for(TI e = begin; e < end; e++){
                    typename PENDULUM::State s, ns; s.theta = states[2 * e]; s.theta_dot = states[2 * e + 1];
                    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 1, false>> a;
                    rlt::set(a, 0, 0, act_t[e]);
                    rlt::step(device, env, env_params, s, a, ns, rng);
                    T r = rlt::reward(device, env, env_params, s, a, ns, rng);
                    bool terminated_flag = rlt::terminated(device, env, env_params, ns, rng);
                    episode_step[e] += 1;
                    episode_return[e] += r;
                    truncated[e] = terminated_flag || ((TI)episode_step[e] == step_limit);
                    rew_t[e] = r;
                    states[2 * e] = ns.theta; states[2 * e + 1] = ns.theta_dot;
                }
            };
            auto fan_out = [&](auto& f){
                if(num_threads <= 1){ f(0, N); return; }
                std::vector<std::thread> threads;
                TI per = (N + num_threads - 1) / num_threads;
                for(int th = 0; th < num_threads; th++){
                    TI b = th * per, e = std::min<TI>(N, b + per);
                    if(b < e) threads.emplace_back([&f, b, e](){ f(b, e); });
                }
                for(auto& th: threads) th.join();
            };
            fan_out(prologue);
            for(TI c = 0; c < N; c += CHUNK){
                rlt::Matrix<rlt::matrix::Specification<T, TI, CHUNK, 3, true, rlt::matrix::layouts::RowMajorAlignment<TI, 1>>> in;
                rlt::Matrix<rlt::matrix::Specification<T, TI, CHUNK, 1, true, rlt::matrix::layouts::RowMajorAlignment<TI, 1>>> out;
                in._data = obs_t + (size_t)c * 3;
                out._data = act_t + c;
                rlt::evaluate(device, net, in, out, buffers, rng);
            }
            fan_out(epilogue);
        }
        rlt::free(device, net); rlt::free(device, buffers);
        return rc;
    }
};

// GAE through the reference's own Dataset + estimate_generalized_advantages (rl/algorithms/ppo/operations_generic.h:59-95)
template <TI N, TI STEPS>
static void gae_case(const float* rewards, const float* all_values, const uint8_t* terminated, const uint8_t* truncated, float* advantages, float* target_values){
    using RUNNER_SPEC = rlt::rl::components::on_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, bool, N>;
    using DATASET_SPEC = rlt::rl::components::on_policy_runner::DatasetSpecification<RUNNER_SPEC, STEPS>;
    using PARAMETERS = rlt::rl::algorithms::ppo::DefaultParameters<TYPE_POLICY, TI, 64>;
    DEVICE device;
    rlt::rl::components::on_policy_runner::Dataset<DATASET_SPEC> dataset;
    rlt::malloc(device, dataset);
    for(TI i = 0; i < STEPS * N; i++){
        rlt::set(dataset.rewards, i, 0, rewards[i]); rlt::set(dataset.terminated, i, 0, (T)terminated[i]); rlt::set(dataset.truncated, i, 0, (T)truncated[i]);
    }
    for(TI i = 0; i < (STEPS + 1) * N; i++) rlt::set(dataset.all_values, i, 0, all_values[i]);
    rlt::estimate_generalized_advantages(device, dataset, PARAMETERS{});
    for(TI i = 0; i < STEPS * N; i++){ advantages[i] = rlt::get(dataset.advantages, i, 0); target_values[i] = rlt::get(dataset.target_values, i, 0); }
    rlt::free(device, dataset);
}

// On-policy collect through the reference's own runner (rl/components/on_policy_runner/operations_generic.h:69-146,
// operations_generic_per_env.h:9-79) with the PPO actor type (rl/algorithms/ppo/loop/core/config.h:54-67 without the
// identity standardisation layer): sequential< mlp_unconditional_stddev 3 -> 64 -> 64 -> 1 >.
// actor_params: W1 b1 W2 b2 W3 b3 log_std (flat). datasets receives n_collects x [(STEPS+1)*N, 13] (the whole data matrix
// after each collect, zero-initialised before the first).
template <TI N, TI STEPS, TI STEP_LIMIT, act::ActivationFunction HACT>
static void collect_case(const float* actor_params, uint32_t seed, int n_collects, float* datasets, float* states_out, int32_t* episode_step_out,
                         uint8_t* truncated_out, float* episode_return_out, uint64_t* runner_step_out){
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, HACT, act::IDENTITY>;
    using ACTOR_MLP = rlt::nn_models::mlp_unconditional_stddev::BindConfiguration<ACTOR_CONFIG>;
    using MODULE_CHAIN = rlt::nn_models::sequential::Module<ACTOR_MLP>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, MODULE_CHAIN, rlt::tensor::Shape<TI, 1, N, 3>>;
    using RUNNER_SPEC = rlt::rl::components::on_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, typename ACTOR::template State<>, N, STEP_LIMIT>;
    using RUNNER = rlt::rl::components::OnPolicyRunner<RUNNER_SPEC>;
    using DATASET_SPEC = rlt::rl::components::on_policy_runner::DatasetSpecification<RUNNER_SPEC, STEPS>;
    using DATASET = rlt::rl::components::on_policy_runner::Dataset<DATASET_SPEC>;
    static_assert(DATASET::DATA_DIM == 13);
    DEVICE device;
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    ACTOR actor; typename ACTOR::template Buffer<> buffers; RUNNER runner; DATASET dataset;
    rlt::malloc(device, actor); rlt::malloc(device, buffers); rlt::malloc(device, runner); rlt::malloc(device, dataset);
    { const float* p = actor_params;
      auto& mlp = actor.content;
      load_layer(device, mlp.input_layer, p); load_layer(device, mlp.hidden_layers[0], p); load_layer(device, mlp.output_layer, p);
      rlt::set(device, mlp.log_std.parameters, p[0], 0); }
    rlt::Tensor<rlt::tensor::Specification<PENDULUM, TI, rlt::tensor::Shape<TI, N>>> envs;
    rlt::Tensor<rlt::tensor::Specification<typename PENDULUM::Parameters, TI, rlt::tensor::Shape<TI, N>>> env_parameters;
    rlt::malloc(device, envs); rlt::malloc(device, env_parameters);
    rlt::set_all(device, dataset.data, 0);
    rlt::init(device, runner, envs, env_parameters, actor, rng);
    constexpr size_t DS = (size_t)(STEPS + 1) * N * 13;
    for(int c = 0; c < n_collects; c++){
        rlt::collect(device, dataset, runner, actor, buffers, rng);
        for(TI r = 0; r < (STEPS + 1) * N; r++) for(TI k = 0; k < 13; k++) datasets[c * DS + r * 13 + k] = rlt::get(dataset.data, r, k);
    }
    for(TI e = 0; e < N; e++){
        auto& st = rlt::get(runner.states, 0, e);
        states_out[2 * e] = st.theta; states_out[2 * e + 1] = st.theta_dot;
        episode_step_out[e] = (int32_t)rlt::get(runner.episode_step, 0, e);
        truncated_out[e] = rlt::get(runner.truncated, 0, e) ? 1 : 0;
        episode_return_out[e] = rlt::get(runner.episode_return, 0, e);
    }
    *runner_step_out = runner.step;
    rlt::free(device, envs); rlt::free(device, env_parameters);
    rlt::free(device, actor); rlt::free(device, buffers); rlt::free(device, runner); rlt::free(device, dataset);
}

// PPO update through the reference's own train() (rl/algorithms/ppo/operations_generic.h:96-336) on a caller-provided dataset matrix:
// EPOCHS x (STEPS_TOTAL / BATCH) minibatches, no shuffling, default PPO parameters otherwise (ppo.h:13-38), Adam with the TF defaults.
// Actor = sequential<mlp_unconditional_stddev 3->64->64->1>, critic = sequential<mlp 3->64->64->1>, both ReLU / identity.
// Outputs after the call: parameters, and the gradient and Adam first moment left by the LAST minibatch, actor (4482 = MLP arena +
// log_std) and critic (4481).
template <TI BATCH, TI EPOCHS, bool SHUFFLE>
struct PpoTrainParameters: rlt::rl::algorithms::ppo::DefaultParameters<TYPE_POLICY, TI, BATCH>{
    static constexpr TI N_EPOCHS = EPOCHS;
    static constexpr bool SHUFFLE_EPOCH = SHUFFLE;
};
// SHUFFLE: the reference's per-epoch in-place row shuffle (operations_generic.h:127-158) driven by the engine seeded with `seed`;
// dataset_out receives the matrix as train() leaves it (rows of the shuffled columns permuted).
// Shapes of the Ant PPO configuration (observation 27, action 8) as a type: train() and the dataset only read these constants.
struct AntLike{
    struct Observation{ static constexpr TI DIM = 27; };
    using ObservationPrivileged = Observation;
    static constexpr TI ACTION_DIM = 8;
    static constexpr TI N_AGENTS = 1;
    static constexpr TI EPISODE_STEP_LIMIT = 1000;
    struct Parameters{}; struct State{};
};
// Generic in the environment type: the dataset has OBS + 2 * ACT + 8 columns, the actor arena is the MLP OBS -> 64 -> 64 -> ACT followed
// by log_std[ACT], the critic OBS -> 64 -> 64 -> 1. seconds (may be null) receives the wall time of train() alone.
template <typename ENV, act::ActivationFunction HACT, TI N, TI STEPS, TI BATCH, TI EPOCHS, bool SHUFFLE>
static void ppo_train_case(const float* actor_params, const float* critic_params, const float* dataset_in, uint32_t seed, float* actor_out, float* actor_grad, float* actor_m,
                           float* critic_out, float* critic_grad, float* critic_m, float* dataset_out, double* seconds){
    constexpr TI OBS = ENV::Observation::DIM, ACT = ENV::ACTION_DIM, D = OBS + 2 * ACT + 8;
    constexpr TI N_ACTOR = OBS * 64 + 64 + 64 * 64 + 64 + 64 * ACT + ACT;
    using CAPABILITY = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using INPUT_SHAPE = rlt::tensor::Shape<TI, 1, BATCH, OBS>;
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, ACT, 3, 64, HACT, act::IDENTITY>;
    using CRITIC_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, HACT, act::IDENTITY>;
    using ACTOR = rlt::nn_models::sequential::Build<CAPABILITY, rlt::nn_models::sequential::Module<rlt::nn_models::mlp_unconditional_stddev::BindConfiguration<ACTOR_CONFIG>>, INPUT_SHAPE>;
    using CRITIC = rlt::nn_models::sequential::Build<CAPABILITY, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<CRITIC_CONFIG>>, INPUT_SHAPE>;
    using PARAMETERS = PpoTrainParameters<BATCH, EPOCHS, SHUFFLE>;
    using PPO_SPEC = rlt::rl::algorithms::ppo::Specification<TYPE_POLICY, TI, ENV, ACTOR, CRITIC, PARAMETERS>;
    using PPO = rlt::rl::algorithms::PPO<PPO_SPEC>;
    using PPO_BUFFERS = rlt::rl::algorithms::ppo::Buffers<rlt::rl::algorithms::ppo::BufferSpecification<PPO_SPEC>>;
    using RUNNER_SPEC = rlt::rl::components::on_policy_runner::Specification<TYPE_POLICY, TI, ENV, typename ACTOR::template State<>, N, 100>;
    using DATASET = rlt::rl::components::on_policy_runner::Dataset<rlt::rl::components::on_policy_runner::DatasetSpecification<RUNNER_SPEC, STEPS>>;
    static_assert(DATASET::DATA_DIM == D);
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    DEVICE device;
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    RNG train_rng; rlt::malloc(device, train_rng); rlt::init(device, train_rng, seed);
    PPO ppo; PPO_BUFFERS ppo_buffers; DATASET dataset; OPTIMIZER actor_optimizer, critic_optimizer;
    typename ACTOR::template Buffer<> actor_buffers; typename CRITIC::template Buffer<> critic_buffers;
    rlt::malloc(device, ppo); rlt::malloc(device, ppo_buffers); rlt::malloc(device, dataset); rlt::malloc(device, actor_optimizer); rlt::malloc(device, critic_optimizer);
    rlt::malloc(device, actor_buffers); rlt::malloc(device, critic_buffers);
    rlt::init(device, ppo, actor_optimizer, critic_optimizer, rng);
    { const float* p = actor_params; auto& m = ppo.actor.content;
      load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p);
      for(TI a = 0; a < ACT; a++) rlt::set(device, m.log_std.parameters, p[a], a); }
    { const float* p = critic_params; auto& m = ppo.critic.content;
      load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
    for(TI r = 0; r < (STEPS + 1) * N; r++) for(TI k = 0; k < D; k++) rlt::set(dataset.data, r, k, dataset_in[r * D + k]);
    auto t0 = std::chrono::steady_clock::now();
    rlt::train(device, ppo, dataset, actor_optimizer, critic_optimizer, ppo_buffers, actor_buffers, critic_buffers, train_rng);
    if(seconds) *seconds = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
    if(dataset_out) for(TI r = 0; r < (STEPS + 1) * N; r++) for(TI k = 0; k < D; k++) dataset_out[r * D + k] = rlt::get(dataset.data, r, k);
    auto dump = [&](auto& m, float* params, float* grads, float* mom){
        store_layer(device, m.input_layer, params, PARAMS); store_layer(device, m.hidden_layers[0], params, PARAMS); store_layer(device, m.output_layer, params, PARAMS);
        store_layer(device, m.input_layer, grads, GRADS); store_layer(device, m.hidden_layers[0], grads, GRADS); store_layer(device, m.output_layer, grads, GRADS);
        store_layer(device, m.input_layer, mom, MOM1); store_layer(device, m.hidden_layers[0], mom, MOM1); store_layer(device, m.output_layer, mom, MOM1);
    };
    dump(ppo.actor.content, actor_out, actor_grad, actor_m);
    for(TI a = 0; a < ACT; a++){
        actor_out[N_ACTOR + a] = rlt::get(device, ppo.actor.content.log_std.parameters, a);
        actor_grad[N_ACTOR + a] = rlt::get(device, ppo.actor.content.log_std.gradient, a);
        actor_m[N_ACTOR + a] = rlt::get(device, ppo.actor.content.log_std.gradient_first_order_moment, a);
    }
    dump(ppo.critic.content, critic_out, critic_grad, critic_m);
    rlt::free(device, ppo); rlt::free(device, ppo_buffers); rlt::free(device, dataset); rlt::free(device, actor_optimizer); rlt::free(device, critic_optimizer);
    rlt::free(device, actor_buffers); rlt::free(device, critic_buffers);
}

// Off-policy runner through the reference's own OffPolicyRunner (rl/components/off_policy_runner/operations_generic.h:47-69,162-238,
// operations_generic_per_env.h:8-108; replay buffer rl/components/replay_buffer/operations_generic.h:54-85): n_steps x step<0> with a
// deterministic actor sequential<mlp 3 -> 64 -> 64 -> 1, ReLU / tanh>. Outputs per environment: the replay buffer's data matrix
// [CAPACITY, 10] (observation 3, action 1, reward 1, next observation 3, terminated, truncated), episode_start [CAPACITY], states and
// next_states [CAPACITY, 2], and (position, full, current_episode_start); plus the runner state and the runner's step buffers.
template <TI T_N, TI T_CAPACITY, TI T_LIMIT>
struct OffPolicyParameters: rlt::rl::components::off_policy_runner::ParametersDefault<TYPE_POLICY, TI>{
    static constexpr TI N_ENVIRONMENTS = T_N;
    static constexpr TI REPLAY_BUFFER_CAPACITY = T_CAPACITY;
    static constexpr TI EPISODE_STEP_LIMIT = T_LIMIT;
};
template <TI N, TI CAPACITY, TI LIMIT>
static void offpolicy_case(const float* actor_params, uint32_t seed, int n_steps, float* replay_data, int64_t* episode_start, float* replay_states, float* replay_next_states,
                           int64_t* counters, float* states_out, int32_t* episode_step_out, uint8_t* truncated_out, float* episode_return_out,
                           float* buf_obs, float* buf_act, float* buf_next_obs){
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::TANH>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<ACTOR_CONFIG>>, rlt::tensor::Shape<TI, 1, N, 3>>;
    using POLICIES = rlt::utils::Tuple<TI, ACTOR>;
    using SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, POLICIES, OffPolicyParameters<N, CAPACITY, LIMIT>>;
    using RUNNER = rlt::rl::components::OffPolicyRunner<SPEC>;
    DEVICE device;
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    ACTOR actor; typename ACTOR::template Buffer<> buffers;
    rlt::malloc(device, actor); rlt::malloc(device, buffers);
    { const float* p = actor_params; auto& m = actor.content;
      load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
    RUNNER* runner = new RUNNER();                       // the replay buffers are statically allocated inside the runner's matrices
    rlt::malloc(device, *runner);
    rlt::init(device, *runner);
    for(int s = 0; s < n_steps; s++) rlt::step<0>(device, *runner, actor, buffers, rng);
    for(TI e = 0; e < N; e++){
        auto& rb = rlt::get(runner->replay_buffers, 0, e);
        for(TI r = 0; r < CAPACITY; r++){
            for(TI k = 0; k < 10; k++) replay_data[((size_t)e * CAPACITY + r) * 10 + k] = rlt::get(rb.data, r, k);
            episode_start[(size_t)e * CAPACITY + r] = (int64_t)rlt::get(device, rb.episode_start, r);
            const auto& st = rlt::get(rb.states, r, 0); const auto& ns = rlt::get(rb.next_states, r, 0);
            replay_states[((size_t)e * CAPACITY + r) * 2] = st.theta; replay_states[((size_t)e * CAPACITY + r) * 2 + 1] = st.theta_dot;
            replay_next_states[((size_t)e * CAPACITY + r) * 2] = ns.theta; replay_next_states[((size_t)e * CAPACITY + r) * 2 + 1] = ns.theta_dot;
        }
        counters[3 * e] = (int64_t)rb.position; counters[3 * e + 1] = rb.full ? 1 : 0; counters[3 * e + 2] = (int64_t)rb.current_episode_start;
        const auto& st = rlt::get(runner->states, 0, e);
        states_out[2 * e] = st.theta; states_out[2 * e + 1] = st.theta_dot;
        episode_step_out[e] = (int32_t)rlt::get(runner->episode_step, 0, e);
        truncated_out[e] = rlt::get(runner->truncated, 0, e) ? 1 : 0;
        episode_return_out[e] = rlt::get(runner->episode_return, 0, e);
        for(TI k = 0; k < 3; k++){ buf_obs[3 * e + k] = rlt::get(runner->buffers.observations, e, k); buf_next_obs[3 * e + k] = rlt::get(runner->buffers.next_observations, e, k); }
        buf_act[e] = rlt::get(runner->buffers.actions, e, 0);
    }
    rlt::free(device, *runner); delete runner;
    rlt::free(device, actor); rlt::free(device, buffers);
}

// Replay-buffer sampling through the reference's own gather_batch (rl/components/off_policy_runner/operations_generic.h:239-423) with
// SEQUENCE_LENGTH 1 (the Markovian default: no random sequence lengths, no sampling from the initial state): n_steps x step<0> on a fresh
// runner, then n_gathers x gather_batch on the same engine. Per gather: observations_actions_base [2, BATCH, 4], rewards [BATCH],
// terminated / reset / final_step_mask [BATCH], next_reset_base / next_final_step_mask_base [2, BATCH].
template <TI N, TI CAPACITY, TI LIMIT, TI BATCH>
static void gather_case(const float* actor_params, uint32_t seed, int n_steps, int n_gathers, float* oa_base, float* rewards, uint8_t* terminated, uint8_t* reset,
                        uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, uint32_t* next_draw){
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::TANH>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<ACTOR_CONFIG>>, rlt::tensor::Shape<TI, 1, N, 3>>;
    using POLICIES = rlt::utils::Tuple<TI, ACTOR>;
    using SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, POLICIES, OffPolicyParameters<N, CAPACITY, LIMIT>>;
    using RUNNER = rlt::rl::components::OffPolicyRunner<SPEC>;
    using BATCH_SPEC = rlt::rl::components::off_policy_runner::SequentialBatchSpecification<SPEC, 1, BATCH>;
    using BATCH_TYPE = rlt::rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>;
    DEVICE device;
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    ACTOR actor; typename ACTOR::template Buffer<> buffers;
    rlt::malloc(device, actor); rlt::malloc(device, buffers);
    { const float* p = actor_params; auto& m = actor.content;
      load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
    RUNNER* runner = new RUNNER();
    BATCH_TYPE batch;
    rlt::malloc(device, *runner); rlt::malloc(device, batch);
    rlt::init(device, *runner);
    for(int s = 0; s < n_steps; s++) rlt::step<0>(device, *runner, actor, buffers, rng);
    for(int g = 0; g < n_gathers; g++){
        rlt::gather_batch(device, *runner, batch, rng);
        for(TI q = 0; q < 2; q++) for(TI b = 0; b < BATCH; b++){
            for(TI k = 0; k < 4; k++) oa_base[(((size_t)g * 2 + q) * BATCH + b) * 4 + k] = rlt::get(device, batch.observations_actions_base, q, b, k);
            next_reset_base[((size_t)g * 2 + q) * BATCH + b] = rlt::get(device, batch.next_reset_base, q, b, 0) ? 1 : 0;
            next_final_step_mask_base[((size_t)g * 2 + q) * BATCH + b] = rlt::get(device, batch.next_final_step_mask_base, q, b, 0) ? 1 : 0;
        }
        for(TI b = 0; b < BATCH; b++){
            rewards[(size_t)g * BATCH + b] = rlt::get(device, batch.rewards, 0, b, 0);
            terminated[(size_t)g * BATCH + b] = rlt::get(device, batch.terminated, 0, b, 0) ? 1 : 0;
            reset[(size_t)g * BATCH + b] = rlt::get(device, batch.reset, 0, b, 0) ? 1 : 0;
            final_step_mask[(size_t)g * BATCH + b] = rlt::get(device, batch.final_step_mask, 0, b, 0) ? 1 : 0;
        }
    }
    if(next_draw) *next_draw = (uint32_t)rng.engine();      // where the engine stands afterwards
    rlt::free(device, *runner); delete runner; rlt::free(device, batch);
    rlt::free(device, actor); rlt::free(device, buffers);
}

// The same through gather_batch for sequences: SequentialBatch with SEQUENCE_LENGTH = SEQ and its sampling parameters switched by MODE bits
// (1 = ALWAYS_SAMPLE_FROM_INITIAL_STATE, 2 = RANDOM_SEQ_LENGTH, 8 = the DETERMINISTIC template flag of gather_batch; INCLUDE_FIRST_STEP_IN_TARGETS
// keeps its default, SEQ > 1). Outputs per gather: observations_actions_base [SEQ + 1, BATCH, 4], rewards / terminated / reset / final_step_mask
// [SEQ, BATCH], next_reset_base / next_final_step_mask_base [SEQ + 1, BATCH]. The batch tensors are zeroed before every gather (the reference
// leaves entries behind a sequence's end unwritten).
template <TI SEQ, int MODE>
struct SeqBatchParameters: rlt::rl::components::off_policy_runner::SequentialBatchParameters<TYPE_POLICY, TI, SEQ>{
    static constexpr bool ALWAYS_SAMPLE_FROM_INITIAL_STATE = (MODE & 1) != 0;
    static constexpr bool RANDOM_SEQ_LENGTH = (MODE & 2) != 0;
};
template <TI N, TI CAPACITY, TI LIMIT, TI BATCH, TI SEQ, int MODE>
static void gather_seq_case(const float* actor_params, uint32_t seed, int n_steps, int n_gathers, float* oa_base, float* rewards, uint8_t* terminated, uint8_t* reset,
                            uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, uint32_t* next_draw){
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::TANH>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<ACTOR_CONFIG>>, rlt::tensor::Shape<TI, 1, N, 3>>;
    using POLICIES = rlt::utils::Tuple<TI, ACTOR>;
    using SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, POLICIES, OffPolicyParameters<N, CAPACITY, LIMIT>>;
    using RUNNER = rlt::rl::components::OffPolicyRunner<SPEC>;
    using BATCH_SPEC = rlt::rl::components::off_policy_runner::SequentialBatchSpecification<SPEC, SEQ, BATCH, SeqBatchParameters<SEQ, MODE>>;
    using BATCH_TYPE = rlt::rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>;
    constexpr TI P = SEQ + 1;
    DEVICE device;
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    ACTOR actor; typename ACTOR::template Buffer<> buffers;
    rlt::malloc(device, actor); rlt::malloc(device, buffers);
    { const float* p = actor_params; auto& m = actor.content;
      load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
    RUNNER* runner = new RUNNER();
    BATCH_TYPE batch;
    rlt::malloc(device, *runner); rlt::malloc(device, batch);
    rlt::init(device, *runner);
    for(int s = 0; s < n_steps; s++) rlt::step<0>(device, *runner, actor, buffers, rng);
    for(int g = 0; g < n_gathers; g++){
        rlt::set_all(device, batch.observations_actions_base, 0); rlt::set_all(device, batch.rewards, 0); rlt::set_all(device, batch.terminated, false);
        rlt::gather_batch<DEVICE, SPEC, BATCH_SPEC, RNG, (MODE & 8) != 0>(device, *runner, batch, rng);
        for(TI q = 0; q < P; q++) for(TI b = 0; b < BATCH; b++){
            for(TI k = 0; k < 4; k++) oa_base[(((size_t)g * P + q) * BATCH + b) * 4 + k] = rlt::get(device, batch.observations_actions_base, q, b, k);
            next_reset_base[((size_t)g * P + q) * BATCH + b] = rlt::get(device, batch.next_reset_base, q, b, 0) ? 1 : 0;
            next_final_step_mask_base[((size_t)g * P + q) * BATCH + b] = rlt::get(device, batch.next_final_step_mask_base, q, b, 0) ? 1 : 0;
        }
        for(TI q = 0; q < SEQ; q++) for(TI b = 0; b < BATCH; b++){
            rewards[((size_t)g * SEQ + q) * BATCH + b] = rlt::get(device, batch.rewards, q, b, 0);
            terminated[((size_t)g * SEQ + q) * BATCH + b] = rlt::get(device, batch.terminated, q, b, 0) ? 1 : 0;
            reset[((size_t)g * SEQ + q) * BATCH + b] = rlt::get(device, batch.reset, q, b, 0) ? 1 : 0;
            final_step_mask[((size_t)g * SEQ + q) * BATCH + b] = rlt::get(device, batch.final_step_mask, q, b, 0) ? 1 : 0;
        }
    }
    if(next_draw) *next_draw = (uint32_t)rng.engine();
    rlt::free(device, *runner); delete runner; rlt::free(device, batch);
    rlt::free(device, actor); rlt::free(device, buffers);
}

// The SAC policy head on its own: nn::layers::sample_and_squash LayerGradient forward (external noise) and backward_full
// (nn/layers/sample_and_squash/operations_generic.h:212-280, 290-398) on a [B, 2A] input. log_alpha_gradient_out = the layer's log_alpha gradient
// after one backward from a zeroed gradient.
template <TI B, TI A>
static void sas_case(const float* input, const float* noise, const float* d_output, float log_alpha, float* pre_squashing, float* output, float* log_probs,
                     float* d_input, float* d_log_alpha_per_sample, float* log_alpha_gradient_out){
    using CONFIG = rlt::nn::layers::sample_and_squash::Configuration<TYPE_POLICY, TI>;
    using CAPABILITY = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using LAYER = rlt::nn::layers::sample_and_squash::Layer<CONFIG, CAPABILITY, rlt::tensor::Shape<TI, 1, B, 2 * A>>;
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    LAYER layer; typename LAYER::template Buffer<> buffer;
    rlt::malloc(device, layer); rlt::malloc(device, buffer);
    rlt::init_weights(device, layer, rng); rlt::zero_gradient(device, layer);
    rlt::set(device, layer.log_alpha.parameters, log_alpha, 0);
    rlt::Matrix<rlt::matrix::Specification<T, TI, B, 2 * A>> in, din;
    rlt::Matrix<rlt::matrix::Specification<T, TI, B, A>> dout;
    rlt::malloc(device, in); rlt::malloc(device, din); rlt::malloc(device, dout);
    for(TI b = 0; b < B; b++){
        for(TI k = 0; k < 2 * A; k++) rlt::set(in, b, k, input[b * 2 * A + k]);
        for(TI k = 0; k < A; k++){ rlt::set(dout, b, k, d_output[b * A + k]); rlt::set(buffer.noise, b, k, noise[b * A + k]); }
    }
    rlt::Mode<rlt::nn::layers::sample_and_squash::mode::ExternalNoise<rlt::mode::Default<>>> mode;
    rlt::forward(device, layer, in, buffer, rng, mode);
    rlt::backward_full(device, layer, in, dout, din, buffer, mode);
    for(TI b = 0; b < B; b++){
        for(TI k = 0; k < A; k++){ pre_squashing[b * A + k] = rlt::get(layer.pre_squashing, b, k); output[b * A + k] = rlt::get(layer.output, b, k); }
        for(TI k = 0; k < 2 * A; k++) d_input[b * 2 * A + k] = rlt::get(din, b, k);
        log_probs[b] = rlt::get(layer.log_probabilities, 0, b);
        d_log_alpha_per_sample[b] = rlt::get(buffer.d_log_alpha, 0, b);
    }
    *log_alpha_gradient_out = rlt::get(device, layer.log_alpha.gradient, 0);
    rlt::free(device, layer); rlt::free(device, buffer); rlt::free(device, in); rlt::free(device, din); rlt::free(device, dout);
}
// SAC update through the reference's own train_critic / update_critic_targets / train_actor (rl/algorithms/sac/operations_generic.h:223-336,
// 486-522, 378-456) with the default SAC parameters (gamma 0.99, entropy bonus on the next step, masking of non-terminal steps, target entropy
// -ACTION_DIM, Polyak 0.995) on hand-filled SequentialBatch tensors of sequence length 1: per update critic 0, critic 1 (same batch, own noise),
// target update, actor. Networks: actor sequential<mlp 3 -> H -> H -> 2, sample_and_squash>, critics sequential<mlp 4 -> H -> H -> 1>, ReLU.
// Parameter arrays are W1 b1 W2 b2 W3 b3 per network; outputs are the same arrays after the updates plus gradients / first moments.
template <TI T_BATCH>
struct SacCaseParameters: rlt::rl::algorithms::sac::DefaultParameters<TYPE_POLICY, TI, 1>{
    static constexpr TI ACTOR_BATCH_SIZE = T_BATCH;
    static constexpr TI CRITIC_BATCH_SIZE = T_BATCH;
};
template <typename SAC_PARAMETERS>
struct SacCaseHeadParameters{
    static constexpr T LOG_STD_LOWER_BOUND = SAC_PARAMETERS::LOG_STD_LOWER_BOUND, LOG_STD_UPPER_BOUND = SAC_PARAMETERS::LOG_STD_UPPER_BOUND;
    static constexpr T LOG_PROBABILITY_EPSILON = SAC_PARAMETERS::LOG_PROBABILITY_EPSILON, ALPHA = SAC_PARAMETERS::ALPHA, TARGET_ENTROPY = SAC_PARAMETERS::TARGET_ENTROPY;
    static constexpr bool ADAPTIVE_ALPHA = SAC_PARAMETERS::ADAPTIVE_ALPHA, UPDATE_ALPHA_WITH_ACTOR = false;
};
template <typename LAYER>
static void store_parameters_only(DEVICE& device, LAYER& layer, float*& p){        // for networks without gradient members
    for(TI o = 0; o < LAYER::OUTPUT_DIM; o++) for(TI i = 0; i < LAYER::INPUT_DIM; i++) *p++ = rlt::get(device, layer.weights.parameters, o, i);
    for(TI o = 0; o < LAYER::OUTPUT_DIM; o++) *p++ = rlt::get(device, layer.biases.parameters, o);
}
template <TI BATCH, TI HIDDEN>
static void sac_case(int n_updates, const float* actor_params, float log_alpha, const float* critic_params /*[2]*/, const float* target_params /*[2]*/,
                     const float* oa_base /*[U,2,B,4]*/, const float* rewards /*[U,B]*/, const uint8_t* terminated /*[U,B]*/, const float* noise_critic /*[U,2,B,1]*/,
                     const float* noise_actor /*[U,B,1]*/, float* actor_out /*[3][n]*/, float* log_alpha_out /*[3]*/, float* critic_out /*[2][3][n]*/, float* target_out /*[2][n]*/,
                     float* target_values_out /*[B] of the last critic update*/){
    using SAC_PARAMETERS = SacCaseParameters<BATCH>;
    using ACTOR_MLP = rlt::nn_models::mlp::BindConfiguration<rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 2, 3, HIDDEN, act::RELU, act::IDENTITY>>;
    using SAS_PARAMETERS = SacCaseHeadParameters<SAC_PARAMETERS>;
    using SAS = rlt::nn::layers::sample_and_squash::BindConfiguration<rlt::nn::layers::sample_and_squash::Configuration<TYPE_POLICY, TI, SAS_PARAMETERS>>;
    using CAP_GRADIENT = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using ACTOR = rlt::nn_models::sequential::Build<CAP_GRADIENT, rlt::nn_models::sequential::Module<ACTOR_MLP, rlt::nn_models::sequential::Module<SAS>>, rlt::tensor::Shape<TI, 1, BATCH, 3>>;
    using CRITIC_MLP = rlt::nn_models::mlp::BindConfiguration<rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, HIDDEN, act::RELU, act::IDENTITY>>;
    using CRITIC = rlt::nn_models::sequential::Build<CAP_GRADIENT, rlt::nn_models::sequential::Module<CRITIC_MLP>, rlt::tensor::Shape<TI, 1, BATCH, 4>>;
    using CRITIC_TARGET = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<CRITIC_MLP>, rlt::tensor::Shape<TI, 1, BATCH, 4>>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    using AC_SPEC = rlt::rl::algorithms::sac::Specification<TYPE_POLICY, TI, PENDULUM, ACTOR, CRITIC, CRITIC_TARGET, rlt::nn::parameters::Adam, OPTIMIZER, OPTIMIZER, OPTIMIZER, SAC_PARAMETERS, false>;
    using ACTOR_CRITIC = rlt::rl::algorithms::sac::ActorCritic<AC_SPEC>;
    using EVAL_ACTOR = typename ACTOR::template CHANGE_BATCH_SIZE<TI, 4>;
    using RUNNER_SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, rlt::utils::Tuple<TI, EVAL_ACTOR>, OffPolicyParameters<4, 16, 200>>;
    using BATCH_TYPE = rlt::rl::components::off_policy_runner::SequentialBatch<rlt::rl::components::off_policy_runner::SequentialBatchSpecification<RUNNER_SPEC, 1, BATCH>>;
    using CRITIC_TRAINING_BUFFERS = rlt::rl::algorithms::sac::CriticTrainingBuffers<rlt::rl::algorithms::sac::CriticTrainingBuffersSpecification<AC_SPEC, true>>;
    using ACTOR_TRAINING_BUFFERS = rlt::rl::algorithms::sac::ActorTrainingBuffers<rlt::rl::algorithms::sac::ActorTrainingBuffersSpecification<AC_SPEC, true>>;
    constexpr TI N_ACTOR = 3 * HIDDEN + HIDDEN + HIDDEN * HIDDEN + HIDDEN + HIDDEN * 2 + 2, N_CRITIC = 4 * HIDDEN + HIDDEN + HIDDEN * HIDDEN + HIDDEN + HIDDEN + 1;
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    auto* ac = new ACTOR_CRITIC();
    BATCH_TYPE batch; CRITIC_TRAINING_BUFFERS ctb; ACTOR_TRAINING_BUFFERS atb;
    typename ACTOR::template Buffer<> actor_buffers, actor_target_buffers; typename CRITIC::template Buffer<> critic_buffers; typename CRITIC_TARGET::template Buffer<> critic_target_buffers;
    rlt::Matrix<rlt::matrix::Specification<T, TI, BATCH, 1>> action_noise_critic, action_noise_actor;
    rlt::malloc(device, *ac); rlt::malloc(device, batch); rlt::malloc(device, ctb); rlt::malloc(device, atb);
    rlt::malloc(device, actor_buffers); rlt::malloc(device, actor_target_buffers); rlt::malloc(device, critic_buffers); rlt::malloc(device, critic_target_buffers);
    rlt::malloc(device, action_noise_critic); rlt::malloc(device, action_noise_actor);
    rlt::init(device, *ac, rng);
    { const float* p = actor_params; auto& m = ac->actor.content;
      load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
    rlt::set(device, rlt::get_last_layer(ac->actor).log_alpha.parameters, log_alpha, 0);
    for(int c = 0; c < 2; c++){
        { const float* p = critic_params + c * N_CRITIC; auto& m = ac->critics[c].content;
          load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
        { const float* p = target_params + c * N_CRITIC; auto& m = ac->critics_target[c].content;
          load_layer(device, m.input_layer, p); load_layer(device, m.hidden_layers[0], p); load_layer(device, m.output_layer, p); }
    }
    for(int u = 0; u < n_updates; u++){
        for(TI q = 0; q < 2; q++) for(TI b = 0; b < BATCH; b++){
            for(TI k = 0; k < 4; k++) rlt::set(device, batch.observations_actions_base, oa_base[(((size_t)u * 2 + q) * BATCH + b) * 4 + k], q, b, k);
            rlt::set(device, batch.next_reset_base, true, q, b, 0);
            rlt::set(device, batch.next_final_step_mask_base, q == 1, q, b, 0);
        }
        for(TI b = 0; b < BATCH; b++){
            rlt::set(device, batch.rewards, rewards[(size_t)u * BATCH + b], 0, b, 0);
            rlt::set(device, batch.terminated, terminated[(size_t)u * BATCH + b] != 0, 0, b, 0);
            rlt::set(device, batch.reset, true, 0, b, 0);
            rlt::set(device, batch.final_step_mask, true, 0, b, 0);
        }
        for(int c = 0; c < 2; c++){
            for(TI b = 0; b < BATCH; b++) rlt::set(action_noise_critic, b, 0, noise_critic[((size_t)u * 2 + c) * BATCH + b]);
            rlt::train_critic(device, *ac, ac->critics[c], batch, ac->critic_optimizers[c], actor_target_buffers, critic_buffers, critic_target_buffers, ctb, action_noise_critic, rng);
        }
        if(target_values_out) for(TI b = 0; b < BATCH; b++) target_values_out[b] = rlt::get(device, ctb.target_action_value, 0, b, 0);
        rlt::update_critic_targets(device, *ac);
        for(TI b = 0; b < BATCH; b++) rlt::set(action_noise_actor, b, 0, noise_actor[(size_t)u * BATCH + b]);
        rlt::train_actor(device, *ac, batch, ac->actor_optimizer, actor_buffers, critic_buffers, atb, action_noise_actor, rng);
    }
    auto dump = [&](auto& m, float*& out, Which what){ store_layer(device, m.input_layer, out, what); store_layer(device, m.hidden_layers[0], out, what); store_layer(device, m.output_layer, out, what); };
    { float* o = actor_out; dump(ac->actor.content, o, PARAMS); dump(ac->actor.content, o, GRADS); dump(ac->actor.content, o, MOM1); }
    auto& la = rlt::get_last_layer(ac->actor).log_alpha;
    log_alpha_out[0] = rlt::get(device, la.parameters, 0); log_alpha_out[1] = rlt::get(device, la.gradient, 0); log_alpha_out[2] = rlt::get(device, la.gradient_first_order_moment, 0);
    for(int c = 0; c < 2; c++){
        float* o = critic_out + (size_t)c * 3 * N_CRITIC;
        dump(ac->critics[c].content, o, PARAMS); dump(ac->critics[c].content, o, GRADS); dump(ac->critics[c].content, o, MOM1);
        float* t = target_out + (size_t)c * N_CRITIC;
        auto& tm = ac->critics_target[c].content;
        store_parameters_only(device, tm.input_layer, t); store_parameters_only(device, tm.hidden_layers[0], t); store_parameters_only(device, tm.output_layer, t);
    }
    rlt::free(device, *ac); delete ac; rlt::free(device, batch); rlt::free(device, ctb); rlt::free(device, atb);
    rlt::free(device, actor_buffers); rlt::free(device, actor_target_buffers); rlt::free(device, critic_buffers); rlt::free(device, critic_target_buffers);
    rlt::free(device, action_noise_critic); rlt::free(device, action_noise_actor);
}

// Observation normalisation through the reference's own RunningNormalizer::update (rl/components/running_normalizer/operations_generic.h:27-47)
// on n_updates consecutive [ROWS, DIM] batches, then set_statistics + evaluate of a standardize layer
// (nn/layers/standardize/operations_generic.h:52-86) on the last batch. The layer's backward_input (:105-124) cannot be instantiated: it names
// LAYER_SPEC::T, which the layer's specification does not define (it is never reached in the reference, where the layer comes first).
template <TI ROWS, TI DIM>
static void normalizer_case(int n_updates, const float* data, float* mean_out, float* std_out, float* layer_mean, float* layer_precision, float* output){
    using NORMALIZER = rlt::rl::components::RunningNormalizer<rlt::rl::components::running_normalizer::Specification<TYPE_POLICY, TI, DIM>>;
    using LAYER = rlt::nn::layers::standardize::Layer<rlt::nn::layers::standardize::Configuration<TYPE_POLICY, TI>, rlt::nn::capability::Backward<>, rlt::tensor::Shape<TI, 1, ROWS, DIM>>;
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    NORMALIZER normalizer; LAYER layer; typename LAYER::template Buffer<> buffer;
    rlt::Matrix<rlt::matrix::Specification<T, TI, ROWS, DIM>> batch, out;
    rlt::malloc(device, normalizer); rlt::malloc(device, layer); rlt::malloc(device, batch); rlt::malloc(device, out);
    rlt::init(device, normalizer); rlt::init_weights(device, layer, rng);
    for(int u = 0; u < n_updates; u++){
        for(TI r = 0; r < ROWS; r++) for(TI c = 0; c < DIM; c++) rlt::set(batch, r, c, data[((size_t)u * ROWS + r) * DIM + c]);
        rlt::update(device, normalizer, batch);
        for(TI c = 0; c < DIM; c++){ mean_out[(size_t)u * DIM + c] = rlt::get(normalizer.mean, 0, c); std_out[(size_t)u * DIM + c] = rlt::get(normalizer.std, 0, c); }
    }
    rlt::set_statistics(device, layer, normalizer.mean, normalizer.std);
    rlt::evaluate(device, layer, batch, out, buffer, rng);
    for(TI c = 0; c < DIM; c++){ layer_mean[c] = rlt::get(device, layer.mean.parameters, c); layer_precision[c] = rlt::get(device, layer.precision.parameters, c); }
    for(TI r = 0; r < ROWS; r++) for(TI c = 0; c < DIM; c++) output[r * DIM + c] = rlt::get(out, r, c);
    rlt::free(device, normalizer); rlt::free(device, layer); rlt::free(device, batch); rlt::free(device, out);
}

// AcrobotSwingup through the reference's own observe / step / reward (rl/environments/acrobot/operations_generic.h) and a deterministic
// actor 6 -> 64 -> 64 -> 1 (ReLU, tanh) evaluated one environment at a time; the runner semantics of Rollout<> above. states [N, 4];
// a reset takes (theta_1, theta_2) from reset_states [R, N, 2] and zeroes the velocities (sample_initial_state of AcrobotSwingup, :46-53).
using ACROBOT = rlt::rl::environments::AcrobotSwingup<rlt::rl::environments::acrobot::Specification<T, TI, rlt::rl::environments::acrobot::DefaultParameters<T>>>;
// the variant that TERMINATES (reward -1 per step until the tip is above the bar, :154-156, 193-195); its initial state is four draws (:38-44)
using ACROBOT_TERMINATING = rlt::rl::environments::Acrobot<rlt::rl::environments::acrobot::Specification<T, TI, rlt::rl::environments::acrobot::DefaultParameters<T>>>;
static void acrobot_load(typename ACROBOT::State& s, const float* p){ s.theta_1 = p[0]; s.theta_2 = p[1]; s.theta_1_dot = p[2]; s.theta_2_dot = p[3]; }
static void acrobot_store(const typename ACROBOT::State& s, float* p){ p[0] = s.theta_1; p[1] = s.theta_2; p[2] = s.theta_1_dot; p[3] = s.theta_2_dot; }
// RESET_DIM values of reset_states [R, N, RESET_DIM] overwrite the leading state components at a reset, the rest are zeroed; terminated_out
// [T * N] (may be null) receives the environment's terminated flag of every transition
template <typename ACROBOT, TI RESET_DIM>
static int acrobot_rollout(const float* params, TI N, TI Tsteps, float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                           const float* reset_states, TI R, TI step_limit, float* obs, float* actions, float* rew, uint8_t* terminated_out){
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::TANH>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, rlt::nn::capability::Forward<>, rlt::tensor::Shape<TI, 1, 1, 6>>;
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    NET net; typename NET::template Buffer<> buffers;
    rlt::malloc(device, net); rlt::malloc(device, buffers);
    { const float* p = params; load_layer(device, net.input_layer, p); load_layer(device, net.hidden_layers[0], p); load_layer(device, net.output_layer, p); }
    ACROBOT env; typename ACROBOT::Parameters env_params;
    std::vector<TI> reset_count(N, 0);
    int rc = 0;
    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 6>> o; rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 1>> a;
    rlt::malloc(device, o); rlt::malloc(device, a);
    for(TI t = 0; t < Tsteps; t++){
        for(TI e = 0; e < N; e++){
            float* st = states + 4 * e;
            if(truncated[e]){
                if(reset_count[e] >= R){ rc = -2; continue; }
                for(TI k = 0; k < 4; k++) st[k] = k < RESET_DIM ? reset_states[((size_t)reset_count[e] * N + e) * RESET_DIM + k] : 0;
                reset_count[e]++; episode_step[e] = 0; episode_return[e] = 0;
            }
            typename ACROBOT::State s, ns; acrobot_load(s, st);
            rlt::observe(device, env, env_params, s, typename ACROBOT::Observation{}, o, rng);
            for(TI k = 0; k < 6; k++) obs[((size_t)t * N + e) * 6 + k] = rlt::get(o, 0, k);
            rlt::evaluate(device, net, o, a, buffers, rng);
            actions[(size_t)t * N + e] = rlt::get(a, 0, 0);
            rlt::step(device, env, env_params, s, a, ns, rng);
            T r = rlt::reward(device, env, env_params, s, a, ns, rng);
            bool terminated_flag = rlt::terminated(device, env, env_params, ns, rng);
            episode_step[e] += 1; episode_return[e] += r;
            truncated[e] = terminated_flag || ((TI)episode_step[e] == step_limit);
            rew[(size_t)t * N + e] = r;
            if(terminated_out) terminated_out[(size_t)t * N + e] = terminated_flag ? 1 : 0;
            acrobot_store(ns, st);
        }
    }
    rlt::free(device, net); rlt::free(device, buffers); rlt::free(device, o); rlt::free(device, a);
    return rc;
}

// L2F quadrotor: the environment of the reference's own GPU throughput harness (src/rl/environments/l2f/cuda/benchmark.cu:31-60: rotor
// dynamics by integration, a constant disturbance force / torque in the state, the default "crazyflie" parameter set, state limits far out),
// stepped through the reference's step() (rl/environments/l2f/operations_generic.h:93-131). State rows are position 3, orientation
// quaternion 4 (w first), linear velocity 3, angular velocity 3, disturbance force 3, disturbance torque 3, rotor speeds 4 = 23 floats.
namespace l2f_harness {
    using namespace rlt::rl::environments::l2f;
    struct STATIC_PARAMETERS{
        static constexpr TI N_SUBSTEPS = 1;
        static constexpr TI ACTION_HISTORY_LENGTH = 16;
        static constexpr bool CLOSED_FORM = false;
        using STATE_BASE = StateBase<StateSpecification<T, TI>>;
        using STATE_TYPE = StateRotors<StateRotorsSpecification<T, TI, CLOSED_FORM, StateRandomForce<StateSpecification<T, TI, STATE_BASE>>>>;
        using OBSERVATION_TYPE = observation::Position<observation::PositionSpecification<T, TI, observation::OrientationRotationMatrix<observation::OrientationRotationMatrixSpecification<T, TI,
                                 observation::LinearVelocity<observation::LinearVelocitySpecification<T, TI, observation::AngularVelocity<observation::AngularVelocitySpecification<T, TI>>>>>>>>;
        using OBSERVATION_TYPE_PRIVILEGED = OBSERVATION_TYPE;
        static constexpr bool PRIVILEGED_OBSERVATION_NOISE = false;
        using DEFAULT_STUB = parameters::DEFAULT_PARAMETERS_FACTORY<T, TI>;
        using PARAMETERS = typename DEFAULT_STUB::PARAMETERS_TYPE;
        static constexpr auto PARAMETER_VALUES = DEFAULT_STUB::nominal_parameters;
        static constexpr T STATE_LIMIT_POSITION = 100000;
        static constexpr T STATE_LIMIT_VELOCITY = 100000;
        static constexpr T STATE_LIMIT_ANGULAR_VELOCITY = 100000;
    };
    using ENVIRONMENT = rlt::rl::environments::Multirotor<rlt::rl::environments::l2f::Specification<T, TI, STATIC_PARAMETERS>>;
    static void load(ENVIRONMENT::State& s, const float* r){
        for(int k = 0; k < 3; k++){ s.position[k] = r[k]; s.linear_velocity[k] = r[7 + k]; s.angular_velocity[k] = r[10 + k]; s.force[k] = r[13 + k]; s.torque[k] = r[16 + k]; }
        for(int k = 0; k < 4; k++){ s.orientation[k] = r[3 + k]; s.rpm[k] = r[19 + k]; }
    }
    static void store(const ENVIRONMENT::State& s, float* r){
        for(int k = 0; k < 3; k++){ r[k] = s.position[k]; r[7 + k] = s.linear_velocity[k]; r[10 + k] = s.angular_velocity[k]; r[13 + k] = s.force[k]; r[16 + k] = s.torque[k]; }
        for(int k = 0; k < 4; k++){ r[3 + k] = s.orientation[k]; r[19 + k] = s.rpm[k]; }
    }
}

extern "C" {

int ref_offpolicy_gather(int N, int capacity, int step_limit, int batch, const float* actor_params, uint32_t seed, int n_steps, int n_gathers, float* oa_base, float* rewards,
                         uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, uint32_t* next_draw){
#define GATHER_CASE(n, c, l, b) if(N == n && capacity == c && step_limit == l && batch == b){ gather_case<n, c, l, b>(actor_params, seed, n_steps, n_gathers, oa_base, rewards, terminated, reset, next_reset_base, final_step_mask, next_final_step_mask_base, next_draw); return 0; }
    GATHER_CASE(8, 64, 50, 32)
    GATHER_CASE(33, 40, 17, 100)
    GATHER_CASE(5, 300, 60, 64)
#undef GATHER_CASE
    return -1;
}

// the parameter values the step reads, as the reference's own structs hold them: parameters.dynamics (85 floats in declaration order:
// rotor positions, thrust directions, torque directions [4][3] each, thrust coefficients [4][3], torque constants, rising and falling time
// constants [4] each, mass, gravity [3], J, J_inv [3][3] each, hovering throttle, action limits min / max), then dt, then the action noise
int ref_l2f_parameters(float* dynamics, float* dt, float* action_noise){
    DEVICE device;
    l2f_harness::ENVIRONMENT env; l2f_harness::ENVIRONMENT::Parameters parameters;
    rlt::init(device, env); rlt::initial_parameters(device, env, parameters);
    static_assert(sizeof(parameters.dynamics) == 85 * sizeof(float));
    std::memcpy(dynamics, &parameters.dynamics, sizeof(parameters.dynamics));
    *dt = parameters.integration.dt; *action_noise = parameters.mdp.action_noise.normalized_rpm;
    return 0;
}
// the MDP side of the default parameter set as 18 floats: reward (Squared: non_negative flag, scale, constant, termination penalty, the weights
// position, position clip, orientation, linear velocity, angular velocity, linear acceleration, angular acceleration, action, d_action,
// position error integral), termination (enabled flag, position / linear velocity / angular velocity thresholds)
int ref_l2f_mdp(float* mdp){
    DEVICE device;
    l2f_harness::ENVIRONMENT env; l2f_harness::ENVIRONMENT::Parameters parameters;
    rlt::init(device, env); rlt::initial_parameters(device, env, parameters);
    const auto& r = parameters.mdp.reward; const auto& t = parameters.mdp.termination;
    const float values[18] = {r.non_negative ? 1.0f : 0.0f, r.scale, r.constant, r.termination_penalty, r.position, r.position_clip, r.orientation, r.linear_velocity, r.angular_velocity,
                              r.linear_acceleration, r.angular_acceleration, r.action, r.d_action, r.position_error_integral, t.enabled ? 1.0f : 0.0f, t.position_threshold,
                              t.linear_velocity_threshold, t.angular_velocity_threshold};
    std::memcpy(mdp, values, sizeof(values));
    return 0;
}
// observe(state) [n, 18] (position, rotation matrix, linear velocity, angular velocity), reward(state, action, next_state) [n] and
// terminated(next_state) [n] through the reference's own functions, row by row
int ref_l2f_functions(int n, const float* states, const float* actions, const float* next_states, float* observations, float* rewards, uint8_t* terminated_out){
    DEVICE device;
    l2f_harness::ENVIRONMENT env; l2f_harness::ENVIRONMENT::Parameters parameters;
    rlt::init(device, env); rlt::initial_parameters(device, env, parameters);
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 4, false>> action;
    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 18, false>> observation;
    static_assert(l2f_harness::ENVIRONMENT::Observation::DIM == 18);
    for(int i = 0; i < n; i++){
        l2f_harness::ENVIRONMENT::State state, next;
        l2f_harness::load(state, states + (size_t)i * 23); l2f_harness::load(next, next_states + (size_t)i * 23);
        for(TI k = 0; k < 4; k++) rlt::set(action, 0, k, actions[(size_t)i * 4 + k]);
        rlt::observe(device, env, parameters, state, typename l2f_harness::ENVIRONMENT::Observation{}, observation, rng);
        for(TI k = 0; k < 18; k++) observations[(size_t)i * 18 + k] = rlt::get(observation, 0, k);
        rewards[i] = rlt::reward(device, env, parameters, state, action, next, rng);
        terminated_out[i] = rlt::terminated(device, env, parameters, next, rng) ? 1 : 0;
    }
    return 0;
}
// the initial-state distribution of the harness configuration: mdp.init (guidance, max_position, max_angle, max_linear_velocity,
// max_angular_velocity, relative_rpm, min_rpm, max_rpm) and the disturbance distributions (force mean / std, torque mean / std)
int ref_l2f_init(float* init){
    DEVICE device;
    l2f_harness::ENVIRONMENT env; l2f_harness::ENVIRONMENT::Parameters parameters;
    rlt::init(device, env); rlt::initial_parameters(device, env, parameters);
    const auto& i = parameters.mdp.init; const auto& d = parameters.disturbances;
    const float values[12] = {i.guidance, i.max_position, i.max_angle, i.max_linear_velocity, i.max_angular_velocity, i.relative_rpm ? 1.0f : 0.0f, i.min_rpm, i.max_rpm,
                              (float)d.random_force.mean, (float)d.random_force.std, (float)d.random_torque.mean, (float)d.random_torque.std};
    std::memcpy(init, values, sizeof(values));
    return 0;
}
// n x sample_initial_state on one engine (nominal parameters)
int ref_l2f_initial_states(uint32_t seed, int n, float* out){
    DEVICE device;
    l2f_harness::ENVIRONMENT env; l2f_harness::ENVIRONMENT::Parameters parameters;
    rlt::init(device, env); rlt::initial_parameters(device, env, parameters);
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    for(int i = 0; i < n; i++){
        l2f_harness::ENVIRONMENT::State state;
        rlt::sample_initial_state(device, env, parameters, state, rng);
        l2f_harness::store(state, out + (size_t)i * 23);
    }
    return 0;
}
// n quadrotors, n_steps x step() each with its own constant action [n, 4] (normalised, as a policy emits it); states [n, 23] in, out [n, 23]
int ref_l2f_steps(int n, int n_steps, const float* states, const float* actions, float* out){
    DEVICE device;
    l2f_harness::ENVIRONMENT env; l2f_harness::ENVIRONMENT::Parameters parameters;
    rlt::init(device, env); rlt::initial_parameters(device, env, parameters);
    RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 4, false>> action;
    for(int i = 0; i < n; i++){
        l2f_harness::ENVIRONMENT::State state, next;
        l2f_harness::load(state, states + (size_t)i * 23);
        for(TI k = 0; k < 4; k++) rlt::set(action, 0, k, actions[(size_t)i * 4 + k]);
        for(int s = 0; s < n_steps; s++){ rlt::step(device, env, parameters, state, action, next, rng); state = next; }
        l2f_harness::store(state, out + (size_t)i * 23);
    }
    return 0;
}

// cases: 0 = (N 4, capacity 256, limit 20, batch 32, sequence 5), 1 = (N 3, capacity 300, limit 17, batch 16, sequence 8); modes as in gather_seq_case.
// (MAX_EPISODE_LENGTH is the environment's own 200, whatever the runner's step limit: sampling from the initial state needs a capacity above it.)
int ref_offpolicy_gather_sequences(int which, int mode, const float* actor_params, uint32_t seed, int n_steps, int n_gathers, float* oa_base, float* rewards,
                                   uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, uint32_t* next_draw){
#define GATHER_SEQ_CASE(w, n, c, l, b, q, m) if(which == w && mode == m){ gather_seq_case<n, c, l, b, q, m>(actor_params, seed, n_steps, n_gathers, oa_base, rewards, terminated, reset, next_reset_base, final_step_mask, next_final_step_mask_base, next_draw); return 0; }
#define GATHER_SEQ_MODES(w, n, c, l, b, q) GATHER_SEQ_CASE(w, n, c, l, b, q, 3) GATHER_SEQ_CASE(w, n, c, l, b, q, 0) GATHER_SEQ_CASE(w, n, c, l, b, q, 1) GATHER_SEQ_CASE(w, n, c, l, b, q, 8) GATHER_SEQ_CASE(w, n, c, l, b, q, 9) GATHER_SEQ_CASE(w, n, c, l, b, q, 2)
    GATHER_SEQ_MODES(0, 4, 256, 20, 32, 5)
    GATHER_SEQ_MODES(1, 3, 300, 17, 16, 8)
#undef GATHER_SEQ_MODES
#undef GATHER_SEQ_CASE
    return -1;
}

int ref_offpolicy_steps(int N, int capacity, int step_limit, const float* actor_params, uint32_t seed, int n_steps, float* replay_data, int64_t* episode_start,
                         float* replay_states, float* replay_next_states, int64_t* counters, float* states_out, int32_t* episode_step_out, uint8_t* truncated_out,
                         float* episode_return_out, float* buf_obs, float* buf_act, float* buf_next_obs){
#define OFFPOLICY_CASE(n, c, l) if(N == n && capacity == c && step_limit == l){ offpolicy_case<n, c, l>(actor_params, seed, n_steps, replay_data, episode_start, replay_states, replay_next_states, counters, states_out, episode_step_out, truncated_out, episode_return_out, buf_obs, buf_act, buf_next_obs); return 0; }
    OFFPOLICY_CASE(8, 64, 50)
    OFFPOLICY_CASE(33, 40, 17)
#undef OFFPOLICY_CASE
    return -1;
}

// env: 0 = Pendulum shapes (3 / 1, ReLU), 1 = Ant shapes (27 / 8, tanh)
int ref_ppo_train(int env, int N, int steps, int batch, int epochs, int shuffle, uint32_t seed, const float* actor_params, const float* critic_params, const float* dataset_in,
                  float* actor_out, float* actor_grad, float* actor_m, float* critic_out, float* critic_grad, float* critic_m, float* dataset_out, double* seconds){
#define PPO_CASE(id, ENV, HACT, n, s, b, e, sh) if(env == id && N == n && steps == s && batch == b && epochs == e && (shuffle != 0) == sh){ \
        ppo_train_case<ENV, HACT, n, s, b, e, sh>(actor_params, critic_params, dataset_in, seed, actor_out, actor_grad, actor_m, critic_out, critic_grad, critic_m, dataset_out, seconds); return 0; }
    PPO_CASE(0, PENDULUM, act::RELU, 64, 64, 4096, 1, false)
    PPO_CASE(0, PENDULUM, act::RELU, 64, 64, 512, 2, false)
    PPO_CASE(0, PENDULUM, act::RELU, 5, 37, 37, 3, false)
    PPO_CASE(0, PENDULUM, act::RELU, 64, 64, 512, 2, true)
    PPO_CASE(0, PENDULUM, act::RELU, 5, 37, 37, 3, true)
    PPO_CASE(1, AntLike, act::TANH, 64, 1024, 2048, 1, false)
    PPO_CASE(1, AntLike, act::TANH, 64, 1024, 2048, 1, true)
    PPO_CASE(1, AntLike, act::TANH, 64, 1024, 2048, 10, true)
#undef PPO_CASE
    return -1;
}
int ref_acrobot_rollout(const float* params, int N, int Tsteps, float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                        const float* reset_states, int R, int step_limit, float* obs, float* actions, float* rew){
    return acrobot_rollout<ACROBOT, 2>(params, N, Tsteps, states, episode_step, truncated, episode_return, reset_states, R, step_limit, obs, actions, rew, nullptr);
}
int ref_acrobot_terminating_rollout(const float* params, int N, int Tsteps, float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                                    const float* reset_states, int R, int step_limit, float* obs, float* actions, float* rew, uint8_t* terminated){
    return acrobot_rollout<ACROBOT_TERMINATING, 4>(params, N, Tsteps, states, episode_step, truncated, episode_return, reset_states, R, step_limit, obs, actions, rew, terminated);
}
void ref_acrobot_terminating_initial_states(uint32_t seed, int n, float* states){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    ACROBOT_TERMINATING env; typename ACROBOT_TERMINATING::Parameters env_params;
    for(int e = 0; e < n; e++){ typename ACROBOT_TERMINATING::State s; rlt::sample_initial_state(device, env, env_params, s, rng); acrobot_store(s, states + 4 * e); }
}
void ref_acrobot_step(int n, const float* states, const float* actions, float* next_states, float* rewards, float* obs, float* next_obs){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    ACROBOT env; typename ACROBOT::Parameters env_params;
    rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 6>> o; rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 1>> a;
    rlt::malloc(device, o); rlt::malloc(device, a);
    for(int e = 0; e < n; e++){
        typename ACROBOT::State s, ns; acrobot_load(s, states + 4 * e);
        rlt::set(a, 0, 0, actions[e]);
        rlt::step(device, env, env_params, s, a, ns, rng);
        rewards[e] = rlt::reward(device, env, env_params, s, a, ns, rng);
        acrobot_store(ns, next_states + 4 * e);
        rlt::observe(device, env, env_params, s, typename ACROBOT::Observation{}, o, rng);
        for(int k = 0; k < 6; k++) obs[6 * e + k] = rlt::get(o, 0, k);
        rlt::observe(device, env, env_params, ns, typename ACROBOT::Observation{}, o, rng);
        for(int k = 0; k < 6; k++) next_obs[6 * e + k] = rlt::get(o, 0, k);
    }
    rlt::free(device, o); rlt::free(device, a);
}
void ref_acrobot_initial_states(uint32_t seed, int n, float* states){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    ACROBOT env; typename ACROBOT::Parameters env_params;
    for(int e = 0; e < n; e++){ typename ACROBOT::State s; rlt::sample_initial_state(device, env, env_params, s, rng); acrobot_store(s, states + 4 * e); }
}
int ref_normalizer(int rows, int dim, int n_updates, const float* data, float* mean_out, float* std_out, float* layer_mean, float* layer_precision, float* output){
#define NORMALIZER_CASE(r, d) if(rows == r && dim == d){ normalizer_case<r, d>(n_updates, data, mean_out, std_out, layer_mean, layer_precision, output); return 0; }
    NORMALIZER_CASE(4096, 27)
    NORMALIZER_CASE(333, 3)
    NORMALIZER_CASE(50, 5)
#undef NORMALIZER_CASE
    return -1;
}
int ref_sac_updates(int batch, int hidden, int n_updates, const float* actor_params, float log_alpha, const float* critic_params, const float* target_params,
                    const float* oa_base, const float* rewards, const uint8_t* terminated, const float* noise_critic, const float* noise_actor, float* actor_out,
                    float* log_alpha_out, float* critic_out, float* target_out, float* target_values_out){
#define SAC_CASE(b, h) if(batch == b && hidden == h){ sac_case<b, h>(n_updates, actor_params, log_alpha, critic_params, target_params, oa_base, rewards, terminated, noise_critic, noise_actor, actor_out, log_alpha_out, critic_out, target_out, target_values_out); return 0; }
    SAC_CASE(256, 64)
    SAC_CASE(256, 256)
    SAC_CASE(100, 32)
#undef SAC_CASE
    return -1;
}
int ref_sample_and_squash(int B, int A, const float* input, const float* noise, const float* d_output, float log_alpha, float* pre_squashing, float* output,
                          float* log_probs, float* d_input, float* d_log_alpha_per_sample, float* log_alpha_gradient_out){
#define SAS_CASE(b, a) if(B == b && A == a){ sas_case<b, a>(input, noise, d_output, log_alpha, pre_squashing, output, log_probs, d_input, d_log_alpha_per_sample, log_alpha_gradient_out); return 0; }
    SAS_CASE(256, 1)
    SAS_CASE(100, 8)
    SAS_CASE(7, 3)
#undef SAS_CASE
    return -1;
}
// utils::polyak::update / update_squared (utils/polyak/operations_generic.h:10-40) on a [41, 29] matrix, n_updates times in a row
void ref_polyak_update(const float* source, float* target, float polyak, int square, int n_updates){
    DEVICE device;
    rlt::Matrix<rlt::matrix::Specification<float, TI, 41, 29>> src, dst;
    rlt::malloc(device, src); rlt::malloc(device, dst);
    for(TI r = 0; r < 41; r++) for(TI c = 0; c < 29; c++){ rlt::set(src, r, c, source[r * 29 + c]); rlt::set(dst, r, c, target[r * 29 + c]); }
    for(int i = 0; i < n_updates; i++){
        if(square) rlt::utils::polyak::update_squared(device, src, dst, polyak);
        else rlt::utils::polyak::update(device, src, dst, polyak);
    }
    for(TI r = 0; r < 41; r++) for(TI c = 0; c < 29; c++) target[r * 29 + c] = rlt::get(dst, r, c);
    rlt::free(device, src); rlt::free(device, dst);
}
// std::uniform_int_distribution<TI>(lo, hi) as random/operations_cpu.h:27-29 drives it (TI = the CPU device's index type)
void ref_rng_uniform_int(uint32_t seed, int n, const uint64_t* lo, const uint64_t* hi, uint64_t* out){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    for(int i = 0; i < n; i++) out[i] = rlt::random::uniform_int_distribution(device.random, (TI)lo[i], (TI)hi[i], rng);
}

int ref_collect(int N, int steps, int step_limit, int hidden_act, const float* actor_params, uint32_t seed, int n_collects, float* datasets,
                float* states_out, int32_t* episode_step_out, uint8_t* truncated_out, float* episode_return_out, uint64_t* runner_step_out){
#define COLLECT_CASE(n, s, l, a, A) if(N == n && steps == s && step_limit == l && hidden_act == a){ \
        collect_case<n, s, l, A>(actor_params, seed, n_collects, datasets, states_out, episode_step_out, truncated_out, episode_return_out, runner_step_out); return 0; }
    COLLECT_CASE(64, 64, 100, 1, act::RELU)
    COLLECT_CASE(5, 37, 20, 1, act::RELU)
    COLLECT_CASE(7, 50, 0, 1, act::RELU)
    COLLECT_CASE(33, 25, 10, 2, act::TANH)
#undef COLLECT_CASE
    return -1;
}

int ref_gae(int N, int steps, const float* rewards, const float* all_values, const uint8_t* terminated, const uint8_t* truncated, float* advantages, float* target_values){
    if(N == 64 && steps == 1024){ gae_case<64, 1024>(rewards, all_values, terminated, truncated, advantages, target_values); return 0; }
    if(N == 5 && steps == 37){ gae_case<5, 37>(rewards, all_values, terminated, truncated, advantages, target_values); return 0; }
    if(N == 64 && steps == 64){ gae_case<64, 64>(rewards, all_values, terminated, truncated, advantages, target_values); return 0; }
    return -1;
}
// Gaussian head: random/operations_generic.h:87-121
void ref_normal_functions(int n, const float* mean, const float* log_std, const float* value, float* lp, float* dmean, float* dlogstd){
    DEVICE device;
    for(int i = 0; i < n; i++){
        lp[i] = rlt::random::normal_distribution::log_prob(device.random, mean[i], log_std[i], value[i]);
        dmean[i] = rlt::random::normal_distribution::d_log_prob_d_mean(device.random, mean[i], log_std[i], value[i]);
        dlogstd[i] = rlt::random::normal_distribution::d_log_prob_d_log_std(device.random, mean[i], log_std[i], value[i]);
    }
}

int ref_num_cases(){ return (int)registry().size(); }
const char* ref_case_name(int i){
    auto it = registry().begin(); std::advance(it, i); return it->first.c_str();
}
// dims[7] = batch, input_dim, hidden_dim, output_dim, num_layers, hidden_act, output_act  (activation ids: see act_from_int)
int ref_case_dims(const char* name, int* dims){
    auto it = registry().find(name); if(it == registry().end()) return -1;
    const MlpVTable& v = it->second;
    dims[0] = v.batch; dims[1] = v.input_dim; dims[2] = v.hidden_dim; dims[3] = v.output_dim; dims[4] = v.num_layers;
    dims[5] = act_to_int((act::ActivationFunction)v.hidden_act); dims[6] = act_to_int((act::ActivationFunction)v.output_act);
    return 0;
}
int ref_mlp_run(const char* name, const float* params_in, uint32_t init_seed, const float* x, const float* target, int mode, int n_steps,
                float* params_out, float* grads_out, float* m_out, float* v_out, float* pre_out, float* act_out, float* d_input_out, double* seconds){
    auto it = registry().find(name); if(it == registry().end()) return -1;
    it->second.run(params_in, init_seed, x, target, mode, n_steps, params_out, grads_out, m_out, v_out, pre_out, act_out, d_input_out, seconds);
    return 0;
}

// The training network of the sharded configuration (64 -> 256 -> 256 -> 256 -> 16, ReLU, identity) stepped over chunks of chunk_rows rows
// (1024: fast enough for a live comparison; 65536: the chunk size of the GPU path, used to generate a fixture).
int ref_mlp_c5_chunked(int chunk_rows, const float* params_in, const float* x, const float* target, int n_chunks, int total_rows, int do_step,
                       float* params_out, float* grads_out, float* m_out, float* v_out, float* pre_out, float* act_out){
    switch(chunk_rows){
        case 1024:  MlpCase<1024, 64, 256, 16, 4, act::RELU, act::IDENTITY>::run_chunked(params_in, x, target, n_chunks, total_rows, do_step, params_out, grads_out, m_out, v_out, pre_out, act_out); return 0;
        case 65536: MlpCase<65536, 64, 256, 16, 4, act::RELU, act::IDENTITY>::run_chunked(params_in, x, target, n_chunks, total_rows, do_step, params_out, grads_out, m_out, v_out, pre_out, act_out); return 0;
        default: return -1;
    }
}

// raw reference RNG streams (random/operations_cpu.h): engine seeded with seed+1
void ref_rng_uniform(uint32_t seed, int n, float lo, float hi, float* out){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    for(int i = 0; i < n; i++) out[i] = rlt::random::uniform_real_distribution(device.random, lo, hi, rng);
}
void ref_rng_normal(uint32_t seed, int n, float mean, float std, float* out){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    for(int i = 0; i < n; i++) out[i] = rlt::random::normal_distribution::sample(device.random, mean, std, rng);
}
// interleaved stream: kinds[i] == 0 -> uniform(lo[i], hi[i]); 1 -> normal(mean=lo[i], std=hi[i])
void ref_rng_mixed(uint32_t seed, int n, const uint8_t* kinds, const float* a, const float* b, float* out){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    for(int i = 0; i < n; i++){
        out[i] = kinds[i] == 0 ? rlt::random::uniform_real_distribution(device.random, a[i], b[i], rng)
                               : rlt::random::normal_distribution::sample(device.random, a[i], b[i], rng);
    }
}
// n envs, sample_initial_state in env order from one engine; states [n,2]
void ref_pendulum_initial_states(uint32_t seed, int n, float* states){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, seed);
    PENDULUM env; typename PENDULUM::Parameters env_params;
    for(int e = 0; e < n; e++){
        typename PENDULUM::State s;
        rlt::sample_initial_state(device, env, env_params, s, rng);
        states[2 * e] = s.theta; states[2 * e + 1] = s.theta_dot;
    }
}
// element-wise reference env functions on n independent (state, action) pairs
void ref_pendulum_step(int n, const float* states, const float* actions, float* next_states, float* rewards, float* obs, float* next_obs){
    DEVICE device; RNG rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    PENDULUM env; typename PENDULUM::Parameters env_params;
    for(int e = 0; e < n; e++){
        typename PENDULUM::State s, ns; s.theta = states[2 * e]; s.theta_dot = states[2 * e + 1];
        rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 1, false>> a; rlt::set(a, 0, 0, actions[e]);
        rlt::Matrix<rlt::matrix::Specification<T, TI, 1, 3, false>> o;
        rlt::step(device, env, env_params, s, a, ns, rng);
        rewards[e] = rlt::reward(device, env, env_params, s, a, ns, rng);
        next_states[2 * e] = ns.theta; next_states[2 * e + 1] = ns.theta_dot;
        if(obs){ rlt::observe(device, env, env_params, s, typename PENDULUM::Observation{}, o, rng); for(int k = 0; k < 3; k++) obs[3 * e + k] = rlt::get(o, 0, k); }
        if(next_obs){ rlt::observe(device, env, env_params, ns, typename PENDULUM::Observation{}, o, rng); for(int k = 0; k < 3; k++) next_obs[3 * e + k] = rlt::get(o, 0, k); }
    }
}
int ref_pendulum_episode_step_limit(){ return (int)PENDULUM::EPISODE_STEP_LIMIT; }

// chunk: batch size of each reference evaluate() call (compile-time in the reference): 1, 256 or 65536
int ref_pendulum_rollout(int chunk, const float* params, int N, int Tsteps, float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                         const float* reset_states, int R, int step_limit, float* obs, float* actions, float* rew, int num_threads){
    switch(chunk){
        case 1:     return Rollout<1>::run(params, N, Tsteps, states, episode_step, truncated, episode_return, reset_states, R, step_limit, obs, actions, rew, num_threads);
        case 256:   return Rollout<256>::run(params, N, Tsteps, states, episode_step, truncated, episode_return, reset_states, R, step_limit, obs, actions, rew, num_threads);
        case 65536: return Rollout<65536>::run(params, N, Tsteps, states, episode_step, truncated, episode_return, reset_states, R, step_limit, obs, actions, rew, num_threads);
        default: return -3;
    }
}
int ref_uses_openblas(){
#ifdef REF_USE_OPENBLAS
    return 1;
#else
    return 0;
#endif
}
}
