// TEST / BENCHMARK INFRASTRUCTURE ONLY: the UNMODIFIED reference compiled with ITS OWN CUDA device (devices::CUDA: cuBLAS SGEMM per dense
// layer, its own bias / activation / Adam kernels), as the second baseline next to the reference's CPU path: what the reference itself does
// on the same GPU. Built by `make ref_cuda REFERENCE=...` into oracle/_ref/libref_cuda.so from the headers where they lie; nothing of the
// reference is copied. Only bench.py's reference measurements and tests/ load it; the product never does.
//
// The reference's graph-dump helper (devices/cuda.h:198-208) calls cudaGraphGetEdges with five arguments under CUDART_VERSION >= 12030; the
// CUDA 12.9 runtime gives that form another name, so the header does not compile against this toolkit as it stands. The overload below is
// declared before the reference is included and forwards to the four-argument runtime call; no reference source is modified, and the
// helper is never called here.
#include <cuda_runtime.h>
#include <cstddef>
static inline cudaError_t cudaGraphGetEdges(cudaGraph_t graph, cudaGraphNode_t* from, cudaGraphNode_t* to, std::nullptr_t, size_t* count){
    return cudaGraphGetEdges(graph, from, to, count);
}

// Include order as in the reference's own CUDA test (tests/src/nn/cuda/cuda_basics.cu:1-19).
#include <rl_tools/operations/cpu/group_1.h>
#include <rl_tools/operations/cuda/group_1.h>
#include <rl_tools/operations/cpu/group_2.h>
#include <rl_tools/operations/cuda/group_2.h>
#include <rl_tools/operations/cpu/group_3.h>
#include <rl_tools/operations/cuda/group_3.h>

#include <rl_tools/nn/optimizers/adam/instance/operations_generic.h>
#include <rl_tools/nn/optimizers/adam/instance/operations_cuda.h>
#include <rl_tools/nn/operations_cuda.h>
#include <rl_tools/nn/loss_functions/mse/operations_cuda.h>
#include <rl_tools/nn_models/operations_generic.h>
#include <rl_tools/nn_models/operations_cpu.h>
#include <rl_tools/nn/optimizers/adam/operations_cuda.h>
#include <rl_tools/nn_models/sequential/operations_generic.h>
#include <rl_tools/rl/environments/pendulum/operations_generic.h>
#include <rl_tools/rl/components/off_policy_runner/operations_cuda.h>

#include <cstdio>
#include <memory>
#include <vector>

namespace rlt = rl_tools;
using DEVICE_CPU = rlt::devices::DefaultCPU;
using DEVICE_CUDA = rlt::devices::DefaultCUDA;
using T = float;
using TI = typename DEVICE_CUDA::index_t;
using TYPE_POLICY = rlt::numeric_types::Policy<T>;
namespace act = rlt::nn::activation_functions;

namespace {

template <typename LAYER_CPU>
void load_layer(DEVICE_CPU& cpu, LAYER_CPU& layer, const float*& p){
    for(TI o = 0; o < LAYER_CPU::OUTPUT_DIM; o++) for(TI i = 0; i < LAYER_CPU::INPUT_DIM; i++) rlt::set(cpu, layer.weights.parameters, *p++, o, i);
    for(TI o = 0; o < LAYER_CPU::OUTPUT_DIM; o++) rlt::set(cpu, layer.biases.parameters, *p++, o);
}
template <typename LAYER_CPU>
void store_layer(DEVICE_CPU& cpu, LAYER_CPU& layer, float*& p, bool gradient){
    for(TI o = 0; o < LAYER_CPU::OUTPUT_DIM; o++) for(TI i = 0; i < LAYER_CPU::INPUT_DIM; i++) *p++ = gradient ? rlt::get(cpu, layer.weights.gradient, o, i) : rlt::get(cpu, layer.weights.parameters, o, i);
    for(TI o = 0; o < LAYER_CPU::OUTPUT_DIM; o++) *p++ = gradient ? rlt::get(cpu, layer.biases.gradient, o) : rlt::get(cpu, layer.biases.parameters, o);
}

// One training step of the reference on ITS CUDA device, as bench.py's `mlp_train` line defines a step: zero_gradient, then per chunk of
// CHUNK rows forward + MSE gradient (weight chunk / rows, so that the accumulated gradient is the mean over all rows) + backward, then one
// Adam step. x_dev / y_dev are device pointers to [rows, INPUT] / [rows, OUTPUT] row-major fp32. Parameters W_l b_l per layer, in and out.
template <TI CHUNK, TI INPUT_DIM, TI HIDDEN_DIM, TI OUTPUT_DIM, TI NUM_LAYERS>
int mlp_train(long long rows, int steps, int warmup, const float* params_in, const float* x_dev, const float* y_dev, float* ms_per_step, float* params_out, float* grads_out){
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, OUTPUT_DIM, NUM_LAYERS, HIDDEN_DIM, act::RELU, act::IDENTITY>;
    using CAPABILITY = rlt::nn::capability::Gradient<rlt::nn::parameters::Adam>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, CAPABILITY, rlt::tensor::Shape<TI, 1, CHUNK, INPUT_DIM>>;
    using OPTIMIZER = rlt::nn::optimizers::Adam<rlt::nn::optimizers::adam::Specification<TYPE_POLICY, TI>>;
    if(rows <= 0 || rows % CHUNK) return -1;
    DEVICE_CPU cpu; DEVICE_CUDA cuda;
    rlt::init(cuda);
    auto net_cpu = new NET(); NET net; typename NET::template Buffer<> buffers; OPTIMIZER optimizer;
    rlt::malloc(cpu, *net_cpu); rlt::malloc(cuda, net); rlt::malloc(cuda, buffers); rlt::malloc(cuda, optimizer);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng_cpu; rlt::malloc(cpu, rng_cpu); rlt::init(cpu, rng_cpu, 0);
    DEVICE_CUDA::SPEC::RANDOM::ENGINE<> rng; rlt::malloc(cuda, rng); rlt::init(cuda, rng);
    rlt::init_weights(cpu, *net_cpu, rng_cpu);
    { const float* p = params_in; load_layer(cpu, net_cpu->input_layer, p);
      for(TI l = 0; l < NET::NUM_HIDDEN_LAYERS; l++) load_layer(cpu, net_cpu->hidden_layers[l], p);
      load_layer(cpu, net_cpu->output_layer, p); }
    rlt::zero_gradient(cpu, *net_cpu);
    rlt::copy(cpu, cuda, *net_cpu, net);
    rlt::init(cuda, optimizer);
    rlt::reset_optimizer_state(cuda, optimizer, net);
    rlt::Matrix<rlt::matrix::Specification<T, TI, CHUNK, INPUT_DIM>> x;
    rlt::Matrix<rlt::matrix::Specification<T, TI, CHUNK, OUTPUT_DIM>> y, d_out;
    rlt::malloc(cuda, d_out);
    const long long n_chunks = rows / CHUNK;
    // the loss weight as a one-element DEVICE tensor: the reference's CUDA overload of the MSE gradient takes it in that form only
    // (nn/loss_functions/mse/operations_cuda.h:40-58; a scalar weight would select the generic host loop)
    rlt::Tensor<rlt::tensor::Specification<T, TI, rlt::tensor::Shape<TI, 1>>> weight_cpu, weight;
    rlt::malloc(cpu, weight_cpu); rlt::malloc(cuda, weight);
    rlt::set(cpu, weight_cpu, (T)((double)CHUNK / (double)rows), 0);
    rlt::copy(cpu, cuda, weight_cpu, weight);
    auto step = [&](){
        rlt::zero_gradient(cuda, net);
        for(long long c = 0; c < n_chunks; c++){
            x._data = const_cast<float*>(x_dev) + c * (long long)CHUNK * INPUT_DIM;
            y._data = const_cast<float*>(y_dev) + c * (long long)CHUNK * OUTPUT_DIM;
            rlt::forward(cuda, net, x, buffers, rng);
            auto out = rlt::output(cuda, net); auto out_m = rlt::matrix_view(cuda, out);
            rlt::nn::loss_functions::mse::gradient(cuda, out_m, y, d_out, weight);
            rlt::backward(cuda, net, x, d_out, buffers);
        }
        rlt::step(cuda, optimizer, net);
    };
    for(int i = 0; i < warmup; i++) step();
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaDeviceSynchronize();
    cudaEventRecord(e0, cuda.stream);
    for(int i = 0; i < steps; i++) step();
    cudaEventRecord(e1, cuda.stream);
    cudaEventSynchronize(e1);
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    if(ms_per_step) *ms_per_step = steps > 0 ? ms / steps : 0;
    int rc = cudaGetLastError() == cudaSuccess ? 0 : -2;
    rlt::copy(cuda, cpu, net, *net_cpu);
    for(int what = 0; what < 2; what++){                        // parameters, then the gradient accumulated by the last step
        float* p = what ? grads_out : params_out;
        if(!p) continue;
        store_layer(cpu, net_cpu->input_layer, p, what == 1);
        for(TI l = 0; l < NET::NUM_HIDDEN_LAYERS; l++) store_layer(cpu, net_cpu->hidden_layers[l], p, what == 1);
        store_layer(cpu, net_cpu->output_layer, p, what == 1);
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    rlt::free(cpu, weight_cpu); rlt::free(cuda, weight); rlt::free(cuda, rng); rlt::free(cuda, d_out); rlt::free(cuda, net); rlt::free(cuda, buffers); rlt::free(cuda, optimizer); rlt::free(cpu, *net_cpu); delete net_cpu;
    return rc;
}

// The reference's own off-policy runner on ITS CUDA device: `step<0>` = prologue kernel, policy `evaluate` (per layer: bias kernel, cublasSgemm,
// activation kernel), epilogue kernel (rl/components/off_policy_runner/operations_cuda.h:184-204), N environments, each step appended to the
// per-environment replay buffers. Deterministic actor 3 -> 64 -> 64 -> 1 (ReLU, ReLU, tanh) as in the benchmark workload.
template <TI T_N, TI T_CAPACITY, TI T_LIMIT>
struct RolloutParameters: rlt::rl::components::off_policy_runner::ParametersDefault<TYPE_POLICY, TI>{
    static constexpr TI N_ENVIRONMENTS = T_N;
    static constexpr TI REPLAY_BUFFER_CAPACITY = T_CAPACITY;
    static constexpr TI EPISODE_STEP_LIMIT = T_LIMIT;
};
template <TI N, TI CAPACITY, TI LIMIT>
int rollout(int steps, int warmup, const float* params_in, float* ms_per_rollout, float* mean_return_probe){
    using PENDULUM = rlt::rl::environments::Pendulum<rlt::rl::environments::pendulum::Specification<T, TI, rlt::rl::environments::pendulum::DefaultParameters<T>>>;
    using ACTOR_CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, 1, 3, 64, act::RELU, act::TANH>;
    using ACTOR = rlt::nn_models::sequential::Build<rlt::nn::capability::Forward<>, rlt::nn_models::sequential::Module<rlt::nn_models::mlp::BindConfiguration<ACTOR_CONFIG>>, rlt::tensor::Shape<TI, 1, N, 3>>;
    using SPEC = rlt::rl::components::off_policy_runner::Specification<TYPE_POLICY, TI, PENDULUM, rlt::utils::Tuple<TI, ACTOR>, RolloutParameters<N, CAPACITY, LIMIT>>;
    using RUNNER = rlt::rl::components::OffPolicyRunner<SPEC>;
    using RNG = DEVICE_CUDA::SPEC::RANDOM::ENGINE<DEVICE_CUDA::SPEC::RANDOM::Specification<TI, N>>;
    DEVICE_CPU cpu; DEVICE_CUDA cuda;
    rlt::init(cuda);
    ACTOR actor_cpu, actor; typename ACTOR::template Buffer<> buffers;
    rlt::malloc(cpu, actor_cpu); rlt::malloc(cuda, actor); rlt::malloc(cuda, buffers);
    DEVICE_CPU::SPEC::RANDOM::ENGINE<> rng_cpu; rlt::malloc(cpu, rng_cpu); rlt::init(cpu, rng_cpu, 0);
    rlt::init_weights(cpu, actor_cpu, rng_cpu);
    { const float* p = params_in; auto& m = actor_cpu.content; load_layer(cpu, m.input_layer, p); load_layer(cpu, m.hidden_layers[0], p); load_layer(cpu, m.output_layer, p); }
    rlt::copy(cpu, cuda, actor_cpu, actor);
    RNG rng; rlt::malloc(cuda, rng); rlt::init(cuda, rng, 1);
    std::unique_ptr<RUNNER> runner(new RUNNER());
    rlt::malloc(cuda, *runner);
    rlt::init(cuda, *runner);
    auto run = [&](){ for(int s = 0; s < (int)LIMIT; s++) rlt::step<0>(cuda, *runner, actor, buffers, rng); };
    for(int i = 0; i < warmup; i++) run();
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaDeviceSynchronize();
    cudaEventRecord(e0, cuda.stream);
    for(int i = 0; i < steps; i++) run();
    cudaEventRecord(e1, cuda.stream);
    cudaEventSynchronize(e1);
    float ms = 0; cudaEventElapsedTime(&ms, e0, e1);
    if(ms_per_rollout) *ms_per_rollout = steps > 0 ? ms / steps : 0;
    int rc = cudaGetLastError() == cudaSuccess ? 0 : -2;
    if(mean_return_probe){                                     // evidence that the environments were stepped: the mean episode return so far
        std::vector<float> returns(N);
        cudaMemcpy(returns.data(), runner->episode_return._data, N * sizeof(float), cudaMemcpyDeviceToHost);
        double sum = 0; for(float r : returns) sum += r;
        *mean_return_probe = (float)(sum / N);
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    rlt::free(cuda, *runner); rlt::free(cuda, rng); rlt::free(cuda, actor); rlt::free(cuda, buffers); rlt::free(cpu, actor_cpu);
    return rc;
}

}  // namespace

extern "C" {

// case 0: the benchmark network 64 -> 256 -> 256 -> 256 -> 16 in 65,536-row chunks; case 1: the same network in 1,024-row chunks (parity sizes);
// case 2: the SAC critic 4 -> 256 -> 256 -> 1 at batch 256
int ref_cuda_mlp_train(int which, long long rows, int steps, int warmup, const float* params_in, const float* x_dev, const float* y_dev, float* ms_per_step,
                       float* params_out, float* grads_out){
    switch(which){
        case 0: return mlp_train<65536, 64, 256, 16, 4>(rows, steps, warmup, params_in, x_dev, y_dev, ms_per_step, params_out, grads_out);
        case 1: return mlp_train<1024, 64, 256, 16, 4>(rows, steps, warmup, params_in, x_dev, y_dev, ms_per_step, params_out, grads_out);
        case 2: return mlp_train<256, 4, 256, 1, 3>(rows, steps, warmup, params_in, x_dev, y_dev, ms_per_step, params_out, grads_out);
    }
    return -3;
}

// `steps` timed rollouts of 200 runner steps each (after `warmup` untimed ones) on 65,536 environments (which = 0) or 512 (which = 1), episode
// step limit 200, replay capacity 256 per environment. params: W1 b1 W2 b2 W3 b3 of the actor.
int ref_cuda_rollout(int which, int steps, int warmup, const float* params_in, float* ms_per_rollout, float* mean_return_probe){
    switch(which){
        case 0: return rollout<65536, 256, 200>(steps, warmup, params_in, ms_per_rollout, mean_return_probe);
        case 1: return rollout<512, 256, 200>(steps, warmup, params_in, ms_per_rollout, mean_return_probe);
    }
    return -3;
}

}
