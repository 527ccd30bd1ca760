// Fixture generator (test infrastructure): the reference's OWN code export, `save_code(device, network, name)` (nn_models/mlp/persist_code.h:
// 100-103), of a forward-only MLP whose parameters are read from a raw float32 file (W b per layer), as the checkpoint step writes an actor
// (rl/loop/steps/checkpoint/operations_cpu.h:54-58). Compiled and run by make_golden.py (target `export`) where the reference tree exists:
//   g++ -std=c++17 -O1 -I<reference>/include export_golden.cpp -o export_golden && ./export_golden <case> <params.bin> <name> > text
// A program of its own rather than a function of the reference driver library: called inside a Python process that has numpy loaded, the
// writer's stream formatting crashed; as a process of its own it does not.
#include <rl_tools/operations/cpu.h>
#include <rl_tools/nn/optimizers/adam/instance/operations_generic.h>
#include <rl_tools/nn/operations_generic.h>
#include <rl_tools/nn/layers/dense/operations_cpu.h>
#include <rl_tools/nn_models/mlp/operations_generic.h>
#include <rl_tools/numeric_types/persist_code.h>
#include <rl_tools/containers/matrix/persist_code.h>
#include <rl_tools/containers/tensor/persist_code.h>
#include <rl_tools/nn/capability/persist_code.h>
#include <rl_tools/nn/parameters/persist_code.h>
#include <rl_tools/nn/optimizers/adam/instance/persist_code.h>
#include <rl_tools/nn/layers/dense/persist_code.h>
#include <rl_tools/nn_models/mlp/persist_code.h>
#include <cstdio>
#include <cstdlib>
#include <iostream>
#include <vector>
namespace rlt = rl_tools;
using DEVICE = rlt::devices::DefaultCPU;
using T = float;
using TI = typename DEVICE::index_t;
using TYPE_POLICY = rlt::numeric_types::Policy<T>;
namespace act = rlt::nn::activation_functions;

template <typename LAYER>
static void load_layer(DEVICE& device, LAYER& layer, const float*& p){
    for(TI o = 0; o < LAYER::OUTPUT_DIM; o++) for(TI i = 0; i < LAYER::INPUT_DIM; i++) rlt::set(device, layer.weights.parameters, *p++, o, i);
    for(TI o = 0; o < LAYER::OUTPUT_DIM; o++) rlt::set(device, layer.biases.parameters, *p++, o);
}
template <TI IN, TI HIDDEN, TI OUT, TI LAYERS, TI BATCH, act::ActivationFunction HACT, act::ActivationFunction OACT>
static int run(const char* file, const char* name){
    using CONFIG = rlt::nn_models::mlp::Configuration<TYPE_POLICY, TI, OUT, LAYERS, HIDDEN, HACT, OACT>;
    using NET = rlt::nn_models::mlp::NeuralNetwork<CONFIG, rlt::nn::capability::Forward<>, rlt::tensor::Shape<TI, 1, BATCH, IN>>;
    constexpr TI N = IN * HIDDEN + HIDDEN + (LAYERS - 2) * (HIDDEN * HIDDEN + HIDDEN) + HIDDEN * OUT + OUT;
    std::vector<float> params(N);
    FILE* f = std::fopen(file, "rb");
    if(!f || std::fread(params.data(), sizeof(float), N, f) != N){ std::fprintf(stderr, "cannot read %zu parameters from %s\n", (size_t)N, file); return 2; }
    std::fclose(f);
    DEVICE device;
    NET net; rlt::malloc(device, net);
    const float* p = params.data();
    load_layer(device, net.input_layer, p);
    for(TI l = 0; l < NET::NUM_HIDDEN_LAYERS; l++) load_layer(device, net.hidden_layers[l], p);
    load_layer(device, net.output_layer, p);
    std::cout << rlt::save_code(device, net, std::string(name), true);
    rlt::free(device, net);
    return 0;
}
int main(int argc, char** argv){
    if(argc != 4){ std::fprintf(stderr, "usage: export_golden <case> <params.bin> <name>\n"); return 1; }
    switch(std::atoi(argv[1])){
        case 0: return run<3, 8, 2, 3, 4, act::RELU, act::IDENTITY>(argv[2], argv[3]);      // small, batch 4
        case 1: return run<3, 64, 1, 3, 1, act::RELU, act::TANH>(argv[2], argv[3]);          // the rollout actor
        case 2: return run<5, 16, 3, 4, 2, act::TANH, act::SIGMOID>(argv[2], argv[3]);       // two hidden layers
    }
    return 1;
}
