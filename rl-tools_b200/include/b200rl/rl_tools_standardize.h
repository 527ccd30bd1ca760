// Header-only adapter, part 6: observation normalisation on `devices::B200`.
//
// Include after <b200rl/rl_tools_device.h>, <rl_tools/nn/layers/standardize/operations_generic.h> and
// <rl_tools/rl/components/running_normalizer/operations_generic.h>, and BEFORE the model headers (nn_models/sequential/operations_generic.h)
// that recurse into the layer (the same ordering rule the reference's own layer headers follow).
//
// Overloads, on the device tag, of what the PPO loop calls every step (rl/algorithms/ppo/loop/core/operations_generic.h:99-131):
// update(device, normalizer, observations), set_statistics(device, layer, normalizer.mean, normalizer.std), and the standardize layer's
// evaluate / forward on matrices (the reference's CUDA forms: nn/layers/standardize/operations_cuda.h). The layer has no trainable
// parameters; its backward / update / zero_gradient stay the reference's generic no-ops.
#pragma once
#include "rl_tools_device.h"

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    // rl/components/running_normalizer/operations_generic.h:27-47
    template <typename DEV_SPEC, typename SPEC, typename DATA_SPEC>
    void update(devices::B200<DEV_SPEC>& device, rl::components::RunningNormalizer<SPEC>& normalizer, Matrix<DATA_SPEC>& data){
        static_assert(DATA_SPEC::COLS == SPEC::DIM, "Data dimension must match normalizer dimension");
        static_assert(DATA_SPEC::ROWS > 1 && utils::typing::is_same_v<typename SPEC::TYPE_POLICY::DEFAULT, float>);
        normalizer.age++;
        b200::note(device, b200rl_running_normalizer_update(data._data, (int)rl_tools::b200::ld(data), (int)DATA_SPEC::ROWS, (int)SPEC::DIM, normalizer.mean._data, normalizer.std._data,
                                                            (unsigned long long)normalizer.age, device.stream));
    }
    // rl/components/running_normalizer/operations_generic.h:20-25 (set_all on 1 x DIM matrices)
    template <typename DEV_SPEC, typename SPEC>
    void init(devices::B200<DEV_SPEC>& device, rl::components::RunningNormalizer<SPEC>& normalizer){
        normalizer.age = 0;
        b200::note(device, b200rl_fill(normalizer.mean._data, SPEC::DIM, 0.0f, device.stream));
        b200::note(device, b200rl_fill(normalizer.std._data, SPEC::DIM, 1.0f, device.stream));
    }
    // nn/layers/standardize/operations_generic.h:47-50, 52-66
    template<typename DEV_SPEC, typename SPEC, typename RNG>
    void init_weights(devices::B200<DEV_SPEC>& device, nn::layers::standardize::LayerForward<SPEC>& layer, RNG&){
        b200::note(device, b200rl_fill(layer.mean.parameters._data, SPEC::INPUT_DIM, 0.0f, device.stream));
        b200::note(device, b200rl_fill(layer.precision.parameters._data, SPEC::INPUT_DIM, 1.0f, device.stream));
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename MEAN_SPEC, typename STD_SPEC>
    void set_statistics(devices::B200<DEV_SPEC>& device, nn::layers::standardize::LayerForward<LAYER_SPEC>& layer, const Matrix<MEAN_SPEC>& mean, const Matrix<STD_SPEC>& std){
        static_assert(MEAN_SPEC::ROWS == 1 && MEAN_SPEC::COLS == LAYER_SPEC::INPUT_DIM && STD_SPEC::ROWS == 1 && STD_SPEC::COLS == LAYER_SPEC::INPUT_DIM);
        b200::note(device, b200rl_standardize_set_statistics(mean._data, std._data, (int)LAYER_SPEC::INPUT_DIM, layer.mean.parameters._data, layer.precision.parameters._data, device.stream));
    }
    // :69-92
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename OUTPUT_SPEC, typename RNG, typename MODE = mode::Default<>>
    void evaluate(devices::B200<DEV_SPEC>& device, const nn::layers::standardize::LayerForward<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<OUTPUT_SPEC>& output,
                  nn::layers::standardize::Buffer&, RNG&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(nn::layers::standardize::check_input_output<LAYER_SPEC, INPUT_SPEC, OUTPUT_SPEC>);
        b200::note(device, b200rl_standardize_forward(input._data, (int)rl_tools::b200::ld(input), layer.mean.parameters._data, layer.precision.parameters._data, output._data,
                                                      (int)rl_tools::b200::ld(output), (int)INPUT_SPEC::ROWS, (int)LAYER_SPEC::INPUT_DIM, device.stream));
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename OUTPUT_SPEC, typename RNG, typename MODE = mode::Default<>>
    void forward(devices::B200<DEV_SPEC>& device, nn::layers::standardize::LayerBackward<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<OUTPUT_SPEC>& output,
                 nn::layers::standardize::Buffer& buffer, RNG& rng, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        evaluate(device, layer, input, output, buffer, rng, mode);
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename RNG, typename MODE = mode::Default<>>
    void forward(devices::B200<DEV_SPEC>& device, nn::layers::standardize::LayerGradient<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, nn::layers::standardize::Buffer& buffer,
                 RNG& rng, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        evaluate(device, layer, input, layer.output, buffer, rng, mode);
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
