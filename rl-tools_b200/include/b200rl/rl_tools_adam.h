// Header-only adapter, Adam part: init / reset_optimizer_state / step of nn::optimizers::Adam on `devices::B200`.
//
// rl_tools_operations.h includes this file, so user code that calls these verbs itself needs nothing more. Include it EARLIER -- after the
// model headers (nn_models/mlp, nn_models/sequential, ...) and before a reference header whose templates call `init(device, optimizer)`,
// `reset_optimizer_state(device, optimizer, model)` or `step(device, optimizer, model)` for you (rl/algorithms/sac/operations_generic.h does) --
// when the reference's generic code is to pick them up: an optimizer and a model are no Matrix / Tensor, so argument-dependent lookup does not
// reach namespace rl_tools from inside those templates, and only overloads declared before them are candidates. The same rule makes the
// reference put nn/optimizers/adam/operations_generic.h after the models it steps.
#pragma once
#include <b200rl/rl_tools_device.h>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    // ---- Adam: nn/optimizers/adam/operations_cuda.h:39-69, instance/operations_cuda.h:60-70 ------------------------
    template<typename DEV_SPEC, typename SPEC>
    void init(devices::B200<DEV_SPEC>& device, nn::optimizers::Adam<SPEC>& optimizer){
        using PARAMETERS = typename SPEC::DEFAULT_PARAMETERS;
        static_assert(utils::typing::is_same_v<typename SPEC::T, float>, "fp32 only");
        static_assert(!PARAMETERS::ENABLE_WEIGHT_DECAY && !PARAMETERS::ENABLE_BIAS_LR_FACTOR && !PARAMETERS::ENABLE_GRADIENT_CLIPPING, "only the default (plain) Adam update is implemented");
        typename nn::optimizers::Adam<SPEC>::PARAMETERS host{PARAMETERS::ALPHA, PARAMETERS::BETA_1, PARAMETERS::BETA_2, PARAMETERS::EPSILON, PARAMETERS::EPSILON_SQRT,
                                                             PARAMETERS::WEIGHT_DECAY, PARAMETERS::WEIGHT_DECAY_INPUT, PARAMETERS::WEIGHT_DECAY_OUTPUT, PARAMETERS::BIAS_LR_FACTOR};
        b200::note(device, b200rl_memcpy(optimizer.parameters._data, &host, sizeof(host), 0, device.stream));
    }
    template<typename DEV_SPEC, typename SPEC, typename MODEL>
    void reset_optimizer_state(devices::B200<DEV_SPEC>& device, nn::optimizers::Adam<SPEC>& optimizer, MODEL& model){
        typename SPEC::TI one = 1;                        // age starts at 1 (nn/optimizers/adam/operations_generic.h:43-46)
        b200::note(device, b200rl_memcpy(optimizer.age._data, &one, sizeof(one), 0, device.stream));
        _reset_optimizer_state(device, model, optimizer);
    }
    template<typename DEV_SPEC, typename SPEC, typename MODEL>
    void step(devices::B200<DEV_SPEC>& device, nn::optimizers::Adam<SPEC>& optimizer, MODEL& model){
        static_assert(sizeof(typename SPEC::TI) == 4, "the age is a 32-bit counter");
        b200::note(device, b200rl_adam_advance_dev(reinterpret_cast<const float*>(optimizer.parameters._data), reinterpret_cast<uint32_t*>(optimizer.age._data),
                                                   optimizer.first_order_moment_bias_correction._data, optimizer.second_order_moment_bias_correction._data, device.stream));
        update(device, model, optimizer);
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
