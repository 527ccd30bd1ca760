// Header-only adapter, part 1: the device tag `rl_tools::devices::B200` for RLtools' overload-on-device-type API.
//
// Include AFTER <rl_tools/operations/cpu.h> (the host device is needed for host<->device copies and for the host-side
// math/random/logging sub-devices) and BEFORE the reference's generic nn / nn_models headers; then include
// <b200rl/rl_tools_operations.h>. User code is compiled with the host compiler only and linked against libb200rl.so.
//
// Mirrors the interface of the reference's CUDA device (devices/cuda.h:16-125: index_t = unsigned int,
// DEVICE_ID = DeviceId::CUDA, SPEC::{MATH, RANDOM, LOGGING}, members math / random / logger / stream,
// graph_capture_active) without cuBLAS / cuRAND handles. Errors are sticky in `device.status` (the reference prints
// and continues); `check_status(device)` returns it.
#pragma once
#include <b200rl.h>
#include <rl_tools/containers/matrix/matrix.h>
#include <rl_tools/containers/tensor/tensor.h>
#include <rl_tools/nn/optimizers/adam/adam.h>
#include <rl_tools/nn/layers/dense/layer.h>
#include <vector>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools::devices{
    namespace b200{
        struct Base{
            static constexpr DeviceId DEVICE_ID = DeviceId::CUDA;
            using index_t = unsigned int;
            static constexpr index_t MAX_INDEX = -1;
        };
    }
    struct DefaultB200Specification{
        using MATH = devices::math::CPU;                 // scalar host-side math (hyper-parameters, bounds)
        using MATH_DEVICE_ACCURATE = devices::math::CPU;
        using RANDOM = devices::random::CPU;             // the CPU engine is the source of truth for parity
        using LOGGING = devices::logging::CPU;
        static constexpr bool TAG = false;
        static constexpr bool KERNEL = false;
    };
    template <typename T_SPEC>
    struct B200: b200::Base{
        template <typename OTHER_DEVICE>
        static constexpr bool compatible = OTHER_DEVICE::DEVICE_ID == DeviceId::CUDA;
        using SPEC = T_SPEC;
        typename SPEC::MATH math;
        typename SPEC::RANDOM random;
        typename SPEC::LOGGING* logger = nullptr;
        b200rl_stream_t stream = nullptr;                // cudaStream_t; nullptr = the default stream
        bool graph_capture_active = false;
        int status = B200RL_OK;                          // first failure of any call on this device
    };
    using DefaultB200 = B200<DefaultB200Specification>;
}
RL_TOOLS_NAMESPACE_WRAPPER_END

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    namespace b200{
        template <typename DEVICE>
        inline void note(DEVICE& device, int rc){ if(rc != B200RL_OK && device.status == B200RL_OK) device.status = rc; }
        // row pitch of a matrix as the C ABI wants it (>= the row length): the reference's matrix view of a one-dimensional tensor is a single
        // row whose nominal pitch is 1 (containers/tensor/operations_generic.h:1053-1066), where the pitch is never used
        template<typename SPEC>
        constexpr typename SPEC::TI ld(const Matrix<SPEC>& m){ return SPEC::ROWS == 1 && row_pitch(m) < SPEC::COLS ? SPEC::COLS : row_pitch(m); }
        // a tensor whose last dimension is contiguous and whose leading dimensions collapse into rows of one pitch
        template<typename SPEC, typename TI, TI I>
        constexpr bool collapsible_from(){
            constexpr TI N = length(typename SPEC::SHAPE{});
            if constexpr(I + 2 >= N) return true;
            else return get<I>(typename SPEC::STRIDE{}) == get<I + 1>(typename SPEC::STRIDE{}) * get<I + 1>(typename SPEC::SHAPE{}) && collapsible_from<SPEC, TI, I + 1>();
        }
        template<typename SPEC>
        struct Rows{
            using TI = typename SPEC::TI;
            static constexpr TI N = length(typename SPEC::SHAPE{});
            static_assert(N >= 1);
            static_assert(get<N - 1>(typename SPEC::STRIDE{}) == 1, "the last dimension must be contiguous");
            static_assert(collapsible_from<SPEC, TI, 0>(), "the leading dimensions must collapse into rows of one pitch");
            static constexpr TI COLS = get<N - 1>(typename SPEC::SHAPE{});
            static constexpr TI ROWS = get<0>(tensor::CumulativeProduct<typename SPEC::SHAPE>{}) / COLS;      // the SHAPE's product: a view's SIZE may be its parent's
            static constexpr TI PITCH = N >= 2 ? get<(N >= 2 ? N - 2 : 0)>(typename SPEC::STRIDE{}) : COLS;
        };
    }
    template <typename SPEC>
    void init(devices::B200<SPEC>& device){ device.status = B200RL_OK; }
    template <typename SPEC>
    int check_status(devices::B200<SPEC>& device){
        b200::note(device, b200rl_stream_synchronize(device.stream));
        return device.status;
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END

// init_weights of a dense layer likewise has to be declared before the reference's generic dense operations: their three-argument
// init_weights(device, layer, rng) forwards to the four-argument form below with no argument from namespace rl_tools.
// The draws are made on the HOST with the reference's own uniform_real_distribution on the caller's engine, in the reference's order
// (per output row the bias, then the row's weights; nn/layers/dense/operations_generic.h:59-87), then uploaded: the parameters are
// bit-identical to those of the CPU device for the same engine state, and the engine advances identically.
// Replaces nn/layers/dense/operations_cuda.h:17-67 (which draws on its device engines instead).
RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    template<typename DEV_SPEC, typename SPEC, typename INITIALIZER_SPEC, typename RNG>
    void init_weights(devices::B200<DEV_SPEC>& device, nn::layers::dense::LayerForward<SPEC>& layer, const nn::layers::dense::KaimingUniform<INITIALIZER_SPEC>&, RNG& rng){
        using T = typename SPEC::TYPE_POLICY::DEFAULT;
        static_assert(utils::typing::is_same_v<T, float>, "fp32 only");
        T gain;
        if constexpr(INITIALIZER_SPEC::INIT_LEGACY){
            const T negative_slope = math::sqrt(device.math, (T)5);
            gain = math::sqrt(device.math, (T)2.0 / (1 + negative_slope * negative_slope));
        }
        else gain = math::sqrt(device.math, (T)2.0) * INITIALIZER_SPEC::SCALE;
        const T std = gain / math::sqrt(device.math, (T)SPEC::INPUT_DIM);
        const T weight_bound = math::sqrt(device.math, (T)3.0) * std, bias_bound = 1 / math::sqrt(device.math, (T)SPEC::INPUT_DIM);
        std::vector<T> w((size_t)SPEC::OUTPUT_DIM * SPEC::INPUT_DIM), b((size_t)SPEC::OUTPUT_DIM);
        for(typename SPEC::TI i = 0; i < SPEC::OUTPUT_DIM; i++){
            b[i] = INITIALIZER_SPEC::INIT_LEGACY ? random::uniform_real_distribution(device.random, -bias_bound, bias_bound, rng) : (T)0;
            for(typename SPEC::TI j = 0; j < SPEC::INPUT_DIM; j++) w[(size_t)i * SPEC::INPUT_DIM + j] = random::uniform_real_distribution(device.random, -weight_bound, weight_bound, rng);
        }
        b200::note(device, b200rl_memcpy(layer.weights.parameters._data, w.data(), w.size() * sizeof(T), 0, device.stream));
        b200::note(device, b200rl_memcpy(layer.biases.parameters._data, b.data(), b.size() * sizeof(T), 0, device.stream));
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END

// The per-parameter Adam update must be declared BEFORE the reference's generic layer headers are included: the generic
// dense `update(device, layer, optimizer)` calls `update(device, layer.weights, optimizer)`, and none of those argument
// types lives directly in namespace rl_tools, so argument-dependent lookup does not reach overloads declared later (the
// reference has the same ordering rule, see the note at the top of nn/optimizers/adam/adam.h).
// Replaces nn/optimizers/adam/instance/operations_cuda.h:60-70.
RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    template<typename DEV_SPEC, typename SPEC, typename ADAM_SPEC>
    void update(devices::B200<DEV_SPEC>& device, nn::parameters::Adam::Instance<SPEC>& parameter, nn::optimizers::Adam<ADAM_SPEC>& optimizer){
        static_assert(tensor::dense_row_major_layout<typename decltype(parameter.parameters)::SPEC>(), "only dense parameter tensors");
        b200::note(device, b200rl_adam_update_dev(parameter.parameters._data, parameter.gradient._data, parameter.gradient_first_order_moment._data,
                                                  parameter.gradient_second_order_moment._data, decltype(parameter.parameters)::SPEC::SIZE,
                                                  reinterpret_cast<const float*>(optimizer.parameters._data), optimizer.first_order_moment_bias_correction._data,
                                                  optimizer.second_order_moment_bias_correction._data, device.stream));
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END

// The target-network update is declared here as well, ahead of everything: the reference calls it by its qualified name
// (rl/algorithms/sac/operations_generic.h:486-496), which considers only the overloads declared before that call.
RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    // ---- Polyak (target-network) update: utils/polyak/operations_cuda.h:31-52 ---------------------------------------
    namespace utils::polyak{
        template<typename DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC, bool SQUARE = false>
        void update(devices::B200<DEV_SPEC>& device, const Matrix<SOURCE_SPEC>& source, Matrix<TARGET_SPEC>& target, const typename SOURCE_SPEC::T polyak){
            static_assert(containers::check_structure<SOURCE_SPEC, TARGET_SPEC> && utils::typing::is_same_v<typename SOURCE_SPEC::T, float>);
            rl_tools::b200::note(device, b200rl_polyak_update(source._data, rl_tools::b200::ld(source), target._data, rl_tools::b200::ld(target), SOURCE_SPEC::ROWS, SOURCE_SPEC::COLS, polyak, SQUARE ? 1 : 0, device.stream));
        }
        template<typename DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
        void update_squared(devices::B200<DEV_SPEC>& device, const Matrix<SOURCE_SPEC>& source, Matrix<TARGET_SPEC>& target, const typename SOURCE_SPEC::T polyak){
            update<DEV_SPEC, SOURCE_SPEC, TARGET_SPEC, true>(device, source, target, polyak);
        }
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
