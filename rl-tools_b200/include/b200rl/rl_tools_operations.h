// Header-only adapter, part 2: RLtools operations overloaded on `devices::B200`, forwarding to the C ABI of libb200rl.so.
//
// Include after <b200rl/rl_tools_device.h> and after the reference's generic headers for containers, nn layers,
// optimizers and models (their generic recursions -- nn_models::mlp forward/backward/update, zero_gradient,
// _reset_optimizer_state, malloc/free/copy of whole networks -- reach the overloads below through the device type).
// Only fp32 containers with column pitch 1 are supported (the same restriction the reference's CUDA dense layer has,
// nn/layers/dense/operations_cuda.h:240-242).
#pragma once
#include "rl_tools_device.h"

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    // ---- containers: containers/matrix/operations_cuda.h:16-40, containers/tensor/operations_cuda.h:16-40 ----------
    template<typename DEV_SPEC, typename T, typename T_TI, T_TI SIZE_BYTES, bool T_CONST>
    void malloc(devices::B200<DEV_SPEC>& device, matrix::MatrixDynamic<T, T_TI, SIZE_BYTES, T_CONST>& matrix){
        void* p = nullptr;
        b200::note(device, b200rl_device_malloc(&p, SIZE_BYTES));
        matrix._data = static_cast<T*>(p);
    }
    template<typename DEV_SPEC, typename T, typename T_TI, T_TI SIZE_BYTES, bool T_CONST>
    void free(devices::B200<DEV_SPEC>& device, matrix::MatrixDynamic<T, T_TI, SIZE_BYTES, T_CONST>& matrix){
        b200::note(device, b200rl_device_free(const_cast<typename utils::typing::remove_const<T>::type*>(matrix._data)));
        matrix._data = nullptr;
    }
    template<typename DEV_SPEC, typename T, typename T_TI, T_TI SIZE, bool T_CONST>
    void malloc(devices::B200<DEV_SPEC>& device, tensor::TensorDynamic<T, T_TI, SIZE, T_CONST>& tensor){
        void* p = nullptr;
        b200::note(device, b200rl_device_malloc(&p, SIZE * sizeof(T)));
        tensor._data = static_cast<T*>(p);
    }
    template<typename DEV_SPEC, typename T, typename T_TI, T_TI SIZE, bool T_CONST>
    void free(devices::B200<DEV_SPEC>& device, tensor::TensorDynamic<T, T_TI, SIZE, T_CONST>& tensor){
        b200::note(device, b200rl_device_free(const_cast<typename utils::typing::remove_const<T>::type*>(tensor._data)));
        tensor._data = nullptr;
    }

    namespace b200{
        // row-wise copy between two matrices of the same shape with independent row pitches (views included)
        template<typename DEVICE, typename SOURCE_SPEC, typename TARGET_SPEC>
        void copy_matrix(DEVICE& device, const Matrix<SOURCE_SPEC>& source, Matrix<TARGET_SPEC>& target, int kind){
            static_assert(containers::check_structure<SOURCE_SPEC, TARGET_SPEC>);
            static_assert(utils::typing::is_same_v<typename SOURCE_SPEC::T, typename TARGET_SPEC::T>, "copy converts no types");
            static_assert(SOURCE_SPEC::COL_PITCH == 1 && TARGET_SPEC::COL_PITCH == 1, "column pitch must be 1");
            using T = typename SOURCE_SPEC::T;
            note(device, b200rl_memcpy_2d(target._data, rl_tools::b200::ld(target) * sizeof(T), source._data, rl_tools::b200::ld(source) * sizeof(T),
                                          SOURCE_SPEC::COLS * sizeof(T), SOURCE_SPEC::ROWS, kind, device.stream));
        }
        template<typename DEVICE, typename SOURCE_SPEC, typename TARGET_SPEC>
        void copy_tensor(DEVICE& device, const Tensor<SOURCE_SPEC>& source, Tensor<TARGET_SPEC>& target, int kind){
            static_assert(tensor::same_dimensions<SOURCE_SPEC, TARGET_SPEC>());
            static_assert(utils::typing::is_same_v<typename utils::typing::remove_const<typename SOURCE_SPEC::T>::type, typename TARGET_SPEC::T>, "copy converts no types");
            using T = typename TARGET_SPEC::T;
            if constexpr(tensor::dense_row_major_layout<SOURCE_SPEC>() && tensor::dense_row_major_layout<TARGET_SPEC>()){
                note(device, b200rl_memcpy(target._data, source._data, SOURCE_SPEC::SIZE * sizeof(T), kind, device.stream));
            }
            else{                                           // views of a wider table (view_range over the last dimension): a pitched row copy
                using S = Rows<SOURCE_SPEC>; using D = Rows<TARGET_SPEC>;
                note(device, b200rl_memcpy_2d(target._data, D::PITCH * sizeof(T), source._data, S::PITCH * sizeof(T), S::COLS * sizeof(T), S::ROWS, kind, device.stream));
            }
        }
    }
    // containers/matrix/operations_cuda.h:105-195 (host<->device copies synchronise the stream, as there)
    template<typename S_DEV_SPEC, typename T_DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
    void copy(devices::CPU<S_DEV_SPEC>&, devices::B200<T_DEV_SPEC>& device, const Matrix<SOURCE_SPEC>& source, Matrix<TARGET_SPEC>& target){ b200::copy_matrix(device, source, target, 0); }
    template<typename S_DEV_SPEC, typename T_DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
    void copy(devices::B200<S_DEV_SPEC>& device, devices::CPU<T_DEV_SPEC>&, const Matrix<SOURCE_SPEC>& source, Matrix<TARGET_SPEC>& target){ b200::copy_matrix(device, source, target, 1); }
    template<typename S_DEV_SPEC, typename T_DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
    void copy(devices::B200<S_DEV_SPEC>& device, devices::B200<T_DEV_SPEC>&, const Matrix<SOURCE_SPEC>& source, Matrix<TARGET_SPEC>& target){ b200::copy_matrix(device, source, target, 2); }
    // containers/tensor/operations_cuda.h:74-166
    template<typename S_DEV_SPEC, typename T_DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
    void copy(devices::CPU<S_DEV_SPEC>&, devices::B200<T_DEV_SPEC>& device, const Tensor<SOURCE_SPEC>& source, Tensor<TARGET_SPEC>& target){ b200::copy_tensor(device, source, target, 0); }
    template<typename S_DEV_SPEC, typename T_DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
    void copy(devices::B200<S_DEV_SPEC>& device, devices::CPU<T_DEV_SPEC>&, const Tensor<SOURCE_SPEC>& source, Tensor<TARGET_SPEC>& target){ b200::copy_tensor(device, source, target, 1); }
    template<typename S_DEV_SPEC, typename T_DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC>
    void copy(devices::B200<S_DEV_SPEC>& device, devices::B200<T_DEV_SPEC>&, const Tensor<SOURCE_SPEC>& source, Tensor<TARGET_SPEC>& target){ b200::copy_tensor(device, source, target, 2); }

    // containers/matrix/operations_cuda.h:47-61 (set_all kernel) -> one fill launch per row block
    template<typename DEV_SPEC, typename SPEC, typename VALUE_T>
    void set_all(devices::B200<DEV_SPEC>& device, Matrix<SPEC>& m, VALUE_T value){
        static_assert(utils::typing::is_same_v<typename SPEC::T, float>, "fp32 only");
        static_assert(SPEC::COL_PITCH == 1);
        if(rl_tools::b200::ld(m) == SPEC::COLS){
            b200::note(device, b200rl_fill(m._data, (size_t)SPEC::ROWS * SPEC::COLS, (float)value, device.stream));
        }
        else{
            for(typename SPEC::TI r = 0; r < SPEC::ROWS; r++) b200::note(device, b200rl_fill(m._data + r * rl_tools::b200::ld(m), SPEC::COLS, (float)value, device.stream));
        }
    }
    template<typename DEV_SPEC, typename SPEC>
    void set_all(devices::B200<DEV_SPEC>& device, Tensor<SPEC>& t, typename SPEC::T value){
        static_assert(utils::typing::is_same_v<typename SPEC::T, float>, "fp32 only");
        static_assert(tensor::dense_row_major_layout<SPEC>(), "only dense tensors");
        b200::note(device, b200rl_fill(t._data, SPEC::SIZE, value, device.stream));
    }

    // containers/matrix/operations_cuda.h:197-223 draws on the device engines; here the draws come from the caller's HOST engine through
    // the reference's own normal_distribution::sample, in the generic randn's order (containers/matrix/operations_generic.h:631-639), so
    // that a matrix filled on this device equals the one the CPU device fills from the same engine state
    template<typename DEV_SPEC, typename SPEC, typename RNG>
    void randn(devices::B200<DEV_SPEC>& device, Matrix<SPEC>& m, RNG& rng){
        using T = typename SPEC::T;
        static_assert(utils::typing::is_same_v<T, float> && SPEC::COL_PITCH == 1, "fp32, column pitch 1");
        std::vector<T> host((size_t)SPEC::ROWS * SPEC::COLS);
        for(size_t i = 0; i < host.size(); i++) host[i] = random::normal_distribution::sample(device.random, (T)0, (T)1, rng);
        b200::note(device, b200rl_memcpy_2d(m._data, rl_tools::b200::ld(m) * sizeof(T), host.data(), SPEC::COLS * sizeof(T), SPEC::COLS * sizeof(T), SPEC::ROWS, 0, device.stream));
    }

    // ---- dense layer: nn/layers/dense/operations_cuda.h:236-413 ---------------------------------------------------
    namespace b200{
        template <nn::activation_functions::ActivationFunction F>
        constexpr int activation_id(){
            using namespace nn::activation_functions;
            static_assert(F == IDENTITY || F == RELU || F == TANH || F == FAST_TANH || F == SIGMOID, "activation not supported by libb200rl");
            return F == IDENTITY ? B200RL_ACT_IDENTITY : F == RELU ? B200RL_ACT_RELU : F == TANH ? B200RL_ACT_TANH : F == FAST_TANH ? B200RL_ACT_FAST_TANH : B200RL_ACT_SIGMOID;
        }
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename OUTPUT_SPEC, typename RNG, typename MODE = mode::Default<>>
    void evaluate(devices::B200<DEV_SPEC>& device, const nn::layers::dense::LayerForward<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<OUTPUT_SPEC>& output,
                  nn::layers::dense::Buffer&, RNG&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(nn::layers::dense::check_input_output<LAYER_SPEC, INPUT_SPEC, OUTPUT_SPEC>);
        static_assert(INPUT_SPEC::COL_PITCH == 1 && OUTPUT_SPEC::COL_PITCH == 1);
        b200::note(device, b200rl_dense_forward(layer.weights.parameters._data, layer.biases.parameters._data, input._data, rl_tools::b200::ld(input), nullptr, 0,
                                                output._data, rl_tools::b200::ld(output), INPUT_SPEC::ROWS, LAYER_SPEC::INPUT_DIM, LAYER_SPEC::OUTPUT_DIM,
                                                b200::activation_id<LAYER_SPEC::ACTIVATION_FUNCTION>(), device.stream));
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename OUTPUT_SPEC, typename RNG, typename MODE = mode::Default<>>
    void forward(devices::B200<DEV_SPEC>& device, nn::layers::dense::LayerBackward<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<OUTPUT_SPEC>& output,
                 nn::layers::dense::Buffer&, RNG&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(nn::layers::dense::check_input_output<LAYER_SPEC, INPUT_SPEC, OUTPUT_SPEC>);
        static_assert(INPUT_SPEC::COL_PITCH == 1 && OUTPUT_SPEC::COL_PITCH == 1);
        b200::note(device, b200rl_dense_forward(layer.weights.parameters._data, layer.biases.parameters._data, input._data, rl_tools::b200::ld(input),
                                                layer.pre_activations._data, rl_tools::b200::ld(layer.pre_activations), output._data, rl_tools::b200::ld(output),
                                                INPUT_SPEC::ROWS, LAYER_SPEC::INPUT_DIM, LAYER_SPEC::OUTPUT_DIM, b200::activation_id<LAYER_SPEC::ACTIVATION_FUNCTION>(), device.stream));
    }
    namespace b200{
        // the reference's signatures carry no scratch buffer, so the allocation-free entry point is used
        template<typename DEVICE, typename LAYER, typename INPUT_SPEC, typename D_OUTPUT_SPEC>
        void dense_backward(DEVICE& device, LAYER& layer, const float* input, unsigned input_pitch, Matrix<D_OUTPUT_SPEC>& d_output, float* d_W, float* d_b, float* d_input, unsigned d_input_pitch, const Matrix<INPUT_SPEC>*){
            using LAYER_SPEC = typename LAYER::SPEC;
            note(device, b200rl_dense_backward_static_scratch(layer.weights.parameters._data, input, input_pitch, layer.pre_activations._data, rl_tools::b200::ld(layer.pre_activations),
                                                              d_output._data, rl_tools::b200::ld(d_output), d_W, d_b, d_input, d_input_pitch, D_OUTPUT_SPEC::ROWS, LAYER_SPEC::INPUT_DIM,
                                                              LAYER_SPEC::OUTPUT_DIM, activation_id<LAYER_SPEC::ACTIVATION_FUNCTION>(), device.stream));
        }
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename D_OUTPUT_SPEC, typename D_INPUT_SPEC, typename MODE = mode::Default<>>
    void backward_input(devices::B200<DEV_SPEC>& device, nn::layers::dense::LayerBackward<LAYER_SPEC>& layer, Matrix<D_OUTPUT_SPEC>& d_output, Matrix<D_INPUT_SPEC>& d_input,
                        nn::layers::dense::Buffer&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(nn::layers::dense::check_input_output<LAYER_SPEC, D_INPUT_SPEC, D_OUTPUT_SPEC>);
        b200::dense_backward(device, layer, nullptr, 0, d_output, nullptr, nullptr, d_input._data, rl_tools::b200::ld(d_input), (const Matrix<D_INPUT_SPEC>*)nullptr);
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename D_OUTPUT_SPEC, typename MODE = mode::Default<>>
    void backward(devices::B200<DEV_SPEC>& device, nn::layers::dense::LayerGradient<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<D_OUTPUT_SPEC>& d_output,
                  nn::layers::dense::Buffer&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(nn::layers::dense::check_input_output<LAYER_SPEC, INPUT_SPEC, D_OUTPUT_SPEC>);
        b200::dense_backward(device, layer, input._data, rl_tools::b200::ld(input), d_output, layer.weights.gradient._data, layer.biases.gradient._data, nullptr, 0, &input);
    }
    template<typename DEV_SPEC, typename LAYER_SPEC, typename INPUT_SPEC, typename D_OUTPUT_SPEC, typename D_INPUT_SPEC, typename MODE = mode::Default<>>
    void backward_full(devices::B200<DEV_SPEC>& device, nn::layers::dense::LayerGradient<LAYER_SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<D_OUTPUT_SPEC>& d_output,
                       Matrix<D_INPUT_SPEC>& d_input, nn::layers::dense::Buffer&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(nn::layers::dense::check_input_output<LAYER_SPEC, INPUT_SPEC, D_OUTPUT_SPEC>);
        b200::dense_backward(device, layer, input._data, rl_tools::b200::ld(input), d_output, layer.weights.gradient._data, layer.biases.gradient._data, d_input._data, rl_tools::b200::ld(d_input), &input);
    }

    // ---- MSE: nn/loss_functions/mse/operations_cuda.h:41-58 -------------------------------------------------------
    namespace nn::loss_functions::mse{
        template<typename DEV_SPEC, typename SPEC_A, typename SPEC_B, typename SPEC_DA>
        void gradient(devices::B200<DEV_SPEC>& device, Matrix<SPEC_A>& a, Matrix<SPEC_B>& b, Matrix<SPEC_DA>& d_a, typename SPEC_A::T loss_weight = 1){
            static_assert(containers::check_structure<SPEC_A, SPEC_B> && containers::check_structure<SPEC_A, SPEC_DA>);
            rl_tools::b200::note(device, b200rl_mse_gradient(a._data, rl_tools::b200::ld(a), b._data, rl_tools::b200::ld(b), d_a._data, rl_tools::b200::ld(d_a), SPEC_A::ROWS, SPEC_A::COLS, loss_weight, device.stream));
        }
        // nn/loss_functions/mse/operations_generic.h:9-22 (the reference has no CUDA form: its generic loop would read device memory on the host)
        template<typename DEV_SPEC, typename SPEC_A, typename SPEC_B>
        typename SPEC_A::T evaluate(devices::B200<DEV_SPEC>& device, Matrix<SPEC_A>& a, Matrix<SPEC_B>& b, typename SPEC_A::T loss_weight = 1){
            static_assert(containers::check_structure<SPEC_A, SPEC_B>);
            float loss = 0;
            rl_tools::b200::note(device, b200rl_mse_evaluate(a._data, rl_tools::b200::ld(a), b._data, rl_tools::b200::ld(b), SPEC_A::ROWS, SPEC_A::COLS, loss_weight, &loss, device.stream));
            return loss;
        }
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END

#include <b200rl/rl_tools_adam.h>
