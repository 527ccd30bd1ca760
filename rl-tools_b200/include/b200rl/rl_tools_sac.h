// Header-only adapter, SAC part: everything the reference's generic `train_critic`, `update_critic_targets` and `train_actor`
// (rl/algorithms/sac/operations_generic.h:243-336, 486-522, 378-456) need so that they run UNCHANGED on `devices::B200` -- the same set of
// overloads the reference's own CUDA device adds (rl/algorithms/sac/operations_cuda.h, nn/layers/sample_and_squash/operations_cuda.h,
// containers/tensor/operations_cuda.h), each a call into libb200rl.so instead of a kernel compiled on the user's side:
//   sample_and_squash layer   evaluate / forward / backward_full with external noise
//   SAC                       target_action_values, min_value_d_output, mask_actions, mask_gradient
//   tensors                   cast_reduce_sum, scale, set_all(tensor, one-element tensor), copy of row-pitched views
//   MSE                       gradient with the loss weight in a one-element device tensor
//
// Include AFTER the model headers (nn_models/mlp, nn_models/sequential: `output(device, model)` must be visible here) and BEFORE
// <rl_tools/rl/algorithms/sac/operations_generic.h>: `min_value_d_output` takes no Matrix / Tensor argument and the MSE gradient is called
// by its qualified name there, so neither is found by argument-dependent lookup from inside the reference's templates unless declared first.
//
// Scope: sequence length 1 (every step of the batch is a final step and a reset, the configuration of the reference's SAC loops for
// feed-forward policies). The masks are honoured row by row as the reference does; the log_alpha gradient is divided by the number of rows,
// which equals the reference's number of resets in that configuration.
#pragma once
#include <b200rl/rl_tools_device.h>
#include <b200rl/rl_tools_adam.h>                    // the generic init / train_* call init, reset_optimizer_state and step for the caller
#include <rl_tools/nn/layers/sample_and_squash/layer.h>
#include <rl_tools/nn/layers/gru/layer.h>
#include <rl_tools/rl/components/off_policy_runner/off_policy_runner.h>
#include <rl_tools/rl/algorithms/sac/sac.h>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    namespace b200{
        template<typename SPEC> constexpr bool is_mask(){ return sizeof(typename SPEC::T) == 1 && tensor::dense_row_major_layout<SPEC>(); }
    }

    // ---- tensors: containers/tensor/operations_cuda.h:308-357 ---------------------------------------------------------------------
    template<typename TARGET_TYPE, typename DEV_SPEC, typename SPEC, typename RESULT_SPEC>
    void cast_reduce_sum(devices::B200<DEV_SPEC>& device, const Tensor<SPEC>& t, Tensor<RESULT_SPEC>& result){
        static_assert(RESULT_SPEC::SHAPE::LENGTH == 1 && RESULT_SPEC::SHAPE::template GET<0> == 1);
        static_assert(utils::typing::is_same_v<TARGET_TYPE, float> && utils::typing::is_same_v<typename RESULT_SPEC::T, float>, "fp32 result");
        static_assert(b200::is_mask<SPEC>(), "a dense tensor of one-byte flags");
        b200::note(device, b200rl_mask_count(reinterpret_cast<const uint8_t*>(t._data), SPEC::SIZE, result._data, device.stream));
    }
    template<typename DEV_SPEC, typename SPEC>
    void scale(devices::B200<DEV_SPEC>& device, Tensor<SPEC>& t, typename SPEC::T factor, bool reciprocal = false){
        static_assert(utils::typing::is_same_v<typename SPEC::T, float> && tensor::dense_row_major_layout<SPEC>(), "dense fp32 tensors");
        b200::note(device, b200rl_scale(t._data, SPEC::SIZE, factor, reciprocal ? 1 : 0, device.stream));
    }
    template<typename DEV_SPEC, typename SPEC, typename VALUE_SPEC>
    void set_all(devices::B200<DEV_SPEC>& device, Tensor<SPEC>& t, Tensor<VALUE_SPEC>& value){
        static_assert(VALUE_SPEC::SHAPE::LENGTH == 1 && VALUE_SPEC::SHAPE::template GET<0> == 1);
        static_assert(utils::typing::is_same_v<typename SPEC::T, float> && tensor::dense_row_major_layout<SPEC>(), "dense fp32 tensors");
        b200::note(device, b200rl_fill_from_device(t._data, SPEC::SIZE, value._data, device.stream));
    }

    // ---- MSE with a device-resident loss weight: nn/loss_functions/mse/operations_generic.h:66-86 ------------------------------------
    namespace nn::loss_functions::mse{
        template<typename DEV_SPEC, typename SPEC_A, typename SPEC_B, typename SPEC_DA, typename LOSS_WEIGHT_SPEC>
        void gradient(devices::B200<DEV_SPEC>& device, Matrix<SPEC_A>& a, Matrix<SPEC_B>& b, Matrix<SPEC_DA>& d_a, Tensor<LOSS_WEIGHT_SPEC>& loss_weight){
            static_assert(containers::check_structure<SPEC_A, SPEC_B> && containers::check_structure<SPEC_A, SPEC_DA>);
            static_assert(LOSS_WEIGHT_SPEC::SHAPE::LENGTH == 1 && LOSS_WEIGHT_SPEC::SHAPE::template GET<0> == 1, "a one-element loss weight");
            rl_tools::b200::note(device, b200rl_mse_gradient_dev_weight(a._data, rl_tools::b200::ld(a), b._data, rl_tools::b200::ld(b), d_a._data, rl_tools::b200::ld(d_a), SPEC_A::ROWS, SPEC_A::COLS,
                                                                        loss_weight._data, device.stream));
        }
    }

    // ---- sample-and-squash layer: nn/layers/sample_and_squash/operations_cuda.h:14-119 --------------------------------------------------
    namespace b200{
        template<typename PARAMETERS>
        constexpr bool default_head_parameters(){
            return PARAMETERS::LOG_STD_LOWER_BOUND == -20 && PARAMETERS::LOG_STD_UPPER_BOUND == 2 && (float)PARAMETERS::LOG_PROBABILITY_EPSILON == 1e-6f;
        }
    }
    template <typename DEV_SPEC, typename SPEC, typename INPUT_SPEC, typename OUTPUT_SPEC, typename BUFFER_SPEC, typename RNG, typename MODE = mode::Default<>>
    void evaluate(devices::B200<DEV_SPEC>& device, const nn::layers::sample_and_squash::LayerForward<SPEC>&, const Matrix<INPUT_SPEC>& input, Matrix<OUTPUT_SPEC>& output,
                  nn::layers::sample_and_squash::Buffer<BUFFER_SPEC>& buffer, RNG&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(mode::is<MODE, nn::layers::sample_and_squash::mode::ExternalNoise>, "the noise comes from buffer.noise (fill it with randn on the device tag)");
        static_assert(INPUT_SPEC::COLS == 2 * SPEC::DIM && OUTPUT_SPEC::COLS == SPEC::DIM && INPUT_SPEC::ROWS == OUTPUT_SPEC::ROWS);
        static_assert(b200::default_head_parameters<typename SPEC::PARAMETERS>(), "libb200rl implements the default clamp bounds and epsilon");
        b200::note(device, b200rl_sample_and_squash_forward(input._data, rl_tools::b200::ld(input), buffer.noise._data, rl_tools::b200::ld(buffer.noise), INPUT_SPEC::ROWS, SPEC::DIM, nullptr,
                                                            output._data, rl_tools::b200::ld(output), buffer.log_probabilities._data, device.stream));
    }
    template <typename DEV_SPEC, typename SPEC, typename INPUT_SPEC, typename BUFFER_SPEC, typename RNG, typename MODE = mode::Default<>>
    void forward(devices::B200<DEV_SPEC>& device, nn::layers::sample_and_squash::LayerGradient<SPEC>& layer, const Matrix<INPUT_SPEC>& input,
                 nn::layers::sample_and_squash::Buffer<BUFFER_SPEC>& buffer, RNG&, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(mode::is<MODE, nn::layers::sample_and_squash::mode::ExternalNoise>, "the noise comes from buffer.noise (fill it with randn on the device tag)");
        static_assert(INPUT_SPEC::COLS == 2 * SPEC::DIM && INPUT_SPEC::ROWS == SPEC::INTERNAL_BATCH_SIZE);
        static_assert(b200::default_head_parameters<typename SPEC::PARAMETERS>(), "libb200rl implements the default clamp bounds and epsilon");
        copy(device, device, buffer.noise, layer.noise);
        b200::note(device, b200rl_sample_and_squash_forward(input._data, rl_tools::b200::ld(input), layer.noise._data, rl_tools::b200::ld(layer.noise), INPUT_SPEC::ROWS, SPEC::DIM,
                                                            layer.pre_squashing._data, layer.output._data, rl_tools::b200::ld(layer.output), layer.log_probabilities._data, device.stream));
        static_assert(decltype(layer.pre_squashing)::ROW_PITCH == SPEC::DIM, "pre_squashing is dense");
    }
    template<typename DEV_SPEC, typename SPEC, typename INPUT_SPEC, typename D_OUTPUT_SPEC, typename D_INPUT_SPEC, typename BUFFER_SPEC, typename MODE = mode::Default<>>
    void backward_full(devices::B200<DEV_SPEC>& device, nn::layers::sample_and_squash::LayerGradient<SPEC>& layer, const Matrix<INPUT_SPEC>& input, Matrix<D_OUTPUT_SPEC>& d_output,
                       Matrix<D_INPUT_SPEC>& d_input, nn::layers::sample_and_squash::Buffer<BUFFER_SPEC>& buffer, const Mode<MODE>& = Mode<mode::Default<>>{}){
        static_assert(!mode::is<MODE, nn::layers::sample_and_squash::mode::DisableEntropy>, "the entropy term is always on");
        static_assert(INPUT_SPEC::ROWS == SPEC::INTERNAL_BATCH_SIZE && D_INPUT_SPEC::COLS == 2 * SPEC::DIM && D_OUTPUT_SPEC::COLS == SPEC::DIM);
        static_assert(b200::default_head_parameters<typename SPEC::PARAMETERS>(), "libb200rl implements the default clamp bounds and epsilon");
        b200::note(device, b200rl_sample_and_squash_backward(input._data, rl_tools::b200::ld(input), layer.noise._data, rl_tools::b200::ld(layer.noise), layer.pre_squashing._data,
                                                             layer.output._data, rl_tools::b200::ld(layer.output), d_output._data, rl_tools::b200::ld(d_output), layer.log_alpha.parameters._data,
                                                             (float)SPEC::PARAMETERS::TARGET_ENTROPY, INPUT_SPEC::ROWS, SPEC::DIM, d_input._data, rl_tools::b200::ld(d_input),
                                                             buffer.d_log_alpha._data, layer.log_alpha.gradient._data, device.stream));
    }

    // ---- SAC: rl/algorithms/sac/operations_cuda.h:11-127 ---------------------------------------------------------------------------------
    template <typename DEV_SPEC, typename BATCH_SPEC, typename TRAINING_BUFFER_SPEC, typename NEXT_ACTION_LOG_PROBS_SPEC, typename LOG_ALPHA_PARAMETER>
    void target_action_values(devices::B200<DEV_SPEC>& device, rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>& batch,
                              rl::algorithms::sac::CriticTrainingBuffers<TRAINING_BUFFER_SPEC>& training_buffers, const Matrix<NEXT_ACTION_LOG_PROBS_SPEC>& next_action_log_probs,
                              LOG_ALPHA_PARAMETER& log_alpha){
        using SPEC = typename TRAINING_BUFFER_SPEC::SPEC;
        using PARAMETERS = typename SPEC::PARAMETERS;
        using BATCH = rl::components::off_policy_runner::SequentialBatch<BATCH_SPEC>;
        static_assert(BATCH::SEQUENCE_LENGTHH == 1 && !BATCH_SPEC::PARAMETERS::INCLUDE_FIRST_STEP_IN_TARGETS, "sequence length 1");
        static_assert(NEXT_ACTION_LOG_PROBS_SPEC::ROWS == 1 && NEXT_ACTION_LOG_PROBS_SPEC::COLS == BATCH::BATCH_SIZE);
        auto q1 = matrix_view(device, training_buffers.next_state_action_value_critic_1);
        auto q2 = matrix_view(device, training_buffers.next_state_action_value_critic_2);
        auto target = matrix_view(device, training_buffers.target_action_value);
        static_assert(sizeof(*batch.terminated._data) == 1, "one-byte flags");
        b200::note(device, b200rl_sac_target_action_values(q1._data, rl_tools::b200::ld(q1), q2._data, rl_tools::b200::ld(q2), batch.rewards._data,
                                                           reinterpret_cast<const uint8_t*>(batch.terminated._data), next_action_log_probs._data, log_alpha.parameters._data,
                                                           (float)PARAMETERS::GAMMA, PARAMETERS::IGNORE_TERMINATION ? 1 : 0, PARAMETERS::ENTROPY_BONUS ? 1 : 0,
                                                           PARAMETERS::ENTROPY_BONUS_NEXT_STEP ? 1 : 0, target._data, rl_tools::b200::ld(target), BATCH::BATCH_SIZE, device.stream));
    }
    template <typename DEV_SPEC, typename SPEC, typename TRAINING_BUFFERS_SPEC>
    void min_value_d_output(devices::B200<DEV_SPEC>& device, rl::algorithms::sac::ActorCritic<SPEC>& actor_critic, rl::algorithms::sac::ActorTrainingBuffers<TRAINING_BUFFERS_SPEC>& training_buffers){
        using BUFFERS = rl::algorithms::sac::ActorTrainingBuffers<TRAINING_BUFFERS_SPEC>;
        using TI = typename devices::B200<DEV_SPEC>::index_t;
        constexpr TI CRITIC_INPUT_DIM = get_last(typename SPEC::CRITIC_NETWORK_TYPE::INPUT_SHAPE{});
        constexpr TI ACTION_DIM = SPEC::ENVIRONMENT::ACTION_DIM;
        auto q1_tensor = output(device, actor_critic.critics[0]);
        auto q2_tensor = output(device, actor_critic.critics[1]);
        auto q1 = matrix_view(device, q1_tensor);
        auto q2 = matrix_view(device, q2_tensor);
        auto d1 = matrix_view(device, training_buffers.d_critic_1_input);
        auto d2 = matrix_view(device, training_buffers.d_critic_2_input);
        auto d_actor = matrix_view(device, training_buffers.d_actor_output_squashing);
        static_assert(decltype(d1)::ROW_PITCH == decltype(d2)::ROW_PITCH);
        b200::note(device, b200rl_sac_min_value_d_output(q1._data, rl_tools::b200::ld(q1), q2._data, rl_tools::b200::ld(q2), d1._data, d2._data, rl_tools::b200::ld(d1), CRITIC_INPUT_DIM - ACTION_DIM,
                                                         ACTION_DIM, d_actor._data, rl_tools::b200::ld(d_actor), SPEC::PARAMETERS::SEQUENCE_LENGTH * BUFFERS::BATCH_SIZE, device.stream));
    }
    template <typename DEV_SPEC, typename SOURCE_SPEC, typename TARGET_SPEC, typename MASK_SPEC>
    void mask_actions(devices::B200<DEV_SPEC>& device, Tensor<SOURCE_SPEC>& source, Tensor<TARGET_SPEC>& target, Tensor<MASK_SPEC>& mask, bool invert_mask = false){
        static_assert(tensor::same_dimensions<SOURCE_SPEC, TARGET_SPEC>() && b200::is_mask<MASK_SPEC>());
        using S = b200::Rows<SOURCE_SPEC>; using D = b200::Rows<TARGET_SPEC>;
        static_assert(b200::Rows<MASK_SPEC>::ROWS * b200::Rows<MASK_SPEC>::COLS == S::ROWS, "one flag per (sequence step, batch element)");
        b200::note(device, b200rl_mask_rows(source._data, S::PITCH, target._data, D::PITCH, reinterpret_cast<const uint8_t*>(mask._data), S::ROWS, S::COLS, invert_mask ? 1 : 0,
                                            device.stream));
    }
    template <typename DEV_SPEC, typename SOURCE_SPEC, typename MASK_SPEC>
    void mask_gradient(devices::B200<DEV_SPEC>& device, Tensor<SOURCE_SPEC>& gradient, Tensor<MASK_SPEC>& mask, bool invert_mask = false){
        static_assert(b200::is_mask<MASK_SPEC>());
        using D = b200::Rows<SOURCE_SPEC>;
        static_assert(b200::Rows<MASK_SPEC>::ROWS * b200::Rows<MASK_SPEC>::COLS == D::ROWS, "one flag per (sequence step, batch element)");
        b200::note(device, b200rl_mask_rows(nullptr, 0, gradient._data, D::PITCH, reinterpret_cast<const uint8_t*>(mask._data), D::ROWS, D::COLS, invert_mask ? 1 : 0, device.stream));
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
