// Header-only adapter, whole-model part: nn_models::mlp on `devices::B200` as ONE arena and one C-ABI call per verb.
//
// Include after <b200rl/rl_tools_device.h> and BEFORE <rl_tools/nn_models/mlp/operations_generic.h> (and every model header that recurses
// into an MLP, e.g. nn_models/sequential): calls such as malloc(device, content) or update(device, network, optimizer) inside the
// reference's generic code carry no argument whose type lives directly in namespace rl_tools, so they only see overloads that were
// declared earlier (the same ordering rule the reference states at the top of nn/optimizers/adam/adam.h).
//
// What it replaces, and with what:
//   malloc / free (nn_models/mlp/operations_generic.h:11-26, one allocation per tensor: 8 per layer with Adam) -> ONE device allocation
//       per network; the reference's per-tensor containers are bound into it, so every per-tensor operation of the reference (copy,
//       the per-layer dense overloads, persistence walks) keeps working on the same memory. Order inside the arena: for each layer
//       W [O, I] then b [O] -- the layout of b200rl_mlp_shape -- repeated for gradients and both Adam moments; then the stored
//       pre-activations and outputs, layer after layer, each [batch, O] dense; then the split-batch scratch of the backward pass and the
//       workspace of the forward pass.
//   evaluate / forward / backward / backward_full / backward_input (:77-204)   -> b200rl_mlp_evaluate / _forward / _backward
//   zero_gradient (:122-129), _reset_optimizer_state (:219-228)                 -> one b200rl_fill per arena
//   update (:210-217: one kernel per parameter tensor)                          -> ONE b200rl_adam_update_dev over the flat arena
// A network whose tensors are not laid out this way (bound by hand, or a pitch that is not dense) takes the layer-by-layer path of
// rl_tools_operations.h, which gives the same results.
#pragma once
#include "rl_tools_device.h"
#include <rl_tools/nn_models/mlp/network.h>

RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    namespace b200::mlp{
        constexpr size_t SECTION_ALIGN = 64;            // floats: every section of the arena starts on a 256-byte boundary
        constexpr size_t section(size_t n){ return (n + SECTION_ALIGN - 1) / SECTION_ALIGN * SECTION_ALIGN; }

        template <typename SPEC>
        struct Layout{
            using TI = typename SPEC::TI;
            static constexpr bool HAS_PRE = SPEC::CAPABILITY::TAG != nn::LayerCapability::Forward;
            static constexpr bool HAS_OUT = SPEC::CAPABILITY::TAG == nn::LayerCapability::Gradient;
            static constexpr bool HAS_GRAD = !utils::typing::is_same_v<typename SPEC::CAPABILITY::PARAMETER_TYPE, nn::parameters::Plain>;
            static constexpr bool HAS_ADAM = utils::typing::is_same_v<typename SPEC::CAPABILITY::PARAMETER_TYPE, nn::parameters::Adam>;
            static constexpr size_t N = SPEC::INPUT_LAYER::NUM_WEIGHTS + SPEC::HIDDEN_LAYER::NUM_WEIGHTS * SPEC::NUM_HIDDEN_LAYERS + SPEC::OUTPUT_LAYER::NUM_WEIGHTS;
            static constexpr size_t BATCH = SPEC::INTERNAL_BATCH_SIZE;
            static constexpr size_t ACTS = BATCH * ((size_t)SPEC::HIDDEN_DIM * (SPEC::NUM_LAYERS - 1) + SPEC::OUTPUT_DIM);
            static constexpr size_t OFF_PARAMS = 0;
            static constexpr size_t OFF_GRADS = OFF_PARAMS + section(N);
            static constexpr size_t OFF_M = OFF_GRADS + (HAS_GRAD ? section(N) : 0);
            static constexpr size_t OFF_V = OFF_M + (HAS_ADAM ? section(N) : 0);
            static constexpr size_t OFF_PRE = OFF_V + (HAS_ADAM ? section(N) : 0);
            static constexpr size_t OFF_OUT = OFF_PRE + (HAS_PRE ? section(ACTS) : 0);
            static constexpr size_t OFF_SCRATCH = OFF_OUT + (HAS_OUT ? section(ACTS) : 0);
            static b200rl_mlp_shape shape(){
                b200rl_mlp_shape s{};
                s.n_layers = SPEC::NUM_LAYERS; s.input_dim = SPEC::INPUT_DIM;
                for(TI l = 0; l < SPEC::NUM_LAYERS; l++){
                    const bool last = l + 1 == SPEC::NUM_LAYERS;
                    s.dims[l] = last ? SPEC::OUTPUT_DIM : SPEC::HIDDEN_DIM;
                    s.acts[l] = last ? activation_code(SPEC::OUTPUT_ACTIVATION_FUNCTION) : activation_code(SPEC::HIDDEN_ACTIVATION_FUNCTION);
                }
                return s;
            }
            static constexpr int activation_code(nn::activation_functions::ActivationFunction f){
                using namespace nn::activation_functions;
                return f == IDENTITY ? B200RL_ACT_IDENTITY : f == RELU ? B200RL_ACT_RELU : f == TANH ? B200RL_ACT_TANH : f == FAST_TANH ? B200RL_ACT_FAST_TANH : f == SIGMOID ? B200RL_ACT_SIGMOID : -1;
            }
            static constexpr bool SUPPORTED = SPEC::NUM_LAYERS <= B200RL_MAX_LAYERS && activation_code(SPEC::OUTPUT_ACTIVATION_FUNCTION) >= 0 && activation_code(SPEC::HIDDEN_ACTIVATION_FUNCTION) >= 0;
            static size_t scratch_bytes(){
                if constexpr(!HAS_GRAD) return 0;
                else{ const b200rl_mlp_shape s = shape(); return (b200rl_mlp_backward_scratch_bytes(&s, (int)BATCH) + 255) / 256 * 256; }
            }
            // forward workspace (the weights' tensor-core operand image of the layer in flight; 0 for small batches), behind the scratch
            static size_t workspace_bytes(){ const b200rl_mlp_shape s = shape(); return b200rl_mlp_forward_workspace_bytes(&s, (int)BATCH); }
        };

        // one parameter tensor and whatever optimizer state its type carries
        template <typename S> void bind_parameter(nn::parameters::Plain::Instance<S>& p, float* params, float*, float*, float*){ p.parameters._data = params; }
        template <typename S> void bind_parameter(nn::parameters::Gradient::Instance<S>& p, float* params, float* grads, float*, float*){ p.parameters._data = params; p.gradient._data = grads; }
        template <typename S> void bind_parameter(nn::parameters::Adam::Instance<S>& p, float* params, float* grads, float* m, float* v){
            p.parameters._data = params; p.gradient._data = grads; p.gradient_first_order_moment._data = m; p.gradient_second_order_moment._data = v;
        }
        template <typename S> void bind_activations(nn::layers::dense::LayerForward<S>&, float*, float*){}
        template <typename S> void bind_activations(nn::layers::dense::LayerBackward<S>& l, float* pre, float*){ l.pre_activations._data = pre; }
        template <typename S> void bind_activations(nn::layers::dense::LayerGradient<S>& l, float* pre, float* out){ l.pre_activations._data = pre; l.output._data = out; }

        template <typename NETWORK, typename F>
        void for_each_layer(NETWORK& network, F&& f){
            f(network.input_layer);
            for(typename NETWORK::TI i = 0; i < NETWORK::NUM_HIDDEN_LAYERS; i++) f(network.hidden_layers[i]);
            f(network.output_layer);
        }
        // points every tensor of the network into the arena at `base` (nullptr unbinds)
        template <typename SPEC>
        void bind(nn_models::mlp::NeuralNetworkForward<SPEC>& network, float* base){
            using L = Layout<SPEC>;
            size_t p = 0, a = 0;
            for_each_layer(network, [&](auto& layer){
                using LAYER = utils::typing::remove_reference_t<decltype(layer)>;
                constexpr size_t W = (size_t)LAYER::OUTPUT_DIM * LAYER::INPUT_DIM, B = LAYER::OUTPUT_DIM;
                auto at = [&](size_t section_offset, size_t off) -> float* { return base ? base + section_offset + off : nullptr; };
                bind_parameter(layer.weights, at(L::OFF_PARAMS, p), at(L::OFF_GRADS, p), at(L::OFF_M, p), at(L::OFF_V, p));
                bind_parameter(layer.biases, at(L::OFF_PARAMS, p + W), at(L::OFF_GRADS, p + W), at(L::OFF_M, p + W), at(L::OFF_V, p + W));
                bind_activations(layer, at(L::OFF_PRE, a), at(L::OFF_OUT, a));
                p += W + B; a += L::BATCH * B;
            });
        }
        // the arena a network lives in, or base == nullptr when its tensors are not laid out as bind() lays them out
        template <typename SPEC>
        struct Arena{
            using L = Layout<SPEC>;
            float* base = nullptr;
            float* params() const { return base + L::OFF_PARAMS; }
            float* grads() const { return base + L::OFF_GRADS; }
            float* m() const { return base + L::OFF_M; }
            float* v() const { return base + L::OFF_V; }
            float* pre() const { return base + L::OFF_PRE; }
            float* out() const { return base + L::OFF_OUT; }
            void* scratch() const { return base + L::OFF_SCRATCH; }
            void* workspace() const { return reinterpret_cast<char*>(base + L::OFF_SCRATCH) + L::scratch_bytes(); }
            explicit operator bool() const { return base != nullptr; }
        };
        template <typename S> bool parameter_at(const nn::parameters::Plain::Instance<S>& p, const float* params, const float*, const float*, const float*){ return p.parameters._data == params; }
        template <typename S> bool parameter_at(const nn::parameters::Gradient::Instance<S>& p, const float* params, const float* grads, const float*, const float*){
            return p.parameters._data == params && p.gradient._data == grads;
        }
        template <typename S> bool parameter_at(const nn::parameters::Adam::Instance<S>& p, const float* params, const float* grads, const float* m, const float* v){
            return p.parameters._data == params && p.gradient._data == grads && p.gradient_first_order_moment._data == m && p.gradient_second_order_moment._data == v;
        }
        template <typename S> bool activations_at(const nn::layers::dense::LayerForward<S>&, const float*, const float*){ return true; }
        template <typename S> bool activations_at(const nn::layers::dense::LayerBackward<S>& l, const float* pre, const float*){ return l.pre_activations._data == pre && rl_tools::b200::ld(l.pre_activations) == S::OUTPUT_DIM; }
        template <typename S> bool activations_at(const nn::layers::dense::LayerGradient<S>& l, const float* pre, const float* out){
            return l.pre_activations._data == pre && l.output._data == out && rl_tools::b200::ld(l.pre_activations) == S::OUTPUT_DIM && rl_tools::b200::ld(l.output) == S::OUTPUT_DIM;
        }
        template <typename SPEC>
        Arena<SPEC> arena_of(const nn_models::mlp::NeuralNetworkForward<SPEC>& network){
            using L = Layout<SPEC>;
            Arena<SPEC> arena;
            if constexpr(!L::SUPPORTED || !utils::typing::is_same_v<typename SPEC::TYPE_POLICY::DEFAULT, float>) return arena;
            float* base = const_cast<float*>(reinterpret_cast<const float*>(network.input_layer.weights.parameters._data));
            if(base == nullptr) return arena;
            bool ok = true;
            size_t p = 0, a = 0;
            for_each_layer(network, [&](const auto& layer){
                using LAYER = utils::typing::remove_cv_t<utils::typing::remove_reference_t<decltype(layer)>>;
                constexpr size_t W = (size_t)LAYER::OUTPUT_DIM * LAYER::INPUT_DIM, B = LAYER::OUTPUT_DIM;
                ok = ok && parameter_at(layer.weights, base + L::OFF_PARAMS + p, base + L::OFF_GRADS + p, base + L::OFF_M + p, base + L::OFF_V + p);
                ok = ok && parameter_at(layer.biases, base + L::OFF_PARAMS + p + W, base + L::OFF_GRADS + p + W, base + L::OFF_M + p + W, base + L::OFF_V + p + W);
                ok = ok && activations_at(layer, base + L::OFF_PRE + a, base + L::OFF_OUT + a);
                p += W + B; a += L::BATCH * B;
            });
            if(ok) arena.base = base;
            return arena;
        }
    }

    // ---- storage: nn_models/mlp/operations_generic.h:11-26 ------------------------------------------------------------------------------
    template<typename DEV_SPEC, typename SPEC>
    void malloc(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkForward<SPEC>& network){
        using L = b200::mlp::Layout<SPEC>;
        static_assert(utils::typing::is_same_v<typename SPEC::TYPE_POLICY::DEFAULT, float>, "fp32 only");
        static_assert(SPEC::CAPABILITY::DYNAMIC_ALLOCATION, "device memory is allocated dynamically");
        void* base = nullptr;
        b200::note(device, b200rl_device_malloc(&base, sizeof(float) * L::OFF_SCRATCH + L::scratch_bytes() + L::workspace_bytes()));
        b200::mlp::bind(network, static_cast<float*>(base));
    }
    template<typename DEV_SPEC, typename SPEC>
    void free(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkForward<SPEC>& network){
        b200::note(device, b200rl_device_free(network.input_layer.weights.parameters._data));       // the arena starts with the first layer's weights
        b200::mlp::bind(network, nullptr);
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END

// The verbs below call the per-layer overloads of rl_tools_operations.h when a network is not arena-backed; those are declared later, which
// is fine for calls that pass a Matrix (namespace rl_tools is then an associated namespace). zero_gradient / update / _reset_optimizer_state
// take no such argument, so their fall-back walks the layers through the functions declared right here.
RL_TOOLS_NAMESPACE_WRAPPER_START
namespace rl_tools{
    template<typename DEV_SPEC, typename MODEL_SPEC, typename INPUT_SPEC, typename OUTPUT_SPEC, typename BUFFER_MODEL_SPEC, typename RNG, typename MODE = mode::Default<>>
    void evaluate(devices::B200<DEV_SPEC>& device, const nn_models::mlp::NeuralNetworkForward<MODEL_SPEC>& network, const Matrix<INPUT_SPEC>& input, Matrix<OUTPUT_SPEC>& output,
                  nn_models::mlp::NeuralNetworkBuffers<BUFFER_MODEL_SPEC>& buffers, RNG& rng, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        static_assert(INPUT_SPEC::COLS == MODEL_SPEC::INPUT_DIM && OUTPUT_SPEC::COLS == MODEL_SPEC::OUTPUT_DIM && OUTPUT_SPEC::ROWS >= INPUT_SPEC::ROWS);
        static_assert(INPUT_SPEC::COL_PITCH == 1 && OUTPUT_SPEC::COL_PITCH == 1 && BUFFER_MODEL_SPEC::DIM >= MODEL_SPEC::HIDDEN_DIM);
        static_assert(BUFFER_MODEL_SPEC::INTERNAL_BATCH_SIZE >= INPUT_SPEC::ROWS, "the tick / tock buffers hold the hidden activations of the whole batch");
        const auto arena = b200::mlp::arena_of(network);
        if(arena){
            const b200rl_mlp_shape shape = b200::mlp::Layout<MODEL_SPEC>::shape();
            // the workspace was sized for the network's own batch; a larger evaluation batch goes without it
            const bool ws = INPUT_SPEC::ROWS <= MODEL_SPEC::INTERNAL_BATCH_SIZE;
            b200::note(device, b200rl_mlp_evaluate_ws(&shape, arena.params(), input._data, rl_tools::b200::ld(input), output._data, rl_tools::b200::ld(output), buffers.tick._data, buffers.tock._data,
                                                      INPUT_SPEC::ROWS, ws ? arena.workspace() : nullptr, ws ? b200::mlp::Layout<MODEL_SPEC>::workspace_bytes() : 0, device.stream));
            return;
        }
        // layer by layer (nn_models/mlp/operations_generic.h:77-102)
        constexpr auto BATCH = INPUT_SPEC::ROWS;
        matrix::ViewSpec<BATCH, MODEL_SPEC::HIDDEN_DIM> hidden;
        { auto to = view(device, buffers.tick, hidden); evaluate(device, network.input_layer, input, to, buffers.layer_buffer, rng, mode); }
        for(typename MODEL_SPEC::TI l = 0; l < MODEL_SPEC::NUM_HIDDEN_LAYERS; l++){
            auto from = view(device, l % 2 == 0 ? buffers.tick : buffers.tock, hidden);
            auto to = view(device, l % 2 == 0 ? buffers.tock : buffers.tick, hidden);
            evaluate(device, network.hidden_layers[l], from, to, buffers.layer_buffer, rng, mode);
        }
        auto from = view(device, MODEL_SPEC::NUM_HIDDEN_LAYERS % 2 == 0 ? buffers.tick : buffers.tock, hidden);
        evaluate(device, network.output_layer, from, output, buffers.layer_buffer, rng, mode);
    }

    template<typename DEV_SPEC, typename MODEL_SPEC, typename INPUT_SPEC, typename BUFFER_SPEC, typename RNG, typename MODE = mode::Default<>>
    void forward(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkGradient<MODEL_SPEC>& network, const Matrix<INPUT_SPEC>& input,
                 nn_models::mlp::NeuralNetworkBuffers<BUFFER_SPEC>&, RNG& rng, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        static_assert(INPUT_SPEC::COLS == MODEL_SPEC::INPUT_DIM && INPUT_SPEC::ROWS == MODEL_SPEC::INTERNAL_BATCH_SIZE && INPUT_SPEC::COL_PITCH == 1);
        const auto arena = b200::mlp::arena_of(network);
        if(arena){
            const b200rl_mlp_shape shape = b200::mlp::Layout<MODEL_SPEC>::shape();
            b200::note(device, b200rl_mlp_forward_ws(&shape, arena.params(), input._data, rl_tools::b200::ld(input), arena.pre(), arena.out(), INPUT_SPEC::ROWS,
                                                     arena.workspace(), b200::mlp::Layout<MODEL_SPEC>::workspace_bytes(), device.stream));
            return;
        }
        nn::layers::dense::Buffer layer_buffer;                 // nn_models/mlp/operations_generic.h:103-113
        forward(device, network.input_layer, input, layer_buffer, rng, mode);
        auto current = network.input_layer.output;
        for(typename MODEL_SPEC::TI l = 0; l < MODEL_SPEC::NUM_HIDDEN_LAYERS; l++){
            forward(device, network.hidden_layers[l], current, layer_buffer, rng, mode);
            current = network.hidden_layers[l].output;
        }
        forward(device, network.output_layer, current, layer_buffer, rng, mode);
    }

    namespace b200::mlp{
        // the three backward verbs differ in what they ask for: parameter gradients (grads) and / or the input gradient (d_input)
        template<typename DEVICE, typename NETWORK, typename INPUT_SPEC, typename D_OUTPUT_SPEC, typename BUFFER_MODEL_SPEC>
        bool backward_arena(DEVICE& device, NETWORK& network, const Matrix<INPUT_SPEC>* input, Matrix<D_OUTPUT_SPEC>& d_output, float* d_input, unsigned d_input_pitch, bool want_grads,
                            nn_models::mlp::NeuralNetworkBuffers<BUFFER_MODEL_SPEC>& buffers){
            using MODEL_SPEC = typename NETWORK::SPEC;
            using L = Layout<MODEL_SPEC>;
            const auto arena = arena_of(network);
            // the C entry points take a dense d_output and a dense d_input
            if(!arena || rl_tools::b200::ld(d_output) != D_OUTPUT_SPEC::COLS || (d_input && d_input_pitch != MODEL_SPEC::INPUT_DIM)) return false;
            const b200rl_mlp_shape shape = L::shape();
            // backward_input needs no layer inputs: the first layer's input gradient only reads its weights; any valid pointer serves as x
            const float* x = input ? input->_data : arena.params();
            const int ldx = input ? (int)rl_tools::b200::ld(*input) : (int)MODEL_SPEC::INPUT_DIM;
            // stored layer outputs exist only on networks that can take parameter gradients; the input gradient alone does not read them
            const float* out = L::HAS_OUT ? arena.out() : arena.pre();
            if(want_grads && !L::HAS_OUT) return false;
            note(device, b200rl_mlp_backward(&shape, arena.params(), want_grads ? arena.grads() : nullptr, x, ldx, arena.pre(), out, d_output._data, d_input,
                                             buffers.tick._data, buffers.tock._data, D_OUTPUT_SPEC::ROWS, arena.scratch(), L::scratch_bytes(), device.stream));
            return true;
        }
    }
    template<typename DEV_SPEC, typename MODEL_SPEC, typename INPUT_SPEC, typename D_OUTPUT_SPEC, typename BUFFER_MODEL_SPEC, typename MODE = mode::Default<>>
    void backward(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkGradient<MODEL_SPEC>& network, const Matrix<INPUT_SPEC>& input, Matrix<D_OUTPUT_SPEC>& d_output,
                  nn_models::mlp::NeuralNetworkBuffers<BUFFER_MODEL_SPEC>& buffer, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        static_assert(BUFFER_MODEL_SPEC::INTERNAL_BATCH_SIZE == D_OUTPUT_SPEC::ROWS && BUFFER_MODEL_SPEC::DIM >= MODEL_SPEC::HIDDEN_DIM && D_OUTPUT_SPEC::ROWS == MODEL_SPEC::INTERNAL_BATCH_SIZE);
        if(b200::mlp::backward_arena(device, network, &input, d_output, nullptr, 0, true, buffer)) return;
        // layer by layer (nn_models/mlp/operations_generic.h:180-204): d_pre ping-pongs through tick / tock, the input layer gets the weights-only backward
        constexpr auto H = MODEL_SPEC::NUM_HIDDEN_LAYERS;
        auto previous = H > 0 ? network.hidden_layers[H > 0 ? H - 1 : 0].output : network.input_layer.output;
        backward_full(device, network.output_layer, previous, d_output, buffer.tick, buffer.layer_buffer, mode);
        for(typename MODEL_SPEC::TI l1 = H; l1 > 0; l1--){
            const auto l = l1 - 1;
            previous = l > 0 ? network.hidden_layers[l - 1].output : network.input_layer.output;
            if(l % 2 == (H - 1) % 2) backward_full(device, network.hidden_layers[l], previous, buffer.tick, buffer.tock, buffer.layer_buffer, mode);
            else backward_full(device, network.hidden_layers[l], previous, buffer.tock, buffer.tick, buffer.layer_buffer, mode);
        }
        backward(device, network.input_layer, input, H % 2 == 0 ? buffer.tick : buffer.tock, buffer.layer_buffer, mode);
    }
    template<typename DEV_SPEC, typename MODEL_SPEC, typename INPUT_SPEC, typename D_OUTPUT_SPEC, typename BUFFER_MODEL_SPEC, typename D_INPUT_SPEC, typename MODE = mode::Default<>>
    void backward_full(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkGradient<MODEL_SPEC>& network, const Matrix<INPUT_SPEC>& input, Matrix<D_OUTPUT_SPEC>& d_output,
                       Matrix<D_INPUT_SPEC>& d_input, nn_models::mlp::NeuralNetworkBuffers<BUFFER_MODEL_SPEC>& buffer, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        static_assert(BUFFER_MODEL_SPEC::INTERNAL_BATCH_SIZE == D_OUTPUT_SPEC::ROWS && BUFFER_MODEL_SPEC::DIM >= MODEL_SPEC::HIDDEN_DIM && D_OUTPUT_SPEC::ROWS == MODEL_SPEC::INTERNAL_BATCH_SIZE);
        if(b200::mlp::backward_arena(device, network, &input, d_output, d_input._data, rl_tools::b200::ld(d_input), true, buffer)) return;
        constexpr auto H = MODEL_SPEC::NUM_HIDDEN_LAYERS;                   // nn_models/mlp/operations_generic.h:152-179
        auto previous = H > 0 ? network.hidden_layers[H > 0 ? H - 1 : 0].output : network.input_layer.output;
        backward_full(device, network.output_layer, previous, d_output, buffer.tick, buffer.layer_buffer, mode);
        for(typename MODEL_SPEC::TI l1 = H; l1 > 0; l1--){
            const auto l = l1 - 1;
            previous = l > 0 ? network.hidden_layers[l - 1].output : network.input_layer.output;
            if(l % 2 == (H - 1) % 2) backward_full(device, network.hidden_layers[l], previous, buffer.tick, buffer.tock, buffer.layer_buffer, mode);
            else backward_full(device, network.hidden_layers[l], previous, buffer.tock, buffer.tick, buffer.layer_buffer, mode);
        }
        backward_full(device, network.input_layer, input, H % 2 == 0 ? buffer.tick : buffer.tock, d_input, buffer.layer_buffer, mode);
    }
    template<typename DEV_SPEC, typename MODEL_SPEC, typename D_OUTPUT_SPEC, typename D_INPUT_SPEC, typename BUFFER_MODEL_SPEC, typename MODE = mode::Default<>>
    void backward_input(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkBackward<MODEL_SPEC>& network, Matrix<D_OUTPUT_SPEC>& d_output, Matrix<D_INPUT_SPEC>& d_input,
                        nn_models::mlp::NeuralNetworkBuffers<BUFFER_MODEL_SPEC>& buffer, const Mode<MODE>& mode = Mode<mode::Default<>>{}){
        static_assert(BUFFER_MODEL_SPEC::INTERNAL_BATCH_SIZE == D_OUTPUT_SPEC::ROWS && BUFFER_MODEL_SPEC::DIM >= MODEL_SPEC::HIDDEN_DIM && D_OUTPUT_SPEC::ROWS == MODEL_SPEC::INTERNAL_BATCH_SIZE);
        if(b200::mlp::backward_arena(device, network, (const Matrix<D_INPUT_SPEC>*)nullptr, d_output, d_input._data, rl_tools::b200::ld(d_input), false, buffer)) return;
        constexpr auto H = MODEL_SPEC::NUM_HIDDEN_LAYERS;                   // nn_models/mlp/operations_generic.h:130-150
        backward_input(device, network.output_layer, d_output, buffer.tick, buffer.layer_buffer, mode);
        for(typename MODEL_SPEC::TI l1 = H; l1 > 0; l1--){
            const auto l = l1 - 1;
            if(l % 2 == (H - 1) % 2) backward_input(device, network.hidden_layers[l], buffer.tick, buffer.tock, buffer.layer_buffer, mode);
            else backward_input(device, network.hidden_layers[l], buffer.tock, buffer.tick, buffer.layer_buffer, mode);
        }
        backward_input(device, network.input_layer, H % 2 == 0 ? buffer.tick : buffer.tock, d_input, buffer.layer_buffer, mode);
    }

    // ---- one pass over a flat arena instead of two launches per layer -----------------------------------------------------------------
    namespace b200::mlp{
        template <typename DEVICE, typename T>
        void fill_tensor(DEVICE& device, T& tensor, float value){ note(device, b200rl_fill(tensor._data, T::SPEC::SIZE, value, device.stream)); }
    }
    template<typename DEV_SPEC, typename SPEC>
    void zero_gradient(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkGradient<SPEC>& network){
        const auto arena = b200::mlp::arena_of(network);
        if(arena){ b200::note(device, b200rl_fill(arena.grads(), b200::mlp::Layout<SPEC>::N, 0.0f, device.stream)); return; }
        b200::mlp::for_each_layer(network, [&](auto& layer){ b200::mlp::fill_tensor(device, layer.weights.gradient, 0.0f); b200::mlp::fill_tensor(device, layer.biases.gradient, 0.0f); });
    }
    template<typename DEV_SPEC, typename SPEC, typename OPTIMIZER>
    void _reset_optimizer_state(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkGradient<SPEC>& network, OPTIMIZER&){
        static_assert(b200::mlp::Layout<SPEC>::HAS_ADAM, "optimizer state of Adam parameters");
        const auto arena = b200::mlp::arena_of(network);
        if(arena){
            b200::note(device, b200rl_fill(arena.m(), b200::mlp::Layout<SPEC>::N, 0.0f, device.stream));
            b200::note(device, b200rl_fill(arena.v(), b200::mlp::Layout<SPEC>::N, 0.0f, device.stream));
            return;
        }
        b200::mlp::for_each_layer(network, [&](auto& layer){
            b200::mlp::fill_tensor(device, layer.weights.gradient_first_order_moment, 0.0f); b200::mlp::fill_tensor(device, layer.weights.gradient_second_order_moment, 0.0f);
            b200::mlp::fill_tensor(device, layer.biases.gradient_first_order_moment, 0.0f); b200::mlp::fill_tensor(device, layer.biases.gradient_second_order_moment, 0.0f);
        });
    }
    template<typename DEV_SPEC, typename SPEC, typename ADAM_SPEC>
    void update(devices::B200<DEV_SPEC>& device, nn_models::mlp::NeuralNetworkGradient<SPEC>& network, nn::optimizers::Adam<ADAM_SPEC>& optimizer){
        static_assert(b200::mlp::Layout<SPEC>::HAS_ADAM, "Adam parameters");
        const auto arena = b200::mlp::arena_of(network);
        if(arena){
            b200::note(device, b200rl_adam_update_dev(arena.params(), arena.grads(), arena.m(), arena.v(), b200::mlp::Layout<SPEC>::N, reinterpret_cast<const float*>(optimizer.parameters._data),
                                                      optimizer.first_order_moment_bias_correction._data, optimizer.second_order_moment_bias_correction._data, device.stream));
            return;
        }
        b200::mlp::for_each_layer(network, [&](auto& layer){ update(device, layer.weights, optimizer); update(device, layer.biases, optimizer); });
    }
}
RL_TOOLS_NAMESPACE_WRAPPER_END
