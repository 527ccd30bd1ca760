"""Export of a trained MLP in the reference's code format: the C++ source that `save_code(device, network, name)` writes for a forward-only
`nn_models::mlp::NeuralNetwork` (nn_models/mlp/persist_code.h:14-103, nn/layers/dense/persist_code.h, nn/parameters/persist_code.h,
containers/tensor/persist_code.h), which the reference's checkpoint step stores as `checkpoint.h` next to an example input / output pair
(rl/loop/steps/checkpoint/operations_cpu.h:54-118) and which its embedded targets compile in. The text is produced here from the flat
parameter arena of `rl_tools_b200.Mlp` (W_l row-major, then b_l, per layer), so that a policy trained on the GPU leaves it in the format the
reference's tooling reads; `tests/test_export.py` holds it byte for byte against the reference's own writer.

Scope: fp32 (`numeric_types::Policy<float>`), three or more layers with one hidden width and one hidden activation (what
`nn_models::mlp::Configuration` can describe), capability `Forward<true, true>`, index type `unsigned long` (the index type of the
reference's CPU device, whose writer defines the format)."""
import numpy as np

NS = "RL_TOOLS_NAMESPACE_WRAPPER ::rl_tools::"
ACTIVATIONS = {"identity": "IDENTITY", "relu": "RELU", "tanh": "TANH", "fast_tanh": "FAST_TANH", "sigmoid": "SIGMOID"}
TI = "unsigned long"
TYPE_POLICY = NS + "numeric_types::Policy<float>"


def hexfloat(value) -> str:
    """A float32 as the reference's writer prints it: std::hexfloat, uppercase, of the value widened to double (no trailing zeros), with
    the `f` suffix."""
    v = float(np.float32(value))
    if v == 0.0:
        return ("-" if np.signbit(np.float32(value)) else "") + "0X0P+0f"
    text = v.hex()                                   # [-]0x1.xxxxxxxxxxxxxp[+-]e
    sign = "-" if text.startswith("-") else ""
    mantissa, exponent = text.lstrip("-")[2:].split("p")
    head, _, frac = mantissa.partition(".")
    frac = frac.rstrip("0")
    return f"{sign}0X{head}{'.' + frac.upper() if frac else ''}P{exponent}f"


def _tensor(values, shape, indent) -> str:
    """containers/tensor/persist_code.h:14-75 for a dense constant tensor named `parameters_memory`."""
    ind = "    " * indent
    dims = ", ".join(str(d) for d in shape)
    return (f"{ind}namespace parameters_memory {{\n"
            f"{ind}    constexpr float memory[] = {{{', '.join(hexfloat(v) for v in values)}}};\n"
            f"{ind}    using SHAPE = {NS}tensor::Shape<{TI}, {dims}>;\n"
            f"{ind}    using SPEC = {NS}tensor::Specification<float, {TI}, SHAPE, true, {NS}tensor::RowMajorStride<SHAPE>, true>;\n"
            f"{ind}    using CONTAINER_TYPE = {NS}Tensor<SPEC>;\n"
            f"{ind}    constexpr CONTAINER_TYPE container = {{(float*)memory}}; \n"
            f"{ind}}}\n")


def _parameter(values, shape, group, category, name, indent) -> str:
    """nn/parameters/persist_code.h (Plain parameters): the tensor plus its parameter specification and instance."""
    ind = "    " * indent
    return (f"{ind}namespace {name} {{\n" + _tensor(values, shape, indent + 1) +
            f"{ind}    using TYPE_POLICY = {TYPE_POLICY};\n"
            f"{ind}    using PARAMETER_SPEC = {NS}nn::parameters::Plain::Specification<TYPE_POLICY, typename parameters_memory::SPEC::TI, typename parameters_memory::SPEC::SHAPE, "
            f"{NS}nn::parameters::groups::{group}, {NS}nn::parameters::categories::{category}, true, true>;\n"
            f"{ind}    constexpr {NS}nn::parameters::Plain::Instance<PARAMETER_SPEC> parameters = {{parameters_memory::container}};\n"
            f"{ind}}}\n")


HEADER_PARAMETER = ("// NOTE: This code export assumes that the endianness of the target platform is the same as the endianness of the source platform\n"
                    "#include <rl_tools/containers/tensor/tensor.h>\n#include <rl_tools/nn/parameters/parameters.h>\n")
HEADER_LAYER = HEADER_PARAMETER + HEADER_PARAMETER + "#include <rl_tools/nn/layers/dense/layer.h>\n#include <rl_tools/numeric_types/policy.h>\n"


def _layer(W, b, activation, group, name, batch, indent) -> str:
    """nn/layers/dense/persist_code.h: weights, biases, then the layer's configuration and the three constructors."""
    ind = "    " * indent
    O, I = W.shape
    init = "{weights::parameters, biases::parameters}"
    return (f"{ind}namespace {name} {{\n" + _parameter(W.reshape(-1), (O, I), group, "Weights", "weights", indent + 1) + _parameter(b, (O,), group, "Biases", "biases", indent + 1) +
            f"{ind}}}\n"
            f"{ind}namespace {name} {{\n"
            f"{ind}    using TYPE_POLICY = {TYPE_POLICY};\n"
            f"{ind}    using CONFIG = {NS}nn::layers::dense::Configuration<TYPE_POLICY, {TI}, {O}, {NS}nn::activation_functions::ActivationFunction::{ACTIVATIONS[activation]}, "
            f"{NS}nn::layers::dense::DefaultInitializer<TYPE_POLICY, {TI}>, {NS}nn::parameters::groups::{group}>; \n"
            f"{ind}    using TEMPLATE = {NS}nn::layers::dense::BindConfiguration<CONFIG>;\n"
            f"{ind}    using INPUT_SHAPE = {NS}tensor::Shape<{TI}, 1, {batch}, {I}>;\n"
            f"{ind}    using CAPABILITY = {NS}nn::capability::Forward<true, true>;\n"
            f"{ind}    using TYPE = {NS}nn::layers::dense::Layer<CONFIG, CAPABILITY, INPUT_SHAPE>;\n"
            f"{ind}    constexpr TYPE module = {init};\n"
            f"{ind}    template <typename T_TYPE = TYPE>\n"
            f"{ind}    constexpr T_TYPE factory = {init};\n"
            f"{ind}    template <typename T_TYPE = TYPE>\n"
            f"{ind}    constexpr T_TYPE factory_function(){{return T_TYPE{init};}}\n"
            f"{ind}}}\n")


def save_code(params, input_dim, dims, activations, name, batch=1) -> str:
    """The reference's `save_code(device, network, name, true)` for the MLP input_dim -> dims[0] -> ... -> dims[-1] with the flat parameter
    arena `params` (numpy array or anything np.asarray takes; a CUDA tensor must be brought to the host by the caller)."""
    params = np.ascontiguousarray(np.asarray(params, np.float32).reshape(-1))
    L = len(dims)
    if L < 3 or len(set(dims[:-1])) != 1 or len(set(activations[:-1])) != 1:
        raise ValueError("nn_models::mlp::Configuration describes input, N equal hidden layers and an output layer with one hidden activation")
    layers, off, fan_in = [], 0, input_dim
    for d in dims:
        W = params[off:off + d * fan_in].reshape(d, fan_in); off += d * fan_in
        layers.append((W, params[off:off + d])); off += d
        fan_in = d
    if off != params.size:
        raise ValueError(f"the arena holds {params.size} parameters, the shape needs {off}")
    names = ["input_layer"] + [f"hidden_layer_{i}" for i in range(L - 2)] + ["output_layer"]
    groups = ["Input"] + ["Normal"] * (L - 2) + ["Output"]
    header = HEADER_LAYER + "#include <rl_tools/nn_models/mlp/network.h>\n" + HEADER_LAYER * (L - 1)
    body = f"namespace {name} {{\n"
    for (W, b), act, group, lname in zip(layers, activations, groups, names):
        body += _layer(W, b, act, group, lname, batch, 1)
    hidden = lambda fmt: ", ".join(fmt.format(i) for i in range(L - 2))
    body += (f"    using TYPE_POLICY = {TYPE_POLICY};\n"
             f"    using CONFIG = {NS}nn_models::mlp::Configuration<TYPE_POLICY, {TI}, {dims[-1]}, {L}, {dims[0]}, {NS}nn::activation_functions::ActivationFunction::{ACTIVATIONS[activations[0]]}, "
             f"{NS}nn::activation_functions::ActivationFunction::{ACTIVATIONS[activations[-1]]}, {NS}nn::layers::dense::DefaultInitializer<TYPE_POLICY, {TI}>>; \n"
             f"    using TEMPLATE = {NS}nn_models::mlp::BindConfiguration<CONFIG>;\n"
             f"    using INPUT_SHAPE = {NS}tensor::Shape<{TI}, 1, {batch}, {input_dim}>;\n"
             f"    using CAPABILITY = {NS}nn::capability::Forward<true, true>;\n"
             f"    using TYPE = {NS}nn_models::mlp::NeuralNetwork<CONFIG, CAPABILITY, INPUT_SHAPE>;\n"
             f"    constexpr TYPE module = {{input_layer::factory<TYPE::SPEC::INPUT_LAYER>, {{{hidden('hidden_layer_{}::factory<TYPE::SPEC::HIDDEN_LAYER>')}}}, output_layer::factory<TYPE::SPEC::OUTPUT_LAYER>}};\n"
             f"    template <typename T_TYPE = TYPE>\n"
             f"    constexpr T_TYPE factory = {{input_layer::factory<typename T_TYPE::SPEC::INPUT_LAYER>, {{{hidden('hidden_layer_{}::factory<typename T_TYPE::SPEC::HIDDEN_LAYER>')}}}, "
             f"output_layer::factory<typename T_TYPE::SPEC::OUTPUT_LAYER>}};\n"
             f"    template <typename T_TYPE = TYPE>\n"
             f"    constexpr T_TYPE factory_function(){{return T_TYPE{{input_layer::factory_function<typename T_TYPE::SPEC::INPUT_LAYER>(), "
             f"{{{hidden('hidden_layer_{}::factory_function<typename T_TYPE::SPEC::HIDDEN_LAYER>()')}}}, output_layer::factory_function<typename T_TYPE::SPEC::OUTPUT_LAYER>()}};}}\n"
             f"}}\n")
    return header + body
