"""The exporter of rl_tools_b200.export against the reference's own code writer (`save_code`, nn_models/mlp/persist_code.h): byte for byte on
the fixture `tests/golden/export_code.npz`, which `tests/golden/make_golden.py export` generates by compiling `export_golden.cpp` against the
reference tree (three networks: batch 4 / batch 1, three and four layers, all activation names that occur, parameters that include zeros of
both signs, one, a subnormal and a value with a full 24-bit mantissa)."""
import os
import sys

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN


@pytest.fixture(scope="module")
def export():
    from __graft_entry__ import load_package
    load_package()
    from rl_tools_b200 import export as module
    return module


@pytest.mark.parametrize("case", sorted(mg.EXPORT_CASES))
def test_exported_source_equals_the_reference_writer(export, case):
    fix = np.load(os.path.join(GOLDEN, "export_code.npz"))
    want = fix[f"code_{case}"].tobytes().decode()
    input_dim, dims, acts, batch = mg.EXPORT_CASES[case]
    got = export.save_code(mg.export_params(case), input_dim, dims, acts, "exported::actor", batch)
    if got != want:
        for i, (a, b) in enumerate(zip(want.split("\n"), got.split("\n"))):
            assert a == b, f"line {i}"
    assert got == want and len(got) > 5000


def test_hexfloat_forms(export):
    """std::hexfloat of a float widened to double, uppercase, no trailing zeros: the forms the writer emits"""
    f = export.hexfloat
    assert f(0.0) == "0X0P+0f" and f(-0.0) == "-0X0P+0f" and f(1.0) == "0X1P+0f" and f(-2.5) == "-0X1.4P+1f"
    assert f(np.float32(0.1)) == "0X1.99999AP-4f" and f(np.float32(1e-40)) == "0X1.16C2P-133f"


def test_shapes_the_format_cannot_describe_are_refused(export):
    with pytest.raises(ValueError):
        export.save_code(np.zeros(3 * 4 + 4 + 4 * 2 + 2, np.float32), 3, [4, 2], ["relu", "identity"], "x")          # two layers: no hidden layer
    with pytest.raises(ValueError):
        export.save_code(np.zeros(10, np.float32), 3, [8, 8, 2], ["relu", "relu", "identity"], "x")                  # arena too short


def test_exported_source_compiles_against_the_reference_and_evaluates(export, orc, tmp_path):
    """The export is consumed as the reference's tooling consumes a checkpoint: a program that includes the generated source next to the
    reference's headers, evaluates `exported::actor::module` on an input with the reference's own `evaluate`, and must reproduce the oracle's
    forward pass of the same parameters bit for bit. Runs where the reference tree is available (it does not travel with the repository)."""
    import subprocess
    import oracle
    reference = os.environ.get("B200RL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
    if not os.path.isdir(os.path.join(reference, "include", "rl_tools")):
        pytest.skip("the reference tree is not available")
    case = 2
    input_dim, dims, acts, batch = mg.EXPORT_CASES[case]
    params = mg.export_params(case)
    (tmp_path / "exported.h").write_text(export.save_code(params, input_dim, dims, acts, "exported::actor", batch))
    x = (mg.det_uniform(77, batch * input_dim) * np.float32(2)).reshape(batch, input_dim)
    (tmp_path / "main.cpp").write_text('''
#include <rl_tools/operations/cpu.h>
#include <rl_tools/nn/optimizers/adam/instance/operations_generic.h>
#include <rl_tools/nn/operations_generic.h>
#include <rl_tools/nn/layers/dense/operations_cpu.h>
#include <rl_tools/nn_models/mlp/operations_generic.h>
#include "exported.h"
#include <cstdio>
namespace rlt = rl_tools;
int main(){
    using DEVICE = rlt::devices::DefaultCPU; using TI = typename DEVICE::index_t;
    using NET = exported::actor::TYPE;
    DEVICE device; typename DEVICE::SPEC::RANDOM::ENGINE<> rng; rlt::malloc(device, rng); rlt::init(device, rng, 0);
    rlt::Tensor<rlt::tensor::Specification<float, TI, typename NET::INPUT_SHAPE>> input;
    rlt::Tensor<rlt::tensor::Specification<float, TI, typename NET::OUTPUT_SHAPE>> output;
    typename NET::template Buffer<> buffer;
    rlt::malloc(device, input); rlt::malloc(device, output); rlt::malloc(device, buffer);
    constexpr TI B = rlt::get<1>(typename NET::INPUT_SHAPE{}), I = rlt::get<2>(typename NET::INPUT_SHAPE{}), O = rlt::get<2>(typename NET::OUTPUT_SHAPE{});
    for(TI b = 0; b < B; b++) for(TI i = 0; i < I; i++){ float v; if(std::scanf("%a", &v) != 1) return 2; rlt::set(device, input, v, 0, b, i); }
    rlt::evaluate(device, exported::actor::module, input, output, buffer, rng);
    for(TI b = 0; b < B; b++) for(TI o = 0; o < O; o++) std::printf("%a\\n", (double)rlt::get(device, output, 0, b, o));
    return 0;
}
''')
    exe = tmp_path / "main"
    subprocess.run(["g++", "-std=c++17", "-O1", "-fno-fast-math", "-ffp-contract=off", "-I" + os.path.join(reference, "include"), "-I" + str(tmp_path), str(tmp_path / "main.cpp"), "-o", str(exe)],
                   check=True)
    res = subprocess.run([str(exe)], input=" ".join(float(v).hex() for v in x.reshape(-1)), capture_output=True, text=True, check=True)
    got = np.float32([float.fromhex(t) for t in res.stdout.split()]).reshape(batch, dims[-1])
    shape = oracle.MlpShape.make(input_dim, dims, acts)
    assert np.array_equal(got, orc.mlp_evaluate(shape, params, x))
