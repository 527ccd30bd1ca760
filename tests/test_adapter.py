"""The header-only C++ adapter (rl-tools_b200/include/b200rl/*.h): the reference's own generic MLP / Adam code
instantiated on devices::B200 must compile with the host compiler alone, and on a GPU agree with the reference CPU
device within the reference's own CPU<->CUDA test threshold (mean abs diff < 1e-6, tests/src/nn/cuda/cuda_basics.cu)."""
import os
import subprocess

import pytest

import __graft_entry__ as entry


def test_adapter_compiles_against_the_reference_headers():
    if not os.path.isdir(os.path.join(entry.REFERENCE_DIR, "include", "rl_tools")):
        pytest.skip("reference tree not present on this machine")
    entry.load_package().build()
    assert entry.build_adapter_test()
    assert os.path.exists(entry.ADAPTER_BIN)


@pytest.mark.gpu
def test_adapter_parity_on_gpu():
    if not os.path.exists(entry.ADAPTER_BIN):
        pytest.skip("adapter_parity binary was not built (needs the reference tree at build time)")
    res = subprocess.run([entry.ADAPTER_BIN], capture_output=True, text=True, timeout=300)
    print(res.stdout)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "ADAPTER PARITY OK" in res.stdout
