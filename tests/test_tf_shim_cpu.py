"""The TensorFlow custom-op shim cannot be compiled or run where TensorFlow is missing; what can be
checked everywhere is that its sources are consistent with the C ABI and with each other: every
``v1g_*`` function the ops call is declared in ``include/v1g.h``, every op the Python glue uses is
registered by the C++ file with the attributes and inputs the glue passes, and the build step says
plainly when TensorFlow is absent."""
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "v1_glif_model_b200", "tf_shim")


def _snake(name):
    return re.sub(r"(?<=[a-z0-9])(?=[A-Z])", "_", name.replace("V1G", "V1g")).lower()


def _registered_ops(cc):
    cc = re.sub(r"//[^\n]*", "", cc)
    ops = {}
    for m in re.finditer(r'REGISTER_OP\("(\w+)"\)(.*?);', cc, re.S):
        body = m.group(2)
        ops[m.group(1)] = {"attrs": set(re.findall(r'\.Attr\("(\w+):', body)),
                           "inputs": re.findall(r'\.Input\("(\w+):', body),
                           "outputs": re.findall(r'\.Output\("(\w+):', body)}
    return ops


def test_ops_call_only_declared_entry_points():
    cc = open(os.path.join(SHIM, "v1g_tf_ops.cc")).read()
    header = open(os.path.join(ROOT, "include", "v1g.h")).read()
    declared = set(re.findall(r"\b(v1g_[a-z0-9_]+)\s*\(", header))
    called = set(re.findall(r"\b(v1g_[a-z0-9_]+)\s*\(", cc))
    assert called and called <= declared, called - declared
    # the op that must not allocate behind TensorFlow's allocator uses the allocation-free entry point
    assert "v1g_compact_spikes_noalloc" in called and "v1g_compact_spikes(" not in cc
    ops = _registered_ops(cc)
    assert {"V1GSynCurrents", "V1GSynCurrentsGrad", "V1GStep", "V1GStepGrad", "V1GCompactSpikes", "V1GRollout",
            "V1GRolloutGrad"} <= set(ops)
    for name in ops:
        assert f'REGISTER_KERNEL_BUILDER(Name("{name}").Device(tf::DEVICE_GPU)' in cc, name


def test_glue_uses_registered_ops_with_their_arguments():
    cc = open(os.path.join(SHIM, "v1g_tf_ops.cc")).read()
    py = open(os.path.join(SHIM, "v1g_tf.py")).read()
    ops = {_snake(k): v for k, v in _registered_ops(cc).items()}
    used = re.findall(r"_ops\.(\w+)\((.*?)\)\n", py, re.S)
    assert len(used) >= 7
    for name, args in used:
        assert name in ops, name
        kwargs = set(re.findall(r"(\w+)=", args))
        allowed = ops[name]["attrs"] | set(ops[name]["inputs"])
        assert kwargs <= allowed, (name, kwargs - allowed)
        assert set(ops[name]["inputs"]) <= kwargs, (name, set(ops[name]["inputs"]) - kwargs)
    # the nine-entry gradient list of calculate_synaptic_currents (models.py:251-261)
    m = re.search(r"return \[d_z, None, tf\.cast\(d_w, weight_values\.dtype\)((?:, None)+)\]", py)
    assert m and m.group(1).count("None") == 6


def test_build_step_reports_missing_tensorflow(capsys):
    from v1_glif_model_b200.tf_shim import build_tf_shim
    try:
        import tensorflow  # noqa: F401
        have_tf = True
    except Exception:  # noqa: BLE001
        have_tf = False
    if not have_tf:
        assert build_tf_shim.build() is None
        assert "TensorFlow: unavailable on this box" in capsys.readouterr().out


def test_shim_source_type_checks_against_the_c_abi():
    """``g++ -fsyntax-only`` over the shim with the real ``include/v1g.h`` and CUDA runtime header, and
    declaration-only stand-ins for the TensorFlow headers (``tests/tf_stub``): every C-ABI call in the
    shim is checked for argument TYPES (pointer constness, integer widths, the state and loss structs),
    not only for its name and argument count."""
    import shutil
    import subprocess
    gxx = shutil.which("g++")
    cuda_inc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "include")
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")):
        pytest.skip("needs g++ and the CUDA runtime header")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    src = os.path.join(root, "v1_glif_model_b200", "tf_shim", "v1g_tf_ops.cc")
    r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-Wall", "-Werror", "-I", os.path.join(root, "tests", "tf_stub"),
                        "-I", os.path.join(root, "include"), "-I", cuda_inc, src], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
