"""Builds ``libv1g_tf_ops.so`` (the TensorFlow custom ops over ``libv1g.so``), in-tree.

    python -m v1_glif_model_b200.tf_shim.build_tf_shim

Runs only where ``import tensorflow`` succeeds; elsewhere it prints why and returns ``None`` (the rest
of the package does not need TensorFlow).  Flags follow TensorFlow's custom-op recipe:
``tf.sysconfig.get_compile_flags()`` / ``get_link_flags()``.
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
PKG = os.path.dirname(HERE)
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
OUT = os.path.join(HERE, "libv1g_tf_ops.so")


def build():
    try:
        import tensorflow as tf
    except Exception as e:  # noqa: BLE001
        print(f"TensorFlow: unavailable on this box ({type(e).__name__}); the custom-op shim is not built")
        return None
    from v1_glif_model_b200 import build as build_lib
    build_lib.build()
    cuda = os.environ.get("CUDA_HOME", "/usr/local/cuda")
    cmd = ["g++", "-std=c++17", "-shared", "-fPIC", "-O2", os.path.join(HERE, "v1g_tf_ops.cc"), "-o", OUT,
           "-I", INCLUDE, "-I", os.path.join(cuda, "include"), "-DGOOGLE_CUDA=1",
           *tf.sysconfig.get_compile_flags(), *tf.sysconfig.get_link_flags(),
           "-L", PKG, "-lv1g", "-Wl,-rpath," + PKG, "-L", os.path.join(cuda, "lib64"), "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError("building the TensorFlow shim failed:\n" + r.stdout + r.stderr)
    return OUT


if __name__ == "__main__":
    print(build())
    sys.exit(0)
