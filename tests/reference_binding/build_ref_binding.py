"""Builds the reference project's OWN torch binding against this repository's library (test infrastructure).

    python tests/reference_binding/build_ref_binding.py [--reference /path/to/reference/checkout]

What it proves: ``Tools/megakernel/qwen_ops.cpp`` of the reference, compiled UNMODIFIED from where it lies, links
against ``libqwen_megakernel.so`` instead of the reference's ``megakernel_5090.cu`` (the four ``launch_ldg_*``
symbols have the reference's signatures), and the reference's own ``Model/Qwen06B_architecture.py`` then drives
this engine.  Outputs go to the git-ignored ``baseline/_ref/``:

    baseline/_ref/qwen_megakernel_C*.so          the reference binding, linked to ../../<package>/libqwen_megakernel.so
    baseline/_ref/Model/Qwen06B_architecture.py  the reference's Python layer, byte for byte (it has to travel to
                                                 the GPU machine, where the reference checkout does not exist)

``tests/test_reference_binding.py`` runs both in a child process (so that the module names do not collide with
this repository's own ``qwen_megakernel_C`` / ``Model`` packages) and is skipped when the outputs are absent.
Nothing in the package imports anything from here.
"""

from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
PKG = os.path.join(ROOT, "qwen3-0.6b-megakernel-rtx-5090_b200")
OUT = os.path.join(ROOT, "baseline", "_ref")


def build(reference: str) -> str:
    import torch
    from torch.utils import cpp_extension
    src = os.path.join(reference, "Tools", "megakernel", "qwen_ops.cpp")
    py = os.path.join(reference, "Model", "Qwen06B_architecture.py")
    if not (os.path.exists(src) and os.path.exists(py)):
        raise SystemExit(f"reference sources not found under {reference}")
    sys.path.insert(0, PKG)
    import build as pkg_build
    pkg_build.build()
    os.makedirs(os.path.join(OUT, "Model"), exist_ok=True)
    ext = os.path.join(OUT, "qwen_megakernel_C" + sysconfig.get_config_var("EXT_SUFFIX"))
    torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cuda_home = cpp_extension.CUDA_HOME or "/usr/local/cuda"
    cmd = ["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-DTORCH_EXTENSION_NAME=qwen_megakernel_C",
           "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={int(torch._C._GLIBCXX_USE_CXX11_ABI)}",
           *[f"-I{p}" for p in cpp_extension.include_paths()], f"-I{os.path.join(cuda_home, 'include')}",
           f"-I{sysconfig.get_paths()['include']}", src, "-o", ext,
           f"-L{torch_lib}", "-ltorch", "-ltorch_cpu", "-ltorch_cuda", "-ltorch_python", "-lc10", "-lc10_cuda",
           f"-L{os.path.join(cuda_home, 'lib64')}", "-lcudart",
           f"-L{PKG}", "-lqwen_megakernel",
           f"-Wl,-rpath,{torch_lib}", "-Wl,-rpath,$ORIGIN/../../qwen3-0.6b-megakernel-rtx-5090_b200"]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise SystemExit("g++ failed:\n" + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)
    shutil.copyfile(py, os.path.join(OUT, "Model", "Qwen06B_architecture.py"))
    open(os.path.join(OUT, "Model", "__init__.py"), "w").close()
    return ext


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("QMK_REFERENCE_CHECKOUT", "/root/reference"))
    print(build(ap.parse_args().reference))
