"""Builds the REFERENCE's own trainer-side extension, unmodified, for the hand-off tests.

    python build_ref_trainer.py <reference root> <output directory>

Compiles training_backend/ipc_service.cpp, helper_multiprocess.cpp and ipc_cuda_kernel.cu from where
the reference lies (nothing is copied) with torch's extension builder, the way the reference's own
training_backend/setup.py does (a CUDAExtension named ipc_service), for sm_100a, and leaves
<output directory>/ipc_service.so.  Test infrastructure only: tests/test_gpu_reference_trainer.py imports
that module in a second process and lets it consume batches from this repository's sampling_server.
"""
import os
import shutil
import sys


def main():
    ref, out = os.path.abspath(sys.argv[1]), os.path.abspath(sys.argv[2])
    src = os.path.join(ref, "training_backend")
    sources = [os.path.join(src, f) for f in ("ipc_service.cpp", "helper_multiprocess.cpp", "ipc_cuda_kernel.cu")]
    for s in sources:
        if not os.path.exists(s):
            raise SystemExit("missing reference source: " + s)
    # the distribution's own compiler: objects made by another g++ wrapper on PATH crashed in iostream
    # code (std::cout << int) once loaded next to torch
    if os.path.exists("/usr/bin/g++") and os.path.exists("/usr/bin/gcc"):
        os.environ["CXX"] = "/usr/bin/g++"
        os.environ["CC"] = "/usr/bin/gcc"
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    os.environ.setdefault("CUDA_HOME", "/usr/local/cuda")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load
    build_dir = os.path.join(out, "ipc_service_build")
    os.makedirs(build_dir, exist_ok=True)
    load(name="ipc_service", sources=sources, build_directory=build_dir, verbose=False, is_python_module=False)
    shutil.copy2(os.path.join(build_dir, "ipc_service.so"), os.path.join(out, "ipc_service.so"))
    shutil.rmtree(build_dir, ignore_errors=True)
    print("built", os.path.join(out, "ipc_service.so"))


if __name__ == "__main__":
    main()
