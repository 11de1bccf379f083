"""Builds the native libraries of this package in-tree with nvcc for sm_100a.

    python polarai-framework_b200/build.py            # everything
    python polarai-framework_b200/build.py --force    # ignore timestamps

libpolar_b200.so    - the builtin kernels and their C ABI (include/polar_b200.h)
libpolar_rt_cuda.so - the PolarAI device-runtime plugin (initContext/closeContext)
                      built against the reference's runtime headers when the
                      reference tree is present (environment variable
                      POLAR_REFERENCE_ROOT); otherwise a prebuilt file is kept.
"""
import concurrent.futures
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
OBJ = os.path.join(HERE, "build")
LIB = os.path.join(HERE, "lib")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-ccbin", "/usr/bin/g++"] + ARCH

KERNEL_SOURCES = ["common.cu", "elementwise.cu", "extra_builtins.cu", "gemm_ffma.cu", "gemm_skinny.cu", "gemm_tc.cu", "peer_collective.cu", "dispatch.cu"]


def _newer(src, dst, extra=()):
    if not os.path.exists(dst):
        return True
    t = os.path.getmtime(dst)
    return any(os.path.getmtime(s) > t for s in (src,) + tuple(extra) if os.path.exists(s))


def _run(cmd):
    out = subprocess.run(cmd, capture_output=True, text=True)
    if out.returncode != 0:
        raise RuntimeError("command failed: " + " ".join(cmd) + "\n" + out.stdout + out.stderr)
    return out.stdout + out.stderr


def _headers():
    hs = [os.path.join(ROOT, "include", f) for f in os.listdir(os.path.join(ROOT, "include"))]
    hs += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".hpp", ".h"))]
    return tuple(hs)


def build_kernels(force=False, verbose=False):
    os.makedirs(OBJ, exist_ok=True)
    os.makedirs(LIB, exist_ok=True)
    hdrs = _headers()
    jobs = []
    objs = []
    for src in KERNEL_SOURCES:
        s = os.path.join(CSRC, src)
        o = os.path.join(OBJ, src.replace(".cu", ".o"))
        objs.append(o)
        if force or _newer(s, o, hdrs):
            jobs.append([NVCC] + NVCC_FLAGS + (["-Xptxas", "-v"] if verbose else []) + ["-c", s, "-o", o])
    with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
        for log in ex.map(_run, jobs):
            if verbose and log:
                print(log)
    lib = os.path.join(LIB, "libpolar_b200.so")
    if force or jobs or not os.path.exists(lib):
        _run([NVCC, "-shared", "-o", lib] + objs + ARCH + ["-ccbin", "/usr/bin/g++"])
    return lib


def reference_root():
    r = os.environ.get("POLAR_REFERENCE_ROOT", "/root/reference")
    return r if os.path.isdir(os.path.join(r, "include", "polarai")) else None


def build_runtime(force=False):
    """The device-runtime plugin.  Needs the reference's headers to compile."""
    lib = os.path.join(LIB, "libpolar_rt_cuda.so")
    rt_dir = os.path.join(CSRC, "rt")
    if not os.path.isdir(rt_dir):
        return None
    ref = reference_root()
    if ref is None:
        if os.path.exists(lib):
            return lib
        raise RuntimeError("libpolar_rt_cuda.so is not built and the reference headers are absent")
    srcs = [os.path.join(rt_dir, f) for f in sorted(os.listdir(rt_dir)) if f.endswith((".cpp", ".cu"))]
    deps = tuple(os.path.join(rt_dir, f) for f in os.listdir(rt_dir)) + _headers()
    if not (force or any(_newer(s, lib, deps) for s in srcs)):
        return lib
    stubs = os.path.join(OBJ, "export_stubs")
    os.makedirs(stubs, exist_ok=True)
    # The reference's CMake generates one <target>_export.h per library; an
    # in-tree build of the plugin only needs the macros to exist.
    for name in ["polar_core", "polar_utils", "polar_loaders", "polar_operation", "polar_backend_generic",
                 "polar_rt_support", "polar_io", "polar_rt_cuda", "polar_generic_backend_driver"]:
        with open(os.path.join(stubs, name + "_export.h"), "w") as fh:
            macro = name.upper()
            fh.write(f"#pragma once\n#define {macro}_EXPORT\n#define {macro}_NO_EXPORT\n")
    cmd = [NVCC] + NVCC_FLAGS + ["-shared", "-o", lib, "-I", os.path.join(ref, "include"),
                                 "-I", os.path.join(ref, "src", "backend", "generic"),
                                 "-I", stubs, "-I", os.path.join(ROOT, "include"),
                                 "-Xcompiler", "-fno-rtti", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN",
                                 "-L", LIB, "-lpolar_b200"] + srcs
    _run(cmd)
    return lib


REF_TESTS = ["AddOperation", "CombineOperation", "Conv2DOperation", "DivideOperation", "LogLossOperation",
             "MatMulOperation", "MulConcatOperation", "MulOperation", "Pool2DOperation", "ReLUOperation",
             "SigmoidOperation", "SoftmaxOperation"]


def build_reference_host(force=False):
    """The unchanged PolarAI frontend (graph, autograd, operations, loaders), runtime
    driver, support routines and LayerAllocator compiled from the reference tree
    where it lies; this package's Executor on top; and the reference's own
    integration tests for the builtins on this path, built against the stand-in
    gtest header in tests/ref_integration/.  Everything lands under lib/ (not
    tracked).  Without the reference tree, prebuilt files are kept."""
    out_dir = os.path.join(LIB, "ref")
    frontend = os.path.join(out_dir, "libpolar_frontend.so")
    executor = os.path.join(LIB, "libpolar_b200_executor.so")
    tests_bin = os.path.join(out_dir, "ref_integration_tests")
    ref = reference_root()
    if ref is None:
        return [p for p in (frontend, executor, tests_bin, os.path.join(out_dir, "autograd_parity"),
                            os.path.join(out_dir, "data_parallel_executor"), os.path.join(out_dir, "lspolar"))
                if os.path.exists(p)]
    os.makedirs(out_dir, exist_ok=True)
    obj_dir = os.path.join(OBJ, "ref")
    gen = os.path.join(obj_dir, "gen")
    os.makedirs(gen, exist_ok=True)
    stubs = os.path.join(OBJ, "export_stubs")
    os.makedirs(stubs, exist_ok=True)
    for name in ["polar_core", "polar_utils", "polar_loaders", "polar_operation", "polar_backend_generic",
                 "polar_rt_support", "polar_io", "polar_rt_cuda", "polar_generic_be_driver"]:
        with open(os.path.join(stubs, name + "_export.h"), "w") as fh:
            macro = name.upper()
            fh.write(f"#pragma once\n#define {macro}_EXPORT\n#define {macro}_NO_EXPORT\n")
    # The driver's generated config.h: the one build-time switch the integration
    # needs - the CUDA runtime library is on the list the RuntimeDriver loads.
    with open(os.path.join(gen, "config.h"), "w") as fh:
        fh.write('#pragma once\n#include <string>\n#include <vector>\n'
                 'inline std::vector<std::string> getListOfLibraries() { return {"libpolar_rt_cuda.so"}; }\n')
    gxx = "/usr/bin/g++"
    flags = ["-std=c++17", "-O2", "-fPIC", "-fno-rtti", "-fno-exceptions", "-w",
             "-DATHENA_MAJOR_VERSION=\"0\"", "-DATHENA_MINOR_VERSION=\"1\"", "-DATHENA_PATCH_VERSION=\"0\"",
             "-I", os.path.join(ref, "include"), "-I", os.path.join(ref, "src"),
             "-I", os.path.join(ref, "src", "backend", "generic"), "-I", stubs, "-I", gen]
    srcs = []
    for sub in ("core", "operation", "loaders", "utils", "io"):
        for d, _, files in os.walk(os.path.join(ref, "src", sub)):
            srcs += [os.path.join(d, f) for f in files if f.endswith(".cpp")]
    g = os.path.join(ref, "src", "backend", "generic")
    srcs += [os.path.join(g, "runtime", "driver", "RuntimeDriver.cpp"),
             os.path.join(g, "runtime", "driver", "DynamicLibrary_posix.cpp"),
             os.path.join(g, "runtime", "support", "routines.cpp"),
             os.path.join(g, "lib", "allocators", "LayerAllocator.cpp")]
    if force or not os.path.exists(frontend):
        jobs, objs = [], []
        for i, src in enumerate(sorted(srcs)):
            o = os.path.join(obj_dir, f"{i:03d}_{os.path.basename(src)[:-4]}.o")
            objs.append(o)
            jobs.append([gxx] + flags + ["-c", src, "-o", o])
        with concurrent.futures.ThreadPoolExecutor(max_workers=8) as ex:
            list(ex.map(_run, jobs))
        _run([gxx, "-shared", "-o", frontend] + objs + ["-ldl", "-lpthread", "-Wl,-rpath,$ORIGIN/.."])
    ex_src = os.path.join(CSRC, "executor", "direct_executor.cpp")
    if force or _newer(ex_src, executor, (frontend, os.path.join(CSRC, "executor", "data_parallel_plan.hpp"))):
        _run([gxx] + flags + ["-shared", "-o", executor, ex_src, "-L", out_dir, "-lpolar_frontend",
                              "-Wl,-rpath,$ORIGIN/ref:$ORIGIN"])
    shim = os.path.join(ROOT, "tests", "ref_integration")
    main_src = os.path.join(shim, "main.cpp")
    if force or _newer(main_src, tests_bin, (executor, os.path.join(shim, "gtest", "gtest.h"))):
        tdir = os.path.join(ref, "tests", "integration", "operations")
        tsrcs = [os.path.join(tdir, t + ".cpp") for t in REF_TESTS]
        tflags = [f for f in flags if f != "-fno-exceptions"]
        _run([gxx] + tflags + ["-I", shim, "-I", tdir, "-o", tests_bin, main_src] + tsrcs +
             ["-L", LIB, "-lpolar_b200_executor", "-L", out_dir, "-lpolar_frontend", "-ldl", "-lpthread",
              "-Wl,-rpath,$ORIGIN/..:$ORIGIN"])
    # whole-graph parity (autograd included) between the B200 device and a CPU oracle device
    parity_bin = os.path.join(out_dir, "autograd_parity")
    parity_src = os.path.join(shim, "autograd_parity.cpp")
    oracle_c = os.path.join(ROOT, "oracle", "builtins_oracle.c")
    if force or _newer(parity_src, parity_bin, (executor, os.path.join(shim, "oracle_device.hpp"), oracle_c)):
        oracle_o = os.path.join(obj_dir, "builtins_oracle.o")
        _run(["/usr/bin/gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-c", oracle_c, "-o", oracle_o])
        tflags = [f for f in flags if f != "-fno-exceptions"]
        _run([gxx] + tflags + ["-I", shim, "-fopenmp", "-o", parity_bin, parity_src, oracle_o,
                               "-L", LIB, "-lpolar_b200_executor", "-L", out_dir, "-lpolar_frontend", "-ldl",
                               "-lpthread", "-Wl,-rpath,$ORIGIN/..:$ORIGIN"])
    # the Executor's batch-sharded evaluation on several (fake, or real) devices
    dp_bin = os.path.join(out_dir, "data_parallel_executor")
    dp_src = os.path.join(shim, "data_parallel_executor.cpp")
    if force or _newer(dp_src, dp_bin, (executor, os.path.join(shim, "oracle_device.hpp"), oracle_c)):
        oracle_o = os.path.join(obj_dir, "builtins_oracle.o")
        if not os.path.exists(oracle_o) or _newer(oracle_c, oracle_o):
            _run(["/usr/bin/gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-c", oracle_c, "-o", oracle_o])
        tflags = [f for f in flags if f != "-fno-exceptions"]
        _run([gxx] + tflags + ["-I", shim, "-I", os.path.join(ROOT, "include"), "-fopenmp", "-o", dp_bin, dp_src,
                               oracle_o, "-L", LIB, "-lpolar_b200_executor", "-L", out_dir, "-lpolar_frontend", "-ldl",
                               "-lpthread", "-Wl,-rpath,$ORIGIN/..:$ORIGIN"])
    # host-side unit tests of the pool-based BackendAllocator with fake devices
    alloc_bin = os.path.join(out_dir, "pool_allocator_test")
    alloc_src = os.path.join(shim, "pool_allocator_test.cpp")
    rt_dir = os.path.join(CSRC, "rt")
    rt_lib = os.path.join(LIB, "libpolar_rt_cuda.so")
    if force or _newer(alloc_src, alloc_bin, (rt_lib, main_src, os.path.join(shim, "oracle_device.hpp"))):
        oracle_o = os.path.join(obj_dir, "builtins_oracle.o")
        if not os.path.exists(oracle_o):
            _run(["/usr/bin/gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-c", oracle_c, "-o", oracle_o])
        tflags = [f for f in flags if f != "-fno-exceptions"]
        _run([gxx] + tflags + ["-I", shim, "-I", CSRC, "-I", os.path.join(ROOT, "include"),
                               "-I", "/usr/local/cuda/include", "-fopenmp", "-o", alloc_bin, main_src, alloc_src,
                               oracle_o, "-L", LIB, "-lpolar_rt_cuda", "-lpolar_b200", "-ldl", "-lpthread",
                               "-Wl,-rpath,$ORIGIN/..:$ORIGIN"])
    # the reference's device-listing tool, unmodified, against the same driver
    lspolar_bin = os.path.join(out_dir, "lspolar")
    lspolar_src = os.path.join(ref, "utils", "lspolar", "main.cpp")
    if os.path.exists(lspolar_src) and (force or _newer(lspolar_src, lspolar_bin, (frontend,))):
        _run([gxx] + flags + ["-I", os.path.join(g, "runtime", "driver"), "-o", lspolar_bin, lspolar_src, "-L", out_dir, "-lpolar_frontend", "-ldl", "-lpthread",
                              "-Wl,-rpath,$ORIGIN/..:$ORIGIN"])
    return [frontend, executor, tests_bin, parity_bin, dp_bin, alloc_bin, lspolar_bin]


def build_all(force=False, verbose=False):
    libs = [build_kernels(force, verbose)]
    rt = build_runtime(force)
    if rt:
        libs.append(rt)
    libs += build_reference_host(force)
    return libs


if __name__ == "__main__":
    print("\n".join(build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)))
