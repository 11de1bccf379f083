"""Generates the golden fixtures in this folder.  Run from the repo root, in a
checkout where the reference tree is present (oracle/Makefile builds
oracle/_ref/libref_ocl.so from it):

    python tests/golden/make_golden.py

reference_kats.json - the inputs of every known-answer test the reference holds
for the builtins on this path (file:line cited per case, paths inside the
reference project), with the outputs of the reference's own OpenCL C kernels
(src/backend/generic/runtime/opencl/kernels.h) compiled as C and run here.
Outputs are stored as uint32 bit patterns of the float32 results.

seeded_cases.npz - seeded inputs of odd sizes for every builtin and all four
matmul transpose forms, with the outputs of the same reference kernels.
"""
import json
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as orc  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))
T = "tests/integration/operations/"


def bits(a):
    return [int(x) for x in np.asarray(a, np.float32).ravel().view(np.uint32)]


def main():
    orc.build()
    ref = orc.RefOcl(threads=1)
    f = lambda *v: np.array(v, np.float32)
    kats = []

    def add(name, cite, builtin, expected, **inputs):
        kats.append({"name": name, "cite": cite, "builtin": builtin,
                     "inputs": {k: (v.tolist() if isinstance(v, np.ndarray) else v)
                                for k, v in inputs.items()},
                     "expected_bits": bits(expected)})

    a, b = f(1, 2, 3, 4), f(7, 8, 9, 10)
    add("AddOp1D", T + "AddOperation.cpp:22-26", "fadd", ref.fadd(a, 1.0, b, 1.0),
        a=a, scaleA=1.0, b=b, scaleB=1.0, shape=[4], stated_target=[8, 10, 12, 14])
    add("AddOp2D", T + "AddOperation.cpp:67-71", "fadd", ref.fadd(a, 1.0, b, 1.0),
        a=a, scaleA=1.0, b=b, scaleB=1.0, shape=[2, 2], stated_target=[8, 10, 12, 14])
    al, be = float(np.float32(0.34)), float(np.float32(0.21))
    add("Combine", T + "CombineOperation.cpp:32-37", "fadd", ref.fadd(a, al, b, be),
        a=a, scaleA=al, b=b, scaleB=be, shape=[2, 2])
    l, r = f(8, 2, 5, 6), f(3, 2, 1, 0.34)
    add("Mul", T + "MulOperation.cpp:32-36", "fmul", ref.fmul(l, r), a=l, b=r, shape=[2, 2])
    add("Divide", T + "DivideOperation.cpp:32-36", "fdivide", ref.fdivide(a, b),
        a=a, b=b, shape=[2, 2])
    loc, g = f(-100, 2, 5, 50), f(17.5)
    add("MulConcat", T + "MulConcatOperation.cpp:32-48", "fmulconcat", ref.fmulconcat(g, loc),
        gradient=g, local=loc, shape=[2, 2])
    x = f(-100, 2, 5, 50)
    add("Sigmoid", T + "SigmoidOperation.cpp:39-43 (DISABLED_ in the reference)", "fsigmoid",
        ref.fsigmoid(x), a=x, shape=[2, 2])
    p, y = f(0.6, 0.2, 0.8, 0.3), f(1, 0, 1, 0)
    add("LogLoss", T + "LogLossOperation.cpp:37-42 (DISABLED_ in the reference)", "flogloss",
        ref.flogloss(p, y), predicted=p, groundTruth=y, shape=[2, 2])

    def mm(name, cite, tl, tr, left, lshape, right, rshape):
        left = np.array(left, np.float32).reshape(lshape)
        right = np.array(right, np.float32).reshape(rshape)
        add(name, cite, "fmatmul", ref.fmatmul(tl, tr, left, right), tl=tl, tr=tr,
            left=left.ravel(), left_shape=list(lshape), right=right.ravel(),
            right_shape=list(rshape))

    mm("MatMulNN", T + "MatMulOperation.cpp:58-64", 0, 0, [3, 4, 5, 10], (1, 4), [6, 7, 8, 11], (4, 1))
    mm("MatMulNNSquare", T + "MatMulOperation.cpp:105-111", 0, 0, [3, 4, 5, 10], (2, 2),
       [6, 7, 8, 11], (2, 2))
    mm("MatMulNNRect", T + "MatMulOperation.cpp:151-157", 0, 0, [3, 4, 5, 10, 6, 7, 12, 6], (2, 4),
       [6, 7, 8, 11, 7, 8, 9, 1, 3, 2, 5, 6], (4, 3))
    mm("MatMulTN", T + "MatMulOperation.cpp:198-204", 1, 0, [3, 6, 4, 7, 5, 12, 10, 6], (4, 2),
       [6, 7, 8, 11, 7, 8, 9, 1, 3, 2, 5, 6], (4, 3))
    mm("MatMulNT", T + "MatMulOperation.cpp:244-250", 0, 1, [3, 4, 5, 10, 6, 7, 12, 6], (2, 4),
       [6, 11, 9, 2, 7, 7, 1, 5, 8, 8, 3, 6], (3, 4))

    with open(os.path.join(HERE, "reference_kats.json"), "w") as fh:
        json.dump({"generator": "tests/golden/make_golden.py",
                   "outputs_from": "reference OpenCL C kernels compiled as C (oracle/_ref)",
                   "cases": kats}, fh, indent=1)

    # Seeded cases, odd sizes.
    rng = np.random.default_rng(0)
    n = 1027
    u = lambda lo, hi, *s: rng.uniform(lo, hi, size=s).astype(np.float32)
    d = {}
    d["a"], d["b"], d["c"] = u(-1, 1, n), u(-1, 1, n), u(-1, 1, n)
    d["den"] = u(0.5, 2, n)
    d["xs"] = np.concatenate([u(-20, 20, n - 8), f(-100, -12, -11.5, 0, 11.5, 12, 50, 100)])
    d["p"] = u(0.0, 1.0, n)
    d["p"][:4] = f(0.0, 1.0, 1e-5, 1 - 1e-5)
    d["y"] = (rng.random(n) < 0.5).astype(np.float32)
    d["ysoft"] = u(0, 1, n)
    d["grad"] = f(-0.73)
    d["out_fill"] = ref.ffill(1.234, n)
    d["out_copy"] = ref.fcopy(d["a"])
    d["out_add"] = ref.fadd(d["a"], 1.0, d["b"], 1.0)
    d["out_combine"] = ref.fadd(d["a"], 0.34, d["b"], -0.21)
    d["out_mul"] = ref.fmul(d["a"], d["b"])
    d["out_divide"] = ref.fdivide(d["a"], d["den"])
    d["out_sigmoid"] = ref.fsigmoid(d["xs"])
    d["out_logloss"] = ref.flogloss(d["p"], d["y"])
    d["out_logloss_soft"] = ref.flogloss(d["p"], d["ysoft"])
    d["out_mulconcat"] = ref.fmulconcat(d["grad"], d["a"])
    m_, n_, k_ = 37, 29, 53
    for tl in (0, 1):
        for tr in (0, 1):
            left = u(-1, 1, *((k_, m_) if tl else (m_, k_)))
            right = u(-1, 1, *((n_, k_) if tr else (k_, n_)))
            tag = f"mm_{'t' if tl else 'f'}_{'t' if tr else 'f'}"
            d[tag + "_left"], d[tag + "_right"] = left, right
            d[tag + "_out"] = ref.fmatmul(tl, tr, left, right)
    np.savez_compressed(os.path.join(HERE, "seeded_cases.npz"), **d)
    print("wrote", len(kats), "KATs and", len(d), "seeded arrays")


if __name__ == "__main__":
    main()
