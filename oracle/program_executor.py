"""Runs a builtin Program (polarai-framework_b200/program.py) on the CPU oracle.
TEST INFRASTRUCTURE ONLY: used by the tests, the smoke check and the bench's
CPU-baseline legs to execute the identical builtin sequence on host cores."""
import numpy as np


class OracleExecutor:
    def __init__(self, program, impl, allreduce=None):
        self.program = program
        self.impl = impl
        self.allreduce = allreduce
        self.t = {n: np.zeros(s, np.float32) for n, s in program.tensors.items()}
        for name, v in program.constants.items():
            self.t[name] = impl.ffill(v, int(np.prod(program.tensors[name]))).reshape(program.tensors[name])

    def set_inputs(self, **arrays):
        for name, a in arrays.items():
            self.t[name] = np.ascontiguousarray(a, np.float32).reshape(self.program.tensors[name])

    def run(self):
        t, o = self.t, self.impl
        for kernel, args in self.program.ops:
            g = lambda i: t[args[i]]
            if kernel == "ALLREDUCE":
                if self.allreduce is not None:
                    t[args[0]] = self.allreduce(t[args[0]])
                continue
            if kernel == "ALLREDUCE_FADD":
                # sum over ranks, then the reference's update fadd(W, sw, g, sg) per pair
                for i in range(2, len(args), 2):
                    w, gname = args[i], args[i + 1]
                    if self.allreduce is not None:
                        t[gname] = self.allreduce(t[gname])
                    t[w] = np.asarray(o.fadd(t[w].ravel(), args[0], t[gname].ravel(), args[1]),
                                      np.float32).reshape(self.program.tensors[w])
                continue
            if kernel == "ALLREDUCE_FADD_PART":
                # the same sum and update for a block of rows of each listed pair
                for i in range(4, len(args), 4):
                    w, gname, r0, rows = args[i], args[i + 1], int(args[i + 2]), int(args[i + 3])
                    sl = slice(r0, r0 + rows) if rows >= 0 else slice(None)
                    piece = np.ascontiguousarray(t[gname][sl])
                    if self.allreduce is not None:
                        piece = self.allreduce(piece)
                    t[gname][sl] = piece
                    t[w][sl] = np.asarray(o.fadd(np.ascontiguousarray(t[w][sl]).ravel(), args[0], piece.ravel(), args[1]),
                                          np.float32).reshape(t[w][sl].shape)
                continue
            if kernel == "fmatmul_t_f_rows":
                # rows [r0, r0 + rows) of left^T . right: the product of that column block of left
                left, right, r0, rows, outn = args[0], args[1], int(args[2]), int(args[3]), args[4]
                t[outn][r0:r0 + rows] = o.fmatmul(True, False, np.ascontiguousarray(t[left][:, r0:r0 + rows]), t[right])
                continue
            if kernel == "fdense_grad":
                # the two builtins it stands for: fmatmul_t_f(H, dZ) and fmatmul_f_t(dZ, W) followed by
                # the Sigmoid derivative chain with H
                d, w, h, dw, din = args
                t[dw] = np.asarray(o.fmatmul(True, False, t[h], t[d]), np.float32).reshape(self.program.tensors[dw])
                r = o.fmatmul(False, True, t[d], t[w])
                one = o.ffill(1.0, t[h].size)
                r = o.fmul(r.ravel(), o.fmul(o.fadd(one, 1.0, t[h].ravel(), -1.0), t[h].ravel()))
                t[din] = np.asarray(r, np.float32).reshape(self.program.tensors[din])
                continue
            out = args[-1]
            shape = self.program.tensors[out]
            if kernel == "fadd":
                r = o.fadd(g(0).ravel(), args[1], g(2).ravel(), args[3])
            elif kernel == "fmul":
                r = o.fmul(g(0).ravel(), g(1).ravel())
            elif kernel == "fdivide":
                r = o.fdivide(g(0).ravel(), g(1).ravel())
            elif kernel == "fsigmoid":
                r = o.fsigmoid(g(0).ravel())
            elif kernel == "flogloss":
                r = o.flogloss(g(0).ravel(), g(1).ravel())
            elif kernel == "fcopy":
                r = o.fcopy(g(0).ravel())
            elif kernel == "ffill":
                r = o.ffill(args[0], int(np.prod(shape)))
            elif kernel == "fmulconcat":
                r = o.fmulconcat(g(0).ravel(), g(1).ravel())
            elif kernel == "fsigmoid_grad":
                # the reference's derivative chain, launch by launch
                one = o.ffill(1.0, g(1).size)
                r = o.fmul(g(0).ravel(), o.fmul(o.fadd(one, 1.0, g(1).ravel(), -1.0), g(1).ravel()))
            elif kernel == "fsigmoid_logloss_grad":
                # LogLoss' then Sigmoid', launch by launch as the reference composes them
                pr, y = g(0).ravel(), g(1).ravel()
                one = o.ffill(1.0, pr.size)
                dldp = o.fdivide(o.fadd(pr, 1.0, y, -1.0), o.fadd(pr, 1.0, o.fmul(pr, pr), -1.0))
                r = o.fmul(dldp, o.fmul(o.fadd(one, 1.0, pr, -1.0), pr))
            elif kernel.startswith("fmatmul_"):
                r = o.fmatmul(kernel[8] == "t", kernel[10] == "t", g(0), g(1))
                if kernel.endswith("_sigmoid"):
                    r = o.fsigmoid(r.ravel())
                elif kernel.endswith("_sigmoid_grad"):
                    one = o.ffill(1.0, g(2).size)
                    r = o.fmul(r.ravel(), o.fmul(o.fadd(one, 1.0, g(2).ravel(), -1.0), g(2).ravel()))
            else:
                raise KeyError(kernel)
            t[out] = np.asarray(r, np.float32).reshape(shape)

    def output(self, name):
        return self.t[name]
