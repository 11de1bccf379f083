"""Builtin programs: the flat list of builtin launches a PolarAI graph compiles to.

The reference's GraphCompiler walks a graph and emits, per node, one builtin call
(src/core/graph/internal/GraphCompiler.cpp:21-110; the operations' gen() methods
under src/operation/internal/ choose the builtin and its argument order).  A
`Program` is that list, with tensors named instead of numbered.  The same program
object is executed by the CUDA runtime (DeviceExecutor below) and, in the tests and
the CPU baseline, by the CPU oracle - both sides run the identical sequence.

Programs for the benchmark configurations are built here from the reference's
operations: MatMul -> fmatmul_{f,t}_{f,t}, Sigmoid -> fsigmoid, LogLoss -> flogloss,
Add/Combine -> fadd, Mul -> fmul, Divide -> fdivide; derivatives are composed as
the operations' genDerivative() methods compose them
(SigmoidOperationInternal.cpp:107-135, LogLossOperationInternal.cpp:127-170).
"ALLREDUCE" is the one step the reference has no counterpart for: the sum of a
gradient over data-parallel ranks.
"""
import ctypes
from dataclasses import dataclass, field

import torch

from .capi import Arg, lib


@dataclass
class Program:
    name: str
    tensors: dict = field(default_factory=dict)      # name -> shape
    ops: list = field(default_factory=list)          # (native kernel name, [tensor names / floats])
    inputs: list = field(default_factory=list)       # tensors the caller fills
    constants: dict = field(default_factory=dict)    # name -> fill value (ConstantLoader)
    outputs: list = field(default_factory=list)

    def tensor(self, name, *shape):
        self.tensors[name] = tuple(int(s) for s in shape)
        return name

    def op(self, kernel, *args):
        self.ops.append((kernel, list(args)))

    def launches(self):
        return sum(1 for k, _ in self.ops if k != "ALLREDUCE")

    def exchanged(self):
        """Names of the gradients the program sums over peer memory, in payload order."""
        names = []
        for k, a in self.ops:
            if k == "ALLREDUCE_FADD":
                names += [a[i] for i in range(3, len(a), 2) if a[i] not in names]
            elif k == "ALLREDUCE_FADD_PART":
                names += [g for _, g, _, _ in exchange_pieces(a) if g not in names]
        return names


def exchange_pieces(args):
    """(weight, gradient, first row, rows) of every piece an ALLREDUCE_FADD_PART op exchanges;
    rows < 0 = the whole tensor.  args = [scale_w, scale_g, channel, overlapped, W, g, row0, rows, ...]."""
    return [(args[i], args[i + 1], int(args[i + 2]), int(args[i + 3])) for i in range(4, len(args), 4)]


def elementwise_chain_program(n):
    """out = sigmoid((a + b) * c / d): Add -> Mul -> Divide -> Sigmoid."""
    p = Program("elementwise_chain")
    for t in "abcd":
        p.tensor(t, n)
    p.inputs = list("abcd")
    p.tensor("t1", n), p.tensor("t2", n), p.tensor("t3", n), p.tensor("out", n)
    p.op("fadd", "a", 1.0, "b", 1.0, "t1")
    p.op("fmul", "t1", "c", "t2")
    p.op("fdivide", "t2", "d", "t3")
    p.op("fsigmoid", "t3", "out")
    p.outputs = ["out"]
    return p


def _logloss_sigmoid_backward(p, P, Y, ones, dZ, tag):
    """dZ = dL/dP * dP/dZ with the reference's derivative chains:
    LogLoss' = (p - y) / (p - p*p)   (LogLossOperationInternal.cpp:127-170)
    Sigmoid' = (1 - p) * p           (SigmoidOperationInternal.cpp:107-135)."""
    shape = p.tensors[P]
    t = lambda s: p.tensor(f"{tag}_{s}", *shape)
    p.op("fadd", P, 1.0, Y, -1.0, t("pmy"))
    p.op("fmul", P, P, t("pp"))
    p.op("fadd", P, 1.0, f"{tag}_pp", -1.0, t("den"))
    p.op("fdivide", f"{tag}_pmy", f"{tag}_den", t("dLdP"))
    p.op("fadd", ones, 1.0, P, -1.0, t("omp"))
    p.op("fmul", f"{tag}_omp", P, t("sp"))
    p.op("fmul", f"{tag}_dLdP", f"{tag}_sp", dZ)


def logreg_program(batch=256, n_in=784, lr=0.1):
    """Logistic-regression step: MatMul -> Sigmoid -> LogLoss, batch gradient,
    one SGD update W <- W - lr * X^T dZ."""
    p = Program("logreg_step")
    p.tensor("X", batch, n_in), p.tensor("W", n_in, 1), p.tensor("Y", batch, 1)
    p.inputs = ["X", "W", "Y"]
    p.tensor("ones", batch, 1)
    p.constants["ones"] = 1.0
    p.tensor("Z", batch, 1), p.tensor("P", batch, 1), p.tensor("L", batch, 1)
    p.tensor("dZ", batch, 1), p.tensor("dW", n_in, 1)
    p.op("fmatmul_f_f", "X", "W", "Z")
    p.op("fsigmoid", "Z", "P")
    p.op("flogloss", "P", "Y", "L")
    _logloss_sigmoid_backward(p, "P", "Y", "ones", "dZ", "b")
    p.op("fmatmul_t_f", "X", "dZ", "dW")
    p.op("ALLREDUCE", "dW")
    p.op("fadd", "W", 1.0, "dW", -lr, "W")
    p.outputs = ["L", "W", "dW"]
    return p


def mlp_program(batch, n_in=784, n_hidden=4096, n_out=10, lr=0.1):
    """2-layer MLP forward + backward + SGD update on `batch` rows (the rows one
    rank holds).  No biases (the reference has no broadcasting add); gradients are
    batch sums (it has no mean)."""
    p = Program("mlp_step")
    p.tensor("X", batch, n_in), p.tensor("Y", batch, n_out)
    p.tensor("W1", n_in, n_hidden), p.tensor("W2", n_hidden, n_out)
    p.inputs = ["X", "Y", "W1", "W2"]
    p.tensor("ones_h", batch, n_hidden), p.tensor("ones_o", batch, n_out)
    p.constants = {"ones_h": 1.0, "ones_o": 1.0}
    for t in ("Z1", "H", "dH", "omh", "sh", "dZ1"):
        p.tensor(t, batch, n_hidden)
    for t in ("Z2", "P", "L", "dZ2"):
        p.tensor(t, batch, n_out)
    p.tensor("dW1", n_in, n_hidden), p.tensor("dW2", n_hidden, n_out)
    # forward
    p.op("fmatmul_f_f", "X", "W1", "Z1")
    p.op("fsigmoid", "Z1", "H")
    p.op("fmatmul_f_f", "H", "W2", "Z2")
    p.op("fsigmoid", "Z2", "P")
    p.op("flogloss", "P", "Y", "L")
    # backward
    _logloss_sigmoid_backward(p, "P", "Y", "ones_o", "dZ2", "o")
    p.op("fmatmul_t_f", "H", "dZ2", "dW2")
    p.op("ALLREDUCE", "dW2")
    p.op("fmatmul_f_t", "dZ2", "W2", "dH")
    p.op("fadd", "ones_h", 1.0, "H", -1.0, "omh")
    p.op("fmul", "omh", "H", "sh")
    p.op("fmul", "dH", "sh", "dZ1")
    p.op("fmatmul_t_f", "X", "dZ1", "dW1")
    p.op("ALLREDUCE", "dW1")
    # update
    p.op("fadd", "W2", 1.0, "dW2", -lr, "W2")
    p.op("fadd", "W1", 1.0, "dW1", -lr, "W1")
    p.outputs = ["L", "W1", "W2", "dW1", "dW2"]
    return p


def fuse_program(program):
    """Rewrites a program with the extended builtins, keeping every result bit-identical:

      fadd(ones,1,S,-1,t1); fmul(t1,S,t2); fmul(G,t2,out)   ->  fsigmoid_grad(G, S, out)
      fadd(P,1,Y,-1,a); fmul(P,P,b); fadd(P,1,b,-1,c); fdivide(a,c,d); fsigmoid_grad(d,P,out)
                                                             ->  fsigmoid_logloss_grad(P, Y, out)
      fmatmul_x_y(L,R,Z); fsigmoid(Z,H)                      ->  fmatmul_x_y_sigmoid(L, R, H)
      fmatmul_x_y(L,R,G); fsigmoid_grad(G,S,out)             ->  fmatmul_x_y_sigmoid_grad(L, R, S, out)
      fmatmul_t_f(H,D,dW); fmatmul_f_t_sigmoid_grad(D,W,H,dIn) ->  fdense_grad(D, W, H, dW, dIn)
                                                                 (one pass over H instead of two; an
                                                                 ALLREDUCE(dW) between them moves behind)

    A rewrite applies only when the intermediates (t1, t2, Z, G) are read by nothing else
    and are not outputs of the program; they are then never written.  `ones` must be a
    constant 1.0 tensor."""
    ops = [(k, list(a)) for k, a in program.ops]

    def readers(name, skip):
        n = 0
        for i, (k, a) in enumerate(ops):
            if i in skip or k == "ALLREDUCE":
                continue
            ins = a[:-1]
            n += sum(1 for x in ins if x == name)
        return n

    def dead_after(name, skip):
        return name not in program.outputs and name not in program.inputs and readers(name, skip) == 0

    changed = True
    while changed:
        changed = False
        for i in range(len(ops)):
            k, a = ops[i]
            # sigmoid derivative chain
            if (k == "fadd" and i + 2 < len(ops) and program.constants.get(a[0]) == 1.0 and a[1] == 1.0
                    and a[3] == -1.0):
                s_, t1 = a[2], a[4]
                k2, a2 = ops[i + 1]
                k3, a3 = ops[i + 2]
                if (k2 == "fmul" and a2[0] == t1 and a2[1] == s_ and k3 == "fmul" and a3[1] == a2[2]
                        and dead_after(t1, {i, i + 1, i + 2}) and dead_after(a2[2], {i, i + 1, i + 2})):
                    ops[i:i + 3] = [("fsigmoid_grad", [a3[0], s_, a3[2]])]
                    changed = True
                    break
            # LogLoss derivative followed by the Sigmoid derivative of the same tensor
            if (k == "fadd" and i + 4 < len(ops) and a[1] == 1.0 and a[3] == -1.0):
                pr, y, pmy = a[0], a[2], a[4]
                (k1, a1), (k2, a2), (k3, a3), (k4, a4) = ops[i + 1:i + 5]
                span = set(range(i, i + 5))
                if (k1 == "fmul" and a1[0] == pr and a1[1] == pr
                        and k2 == "fadd" and a2[:4] == [pr, 1.0, a1[2], -1.0]
                        and k3 == "fdivide" and a3[0] == pmy and a3[1] == a2[4]
                        and k4 == "fsigmoid_grad" and a4[0] == a3[2] and a4[1] == pr
                        and all(dead_after(t, span) for t in (pmy, a1[2], a2[4], a3[2]))):
                    ops[i:i + 5] = [("fsigmoid_logloss_grad", [pr, y, a4[2]])]
                    changed = True
                    break
            # matmul followed by the builtin that consumes its result
            if k.startswith("fmatmul_") and len(k) == 11:
                z = a[2]
                for j in range(i + 1, len(ops)):
                    kj, aj = ops[j]
                    if kj == "ALLREDUCE":
                        continue
                    if z in aj[:-1] or aj[-1] == z:
                        if kj == "fsigmoid" and aj[0] == z and dead_after(z, {i, j}):
                            ops[j] = (k + "_sigmoid", [a[0], a[1], aj[1]])
                            del ops[i]
                            changed = True
                        elif (kj == "fsigmoid_grad" and aj[0] == z and aj[1] != z and dead_after(z, {i, j})
                              and not any(o[1][-1] in (a[0], a[1]) for o in ops[i + 1:j] if o[0] != "ALLREDUCE")):
                            ops[j] = (k + "_sigmoid_grad", [a[0], a[1], aj[1], aj[2]])
                            del ops[i]
                            changed = True
                        break
                if changed:
                    break
            # the two products of a dense layer's backward pass that read its input activations
            if k == "fmatmul_t_f" and i + 1 < len(ops):
                h, d, dw = a
                j = i + 1
                moved = []
                while j < len(ops) and ops[j][0] == "ALLREDUCE" and ops[j][1][0] == dw:
                    moved.append(ops[j])
                    j += 1
                if j < len(ops) and ops[j][0] == "fmatmul_f_t_sigmoid_grad":
                    d2, w, h2, din = ops[j][1]
                    if d2 == d and h2 == h and len({h, d, dw, w, din}) == 5:
                        ops[i:j + 1] = [("fdense_grad", [d, w, h, dw, din])] + moved
                        changed = True
                        break
    fused = Program(program.name + "_fused", dict(program.tensors), ops, list(program.inputs),
                    dict(program.constants), list(program.outputs))
    return fused


def fuse_gradient_exchange(program):
    """Rewrites the data-parallel tail of a program

        ALLREDUCE(g1) ... ALLREDUCE(gk) ... fadd(W1,sw,g1,sg,W1) ... fadd(Wk,sw,gk,sg,Wk)

    into one op  ALLREDUCE_FADD(sw, sg, W1, g1, ..., Wk, gk)  at the place of the first of
    those updates: the sum over ranks and the updates in a single launch
    (polar_b200_allreduce_fadd).  It applies only when every ALLREDUCE'd gradient has exactly
    such an update after the last ALLREDUCE, all with the same two scales, and nothing after the
    first update reads a weight or gradient involved; otherwise the program is returned as is."""
    ops = [(k, list(a)) for k, a in program.ops]
    red = [(i, a[0]) for i, (k, a) in enumerate(ops) if k == "ALLREDUCE"]
    if not red:
        return program
    last_red = max(i for i, _ in red)
    grads = [g for _, g in red]
    upd = {}
    for i, (k, a) in enumerate(ops):
        if k == "fadd" and i > last_red and a[2] in grads and a[0] == a[4] and a[2] not in upd:
            upd[a[2]] = i
    if sorted(upd) != sorted(grads):
        return program
    first = min(upd.values())
    scales = {(ops[i][1][1], ops[i][1][3]) for i in upd.values()}
    if len(scales) != 1:
        return program
    touched = set(grads) | {ops[i][1][0] for i in upd.values()}
    for i in range(first, len(ops)):
        if i in upd.values():
            continue
        if any(isinstance(x, str) and x in touched for x in ops[i][1]):
            return program
    sw, sg = next(iter(scales))
    # payload order: the order the backward pass produces the gradients in
    pairs = []
    for _, g in red:
        pairs += [ops[upd[g]][1][0], g]
    new_ops = []
    for i, op in enumerate(ops):
        if op[0] == "ALLREDUCE" or i in upd.values():
            if i == first:
                new_ops.append(("ALLREDUCE_FADD", [float(sw), float(sg)] + pairs))
            continue
        new_ops.append(op)
    return Program(program.name + "_xchg", dict(program.tensors), new_ops, list(program.inputs),
                   dict(program.constants), list(program.outputs))


def overlap_gradient_exchange(program, tile_rows=256):
    """Rewrites the tail  fmatmul_t_f(X, D, g); ALLREDUCE_FADD(sw, sg, ..., W, g, ...)  so that most of
    the exchange runs WHILE the last gradient is still being computed:

        fmatmul_t_f_rows(X, D, 0, r, g)                    rows [0, r) of g
        ALLREDUCE_FADD_PART(sw, sg, channel 1, overlapped, W, g, 0, r)       on a second stream
        fmatmul_t_f_rows(X, D, r, m - r, g)                the remaining rows, meanwhile
        ALLREDUCE_FADD_PART(sw, sg, channel 0, in order,  W, g, r, m - r, <every other pair, whole>)

    r = two thirds of the rows, rounded down to whole tiles.  The payload is laid out with g first,
    so the second exchange's pieces are contiguous.  Per element the sum over the ranks and the
    update are unchanged; each block of rows is the fmatmul_t_f product of a column block of X, whose
    sum over k the tensor-core kernel may cut into work units differently than for the whole matrix -
    so g agrees with the one-launch form within the fmatmul tolerance (on the CPU oracle, which sums
    sequentially, bit for bit), and the replicas stay bit-identical to each other.
    Returned unchanged when the program has no such tail or g has too few rows to cut."""
    ops = [(k, list(a)) for k, a in program.ops]
    if len(ops) < 2 or ops[-1][0] != "ALLREDUCE_FADD" or ops[-2][0] != "fmatmul_t_f":
        return program
    sw, sg = ops[-1][1][:2]
    pairs = [(ops[-1][1][i], ops[-1][1][i + 1]) for i in range(2, len(ops[-1][1]), 2)]
    x, d, g = ops[-2][1]
    if g not in [gr for _, gr in pairs]:
        return program
    m = program.tensors[g][0]
    r = (2 * m // 3) // tile_rows * tile_rows
    if r < tile_rows or m - r < 64 or r % 4:
        return program
    w = next(wt for wt, gr in pairs if gr == g)
    rest = [(wt, gr) for wt, gr in pairs if gr != g]
    last = [float(sw), float(sg), 0.0, 0.0, w, g, float(r), float(m - r)]
    for wt, gr in rest:
        last += [wt, gr, 0.0, -1.0]
    new_ops = ops[:-2] + [
        ("fmatmul_t_f_rows", [x, d, 0.0, float(r), g]),
        ("ALLREDUCE_FADD_PART", [float(sw), float(sg), 1.0, 1.0, w, g, 0.0, float(r)]),
        ("fmatmul_t_f_rows", [x, d, float(r), float(m - r), g]),
        ("ALLREDUCE_FADD_PART", last),
    ]
    return Program(program.name + "_overlap", dict(program.tensors), new_ops, list(program.inputs),
                   dict(program.constants), list(program.outputs))


class DeviceExecutor:
    """Runs a Program on one GPU: one device tensor per program tensor, every op
    through polar_b200_launch_by_name on torch's current stream.  Argument
    structs are built once, so replaying the program costs one ctypes call per
    launch.  `allreduce` is a callable taking a tensor (torch.distributed over
    NCCL in the data-parallel runs; None = single rank, no-op).  A program with an
    ALLREDUCE_FADD op needs `peers`, a PeerGradients built for program.exchanged():
    those gradients then live in its peer buffer."""

    def __init__(self, program, device="cuda:0", allreduce=None, peers=None):
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device: programs have no CPU path in this package")
        self.program = program
        self.device = torch.device(device)
        self.lib = lib()
        self.allreduce = allreduce
        exchanged = program.exchanged()
        if exchanged and (peers is None or sorted(peers.tensors) != sorted(exchanged)):
            raise ValueError("the program exchanges gradients over peer memory: pass `peers` built for "
                             f"{exchanged}")
        self.peers = peers if exchanged else None
        self.t = {n: (peers.tensors[n] if n in exchanged else torch.empty(s, dtype=torch.float32, device=self.device))
                  for n, s in program.tensors.items()}
        self._keep = []
        self._compiled = []
        fn = self.lib.cdll.polar_b200_launch_by_name
        for kernel, args in program.ops:
            if kernel == "ALLREDUCE":
                self._compiled.append((None, args[0], 0))
                continue
            if kernel == "ALLREDUCE_FADD":
                pairs = [(self.t[args[i]], args[i + 1]) for i in range(2, len(args), 2)]
                self._compiled.append(("peers", (peers.segments(pairs), float(args[0]), float(args[1])), 0))
                continue
            if kernel == "ALLREDUCE_FADD_PART":
                pieces = [(self.t[w], g, r0, rows) for w, g, r0, rows in exchange_pieces(args)]
                seg, first, count = peers.piece_segments(pieces)
                self._compiled.append(("peers_part", (seg, first, count, int(args[2]), bool(args[3]), float(args[0]),
                                                      float(args[1])), 0))
                continue
            arr = (Arg * len(args))()
            for i, a in enumerate(args):
                if isinstance(a, str):
                    tt = self.t[a]
                    shp = (ctypes.c_uint64 * tt.dim())(*tt.shape)
                    self._keep.append(shp)
                    arr[i].is_tensor = 1
                    arr[i].tensor.data = tt.data_ptr()
                    arr[i].tensor.dims = tt.dim()
                    arr[i].tensor.shape = shp
                else:
                    arr[i].is_tensor = 0
                    arr[i].scalar = float(a)
            self._keep.append(arr)
            self._compiled.append((kernel.encode(), arr, len(args)))
        self._fn = fn
        # an exchange marked "overlapped" runs on a second stream, forked from the launch stream where
        # the op stands and joined at the end of the program
        self._side = None
        if any(k == "peers_part" and a[4] for k, a, _ in self._compiled):
            self._side = torch.cuda.Stream(self.device)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
        # one scratch buffer, sized for the most demanding launch of the program
        wsb = self.lib.cdll.polar_b200_launch_workspace_bytes
        need = max([0] + [int(wsb(k, arr, n)) for k, arr, n in self._compiled if isinstance(k, bytes)])
        self.workspace = torch.empty(max(need, 16), dtype=torch.uint8, device=self.device)
        self._ws_ptr, self._ws_bytes = self.workspace.data_ptr(), need
        self.fill_constants()

    def fill_constants(self):
        s = torch.cuda.current_stream(self.device).cuda_stream
        for name, value in self.program.constants.items():
            self.lib.call("polar_b200_ffill", float(value), self.t[name].data_ptr(), self.t[name].numel(), s)

    def set_inputs(self, **arrays):
        for name, a in arrays.items():
            self.t[name].copy_(a if isinstance(a, torch.Tensor) else torch.from_numpy(a))

    def run(self):
        main = torch.cuda.current_stream(self.device)
        s = main.cuda_stream
        forked = False
        for kernel, arr, n in self._compiled:
            if kernel is None:
                if self.allreduce is not None:
                    self.allreduce(self.t[arr])
                continue
            if kernel == "peers":
                self.peers.launch(arr[0], arr[1], arr[2], s)
                continue
            if kernel == "peers_part":
                seg, first, count, channel, overlapped, sw, sg = arr
                if overlapped:
                    self._fork.record(main)
                    self._side.wait_event(self._fork)
                    self.peers.launch_range(channel, first, count, seg, sw, sg, self._side.cuda_stream)
                    forked = True
                else:
                    self.peers.launch_range(channel, first, count, seg, sw, sg, s)
                continue
            rc = self._fn(kernel, arr, n, self._ws_ptr, self._ws_bytes, s)
            if rc != 0:
                self.lib.check(rc)
        if forked:
            self._join.record(self._side)
            main.wait_event(self._join)

    def output(self, name):
        torch.cuda.synchronize(self.device)
        return self.t[name].cpu().numpy()
