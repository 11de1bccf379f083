/*
 * polar_b200.h - C ABI of the B200 (sm_100a) builtin kernels for the PolarAI
 * ("Athena") runtime.
 *
 * One entry point per builtin a PolarAI device runtime must provide.  Each is
 * named after the builtin's native kernel name - the dispatch key a runtime
 * receives in LaunchCommand::nativeKernelName
 * (include/polarai/backend/generic/runtime/LaunchCommand.h:26-31 of the
 * reference; the name table is src/backend/generic/runtime/sycl/SYCLDevice.cpp:57-96)
 * - and takes the builtin's operands in the order of its LaunchCommand
 * arguments, as plain device pointers and element counts.
 *
 * Conventions
 *  - every pointer is a DEVICE pointer to dense row-major fp32 unless said
 *    otherwise; nothing here allocates, copies to the host or synchronises
 *    unless said otherwise;
 *  - `stream` is a cudaStream_t passed as void* (NULL = the legacy default
 *    stream); the launch is asynchronous on it;
 *  - the return value is a polar_b200_status; no entry point aborts the
 *    process (the reference's convention is std::terminate on a CUDA error,
 *    src/backend/generic/runtime/cuda/utils.hpp:20-28);
 *  - `out` may alias an input element-for-element (the reference updates
 *    weights in place: src/core/graph/internal/GraphInternal.cpp:464-465);
 *  - n == 0 (or an empty matrix) is a successful no-op.
 */
#ifndef POLAR_B200_H
#define POLAR_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum polar_b200_status {
  POLAR_B200_OK = 0,
  POLAR_B200_ERR_INVALID = 1,     /* null pointer, bad flag, size overflow */
  POLAR_B200_ERR_CUDA = 2,        /* a CUDA call failed; see polar_b200_last_error */
  POLAR_B200_ERR_UNSUPPORTED = 3, /* unknown kernel name or argument pattern */
  POLAR_B200_ERR_TIMEOUT = 4,     /* a bounded wait gave up: a device-side wait (see
                                     polar_b200_check_device_status) or a collective's
                                     time limit on the host */
  POLAR_B200_ERR_WORKSPACE = 5    /* caller's workspace is too small */
} polar_b200_status;

/* Text of the last error recorded by the calling thread ("" if none). */
const char* polar_b200_last_error(void);
/* Library version, and the compute capability it was built for (100). */
int polar_b200_version(void);
int polar_b200_built_for_sm(void);

/* ---- elementwise builtins ------------------------------------------------ */

/* ffill: out[i] = pattern, bit-exact.  LaunchCommand args: f32 pattern, T out.
 * Replaces sycl/kernels/Fill.hpp:71-74 and opencl/kernels.h:21-30. */
int polar_b200_ffill(float pattern, float* out, uint64_t n, void* stream);

/* fcopy: out[i] = in[i], bit-exact.  Args: T in, T out.
 * Replaces PolarGraph/kernels/CopyOp.cpp:21-23 and opencl/kernels.h:44-53. */
int polar_b200_fcopy(const float* in, float* out, uint64_t n, void* stream);

/* fadd: out[i] = a[i]*scaleA + b[i]*scaleB, two rounded products then a
 * rounded sum (no fused multiply-add).  Args: T a, f32 scaleA, T b, f32 scaleB,
 * T out.  Emitted by AddOperation (1,1) and CombineOperation (alpha,beta).
 * Replaces PolarGraph/kernels/AddOp.cpp:36-48 and opencl/kernels.h:32-42. */
int polar_b200_fadd(const float* a, float scaleA, const float* b, float scaleB,
                    float* out, uint64_t n, void* stream);

/* fmul: out[i] = a[i]*b[i].  Args: T a, T b, T out.
 * Replaces PolarGraph/kernels/MulOp.cpp:36-43 and opencl/kernels.h:119-128. */
int polar_b200_fmul(const float* a, const float* b, float* out, uint64_t n,
                    void* stream);

/* fdivide: out[i] = numerator[i]/denominator[i], IEEE round-to-nearest.
 * Args: T numerator, T denominator, T out.
 * Replaces PolarGraph/kernels/DivideOp.cpp:36-43 and opencl/kernels.h:55-64. */
int polar_b200_fdivide(const float* numerator, const float* denominator,
                       float* out, uint64_t n, void* stream);

/* fsigmoid: r = 1/(1+exp(-x)); then |r-1| < 1e-5 -> 1-1e-5, else |r| < 1e-5
 * -> 1e-5.  Args: T in, T out.
 * Replaces sycl/kernels/Sigmoid.hpp:32-41 and opencl/kernels.h:141-156. */
int polar_b200_fsigmoid(const float* in, float* out, uint64_t n, void* stream);

/* The MLIR form of the same builtin, which has no clamp
 * (PolarGraph/kernels/SigmoidOp.cpp:37-51). */
int polar_b200_fsigmoid_unclamped(const float* in, float* out, uint64_t n,
                                  void* stream);

/* flogloss: out[i] = -y[i]*log(p[i]+eps) - (1-y[i])*log(1-p[i]+eps), eps=1e-5,
 * elementwise (the output has the shape of `predicted`).
 * Args: T predicted, T groundTruth, T out.
 * Replaces sycl/kernels/LogLoss.hpp:33-37 and opencl/kernels.h:66-78. */
int polar_b200_flogloss(const float* predicted, const float* groundTruth,
                        float* out, uint64_t n, void* stream);

/* fmulconcat: out[i] = gradient[0]*localDerivative[i].
 * Args: T gradient, T localDerivative, T out.
 * Replaces PolarGraph/kernels/MulConcatOp.cpp:37-46 and opencl/kernels.h:130-139. */
int polar_b200_fmulconcat(const float* gradient, const float* localDerivative,
                          float* out, uint64_t n, void* stream);

/* ---- the other operation builtins (not on the benchmarked path) ---------- */

/* frelu: out[i] = in[i] > 0 ? in[i] : 0.  Args: T in, T out.
 * Replaces PolarGraph/kernels/ReLUOp.cpp:36-44. */
int polar_b200_frelu(const float* in, float* out, uint64_t n, void* stream);

/* fsoftmax over the WHOLE tensor: out[i] = exp(in[i]) / sum_j exp(in[j]), no maximum
 * subtracted (PolarGraph/kernels/SoftmaxOp.cpp:38-66).  Args: T in, T out.  Needs 8
 * bytes of scratch for the sum: `workspace` (8-byte aligned) or, when NULL, the
 * stream-ordered pool. */
int polar_b200_fsoftmax(const float* in, float* out, uint64_t n, void* workspace,
                        uint64_t workspace_bytes, void* stream);

/* fpool: 2-D max pooling of an [h,w] tensor; out is [(h-windowH)/strideH+1,
 * (w-windowW)/strideW+1]; every maximum starts from -10e5 as in the reference
 * (PolarGraph/kernels/Pool2DOp.cpp:44-84).  As a builtin: T in, four 8-byte integer
 * DATA arguments (windowH, windowW, strideH, strideW), T out. */
int polar_b200_fpool(const float* in, uint64_t h, uint64_t w, uint64_t windowH,
                     uint64_t windowW, uint64_t strideH, uint64_t strideW, float* out,
                     void* stream);

/* fconv2d: single-channel "valid" cross-correlation, out[i,j] = sum_{a,b}
 * in[i+a,j+b]*kernel[a,b] (products rounded, added in row-major kernel order); out is
 * [h-kh+1, w-kw+1]; kernel extents must be odd (PolarGraph/kernels/Conv2DOp.cpp:35-90).
 * Args: T in, T kernel, T out. */
int polar_b200_fconv2d(const float* in, uint64_t h, uint64_t w, const float* kernel,
                       uint64_t kh, uint64_t kw, float* out, void* stream);

/* ftranspose: out[c,r] = in[r,c] for a 2-D tensor in[rows,cols], bit-exact; out is
 * [cols,rows] and must not alias in.  Args: T in, T out.  The reference lists the builtin
 * (include/polarai/core/internal/GenBuiltins.hpp:50 "Transpose 2D tensor (matrix)";
 * PolarGraphOps.td:507-527, kernel name "ftranspose", body empty) but no operation emits it. */
int polar_b200_ftranspose(const float* in, uint64_t rows, uint64_t cols, float* out,
                          void* stream);

/* fslice: out = in[index], the sub-tensor at offset `index` of the first dimension
 * (GenBuiltins.hpp:49 "Get subtensor"; PolarGraphOps.td:134-144 "by first dimension
 * offset": the result has the remaining dimensions), as a bit-exact copy of `inner` =
 * product of the remaining extents floats.  As a builtin: T in, one 8-byte integer DATA
 * argument (index), T out.  The reference's generator functor for Slice returns no value
 * (GenBuiltins.hpp:147-149), so no graph can consume a slice there; here it is reachable
 * by name. */
int polar_b200_fslice(const float* in, uint64_t first_dim, uint64_t inner, uint64_t index,
                      float* out, void* stream);

/* ---- matmul -------------------------------------------------------------- */

/* fmatmul_{f,t}_{f,t}: out[i,j] = sum_k L'[i,k]*R'[k,j] in fp32 accuracy.
 * `left` is stored [m,k], or [k,m] when transLeft; `right` is stored [k,n], or
 * [n,k] when transRight; `out` is [m,n] and is overwritten (no alpha/beta).
 * Args of the builtin: T left, T right, T out; the transposes are part of the
 * kernel NAME (utils/dialects/include/PolarGraph/PolarGraphOps.td:342-352).
 * Replaces PolarGraph/kernels/MatMulOp.cpp:36-85 and opencl/kernels.h:80-117.
 *
 * `workspace` is device scratch of `workspace_bytes` bytes, 256-byte aligned;
 * polar_b200_fmatmul_workspace_bytes gives the size this call needs (0 = none;
 * non-zero when the sum over k is cut into several work units whose partial
 * products are added afterwards in a fixed order: narrow results with a long k,
 * and tensor-core shapes with too few tiles to load every SM).
 * With workspace == NULL the call takes the scratch it needs from the
 * device's stream-ordered memory pool (cudaMallocAsync/cudaFreeAsync on
 * `stream`). */
int polar_b200_fmatmul(int transLeft, int transRight, uint64_t m, uint64_t n,
                       uint64_t k, const float* left, const float* right,
                       float* out, void* workspace, uint64_t workspace_bytes,
                       void* stream);
uint64_t polar_b200_fmatmul_workspace_bytes(int transLeft, int transRight,
                                            uint64_t m, uint64_t n, uint64_t k);

/* A block of rows of fmatmul_t_f: out[row0 .. row0+rows, :] of out[m,n] = left^T . right with
 * left stored [k,m], right [k,n]; the other rows of `out` are not touched.  Bit for bit the
 * rows the product of the column block of `left` gives.  For a step that exchanges a weight
 * gradient between GPUs while the rest of it is still being computed (see
 * polar_b200_allreduce_fadd_range).  row0 and m multiples of 4; the block must be one the
 * tensor-core path serves (rows >= 64, n >= 32, k >= 32, TMA-describable), else
 * POLAR_B200_ERR_UNSUPPORTED.  Native name "fmatmul_t_f_rows": T left, T right, f32 row0,
 * f32 rows (whole numbers), T out. */
int polar_b200_fmatmul_t_f_rows(uint64_t m, uint64_t row0, uint64_t rows, uint64_t n, uint64_t k,
                                const float* left, const float* right, float* out,
                                void* workspace, uint64_t workspace_bytes, void* stream);
uint64_t polar_b200_fmatmul_t_f_rows_workspace_bytes(uint64_t rows, uint64_t n, uint64_t k);

/* fmatmul_t_f / fmatmul_t_t for a narrow result, without any allocation.
 * No counterpart in the reference: it exists for hosts that cannot call
 * cudaMalloc while they run - an application that has already handed all device
 * memory to its own allocator (any further cudaMalloc or pool growth fails), or
 * one on a path where the device-wide synchronisation of cudaMalloc/cudaFree is
 * not acceptable.  polar_b200_fmatmul needs scratch memory for this shape (the
 * sum over the long k dimension is split over CTAs) and takes it from the caller
 * or from the stream-ordered pool; this variant computes the same product,
 *     out[m,n] = sum_k left[k,m] * R'[k,n]      (left stored [k,m]; right stored
 *                                                [k,n], or [n,k] when transRight)
 * with the partial sums in an array that is part of the library image
 * (polar_b200_static_scratch_bytes() = 16 MiB, held by every GPU that loads the
 * library until the process exits).  The caller still owns left, right and out.
 *  - Shapes: n <= 16, k >= 32, m a multiple of 4, left 16-byte aligned; the
 *    scratch needed is splits*m*n*4 bytes with splits about 2*SMs/ceil(m/1024)
 *    (12 MiB for m=4096, n=10).  A product that needs more returns
 *    POLAR_B200_ERR_WORKSPACE; other shapes return POLAR_B200_ERR_UNSUPPORTED.
 *  - The first call on each device looks the array's device address up
 *    (cudaGetSymbolAddress, with the stream's device current); make that first call
 *    outside any stream capture.  With CUDA's default lazy module loading the 16 MiB
 *    are reserved on a GPU when the library's module is first used there, not when the
 *    library is loaded: a host that is about to hand ALL remaining device memory to its
 *    own allocator should make one call per device first (or run with
 *    CUDA_MODULE_LOADING=EAGER), or that first call can fail for lack of memory.
 *  - All calls share the one array per device and it keeps the last call's
 *    contents.  Nothing in it has to start at zero (each call overwrites every
 *    value it later reads).  Two calls whose kernels overlap on the GPU - different
 *    streams, or different host threads - race on it: keep them on one stream or
 *    order them with events.
 *  - Calls no cudaMalloc, cudaFree, or any allocating library routine. */
int polar_b200_fmatmul_tn_small_n_static(int transRight, uint64_t m, uint64_t n,
                                         uint64_t k, const float* left,
                                         const float* right, float* out,
                                         void* stream);
uint64_t polar_b200_static_scratch_bytes(void);

/* The same product on the CUDA cores: one FFMA per term, k ascending per
 * output within a thread.  Kept only as a device-side cross-check of the
 * tensor-core path; no dispatch reaches it unless a caller asks for it. */
int polar_b200_fmatmul_ffma(int transLeft, int transRight, uint64_t m,
                            uint64_t n, uint64_t k, const float* left,
                            const float* right, float* out, void* stream);

/* The tensor-core path alone, with its tuning knobs exposed for tests and
 * benchmarks: tile_n is 128 or 256 (128 x tile_n tiles), or 512 for 256 x 256 tiles
 * (slab_k 16 only), plus 1000 to make the operands exchange roles (see
 * polar_b200_fmatmul_tc_plan; not with stream mode); slab_k is 16 or 32 (floats of k staged per pipeline stage); passes is 3 (fp32-accurate three-product
 * TF32 split) or 1 (plain TF32, about 1e-3 relative); write_hi == 1 makes the
 * split warps store the masked high parts explicitly instead of relying on the
 * tensor core ignoring the low 13 mantissa bits (2: diagnostic, the result is not
 * stored); splits is the number of work
 * units the k range of each tile is cut into (1 = none, 0 = the automatic choice,
 * -1 = stream mode: the CTAs take equal shares of all k slabs of all tiles and a tile
 * may be finished by the next CTA - 128 x 256 tiles only; scratch for the partial
 * products comes from the stream-ordered pool).  Fails with
 * POLAR_B200_ERR_UNSUPPORTED when the operands cannot be described to TMA
 * (bases not 16-byte aligned, or a contiguous extent that is not a multiple of
 * 4 floats). */
int polar_b200_fmatmul_tc(int transLeft, int transRight, uint64_t m, uint64_t n,
                          uint64_t k, const float* left, const float* right,
                          float* out, int tile_n, int slab_k, int passes,
                          int write_hi, int splits, void* stream);

/* Bounded device-side waits.  Every wait inside a kernel of this library (mbarriers of the
 * tensor-core matmuls; the ranks of the gradient exchange waiting for one another) gives
 * up after a limit, records a code in the status word of its device and lets the kernel
 * end, so a lost peer or a stuck pipeline never hangs the GPU.  The reference has no
 * counterpart: its runtimes terminate the process on any error
 * (src/backend/generic/runtime/cuda/utils.hpp:20-28).
 *  - Codes: 0 = none; 101..107 = which wait of the tensor-core matmul; 301 = a peer's
 *    gradients never became ready, 302 = a peer never finished its slice (in both cases no
 *    weight was updated).  The first code recorded since the last clear stays.
 *  - The words live in pinned host memory: reading them needs no CUDA call.  Read after
 *    the stream has been synchronised.  polar_b200_device_status() gives the first
 *    non-zero word of any device, _of(device) one device's word, _clear() clears all.
 *  - polar_b200_check_device_status() turns a non-zero word into POLAR_B200_ERR_TIMEOUT
 *    (text in polar_b200_last_error); POLAR_B200_OK otherwise.
 *  - polar_b200_set_wait_limit_ns sets the limit for launches made afterwards (0 = the
 *    defaults: 2 s in the matmuls, 4 s in the exchange). */
int polar_b200_device_status(void);
int polar_b200_device_status_of(int device);
void polar_b200_device_status_clear(void);
int polar_b200_check_device_status(void);
void polar_b200_set_wait_limit_ns(uint64_t ns);
uint64_t polar_b200_wait_limit_ns(void);

/* Which matmul path polar_b200_fmatmul would take for these sizes:
 * 0 = tcgen05 tensor-core tiles, 1 = skinny (bandwidth-bound CUDA-core) path,
 * 2 = FFMA tiles. */
int polar_b200_fmatmul_path(int transLeft, int transRight, uint64_t m,
                            uint64_t n, uint64_t k);

/* How the tensor-core path would run the product (meaningful when polar_b200_fmatmul_path
 * answers 0): *tile_rows = 128 or 256 (rows of a CTA tile; columns are 256), *exchanged = 1
 * when the operands exchange roles - the kernel computes the transposed product with `right`
 * as its row operand and stores each tile transposed, so that a warp's store instruction
 * writes one 128-byte line of a result row (taken for sums of a few hundred to a few thousand
 * terms, where the epilogue is a visible share of a tile's time) - and *splits = work units per
 * tile (1 = whole tiles, 0 = stream mode, >1 = fixed cuts of k).  For a t_f product with rows
 * just past a tile boundary the answer describes the whole-tile part.  Any pointer may be NULL. */
void polar_b200_fmatmul_tc_plan(int transLeft, int transRight, uint64_t m, uint64_t n, uint64_t k,
                                int* tile_rows, int* exchanged, int* splits);

/* ---- extended builtins (beside, never instead of, the ones above) -------- */

/* fsigmoid_grad: out[i] = gradient[i] * ((1 - s[i]) * s[i]) where s is the OUTPUT of
 * fsigmoid.  One pass over the three launches the reference's Sigmoid derivative
 * compiles to - fadd(ones,1,s,-1), fmul(.,s), fmul(gradient,.)
 * (src/operation/internal/SigmoidOperationInternal.cpp:107-135) - keeping their three
 * roundings, so the result is bit-identical to the chain; 12 instead of 36 bytes per
 * element.  Args as a builtin: T gradient, T sigmoidOut, T out. */
int polar_b200_fsigmoid_grad(const float* gradient, const float* sigmoidOut,
                             float* out, uint64_t n, void* stream);

/* fsigmoid_logloss_grad: dZ[i] for LogLoss applied to a Sigmoid output p with labels y:
 *   ((p - y) / (p - p*p)) * ((1 - p) * p)
 * One pass over the seven launches the reference's derivatives compile to - LogLoss':
 * fadd(p,1,y,-1), fmul(p,p), fadd(p,1,pp,-1), fdivide
 * (src/operation/internal/LogLossOperationInternal.cpp:127-170), then Sigmoid' as in
 * fsigmoid_grad - keeping all seven roundings, so the result is bit-identical to the
 * chain.  Args as a builtin: T predicted, T groundTruth, T out. */
int polar_b200_fsigmoid_logloss_grad(const float* predicted, const float* groundTruth,
                                     float* out, uint64_t n, void* stream);

/* fmatmul with the builtin that follows it fused in, bit-identical to launching the
 * two builtins one after the other (the product is rounded to fp32 before the
 * second step either way):
 *   fmatmul_sigmoid       out = fsigmoid(L'.R')              - the hidden layer forward;
 *                         in the tensor-core kernel the epilogue warps apply it while
 *                         the next tile's k loop runs, and the pre-activation is never
 *                         written;
 *   fmatmul_sigmoid_grad  out = (L'.R') * ((1 - s) * s)      - the hidden layer's
 *                         backward, s = fsigmoid output of the forward pass; in the
 *                         small-k kernel the gradient w.r.t. the activations is never
 *                         written.
 * Shapes served by a kernel without a fused form run the two builtins in sequence
 * (the second one in place).  Native names for polar_b200_launch_by_name:
 * "fmatmul_x_y_sigmoid" (T left, T right, T out) and "fmatmul_x_y_sigmoid_grad"
 * (T left, T right, T sigmoidOut, T out). */
int polar_b200_fmatmul_sigmoid(int transLeft, int transRight, uint64_t m, uint64_t n,
                               uint64_t k, const float* left, const float* right,
                               float* out, void* workspace, uint64_t workspace_bytes,
                               void* stream);
int polar_b200_fmatmul_sigmoid_grad(int transLeft, int transRight, uint64_t m,
                                    uint64_t n, uint64_t k, const float* left,
                                    const float* right, const float* sigmoidOut,
                                    float* out, void* workspace,
                                    uint64_t workspace_bytes, void* stream);

/* fdense_grad: the two products of a dense layer's backward pass that read the layer's input
 * activations H (a Sigmoid output), in ONE pass over H:
 *   dW[kh,n]    = H^T . dZ                      what fmatmul_t_f(H, dZ) gives
 *   dIn[rows,kh] = (dZ . W^T) * ((1 - H) * H)   what fmatmul_f_t_sigmoid_grad(dZ, W, H) gives
 * with dZ [rows,n] the gradient at the layer's n <= 16 outputs and W [kh,n] its weights.  Run
 * separately the two builtins stream H through HBM twice; this one once.  Same arithmetic,
 * same order of every sum as those two launches: both results carry their bits.  Larger n, or
 * pointers that are not 16-byte aligned, run the two builtins in sequence.  As a builtin,
 * "fdense_grad": T dZ, T W, T H, T dW, T dIn - the one native name with TWO result tensors
 * (the last two arguments).  Scratch as for fmatmul (polar_b200_fdense_grad_workspace_bytes). */
int polar_b200_fdense_grad(uint64_t rows, uint64_t kh, uint64_t n, const float* dZ, const float* W,
                           const float* H, float* dW, float* dIn, void* workspace,
                           uint64_t workspace_bytes, void* stream);
uint64_t polar_b200_fdense_grad_workspace_bytes(uint64_t rows, uint64_t kh, uint64_t n);

/* Sum of n floats into *sum (a device double, ADDED to: clear it first), with
 * warp-shuffle + one atomic per block.  Used to report the scalar mean of an
 * elementwise flogloss output; the reference has no reduction builtin. */
int polar_b200_fsum(const float* in, double* sum, uint64_t n, void* stream);

/* The same as an extended builtin with a tensor result, "fsum" (T in, T out): out[0] =
 * (float) of the sum accumulated in double; one partial sum per CTA in scratch, added in a
 * fixed order by a second small kernel, so the result is the same bits run to run.  Lets a
 * host that drives the runtime plugin read a loss back as 4 bytes instead of the whole loss
 * tensor.  Scratch: polar_b200_fsum_f32_workspace_bytes(n) bytes, 8-byte aligned (NULL: the
 * stream-ordered pool). */
int polar_b200_fsum_f32(const float* in, float* out, uint64_t n, void* workspace,
                        uint64_t workspace_bytes, void* stream);
uint64_t polar_b200_fsum_f32_workspace_bytes(uint64_t n);

/* ---- dispatch by native kernel name -------------------------------------- */

typedef struct polar_b200_tensor {
  float* data;            /* device pointer */
  uint64_t dims;          /* number of dimensions (TensorInfo::dims) */
  const uint64_t* shape;  /* host pointer to `dims` extents (TensorInfo::shape) */
} polar_b200_tensor;

typedef struct polar_b200_arg {
  int is_tensor;            /* 1: ArgDesc::TENSOR, 0: ArgDesc::DATA */
  polar_b200_tensor tensor; /* when is_tensor */
  float scalar;             /* DATA of 4 bytes: one f32 */
  int64_t integer;          /* DATA of 8 bytes: one i64 (fpool's window and stride) */
} polar_b200_arg;

/* Native names: the twelve of the benchmarked path, "frelu", "fsoftmax", "fpool",
 * "fconv2d", "ftranspose", "fslice" (the reference's own table names ReLU, Softmax and
 * Transpose all "ftranspose" - PolarGraphOps.td:461-523 - so each gets a name of its own
 * here), and
 * the extended "fsigmoid_grad", "fsigmoid_logloss_grad", "fmatmul_x_y_sigmoid",
 * "fmatmul_x_y_sigmoid_grad", "fmatmul_t_f_rows", "fdense_grad", "fsum".
 *
 * Launches the builtin called `nativeKernelName` ("fadd", "fmatmul_t_f", ...)
 * on arguments in LaunchCommand order; this is what Device::launch forwards to
 * once it has turned each TensorInfo into a device pointer.  Shapes are
 * checked against the builtin's rules (equal element counts; matmul inner
 * dimensions). */
int polar_b200_launch_by_name(const char* nativeKernelName,
                              const polar_b200_arg* args, uint64_t argsCount,
                              void* workspace, uint64_t workspace_bytes,
                              void* stream);

/* ---- Gradient exchange over NVLink peer memory (data-parallel step) -------------
 * No counterpart in the reference: it runs every node on one device
 * (ExecutorImpl.cpp:71-75) and has no collective.  What the fused launch replaces on
 * each rank is the pair "sum dW over ranks" + the reference's own weight update
 * fadd(W, 1, dW, -lr) (AddOperationInternal.cpp:61-66); the update's arithmetic is
 * fadd's, so a replica ends with the bits the two-step form gives for the same sum.
 *
 * A peer buffer = POLAR_B200_PEER_CONTROL_BYTES of control words (zeroed by
 * polar_b200_peer_alloc, then owned by the kernels; one block of
 * POLAR_B200_PEER_CHANNEL_BYTES per channel, whose 64-bit words 20..24 hold the last
 * launch's phase timestamps in ns for profiling) followed by the payload (the
 * gradient vector, padded with zeros to 16 bytes).  Each rank allocates one, exports
 * it as a CUDA IPC handle, and opens every other rank's handle; ranks must be
 * distinct processes on GPUs with peer access (NVLink). */
#define POLAR_B200_MAX_PEERS 16
#define POLAR_B200_MAX_UPDATE_SEGMENTS 8
#define POLAR_B200_PEER_CHANNELS 4
#define POLAR_B200_PEER_CHANNEL_BYTES 256
#define POLAR_B200_PEER_CONTROL_BYTES 1024
#define POLAR_B200_PEER_HANDLE_BYTES 64

int polar_b200_peer_alloc(uint64_t payload_bytes, void** buffer);
int polar_b200_peer_free(void* buffer);
int polar_b200_peer_export(void* buffer, unsigned char handle[POLAR_B200_PEER_HANDLE_BYTES]);
int polar_b200_peer_open(const unsigned char handle[POLAR_B200_PEER_HANDLE_BYTES], void** buffer);
int polar_b200_peer_close(void* buffer);

typedef struct polar_b200_update_segment {
  float* weights;   /* this rank's replica of one weight tensor (16-byte aligned) */
  uint64_t offset;  /* where its gradient starts in the payload, in floats (multiple of 4) */
  uint64_t count;   /* elements */
} polar_b200_update_segment;

/* One launch per rank, all ranks of the group in the same step:
 *   payload <- sum over ranks of payload   (ranks added in ascending order: every rank
 *                                            ends with the same bits, in every buffer)
 *   weights[i] <- fl(fl(weights[i]*scale_w) + fl(payload[offset+i]*scale_g))  per segment
 * `buffers[r]` is rank r's peer buffer as mapped in THIS process (own buffer at
 * buffers[rank]); `n` is the payload length in floats.  The ranks' kernels wait for one
 * another with a bound of 4 s (polar_b200_set_wait_limit_ns); a wait that gives up sets
 * the device's status word to 301 (a peer's gradient never became ready) or 302 (a peer
 * never finished its slice), the launch still terminates and NO weight is updated on any
 * rank.  The launch is cooperative (all its CTAs resident at once).  The launches that produced the payload must precede
 * this one on `stream`.  world == 1 is valid (no exchange, update only). */
int polar_b200_allreduce_fadd(void* const* buffers, uint32_t rank, uint32_t world, uint64_t n,
                              const polar_b200_update_segment* segments, uint32_t n_segments,
                              float scale_w, float scale_g, void* stream);

/* How many of the builtin's trailing tensor arguments it WRITES: 1 for every native name (the
 * reference's convention: the last tensor is the result, e.g. AddOperationInternal.cpp:61-66)
 * except "fdense_grad", which has two.  A runtime takes write locks accordingly. */
int polar_b200_result_count(const char* nativeKernelName);

/* The same exchange for a PART of the payload, floats [first, first + count) (first a multiple
 * of 4; every segment inside the range), on its own `channel` of control words
 * (0 .. POLAR_B200_PEER_CHANNELS-1).  Exchanges on different channels may be in flight at the
 * same time - on two streams of one GPU, in the same order on every rank - which is how a step
 * hides most of its exchange: the first rows of a weight gradient travel while the
 * tensor-core matmul is still computing the remaining rows.  Channel 0 is what
 * polar_b200_allreduce_fadd uses; the other channels launch small CTAs that fit on an SM
 * beside a running tensor-core matmul.  Per element the sum is still taken in ascending
 * rank order: the bits do not depend on how the payload is cut. */
int polar_b200_allreduce_fadd_range(void* const* buffers, uint32_t rank, uint32_t world, uint32_t channel,
                                    uint64_t first, uint64_t count,
                                    const polar_b200_update_segment* segments, uint32_t n_segments,
                                    float scale_w, float scale_g, void* stream);

/* The same exchange with the sum done inside the NVLink switch.  `multicast` is the multicast
 * address of the SAME buffers (the address at which a store reaches every rank's copy and a
 * multimem load returns the sum of all copies; control block first, like the buffers), as a
 * host that owns a multicast object has it - torch's symmetric memory hands one out
 * (`multicast_ptr`), or cuMulticastCreate / cuMulticastBindMem by hand.  `buffers` are still
 * needed: the ranks' flags go through them.  Each rank then moves one slice in and one slice
 * out over its links instead of (world - 1) of each.  The order of the sum is the switch's,
 * not rank order: every rank receives the same bits, and they agree with the plain exchange to
 * rounding.  multicast == NULL is polar_b200_allreduce_fadd_range.  Do not let a rank exit
 * while its memory is bound to the multicast object and other ranks are still running. */
int polar_b200_allreduce_fadd_multicast(void* const* buffers, void* multicast, uint32_t rank, uint32_t world,
                                        uint32_t channel, uint64_t first, uint64_t count,
                                        const polar_b200_update_segment* segments, uint32_t n_segments,
                                        float scale_w, float scale_g, void* stream);

/* Scratch bytes the launch `nativeKernelName(args)` would take from the stream-ordered pool
 * if polar_b200_launch_by_name were given no workspace (0 for every builtin but some
 * fmatmul shapes).  Only shapes are read, not the data pointers. */
uint64_t polar_b200_launch_workspace_bytes(const char* nativeKernelName,
                                           const polar_b200_arg* args, uint64_t argsCount);

/* Number of kernels this library has launched since it was loaded (all
 * threads), for launch accounting in benchmarks. */
uint64_t polar_b200_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* POLAR_B200_H */
