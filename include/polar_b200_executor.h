/*
 * polar_b200_executor.h - the one addition libpolar_b200_executor.so makes to the reference's
 * Executor (include/polarai/backend/generic/Executor.hpp:36-61), whose class it implements
 * member for member.
 *
 * The reference lets a device filter select several devices but evaluates every node on the
 * first (src/backend/generic/lib/ExecutorImpl.cpp:71-75; ath_device_select,
 * src/backend/generic/runtime/support/routines.cpp:73-79).  Here, once the caller has named the
 * input nodes whose first dimension is the batch, evaluate() splits the rows of those inputs -
 * and of every tensor computed from them - evenly over all selected devices, replays the
 * recorded builtin program on each (one host thread and one allocator per device), and sums
 * the results of contractions over the batch (fmatmul_t_f of two batch-shaped operands: the
 * weight gradients) across the devices, in device order, so that every device continues with
 * the same bits.  Weights and other inputs are replicated.  getAllocator() then answers host
 * reads from the devices: replicated tensors from the first, batch-shaped ones gathered.
 * A graph that cannot be split by rows (a whole-tensor builtin on a batch-shaped tensor, a
 * batch that does not divide) runs on the first device as in the reference, with a note on
 * stderr.  Without this call nothing changes.
 */
#ifndef POLAR_B200_EXECUTOR_H
#define POLAR_B200_EXECUTOR_H

#include <cstddef>

namespace polarai::backend::generic {
class Executor;
}

/* inputNodeIds: the indices Graph::create<InputNode>() returned for the batch-shaped inputs. */
void polar_b200_executor_shard_inputs(polarai::backend::generic::Executor& executor, const size_t* inputNodeIds,
                                      size_t count);

#endif /* POLAR_B200_EXECUTOR_H */
