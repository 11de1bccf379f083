/*
 * polar_b200_rt.h - what libpolar_rt_cuda.so exports.
 *
 * 1. The plugin interface a PolarAI RuntimeDriver binds with dlsym
 *    (include/polarai/backend/generic/runtime/api.h:17-20 of the reference;
 *    looked up in src/backend/generic/runtime/driver/RuntimeDriver.cpp:39-46):
 *
 *        polarai::backend::generic::Context* initContext();
 *        void closeContext(polarai::backend::generic::Context*);
 *
 *    The returned Context lists one Device per sm_100 GPU; each Device implements
 *    the reference's abstract classes Device, Event and AllocatorLayerBase
 *    (Device.hpp:34-63, Event.hpp:19-25, AllocatorLayerBase.hpp:22-40) and
 *    replaces src/backend/generic/runtime/cuda/{CudaContext,CudaDevice,
 *    CudaAllocator,CudaEvent}.  These two symbols are C++-typed; C callers use
 *    the handle functions below.
 *
 * 2. A flat C view of the same objects, for hosts that cannot call C++ virtuals
 *    (ctypes, cgo, tests).  Every function forwards to the virtual methods the
 *    executor's support routines would call
 *    (src/backend/generic/runtime/support/routines.cpp:37-112: ath_allocate,
 *    ath_lock, ath_launch, ath_release, ath_barrier, ath_load), through a
 *    BackendAllocator built on the devices' stream-ordered pools.
 *
 * Return values are polar_b200_status codes (polar_b200.h); nothing aborts.
 */
#ifndef POLAR_B200_RT_H
#define POLAR_B200_RT_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* LaunchCommand, ArgDesc and TensorInfo are the reference's own plain-C structs
 * (include/polarai/backend/generic/runtime/LaunchCommand.h:19-31 and
 * TensorInfo.h:17-22); they are only named here. */
struct LaunchCommand;

typedef struct polar_b200_rt polar_b200_rt;

/* initContext() + a BackendAllocator with every device registered.  Enumerates the GPUs
 * without touching them: a GPU gets its context, streams and pool when it is first used.
 * No function of this header changes the calling thread's current CUDA device. */
polar_b200_rt* polar_b200_rt_open(void);
/* Releases devices, pools and pinned host memory, then closeContext(). */
void polar_b200_rt_close(polar_b200_rt* rt);

int polar_b200_rt_device_count(polar_b200_rt* rt);
/* Device::getDeviceName(); unique per GPU ("NVIDIA B200 #0"). */
const char* polar_b200_rt_device_name(polar_b200_rt* rt, int device);

/* ath_allocate on a device: BackendAllocator::allocate(record, device). */
int polar_b200_rt_allocate(polar_b200_rt* rt, int device, uint64_t virtAddr, uint64_t bytes);
/* BackendAllocator::deallocate on every layer that holds the record. */
int polar_b200_rt_deallocate(polar_b200_rt* rt, uint64_t virtAddr, uint64_t bytes);

/* What ath_load does with a MemcpyLoader (routines.cpp:95-105 of the reference; the
 * loader copies into the pointer BackendAllocator::get returns): host write lock, copy
 * `bytes` from `src` into the record's pinned host memory, release.  The whole record is
 * replaced, so the call never waits for the previous version's upload: the record keeps
 * two pinned buffers and fills the one no copy is reading.  On return `src` may be reused,
 * and the upload to every device that holds the record has been STARTED on that device's
 * upload stream, into a fresh block - it overlaps kernels that still read the previous
 * version; the next launch that uses the record waits for it on the device, not on the host. */
int polar_b200_rt_write(polar_b200_rt* rt, uint64_t virtAddr, uint64_t bytes, const void* src);
/* The same without the copy, for a loader that produces its data in place (what
 * AbstractLoaderInternal::load does with the pointer it gets): begin hands out the pinned
 * host buffer to fill, end publishes it and starts the upload. */
int polar_b200_rt_host_begin_write(polar_b200_rt* rt, uint64_t virtAddr, uint64_t bytes, void** host);
int polar_b200_rt_host_end_write(polar_b200_rt* rt, uint64_t virtAddr, uint64_t bytes);
/* What OutputNodeAccessor does: host READ lock (pulls the newest copy to the host: one
 * device-to-host copy on the device's download stream, which waits for the launch that
 * last wrote the record - not for launches queued after it), copy out, release. */
int polar_b200_rt_read(polar_b200_rt* rt, uint64_t virtAddr, uint64_t bytes, void* dst);

/* Makes device memory the caller owns the record's copy on `device` (the runtime never
 * frees or moves it): for tensors that must live in special memory, such as the weight
 * gradients of a data-parallel step in NVLink peer memory (polar_b200_peer_alloc). */
int polar_b200_rt_adopt(polar_b200_rt* rt, int device, uint64_t virtAddr, uint64_t bytes, void* device_ptr);

/* The gradient exchange of a data-parallel step as a runtime call: polar_b200_allreduce_fadd
 * (polar_b200.h) on the device's stream, with the weights named as records - each is locked
 * READ_WRITE for the launch like a builtin's output, so other copies of it become stale.
 * No counterpart in the reference (one device, no collective: ExecutorImpl.cpp:71-75). */
typedef struct polar_b200_rt_update {
  uint64_t weight_va;      /* record of one weight tensor */
  uint64_t weight_bytes;   /* its size */
  uint64_t weight_offset;  /* first element of the record this update touches (floats) */
  uint64_t grad_offset;    /* where the matching gradient elements start in the peer payload (floats) */
  uint64_t count;          /* elements */
} polar_b200_rt_update;
/* channel, first, count: the part of the payload this call exchanges and the channel of control
 * words it uses, as in polar_b200_allreduce_fadd_range (channel 0, first 0, count n = everything).
 * multicast: the buffers' NVLink multicast address for the sum inside the switch, or NULL
 * (polar_b200_allreduce_fadd_multicast). */
int polar_b200_rt_allreduce_fadd(polar_b200_rt* rt, int device, void* const* buffers, void* multicast, uint32_t rank,
                                 uint32_t world, uint32_t channel, uint64_t first, uint64_t count,
                                 const polar_b200_rt_update* updates, uint32_t n_updates, float scale_w,
                                 float scale_g);

/* One builtin: READ_WRITE lock on the last tensor argument, READ locks on the
 * others (as the operations' gen() methods emit), Device::launch, release.
 * The launch is asynchronous; errors of the launch itself are returned. */
int polar_b200_rt_launch(polar_b200_rt* rt, int device, struct LaunchCommand* cmd);
/* ath_barrier over everything launched on the device so far.  Returns
 * POLAR_B200_ERR_TIMEOUT when a kernel's bounded wait gave up on that GPU since the last
 * polar_b200_device_status_clear() (polar_b200_rt_read reports the same). */
int polar_b200_rt_barrier(polar_b200_rt* rt, int device);

/* Device pointer of a record on a device (NULL if absent), and the device's
 * stream, for callers that mix their own CUDA work in. */
void* polar_b200_rt_device_ptr(polar_b200_rt* rt, int device, uint64_t virtAddr, uint64_t bytes);
void* polar_b200_rt_stream(polar_b200_rt* rt, int device);

/* Bytes currently held by a device's pool layer, and an optional cap on them
 * (0 = none): past the cap, unlocked records are offloaded to host memory and
 * freed, oldest first. */
uint64_t polar_b200_rt_bytes_in_use(polar_b200_rt* rt, int device);
int polar_b200_rt_set_memory_limit(polar_b200_rt* rt, int device, uint64_t bytes);

/* Text of the last error seen through this handle. */
const char* polar_b200_rt_last_error(polar_b200_rt* rt);

#ifdef __cplusplus
}
#endif
#endif /* POLAR_B200_RT_H */
