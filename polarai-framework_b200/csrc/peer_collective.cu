// Gradient exchange of the data-parallel step as ONE kernel over NVLink peer memory:
// sum of a gradient vector over ranks fused with the weight update that consumes it.
//
// The reference has no collective (every node runs on devices.front(),
// ExecutorImpl.cpp:71-75 of the reference) and updates weights with a separate
// fadd(W, 1, dW, -lr) launch (AddOperationInternal.cpp:61-66).  Here every rank holds
// its gradient vector G in a buffer its peers have mapped (CUDA IPC); one launch per
// rank then
//   1. tells every peer "my G of step s is complete" and waits for the same from all,
//   2. sums slice `rank` of G over all ranks (loads over NVLink, ranks in ascending
//      order, so every rank computes the same bits) and stores the sum into slice
//      `rank` of EVERY rank's G (stores over NVLink),
//   3. tells every peer "slice `rank` is in place" and waits for the same from all,
//   4. applies W = fl(fl(W*sw) + fl(G*sg)) - fadd's arithmetic - on its own replica.
// Nothing else touches slice r of any rank's G between 1 and 3, so the exchange is in
// place.  No multicast object, no TMA: plain peer loads and stores.
//
// Flags are step numbers that only grow, so nothing is ever reset and a rank that is
// one step ahead cannot confuse a slower one.  Every wait is bounded (four seconds unless
// the host set another limit with polar_b200_set_wait_limit_ns).  A wait that gives up
// records 301 (a peer's gradients never became ready) or 302 (a peer never finished its
// slice) in the device's status word and the launch ends WITHOUT touching the weights:
// a CTA that gave up on "ready" skips its part of the sum and marks the step aborted, the
// rank then never publishes "done", so every rank's second wait runs out too and no rank
// applies an update computed from a partial sum.  The host reads the word after it has
// synchronised the stream (polar_b200_check_device_status -> POLAR_B200_ERR_TIMEOUT).
// All CTAs of a launch wait on other ranks, so the launch is cooperative: the driver starts
// it only when every CTA can be resident at once.
#include <cuda_runtime.h>

#include <cstring>

#include "common.cuh"

namespace polar_b200 {
namespace peer {

constexpr int kMaxWorld = POLAR_B200_MAX_PEERS;
constexpr int kMaxSegments = POLAR_B200_MAX_UPDATE_SEGMENTS;
constexpr int kThreads = 512;
constexpr unsigned long long kDefaultWaitNs = 4000000000ull;   // 4 s

// Control words at the head of every rank's buffer (uint32 each), one block of
// POLAR_B200_PEER_CHANNEL_BYTES per channel: exchanges on different channels (different parts
// of the payload, possibly in flight at the same time on two streams) do not share a word.
constexpr int kReady = 0;                 // [kMaxWorld] written by peer p at index p
constexpr int kDone = kMaxWorld;          // [kMaxWorld]
constexpr int kStep = 2 * kMaxWorld;      // local: last completed step
constexpr int kTicketA = kStep + 1;       // local: CTAs that finished phase 2
constexpr int kTicketB = kStep + 2;       // local: CTAs that finished phase 4
constexpr int kAborted = kStep + 3;       // local: the step in which a CTA of this rank gave up waiting
// %globaltimer (ns) of CTA 0 in the last launch: start, gradients of all ranks ready, slice
// summed and stored, all slices in place, update done.  Five 64-bit words, for profiling.
constexpr int kStamps = 40;
static_assert((kStamps + 10) * 4 <= POLAR_B200_PEER_CHANNEL_BYTES, "control block too small");
static_assert(POLAR_B200_PEER_CHANNEL_BYTES * POLAR_B200_PEER_CHANNELS == POLAR_B200_PEER_CONTROL_BYTES,
              "channels fill the control area");

struct Segment {
  float* w;
  uint64_t offset;   // in floats, into G
  uint64_t count;
};

struct Params {
  unsigned char* base[kMaxWorld];   // every rank's buffer (own one included), control block first
  Segment seg[kMaxSegments];
  uint64_t first4, n4;              // the part of G this launch exchanges, in float4
  uint32_t channel;                 // which control block
  uint32_t rank, world, n_seg;
  float scale_w, scale_g;
  int* status;
  unsigned long long wait_ns;
  // The same buffer's NVLink multicast address (control block first), or nullptr.  With it the
  // slice is summed INSIDE the switch (multimem.ld_reduce) and sent to every rank with one store
  // per element (multimem.st): a rank's links carry one slice in and one slice out instead of
  // (world - 1) of each.
  unsigned char* mc;
  // Threads of each CTA that take part in the slice phase (the first ones); the update phase
  // uses all of them.
  uint32_t slice_threads;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Payload accesses are strong operations at system scope.  Weak (ld.cg/st.cg) and volatile
// forms were measured at two ranks and move the slice in the same 25 us, so the form the
// memory model is clearest about stays.
__device__ __forceinline__ float4 ld_peer(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer(float4* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ float4 multimem_sum(const float4* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void multimem_store(float4* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Threads 0..world-1 of the CTA each watch one peer's word until it reaches `step`.
// Returns false (to every thread of the CTA) when a wait ran out.
__device__ __forceinline__ bool wait_all(const uint32_t* words, uint32_t world, uint32_t step, int* status,
                                         int code, unsigned long long limit_ns) {
  int gave_up = 0;
  if (threadIdx.x < world) {
    const uint32_t* w = words + threadIdx.x;
    const unsigned long long t0 = now_ns();
    // step numbers wrap after 2^32 steps: compare as a signed distance
    while ((int32_t)(ld_acquire_sys(w) - step) < 0) {
      if (now_ns() - t0 > limit_ns) {
        atomicCAS(status, 0, code);   // the first code since the last clear stays
        gave_up = 1;
        break;
      }
      __nanosleep(64);
    }
  }
  return __syncthreads_or(gave_up) == 0;
}

template <int WORLD>   // 0 = any world size up to kMaxWorld
__global__ void __launch_bounds__(kThreads) allreduce_fadd_kernel(const Params p) {
  const uint32_t world = WORLD ? (uint32_t)WORLD : p.world;
  const uint32_t kThreadsNow = blockDim.x;
  const uint32_t ctl_off = p.channel * (POLAR_B200_PEER_CHANNEL_BYTES / 4);
  uint32_t* ctl = reinterpret_cast<uint32_t*>(p.base[p.rank]) + ctl_off;
  const uint32_t step = *(volatile uint32_t*)(ctl + kStep) + 1u;
  unsigned long long* stamps = reinterpret_cast<unsigned long long*>(ctl + kStamps);
  const bool stamper = blockIdx.x == 0 && threadIdx.x == 0;
  if (stamper) stamps[0] = now_ns();

  // 1. my G is complete (the launches that wrote it precede this one in the stream)
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<uint32_t*>(p.base[threadIdx.x]) + ctl_off + kReady + p.rank, step);
  }
  const bool ready = wait_all(ctl + kReady, world, step, p.status, 301, p.wait_ns);
  if (!ready && threadIdx.x == 0) *(volatile uint32_t*)(ctl + kAborted) = step;
  if (stamper) stamps[1] = now_ns();

  // 2. slice `rank`, summed in rank order, to everyone
  if (ready) {
    const uint64_t per = (p.n4 + world - 1) / world;
    const uint64_t lo_rel = (uint64_t)p.rank * per < p.n4 ? (uint64_t)p.rank * per : p.n4;
    const uint64_t lo = p.first4 + lo_rel;
    const uint64_t hi = p.first4 + (lo_rel + per < p.n4 ? lo_rel + per : p.n4);
    // The slice comes in over NVLink and goes out again to everyone: the two directions only run
    // at the same time if some threads are storing while others are loading.  So a thread walks
    // several elements (the host sizes the CTAs for about four each) and asks for the NEXT
    // element's values before it sums and stores the current one.  Issued all at once - one
    // element per thread, everything in flight - the kernel spends one slice's transfer time
    // loading and then another one storing (46 us of a 16 us transfer at eight ranks).
    constexpr int W = WORLD ? WORLD : kMaxWorld;
    const uint32_t st = p.slice_threads;
    const uint64_t stride = (uint64_t)gridDim.x * st;
    auto load_all = [&](float4 (&v)[W], uint64_t i) {
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < (int)world)
          v[r] = ld_peer(reinterpret_cast<const float4*>(p.base[r] + POLAR_B200_PEER_CONTROL_BYTES) + i);
    };
    auto sum_and_store = [&](const float4 (&v)[W], uint64_t i) {
      float4 s = v[0];
#pragma unroll
      for (int r = 1; r < W; ++r)
        if (r < (int)world) {
          s.x = __fadd_rn(s.x, v[r].x);
          s.y = __fadd_rn(s.y, v[r].y);
          s.z = __fadd_rn(s.z, v[r].z);
          s.w = __fadd_rn(s.w, v[r].w);
        }
#pragma unroll
      for (int r = 0; r < W; ++r)
        if (r < (int)world)
          st_peer(reinterpret_cast<float4*>(p.base[r] + POLAR_B200_PEER_CONTROL_BYTES) + i, s);
    };
    // threads beyond the slice phase's share start past the end: they fall through to the barrier
    uint64_t i = threadIdx.x < st ? lo + (uint64_t)blockIdx.x * st + threadIdx.x : hi;
    if (p.mc) {
      // In the switch: one load returns the sum over all ranks (in the switch's order, the same
      // bits for every rank since only this rank asks for this slice), one store delivers it to
      // all.  Two elements' loads are in flight per thread.
      float4* mc4 = reinterpret_cast<float4*>(p.mc + POLAR_B200_PEER_CONTROL_BYTES);
      for (; i < hi; i += 2 * stride) {
        const bool two = i + stride < hi;
        const float4 a = multimem_sum(mc4 + i);
        float4 b = a;
        if (two) b = multimem_sum(mc4 + i + stride);
        multimem_store(mc4 + i, a);
        if (two) multimem_store(mc4 + i + stride, b);
      }
    } else if constexpr (WORLD != 0) {
      float4 cur[W], nxt[W];
      if (i < hi) load_all(cur, i);
      while (i < hi) {
        const uint64_t in = i + stride;
        if (in < hi) load_all(nxt, in);
        sum_and_store(cur, i);
#pragma unroll
        for (int r = 0; r < W; ++r) cur[r] = nxt[r];
        i = in;
      }
    } else {
      // any other number of ranks: sixteen values per element leave no registers for a second set
      float4 v[W];
      for (; i < hi; i += stride) {
        load_all(v, i);
        sum_and_store(v, i);
      }
    }
  }

  // 3. the last CTA to get here tells every peer that slice `rank` is in place
  __threadfence_system();
  __syncthreads();
  if (stamper) stamps[2] = now_ns();
  __shared__ uint32_t last;
  if (threadIdx.x == 0) last = (atomicAdd(ctl + kTicketA, 1u) == gridDim.x - 1) ? 1u : 0u;
  __syncthreads();
  if (last && threadIdx.x < world) {
    if (threadIdx.x == 0) ctl[kTicketA] = 0;
    __threadfence_system();
    // "slice in place" is only said when every CTA of this rank did its part of the sum
    if (*(volatile uint32_t*)(ctl + kAborted) != step)
      st_release_sys(reinterpret_cast<uint32_t*>(p.base[threadIdx.x]) + ctl_off + kDone + p.rank, step);
  }
  const bool done = wait_all(ctl + kDone, world, step, p.status, 302, p.wait_ns);
  if (stamper) stamps[3] = now_ns();

  // 4. fadd(W, sw, G, sg) -> W on this rank's replica; skipped when the sum is not complete
  const float* g = reinterpret_cast<const float*>(p.base[p.rank] + POLAR_B200_PEER_CONTROL_BYTES);
  for (uint32_t sidx = 0; done && sidx < p.n_seg; ++sidx) {
    const Segment sg = p.seg[sidx];
    const float4* g4 = reinterpret_cast<const float4*>(g + sg.offset);
    float4* w4 = reinterpret_cast<float4*>(sg.w);
    const uint64_t c4 = sg.count >> 2;
#pragma unroll 4
    for (uint64_t i = (uint64_t)blockIdx.x * kThreadsNow + threadIdx.x; i < c4; i += (uint64_t)gridDim.x * kThreadsNow) {
      const float4 gv = __ldcg(g4 + i);
      float4 wv = w4[i];
      wv.x = __fadd_rn(__fmul_rn(wv.x, p.scale_w), __fmul_rn(gv.x, p.scale_g));
      wv.y = __fadd_rn(__fmul_rn(wv.y, p.scale_w), __fmul_rn(gv.y, p.scale_g));
      wv.z = __fadd_rn(__fmul_rn(wv.z, p.scale_w), __fmul_rn(gv.z, p.scale_g));
      wv.w = __fadd_rn(__fmul_rn(wv.w, p.scale_w), __fmul_rn(gv.w, p.scale_g));
      w4[i] = wv;
    }
    if (blockIdx.x == 0 && threadIdx.x < (sg.count & 3)) {   // ragged tail of the segment
      const uint64_t i = (c4 << 2) + threadIdx.x;
      sg.w[i] = __fadd_rn(__fmul_rn(sg.w[i], p.scale_w), __fmul_rn(__ldcg(g + sg.offset + i), p.scale_g));
    }
  }

  // the last CTA to finish closes the step
  __syncthreads();
  if (stamper) stamps[4] = now_ns();
  if (threadIdx.x == 0) {
    if (atomicAdd(ctl + kTicketB, 1u) == gridDim.x - 1) {
      ctl[kTicketB] = 0;
      __threadfence();
      *(volatile uint32_t*)(ctl + kStep) = step;
    }
  }
}

}  // namespace peer
}  // namespace polar_b200

using namespace polar_b200;

extern "C" {

int polar_b200_peer_alloc(uint64_t payload_bytes, void** buffer) {
  clear_error();
  if (!buffer) return fail(POLAR_B200_ERR_INVALID, "null result pointer");
  void* p = nullptr;
  const uint64_t total = POLAR_B200_PEER_CONTROL_BYTES + ((payload_bytes + 15) & ~15ull);
  // A plain cudaMalloc: allocations of a stream-ordered pool cannot be exported as IPC handles.
  cudaError_t e = cudaMalloc(&p, total);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaMalloc(peer buffer)", e);
  e = cudaMemset(p, 0, total);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(POLAR_B200_ERR_CUDA, "clearing the peer buffer", e);
  }
  *buffer = p;
  return POLAR_B200_OK;
}

int polar_b200_peer_free(void* buffer) {
  clear_error();
  if (!buffer) return POLAR_B200_OK;
  cudaError_t e = cudaFree(buffer);
  return e == cudaSuccess ? POLAR_B200_OK : fail(POLAR_B200_ERR_CUDA, "cudaFree(peer buffer)", e);
}

int polar_b200_peer_export(void* buffer, unsigned char handle[POLAR_B200_PEER_HANDLE_BYTES]) {
  clear_error();
  static_assert(sizeof(cudaIpcMemHandle_t) == POLAR_B200_PEER_HANDLE_BYTES, "IPC handle size");
  if (!buffer || !handle) return fail(POLAR_B200_ERR_INVALID, "null buffer or handle");
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, buffer);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaIpcGetMemHandle", e);
  memcpy(handle, &h, sizeof h);
  return POLAR_B200_OK;
}

int polar_b200_peer_open(const unsigned char handle[POLAR_B200_PEER_HANDLE_BYTES], void** buffer) {
  clear_error();
  if (!buffer || !handle) return fail(POLAR_B200_ERR_INVALID, "null buffer or handle");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "cudaIpcOpenMemHandle", e);
  *buffer = p;
  return POLAR_B200_OK;
}

int polar_b200_peer_close(void* buffer) {
  clear_error();
  if (!buffer) return POLAR_B200_OK;
  cudaError_t e = cudaIpcCloseMemHandle(buffer);
  return e == cudaSuccess ? POLAR_B200_OK : fail(POLAR_B200_ERR_CUDA, "cudaIpcCloseMemHandle", e);
}

static int allreduce_fadd_impl(void* const* buffers, void* multicast, uint32_t rank, uint32_t world, uint32_t channel,
                               uint64_t first, uint64_t n, const polar_b200_update_segment* segments,
                               uint32_t n_segments, float scale_w, float scale_g, void* stream) {
  clear_error();
  if (!buffers || world == 0 || world > (uint32_t)peer::kMaxWorld || rank >= world)
    return fail(POLAR_B200_ERR_INVALID, "allreduce_fadd: bad rank/world or null buffer list");
  if (n_segments > (uint32_t)peer::kMaxSegments || (n_segments && !segments))
    return fail(POLAR_B200_ERR_INVALID, "allreduce_fadd: too many update segments");
  if (channel >= POLAR_B200_PEER_CHANNELS || (first & 3))
    return fail(POLAR_B200_ERR_INVALID, "allreduce_fadd: bad channel, or a range that does not start on a 16-byte boundary");
  if (n == 0) return POLAR_B200_OK;
  peer::Params p{};
  for (uint32_t r = 0; r < world; ++r) {
    if (!buffers[r] || !aligned16(buffers[r])) return fail(POLAR_B200_ERR_INVALID, "allreduce_fadd: null or unaligned buffer");
    p.base[r] = static_cast<unsigned char*>(buffers[r]);
  }
  for (uint32_t s = 0; s < n_segments; ++s) {
    const polar_b200_update_segment& g = segments[s];
    if (!g.weights || !aligned16(g.weights) || (g.offset & 3) || g.offset < first || g.offset + g.count > first + n)
      return fail(POLAR_B200_ERR_INVALID, "allreduce_fadd: segment outside the exchanged range, or not 16-byte aligned");
    p.seg[s] = peer::Segment{g.weights, g.offset, g.count};
  }
  LaunchDeviceScope on(stream, buffers[rank]);
  int rc = POLAR_B200_OK;
  p.status = device_status_word(&rc);
  if (!p.status) return rc;
  p.wait_ns = wait_limit_ns(peer::kDefaultWaitNs);
  p.first4 = first / 4;
  p.n4 = (n + 3) / 4;   // the buffer is padded to 16 bytes by polar_b200_peer_alloc
  p.channel = channel;
  if (multicast && !aligned16(multicast)) return fail(POLAR_B200_ERR_INVALID, "allreduce_fadd: unaligned multicast address");
  p.mc = world > 1 ? static_cast<unsigned char*>(multicast) : nullptr;
  p.rank = rank; p.world = world; p.n_seg = n_segments;
  p.scale_w = scale_w; p.scale_g = scale_g;
  // Every CTA waits on the other ranks, so all of them must be resident at once: at most one
  // per SM, launched cooperatively (the driver then starts the grid only as a whole, also
  // when other kernels are holding SMs at that moment).  512 threads per CTA on channel 0, the
  // exchange that has the GPU to itself; of those, as many take part in the slice phase as give
  // each about four elements of this rank's slice (see the kernel) - the update phase, plain
  // HBM traffic, wants them all (with CTAs sized for the slice phase alone it took 16 instead
  // of 8 us at eight ranks).  The other channels are meant to run BESIDE a tensor-core
  // matmul that already holds 576 threads and most of the registers of every SM: at most 128
  // threads per CTA fit next to it.
  const unsigned threads = channel == 0 ? peer::kThreads : 128;
  uint64_t want = (p.n4 + 63) / 64;
  unsigned grid = (unsigned)(want < (uint64_t)sm_count() ? (want ? want : 1) : (uint64_t)sm_count());
  const uint64_t slice = (p.n4 + world - 1) / world;
  uint64_t per_cta = ((slice + 3) / 4 + grid - 1) / grid;
  unsigned slice_threads = (unsigned)(((per_cta + 31) / 32) * 32);
  if (slice_threads < 64) slice_threads = 64;
  if (slice_threads > threads) slice_threads = threads;
  p.slice_threads = slice_threads;
  cudaStream_t st = as_stream(stream);
  const void* fn = nullptr;
  switch (world) {
    case 2: fn = reinterpret_cast<const void*>(&peer::allreduce_fadd_kernel<2>); break;
    case 4: fn = reinterpret_cast<const void*>(&peer::allreduce_fadd_kernel<4>); break;
    case 8: fn = reinterpret_cast<const void*>(&peer::allreduce_fadd_kernel<8>); break;
    default: fn = reinterpret_cast<const void*>(&peer::allreduce_fadd_kernel<0>); break;
  }
  void* kargs[] = {&p};
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(grid), dim3(threads), kargs, 0, st);
  if (e != cudaSuccess) return fail(POLAR_B200_ERR_CUDA, "allreduce_fadd cooperative launch", e);
  return check_launch("allreduce_fadd launch");
}

int polar_b200_allreduce_fadd(void* const* buffers, uint32_t rank, uint32_t world, uint64_t n,
                              const polar_b200_update_segment* segments, uint32_t n_segments, float scale_w,
                              float scale_g, void* stream) {
  return allreduce_fadd_impl(buffers, nullptr, rank, world, 0, 0, n, segments, n_segments, scale_w, scale_g, stream);
}

int polar_b200_allreduce_fadd_range(void* const* buffers, uint32_t rank, uint32_t world, uint32_t channel,
                                    uint64_t first, uint64_t count, const polar_b200_update_segment* segments,
                                    uint32_t n_segments, float scale_w, float scale_g, void* stream) {
  return allreduce_fadd_impl(buffers, nullptr, rank, world, channel, first, count, segments, n_segments, scale_w, scale_g,
                             stream);
}

int polar_b200_allreduce_fadd_multicast(void* const* buffers, void* multicast, uint32_t rank, uint32_t world,
                                        uint32_t channel, uint64_t first, uint64_t count,
                                        const polar_b200_update_segment* segments, uint32_t n_segments, float scale_w,
                                        float scale_g, void* stream) {
  return allreduce_fadd_impl(buffers, multicast, rank, world, channel, first, count, segments, n_segments, scale_w,
                             scale_g, stream);
}

}  // extern "C"
