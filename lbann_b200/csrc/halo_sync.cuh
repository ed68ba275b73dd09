// Halo exchange of a depth-partitioned tensor done INSIDE the kernel that consumes it.
//
// A rank's tensor lives in a symmetric buffer as [N][Dl + 2h][plane]: Dl own planes between
// h halo planes per side.  The convolution kernel that reads it
//   1. pushes: the otherwise idle epilogue warps of every CTA copy a slice of this rank's
//      first / last h planes into the halo planes of the rank above / below (plain peer
//      stores over NVLink), fence, and add 1 to an arrival counter at the neighbour;
//   2. computes tiles that touch no halo plane first;
//   3. waits (bounded) on its own arrival counters only before the first TMA load that
//      touches a halo plane, so the transfer runs under the interior tiles.
// The counters only ever grow: the value expected after the k-th launch on a tensor is
// k * (CTAs per launch), and k is counted on the device (`local[0]`), so a launch carries no
// per-step argument and a captured CUDA graph can be replayed.  The last CTA to finish
// advances k.  Nothing here orders a push against the neighbour's reads of the PREVIOUS
// step: the caller runs a rendezvous of the group between two steps (the gradient
// reduction of a training step is one).
//
// Counterpart in the reference: DiHydrogen's halo exchange overlapped with the interior
// convolution (src/layers/learning/base_convolution.cpp:1355-1445 and the call stack below it).
#pragma once
#include "common.cuh"

namespace lb {

struct HaloSync {
  const uint4* src;          // this rank's extended tensor
  uint4* up_dst;             // the same tensor on the rank above (peer mapped), null at the top
  uint4* down_dst;           // ... on the rank below, null at the bottom
  uint32_t* up_flag;         // arrival counter of the rank above's BOTTOM halo (peer mapped)
  uint32_t* down_flag;       // arrival counter of the rank below's TOP halo (peer mapped)
  const uint32_t* top_flag;  // this rank's counters (local memory); null where there is no neighbour
  const uint32_t* bot_flag;
  uint32_t* local;           // [0] launches completed on this tensor, [1] CTAs of this launch done
  long long n, dl, h, pv;    // samples, own planes, halo planes per side, 16-byte vectors per plane
  int enabled;
  int pad_;
};

// Host-side mirror handed over by the Python layer (same field order, plain pointers).
struct HaloSyncArgs {
  void* up_dst;
  void* down_dst;
  void* up_flag;
  void* down_flag;
  void* top_flag;
  void* bot_flag;
  void* local;
  long long h;
};

__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Called by `nthreads` threads of every CTA (thread index tid); the caller then synchronises
// those threads and lets ONE of them call halo_signal.
__device__ __forceinline__ void halo_push(const HaloSync& hs, int tid, int nthreads, int cta,
                                          int nctas) {
  const long long ext = (hs.dl + 2 * hs.h) * hs.pv, edge = hs.h * hs.pv, total = hs.n * edge;
  const long long per = (total + nctas - 1) / nctas;
  const long long b0 = (long long)cta * per;
  const long long b1 = b0 + per < total ? b0 + per : total;
  for (long long i = b0 + tid; i < b1; i += nthreads) {
    const long long n = i / edge, rem = i - n * edge;
    if (hs.up_dst) hs.up_dst[n * ext + edge + hs.dl * hs.pv + rem] = hs.src[n * ext + edge + rem];
    if (hs.down_dst) hs.down_dst[n * ext + rem] = hs.src[n * ext + hs.dl * hs.pv + rem];
  }
  __threadfence_system();
}
__device__ __forceinline__ void halo_signal(const HaloSync& hs) {
  if (hs.up_flag) red_release_sys_add(hs.up_flag, 1u);
  if (hs.down_flag) red_release_sys_add(hs.down_flag, 1u);
}

// One thread: wait until `flag` has reached `target` (wrap-safe), then make the planes that
// the neighbour wrote with ordinary stores visible to this thread's TMA loads.
__device__ __forceinline__ bool halo_wait(const uint32_t* flag, uint32_t target, int* status,
                                          volatile int* abort_flag) {
  if ((int32_t)(ld_acquire_sys_u32(flag) - target) < 0) {
    const uint64_t t0 = globaltimer_ns();
    const uint64_t budget = peer_wait_budget_ns(status);
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys_u32(flag) - target) < 0) {
      if ((++spins & 0x3f) == 0) {
        if (*abort_flag) return false;
        if (globaltimer_ns() - t0 > budget) {
          raise_status(status, abort_flag, kTimeoutPeerFlag);
          return false;
        }
      }
    }
  }
  fence_proxy_async();
  return true;
}

// One thread per CTA, after the CTA's last use of the tensor: the last CTA of the launch
// advances the launch counter.
__device__ __forceinline__ void halo_finish(const HaloSync& hs, int nctas) {
  __threadfence();
  const uint32_t done = atomicAdd(hs.local + 1, 1u);
  if (done == (uint32_t)nctas - 1u) {
    hs.local[1] = 0u;
    __threadfence();
    atomicAdd(hs.local, 1u);
  }
}

// Order in which output planes (or plane bricks) are visited when the halo sync is on:
// index 0 (needs the top halo) goes last, so that the first tiles of a launch are interior.
__device__ __forceinline__ int halo_rotate(int i, int count) {
  return i + 1 < count ? i + 1 : 0;
}

// Fills the device-side struct from the host arguments; x is the extended tensor
// [N][D = Dl + 2h][plane] with `plane_bytes` contiguous bytes per plane and `sample_bytes`
// between samples.  Returns false when the layout is not the one described above.
inline bool make_halo_sync(HaloSync& hs, const HaloSyncArgs* a, const void* x, long long N,
                           long long D, long long plane_bytes, long long sample_bytes) {
  memset(&hs, 0, sizeof(hs));
  if (!a) return true;
  if (a->h < 1 || D <= 2 * a->h || plane_bytes % 16 || sample_bytes != D * plane_bytes) return false;
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(a->up_dst) |
       reinterpret_cast<uintptr_t>(a->down_dst)) & 15) return false;
  if (!a->local) return false;
  hs.src = reinterpret_cast<const uint4*>(x);
  hs.up_dst = reinterpret_cast<uint4*>(a->up_dst);
  hs.down_dst = reinterpret_cast<uint4*>(a->down_dst);
  hs.up_flag = reinterpret_cast<uint32_t*>(a->up_flag);
  hs.down_flag = reinterpret_cast<uint32_t*>(a->down_flag);
  hs.top_flag = reinterpret_cast<const uint32_t*>(a->top_flag);
  hs.bot_flag = reinterpret_cast<const uint32_t*>(a->bot_flag);
  hs.local = reinterpret_cast<uint32_t*>(a->local);
  hs.n = N; hs.h = a->h; hs.dl = D - 2 * a->h; hs.pv = plane_bytes / 16;
  hs.enabled = 1;
  return true;
}

}  // namespace lb
