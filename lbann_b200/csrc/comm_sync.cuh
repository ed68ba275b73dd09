// Peer-pointer tables and the block-level rendezvous shared by the kernels that talk to other
// ranks over peer-mapped ("symmetric") memory: csrc/comm_kernels.cu and csrc/bn_fused.cu.
#pragma once
#include "common.cuh"

namespace lb {

constexpr int kMaxRanks = 8;
constexpr int kCommBlocks = 64;          // upper bound on blocks of a collective kernel
// signal pad layout (uint32): [phase 0..3][block][source rank]
constexpr int kPadWords = 4 * kCommBlocks * kMaxRanks;

struct PeerPtrs {
  void* buf[kMaxRanks];        // data buffers (peer mapped), buf[my_rank] is local
  uint32_t* pad[kMaxRanks];    // signal pads
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Block-level rendezvous with the same block index on every rank of the group.
// Threads 0..world-1 each handle one peer.  Returns false after the wait budget ran out.
//
// The epoch that the flags are compared with is not a launch argument: every flag row
// (phase, block) has a use counter `ctr` in this rank's own memory, read at the start of the
// rendezvous and advanced at its end.  All ranks run the same sequence of kernels, so their
// counters agree, and a launch carries no per-step value - which is what lets a training
// step be captured once as a CUDA graph and replayed.
__device__ __forceinline__ bool block_rendezvous_row(const PeerPtrs& pp, int rank, int world,
                                                     int row, int tid, uint32_t* ctr, int* status) {
  __shared__ int ok_flag;
  __shared__ uint32_t epoch_sh;
  if (tid == 0) {
    ok_flag = 1;
    epoch_sh = ctr[row] + 1;
  }
  __syncthreads();          // all of this block's earlier writes are issued
  const uint32_t epoch = epoch_sh;
  if (tid < world) {
    const int peer = tid;
    __threadfence_system();
    uint32_t* remote = pp.pad[peer] + (size_t)row * kMaxRanks + rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = pp.pad[rank] + (size_t)row * kMaxRanks + peer;
    const uint64_t t0 = globaltimer_ns();
    const uint64_t budget = peer_wait_budget_ns(status);
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > budget) {
        ok_flag = 0;
        if (status) atomicCAS(status, 0, kTimeoutPeerFlag);
        break;
      }
    }
  }
  __syncthreads();
  if (tid == 0) ctr[row] = epoch;
  return ok_flag != 0;
}

// The common form: one-dimensional blocks, the flag row of (phase, blockIdx.x).
__device__ __forceinline__ bool block_rendezvous(const PeerPtrs& pp, int rank, int world,
                                                 int phase, uint32_t* ctr, int* status) {
  return block_rendezvous_row(pp, rank, world, phase * kCommBlocks + blockIdx.x, threadIdx.x, ctr,
                              status);
}

static inline PeerPtrs make_ptrs(void* const* bufs, void* const* pads, int world) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxRanks; ++i) {
    pp.buf[i] = i < world ? bufs[i] : nullptr;
    pp.pad[i] = i < world ? reinterpret_cast<uint32_t*>(pads[i]) : nullptr;
  }
  return pp;
}


}  // namespace lb
