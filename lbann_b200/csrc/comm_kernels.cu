// NVSwitch-native collectives over peer-mapped ("symmetric") buffers.
//
// Every rank of a group owns one buffer of the same size and holds the peer-mapped
// addresses of all the others (CUDA IPC / VMM mappings set up by parallel/symm.py), plus
// a small signal pad per rank.  The kernels below move data with plain peer loads and
// stores over NVLink - no TMA is ever issued on another GPU's memory - and synchronise
// with epoch flags in the signal pads.  Every wait is bounded: when the budget runs out
// the kernel records kTimeoutPeerFlag in the library status word and returns.
//
// They take the place of the reference's Aluminum / NCCL calls (src/comm.cpp:440-625),
// of DiHydrogen's halo exchange and tensor shufflers (src/utils/distconv.cpp:390-432), and
// of the per-weight gradient allreduce (include/lbann/optimizers/optimizer_impl.hpp:101-143).
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
__device__ __forceinline__ bool block_rendezvous(const PeerPtrs& pp, int rank, int world,
                                                 int phase, uint32_t epoch, int* status) {
  __shared__ int ok_flag;
  if (threadIdx.x == 0) ok_flag = 1;
  __syncthreads();          // all of this block's earlier writes are issued
  if ((int)threadIdx.x < world) {
    const int peer = threadIdx.x;
    __threadfence_system();
    uint32_t* remote = pp.pad[peer] + ((size_t)phase * kCommBlocks + blockIdx.x) * kMaxRanks + rank;
    st_release_sys(remote, epoch);
    const uint32_t* mine = pp.pad[rank] + ((size_t)phase * kCommBlocks + blockIdx.x) * kMaxRanks + peer;
    const uint64_t t0 = globaltimer_ns();
    uint32_t spins = 0;
    while ((int32_t)(ld_acquire_sys(mine) - epoch) < 0) {
      if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > LB_WAIT_BUDGET_NS) {
        ok_flag = 0;
        if (status) atomicCAS(status, 0, kTimeoutPeerFlag);
        break;
      }
    }
  }
  __syncthreads();
  return ok_flag != 0;
}

// ---------------------------------------------------------------------------------
// Two-shot all-reduce (sum) in place over fp32 / 16-bit buffers:
//   shot 1: rank r reduces shard r reading the shard from every peer (peer loads),
//   shot 2: and stores the (scaled) result into every peer's buffer (peer stores).
// Shards are split over the blocks; block b only synchronises with block b of the peers.
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_two_shot_kernel(PeerPtrs pp, int rank, int world, long long n, float scale,
                          uint32_t epoch, int* status) {
  constexpr int V = 16 / sizeof(T);
  if (!block_rendezvous(pp, rank, world, 0, epoch, status)) return;
  const long long shard = ((n + world - 1) / world + V - 1) / V * V;
  const long long s0 = (long long)rank * shard;
  const long long s1 = s0 + shard < n ? s0 + shard : n;
  const long long per_block = ((s1 - s0 + gridDim.x - 1) / gridDim.x + V - 1) / V * V;
  const long long b0 = s0 + (long long)blockIdx.x * per_block;
  const long long b1 = b0 + per_block < s1 ? b0 + per_block : s1;
  for (long long i = b0 + (long long)threadIdx.x * V; i < b1; i += (long long)blockDim.x * V) {
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
    if (i + V <= n) {
      for (int p = 0; p < world; ++p) {
        const int q = (rank + p) % world;   // stagger peers to spread NVLink traffic
        uint4 v = *reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(pp.buf[q]) + i);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[j] += to_f32<T>(e[j]);
      }
      uint4 o;
      T* e = reinterpret_cast<T*>(&o);
#pragma unroll
      for (int j = 0; j < V; ++j) e[j] = from_f32<T>(acc[j] * scale);
      for (int p = 0; p < world; ++p) {
        const int q = (rank + p) % world;
        *reinterpret_cast<uint4*>(reinterpret_cast<T*>(pp.buf[q]) + i) = o;
      }
    } else {
      for (int j = 0; j < V && i + j < n; ++j) {
        float a = 0.f;
        for (int q = 0; q < world; ++q) a += to_f32<T>(reinterpret_cast<const T*>(pp.buf[q])[i + j]);
        for (int q = 0; q < world; ++q) reinterpret_cast<T*>(pp.buf[q])[i + j] = from_f32<T>(a * scale);
      }
    }
  }
  block_rendezvous(pp, rank, world, 1, epoch, status);
}

// ---------------------------------------------------------------------------------
// One-shot all-reduce for short vectors (batch-norm statistics, scalars, flags):
// every rank pushes its vector into slot[rank] of every peer's staging buffer, then sums
// the `world` slots locally into `out`.  staging: [world][n] fp32 in the symmetric buffer.
// op: 0 sum, 1 max.
__global__ void __launch_bounds__(256)
allreduce_one_shot_kernel(PeerPtrs pp, int rank, int world, const float* __restrict__ in,
                          float* __restrict__ out, int n, int op, long long slot_stride,
                          uint32_t epoch, int* status) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = in[i];
    for (int q = 0; q < world; ++q)
      reinterpret_cast<float*>(pp.buf[q])[(long long)rank * slot_stride + i] = v;
  }
  if (!block_rendezvous(pp, rank, world, 2, epoch, status)) return;
  const float* mine = reinterpret_cast<const float*>(pp.buf[rank]);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float a = op == 0 ? 0.f : -INFINITY;
    for (int q = 0; q < world; ++q) {
      const float v = __ldcg(mine + (long long)q * slot_stride + i);
      a = op == 0 ? a + v : fmaxf(a, v);
    }
    out[i] = a;
  }
  // peers may overwrite the staging slots on their next call only after everybody read
  block_rendezvous(pp, rank, world, 3, epoch, status);
}

// ---------------------------------------------------------------------------------
// Strided slab copy into a peer buffer followed by a flag: the building block of the
// halo exchange (boundary planes of a partitioned tensor are stored into the neighbour's
// halo planes) and of tensor shuffles.  Copies `rows` rows of `row_bytes` bytes (multiple
// of 16) from src (+ r * src_pitch) to dst (+ r * dst_pitch).
__global__ void __launch_bounds__(256)
put_rows_kernel(const uint8_t* __restrict__ src, long long src_pitch, uint8_t* __restrict__ dst,
                long long dst_pitch, long long rows, long long row_bytes) {
  const long long vec_per_row = row_bytes / 16;
  const long long total = rows * vec_per_row;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vec_per_row, c = i - r * vec_per_row;
    *reinterpret_cast<uint4*>(dst + r * dst_pitch + c * 16) =
        *reinterpret_cast<const uint4*>(src + r * src_pitch + c * 16);
  }
}

// Group barrier as its own (single block) kernel: orders "my puts are visible" with the
// peers' consumers.  phase selects an independent flag row.
__global__ void group_barrier_kernel(PeerPtrs pp, int rank, int world, int phase, uint32_t epoch,
                                     int* status) {
  block_rendezvous(pp, rank, world, phase, epoch, status);
}

static PeerPtrs make_ptrs(void* const* bufs, void* const* pads, int world) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxRanks; ++i) {
    pp.buf[i] = i < world ? bufs[i] : nullptr;
    pp.pad[i] = i < world ? reinterpret_cast<uint32_t*>(pads[i]) : nullptr;
  }
  return pp;
}

}  // namespace lb

extern "C" {

int lb_comm_pad_bytes() { return lb::kPadWords * 4; }
int lb_comm_max_ranks() { return lb::kMaxRanks; }

// bufs / pads: host arrays of `world` device pointers (index = rank in group).
// dtype: 0 fp16, 1 bf16, 2 fp32.  In place on the symmetric buffers; n elements.
int lb_allreduce_two_shot(void* const* bufs, void* const* pads, int rank, int world, long long n,
                          float scale, unsigned epoch, int dtype, int blocks, void* stream_) {
  using namespace lb;
  if (world < 1 || world > kMaxRanks || n <= 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  if (blocks < 1) blocks = 1;
  if (blocks > kCommBlocks) blocks = kCommBlocks;
  if (dtype == kF32)
    allreduce_two_shot_kernel<float><<<blocks, 512, 0, s>>>(pp, rank, world, n, scale, epoch, lbhost::status_word());
  else if (dtype == kBF16)
    allreduce_two_shot_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(pp, rank, world, n, scale, epoch, lbhost::status_word());
  else
    allreduce_two_shot_kernel<__half><<<blocks, 512, 0, s>>>(pp, rank, world, n, scale, epoch, lbhost::status_word());
  return (int)cudaGetLastError();
}

int lb_allreduce_one_shot(void* const* bufs, void* const* pads, int rank, int world,
                          const float* in, float* out, int n, int op, long long slot_stride,
                          unsigned epoch, void* stream_) {
  using namespace lb;
  if (world < 1 || world > kMaxRanks || n <= 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  allreduce_one_shot_kernel<<<1, 256, 0, s>>>(pp, rank, world, in, out, n, op, slot_stride, epoch,
                                              lbhost::status_word());
  return (int)cudaGetLastError();
}

int lb_put_rows(const void* src, long long src_pitch, void* dst, long long dst_pitch,
                long long rows, long long row_bytes, void* stream_) {
  using namespace lb;
  if (rows <= 0 || row_bytes <= 0) return 0;
  if (row_bytes % 16 || src_pitch % 16 || dst_pitch % 16) return -1;
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  const long long total = rows * (row_bytes / 16);
  long long blocks = (total + 255) / 256;
  const long long cap = (long long)lbhost::sm_count() * 4;
  if (blocks > cap) blocks = cap;
  put_rows_kernel<<<(int)blocks, 256, 0, s>>>((const uint8_t*)src, src_pitch, (uint8_t*)dst,
                                               dst_pitch, rows, row_bytes);
  return (int)cudaGetLastError();
}

int lb_group_barrier(void* const* bufs, void* const* pads, int rank, int world, int phase,
                     unsigned epoch, void* stream_) {
  using namespace lb;
  if (world < 1 || world > kMaxRanks || phase < 0 || phase > 3) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  group_barrier_kernel<<<1, 32, 0, s>>>(pp, rank, world, phase, epoch, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
