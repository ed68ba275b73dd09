// NVSwitch-native collectives over peer-mapped ("symmetric") buffers.
//
// Every rank of a group owns one buffer of the same size and holds the peer-mapped
// addresses of all the others (CUDA IPC / VMM mappings set up by parallel/symm.py), plus
// a small signal pad per rank.  The kernels below move data with plain peer loads and
// stores over NVLink - no TMA is ever issued on another GPU's memory - and synchronise
// with epoch flags in the signal pads (epochs counted on the device).  Every wait is bounded: when the budget runs out
// the kernel records kTimeoutPeerFlag in the library status word and returns.
//
// They take the place of the reference's Aluminum / NCCL calls (src/comm.cpp:440-625),
// of DiHydrogen's halo exchange and tensor shufflers (src/utils/distconv.cpp:390-432), and
// of the per-weight gradient allreduce (include/lbann/optimizers/optimizer_impl.hpp:101-143).
#include "comm_sync.cuh"

namespace lb {

// ---------------------------------------------------------------------------------
// Two-shot all-reduce (sum) in place over fp32 / 16-bit buffers:
//   shot 1: rank r reduces shard r reading the shard from every peer (peer loads),
//   shot 2: and stores the (scaled) result into every peer's buffer (peer stores).
// Shards are split over the blocks; block b only synchronises with block b of the peers.
template <typename T>
__global__ void __launch_bounds__(512)
allreduce_two_shot_kernel(PeerPtrs pp, int rank, int world, long long n, float scale,
                          uint32_t* ctr, int* status) {
  constexpr int V = 16 / sizeof(T);
  if (!block_rendezvous(pp, rank, world, 0, ctr, status)) return;
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
  block_rendezvous(pp, rank, world, 1, ctr, status);
}

// ---------------------------------------------------------------------------------
// Reduce-scatter (sum) of a range of an arena whose chunks are OWNED block-cyclically:
// blocks of `own_elems` elements are dealt round-robin, block b belongs to rank b % world
// (the layout of the sharded optimizer, csrc/optim.cu).  Rank r sums, for every block it owns
// inside [e0, e1), the values of all ranks (peer loads over NVLink) and keeps the scaled sum
// in its own buffer; nothing is written to a peer.  The opening rendezvous tells that every
// rank's gradients of the range are complete; the kernel has no closing one - the caller
// keeps the ranks from overwriting their gradients until a later rendezvous of the step
// (the one before the updated weights are used).
template <typename T>
__global__ void __launch_bounds__(512)
reduce_scatter_owned_kernel(PeerPtrs pp, int rank, int world, long long e0, long long e1,
                            long long own_elems, float scale, uint32_t* ctr, int* status) {
  constexpr int V = 16 / sizeof(T);
  __shared__ const T* src[kMaxRanks];      // peers in staggered order (dynamic index: shared, not local)
  if ((int)threadIdx.x < world)
    src[threadIdx.x] = reinterpret_cast<const T*>(pp.buf[(rank + threadIdx.x) % world]);
  if (!block_rendezvous(pp, rank, world, 0, ctr, status)) return;
  const long long b_first = e0 / own_elems, b_end = (e1 + own_elems - 1) / own_elems;
  long long ob = b_first + (((long long)rank - b_first % world) + world) % world;  // first owned block
  if (ob >= b_end) return;
  const long long nob = (b_end - ob + world - 1) / world;
  const long long vpb = own_elems / V;
  const long long total = nob * vpb;
  T* mine = const_cast<T*>(src[0]);
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long k = idx / vpb, v = idx - k * vpb;
    const long long i = (ob + k * world) * own_elems + v * V;
    if (i < e0 || i + V > e1) continue;
    uint4 part[kMaxRanks];
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p >= world) break;
      part[p] = *reinterpret_cast<const uint4*>(src[p] + i);   // src[0] is this rank's own buffer
    }
    float acc[V];
#pragma unroll
    for (int j = 0; j < V; ++j) acc[j] = 0.f;
#pragma unroll
    for (int p = 0; p < kMaxRanks; ++p) {
      if (p >= world) break;
      const T* e = reinterpret_cast<const T*>(&part[p]);
#pragma unroll
      for (int j = 0; j < V; ++j) acc[j] += to_f32<T>(e[j]);
    }
    uint4 o;
    T* e = reinterpret_cast<T*>(&o);
#pragma unroll
    for (int j = 0; j < V; ++j) e[j] = from_f32<T>(acc[j] * scale);
    *reinterpret_cast<uint4*>(mine + i) = o;
  }
}

// ---------------------------------------------------------------------------------
// One-shot all-reduce for short vectors (batch-norm statistics, scalars, flags):
// every rank pushes its vector into slot[rank] of every peer's staging buffer, then sums
// the `world` slots locally into `out`.  staging: [world][n] fp32 in the symmetric buffer.
// op: 0 sum, 1 max.
__global__ void __launch_bounds__(256)
allreduce_one_shot_kernel(PeerPtrs pp, int rank, int world, const float* __restrict__ in,
                          float* __restrict__ out, int n, int op, long long slot_stride,
                          uint32_t* ctr, int* status) {
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = in[i];
    for (int q = 0; q < world; ++q)
      reinterpret_cast<float*>(pp.buf[q])[(long long)rank * slot_stride + i] = v;
  }
  if (!block_rendezvous(pp, rank, world, 2, ctr, status)) return;
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
  block_rendezvous(pp, rank, world, 3, ctr, status);
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

// All-to-all of equal slabs as ONE kernel (tensor shuffles between "every rank holds a depth
// slab of all samples" and "every rank holds all of some samples", either direction): slab i
// of the local source goes to rank i % world, slot (i / world) * world + rank of that rank's
// buffer.  Peer stores, then one rendezvous that makes them visible to the consumers that
// follow in the stream.  Nothing here keeps a destination from being overwritten while it
// is still read: the caller separates two uses of a buffer by another rendezvous of the
// group (one per training step suffices).
__global__ void __launch_bounds__(512)
alltoall_slabs_kernel(PeerPtrs pp, int rank, int world, const uint4* __restrict__ src,
                      long long count, long long slab_vec, uint32_t* ctr, int* status) {
  __shared__ uint4* dst[kMaxRanks];
  if ((int)threadIdx.x < world) dst[threadIdx.x] = reinterpret_cast<uint4*>(pp.buf[threadIdx.x]);
  __syncthreads();
  const long long total = count * slab_vec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long i = idx / slab_vec, v = idx - i * slab_vec;
    const int q = (int)(i % world);
    dst[q][((i / world) * world + rank) * slab_vec + v] = src[idx];
  }
  block_rendezvous(pp, rank, world, 3, ctr, status);
}

// Rows of a local matrix to arbitrary (rank, row) destinations: row j of `src` is stored as
// row dst_row[j] of rank dst_rank[j]'s buffer (negative rank: the row goes nowhere).  One
// kernel with the closing rendezvous inside: the data movement between two GPU subsets
// ("grids") of a trainer, where every sample has one owner on either side
// (what the reference does with El::copy::TranslateBetweenGrids,
// include/lbann/layers/transform/split.hpp:135-243).
__global__ void __launch_bounds__(512)
scatter_rows_kernel(PeerPtrs pp, int rank, int world, const uint4* __restrict__ src,
                    const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                    long long rows, long long row_vec, uint32_t* ctr, int* status) {
  __shared__ uint4* dst[kMaxRanks];
  if ((int)threadIdx.x < world) dst[threadIdx.x] = reinterpret_cast<uint4*>(pp.buf[threadIdx.x]);
  __syncthreads();
  const long long total = rows * row_vec;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long j = idx / row_vec, v = idx - j * row_vec;
    const int q = dst_rank[j];
    if (q < 0 || q >= world) continue;
    dst[q][(long long)dst_row[j] * row_vec + v] = src[idx];
  }
  block_rendezvous(pp, rank, world, 3, ctr, status);
}

// Group barrier as its own (single block) kernel: orders "my puts are visible" with the
// peers' consumers.  phase selects an independent flag row.
__global__ void group_barrier_kernel(PeerPtrs pp, int rank, int world, int phase, uint32_t* ctr,
                                     int* status) {
  block_rendezvous(pp, rank, world, phase, ctr, status);
}

// ---------------------------------------------------------------------------------
// Halo exchange of a depth-partitioned activation as ONE kernel.
//
// Forward: the local tensor x [N][Dl][plane] is copied into the interior of this rank's
// extended buffer [N][Dl + 2h][plane] (a symmetric buffer), the planes beyond the global
// boundary are filled, and - after the neighbours signalled that they no longer read the
// previous contents of their halo planes - the first / last h planes are stored into the
// halo planes of the rank above / below.  A second rendezvous makes the stores visible
// before the consumer (the convolution that follows in the stream) starts.
// `up` / `down`: group ranks of the neighbours, -1 at the global boundary.  `pv`: 16-byte
// vectors per plane.  Every rank has the same Dl.
__global__ void __launch_bounds__(512)
halo_fwd_kernel(PeerPtrs pp, int rank, int world, int up, int down, const uint4* __restrict__ x,
                long long N, long long Dl, long long h, long long pv, uint32_t fill_bits,
                uint32_t* ctr, int* status) {
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long ext_pitch = (Dl + 2 * h) * pv;
  uint4* mine = reinterpret_cast<uint4*>(pp.buf[rank]);
  const long long inner = Dl * pv, edge = h * pv;
  for (long long i = tid; i < N * inner; i += nthreads) {
    const long long n = i / inner, rem = i - n * inner;
    mine[n * ext_pitch + edge + rem] = x[i];
  }
  const uint4 fv = make_uint4(fill_bits, fill_bits, fill_bits, fill_bits);
  if (up < 0 || down < 0) {
    for (long long i = tid; i < N * edge; i += nthreads) {
      const long long n = i / edge, rem = i - n * edge;
      if (up < 0) mine[n * ext_pitch + rem] = fv;
      if (down < 0) mine[n * ext_pitch + edge + inner + rem] = fv;
    }
  }
  if (!block_rendezvous(pp, rank, world, 2, ctr, status)) return;
  uint4* above = up >= 0 ? reinterpret_cast<uint4*>(pp.buf[up]) : nullptr;
  uint4* below = down >= 0 ? reinterpret_cast<uint4*>(pp.buf[down]) : nullptr;
  for (long long i = tid; i < N * edge; i += nthreads) {
    const long long n = i / edge, rem = i - n * edge;
    if (above) above[n * ext_pitch + edge + inner + rem] = x[n * inner + rem];
    if (below) below[n * ext_pitch + rem] = x[n * inner + inner - edge + rem];
  }
  block_rendezvous(pp, rank, world, 3, ctr, status);
}

// Backward: g [N][Dl + 2h][plane] is the gradient of the extended tensor.  The gradients of
// the halo planes belong to the neighbours: they are stored into the neighbours' receive
// areas ([2][N][h][plane]: slot 0 from the rank above, slot 1 from the rank below), the
// planes that receive nothing are copied meanwhile, and after the rendezvous the boundary
// planes are written as own gradient + received gradient.  The closing rendezvous keeps the
// neighbours from overwriting the receive area before it was read.
template <typename T>
__global__ void __launch_bounds__(512)
halo_bwd_kernel(PeerPtrs pp, int rank, int world, int up, int down, const uint4* __restrict__ g,
                uint4* __restrict__ dx, long long N, long long Dl, long long h, long long pv,
                uint32_t* ctr, int* status) {
  constexpr int V = 16 / sizeof(T);
  const long long tid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long nthreads = (long long)gridDim.x * blockDim.x;
  const long long ext_pitch = (Dl + 2 * h) * pv;
  const long long inner = Dl * pv, edge = h * pv;
  uint4* above = up >= 0 ? reinterpret_cast<uint4*>(pp.buf[up]) : nullptr;
  uint4* below = down >= 0 ? reinterpret_cast<uint4*>(pp.buf[down]) : nullptr;
  for (long long i = tid; i < N * edge; i += nthreads) {
    const long long n = i / edge, rem = i - n * edge;
    if (above) above[(N + n) * edge + rem] = g[n * ext_pitch + rem];                  // their slot 1
    if (below) below[n * edge + rem] = g[n * ext_pitch + edge + inner + rem];         // their slot 0
  }
  // planes [lo, hi) receive nothing
  const long long lo = up >= 0 ? (h < Dl ? h : Dl) : 0;
  long long hi = down >= 0 ? Dl - h : Dl;
  if (hi < lo) hi = lo;
  const long long mid = (hi - lo) * pv;
  for (long long i = tid; i < N * mid; i += nthreads) {
    const long long n = i / mid, rem = i - n * mid;
    dx[n * inner + lo * pv + rem] = g[n * ext_pitch + edge + lo * pv + rem];
  }
  if (!block_rendezvous(pp, rank, world, 3, ctr, status)) return;
  const uint4* recv = reinterpret_cast<const uint4*>(pp.buf[rank]);
  const long long nb = lo + (Dl - hi);          // boundary planes
  for (long long i = tid; i < N * nb * pv; i += nthreads) {
    const long long n = i / (nb * pv), r2 = i - n * nb * pv;
    const long long j = r2 / pv, v = r2 - j * pv;
    const long long d = j < lo ? j : hi + (j - lo);
    uint4 acc = g[n * ext_pitch + edge + d * pv + v];
    T* a = reinterpret_cast<T*>(&acc);
    if (up >= 0 && d < h) {
      const uint4 r = __ldcg(recv + n * edge + d * pv + v);
      const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
      for (int k = 0; k < V; ++k) a[k] = from_f32<T>(to_f32<T>(a[k]) + to_f32<T>(e[k]));
    }
    if (down >= 0 && d >= Dl - h) {
      const uint4 r = __ldcg(recv + (N + n) * edge + (d - (Dl - h)) * pv + v);
      const T* e = reinterpret_cast<const T*>(&r);
#pragma unroll
      for (int k = 0; k < V; ++k) a[k] = from_f32<T>(to_f32<T>(a[k]) + to_f32<T>(e[k]));
    }
    dx[n * inner + d * pv + v] = acc;
  }
  block_rendezvous(pp, rank, world, 2, ctr, status);
}

// ---------------------------------------------------------------------------------
// Embedding table partitioned over the ranks of a group (row i lives on rank i % world as
// local row i / world of that rank's fp32 shard in symmetric memory).
//
// Gather (forward): one warp per looked-up index reads the row from its owner with plain
// peer loads and writes it, converted, into the local output.  Scatter (backward): one warp
// per index adds scale * dy to the owner's row with fp32 reductions sent over NVLink; with
// scale = -learning_rate that IS the sparse SGD step, applied where the row lives.  Both
// kernels open with a rendezvous: a peer that has started this kernel has finished whatever
// preceded it in its stream (the previous scatter before a gather, the gather before a
// scatter), so rows are never read half-updated.
// Takes the place of the reference's NVSHMEM kernels (src/layers/misc/dist_embedding.cu:221-360,
// 479-640).
template <typename T>
__global__ void __launch_bounds__(256)
dist_embed_gather_kernel(PeerPtrs pp, int rank, int world, const long long* __restrict__ idx,
                         T* __restrict__ out, long long n, int dim, long long num_embeddings,
                         uint32_t* ctr, int* status) {
  if (!block_rendezvous(pp, rank, world, 2, ctr, status)) return;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long s = warp; s < n; s += nwarps) {
    const long long i = idx[s];
    T* o = out + s * dim;
    if (i < 0 || i >= num_embeddings) {
      for (int k = lane; k < dim; k += 32) o[k] = from_f32<T>(0.f);
      continue;
    }
    const float* row = reinterpret_cast<const float*>(pp.buf[i % world]) + (i / world) * dim;
    if ((dim & 3) == 0) {
      for (int k = lane * 4; k < dim; k += 128) {
        const float4 v = *reinterpret_cast<const float4*>(row + k);
        o[k] = from_f32<T>(v.x);
        o[k + 1] = from_f32<T>(v.y);
        o[k + 2] = from_f32<T>(v.z);
        o[k + 3] = from_f32<T>(v.w);
      }
    } else {
      for (int k = lane; k < dim; k += 32) o[k] = from_f32<T>(row[k]);
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(256)
dist_embed_scatter_kernel(PeerPtrs pp, int rank, int world, const long long* __restrict__ idx,
                          const T* __restrict__ dy, long long n, int dim, long long num_embeddings,
                          float scale, uint32_t* ctr, int* status) {
  if (!block_rendezvous(pp, rank, world, 3, ctr, status)) return;
  const int lane = threadIdx.x & 31;
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long s = warp; s < n; s += nwarps) {
    const long long i = idx[s];
    if (i < 0 || i >= num_embeddings) continue;
    float* row = reinterpret_cast<float*>(pp.buf[i % world]) + (i / world) * dim;
    const T* g = dy + s * dim;
    for (int k = lane; k < dim; k += 32) atomicAdd(row + k, scale * to_f32<T>(g[k]));
  }
}

}  // namespace lb

extern "C" {

int lb_comm_pad_bytes() { return lb::kPadWords * 4; }
int lb_comm_max_ranks() { return lb::kMaxRanks; }

// bufs / pads: host arrays of `world` device pointers (index = rank in group).
// dtype: 0 fp16, 1 bf16, 2 fp32.  In place on the symmetric buffers; n elements.
int lb_allreduce_two_shot(void* const* bufs, void* const* pads, int rank, int world, long long n,
                          float scale, unsigned* ctr, int dtype, int blocks, void* stream_) {
  using namespace lb;
  if (world < 1 || world > kMaxRanks || n <= 0) return -1;
  // the kernel moves 16-byte vectors at bufs[r] + i: a misaligned base would fault on the device
  for (int r = 0; r < world; ++r)
    if (reinterpret_cast<uintptr_t>(bufs[r]) & 15) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  if (blocks < 1) blocks = 1;
  if (blocks > kCommBlocks) blocks = kCommBlocks;
  if (dtype == kF32)
    allreduce_two_shot_kernel<float><<<blocks, 512, 0, s>>>(pp, rank, world, n, scale, ctr, lbhost::status_word());
  else if (dtype == kBF16)
    allreduce_two_shot_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(pp, rank, world, n, scale, ctr, lbhost::status_word());
  else
    allreduce_two_shot_kernel<__half><<<blocks, 512, 0, s>>>(pp, rank, world, n, scale, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

// Reduce-scatter of elements [e0, e1) of the symmetric buffers `bufs` with block-cyclic
// ownership (see reduce_scatter_owned_kernel).  e0, e1 and own_elems are element counts and
// multiples of one 16-byte vector; every base address is 16-byte aligned.
int lb_reduce_scatter_owned(void* const* bufs, void* const* pads, int rank, int world,
                            long long e0, long long e1, long long own_elems, float scale,
                            unsigned* ctr, int dtype, int blocks, void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || e1 <= e0 || own_elems <= 0) return -1;
  const int v = dtype == kF32 ? 4 : 8;
  if (e0 % v || e1 % v || own_elems % v) return -1;
  for (int r = 0; r < world; ++r)
    if (reinterpret_cast<uintptr_t>(bufs[r]) & 15) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  if (blocks < 1) blocks = 1;
  if (blocks > kCommBlocks) blocks = kCommBlocks;
  if (dtype == kF32)
    reduce_scatter_owned_kernel<float><<<blocks, 512, 0, s>>>(pp, rank, world, e0, e1, own_elems, scale, ctr, lbhost::status_word());
  else if (dtype == kBF16)
    reduce_scatter_owned_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(pp, rank, world, e0, e1, own_elems, scale, ctr, lbhost::status_word());
  else
    reduce_scatter_owned_kernel<__half><<<blocks, 512, 0, s>>>(pp, rank, world, e0, e1, own_elems, scale, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

int lb_allreduce_one_shot(void* const* bufs, void* const* pads, int rank, int world,
                          const float* in, float* out, int n, int op, long long slot_stride,
                          unsigned* ctr, void* stream_) {
  using namespace lb;
  if (world < 1 || world > kMaxRanks || n <= 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  allreduce_one_shot_kernel<<<1, 256, 0, s>>>(pp, rank, world, in, out, n, op, slot_stride, ctr,
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

static int halo_blocks(long long vectors) {
  long long b = (vectors + 512 * 8 - 1) / (512 * 8);      // >= 8 vectors per thread
  if (b < 1) b = 1;
  if (b > lb::kCommBlocks) b = lb::kCommBlocks;
  return (int)b;
}

// ext_bufs: the extended buffers of the group's ranks ([N][Dl + 2h][plane_bytes]); x: this
// rank's [N][Dl][plane_bytes].  fill: value of the planes beyond the global boundary.
// Returns -2 when the shape is not covered (plane not a multiple of 16 bytes, Dl < h).
int lb_halo_exchange_fwd(void* const* ext_bufs, void* const* pads, int rank, int world, int up,
                         int down, const void* x, long long N, long long Dl, long long h,
                         long long plane_bytes, float fill, int dtype, unsigned* ctr,
                         void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || up >= world || down >= world) return -1;
  if (plane_bytes % 16 || Dl < h || h < 1 || N < 1) return -2;
  if (reinterpret_cast<uintptr_t>(x) & 15) return -2;
  uint32_t bits;
  if (dtype == kF32) {
    memcpy(&bits, &fill, 4);
  } else {
    uint16_t hb;
    if (dtype == kF16) {
      const __half v = __float2half(fill);
      memcpy(&hb, &v, 2);
    } else {
      const __nv_bfloat16 v = __float2bfloat16(fill);
      memcpy(&hb, &v, 2);
    }
    bits = (uint32_t)hb | ((uint32_t)hb << 16);
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(ext_bufs, pads, world);
  const long long pv = plane_bytes / 16;
  halo_fwd_kernel<<<halo_blocks(N * Dl * pv), 512, 0, s>>>(
      pp, rank, world, up, down, reinterpret_cast<const uint4*>(x), N, Dl, h, pv, bits, ctr,
      lbhost::status_word());
  return (int)cudaGetLastError();
}

// recv_bufs: the receive areas of the group's ranks ([2][N][h][plane_bytes]); g: gradient of
// the extended tensor; dx: [N][Dl][plane_bytes].
int lb_halo_exchange_bwd(void* const* recv_bufs, void* const* pads, int rank, int world, int up,
                         int down, const void* g, void* dx, long long N, long long Dl,
                         long long h, long long plane_bytes, int dtype, unsigned* ctr,
                         void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || up >= world || down >= world) return -1;
  if (plane_bytes % 16 || Dl < h || h < 1 || N < 1) return -2;
  if ((reinterpret_cast<uintptr_t>(g) & 15) || (reinterpret_cast<uintptr_t>(dx) & 15)) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(recv_bufs, pads, world);
  const long long pv = plane_bytes / 16;
  const int blocks = halo_blocks(N * Dl * pv);
  const uint4* gv = reinterpret_cast<const uint4*>(g);
  uint4* dv = reinterpret_cast<uint4*>(dx);
  if (dtype == kF32)
    halo_bwd_kernel<float><<<blocks, 512, 0, s>>>(pp, rank, world, up, down, gv, dv, N, Dl, h, pv, ctr, lbhost::status_word());
  else if (dtype == kBF16)
    halo_bwd_kernel<__nv_bfloat16><<<blocks, 512, 0, s>>>(pp, rank, world, up, down, gv, dv, N, Dl, h, pv, ctr, lbhost::status_word());
  else
    halo_bwd_kernel<__half><<<blocks, 512, 0, s>>>(pp, rank, world, up, down, gv, dv, N, Dl, h, pv, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

// tables: the fp32 shards of the group's ranks.  idx: n int64 indices; out: [n][dim] of dtype.
// Every rank launches the same number of blocks whatever its n (the blocks rendezvous
// pairwise), so ranks with different local batch sizes still meet.
int lb_dist_embed_gather(void* const* tables, void* const* pads, int rank, int world,
                         const long long* idx, void* out, long long n, int dim,
                         long long num_embeddings, int dtype, unsigned* ctr, void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || dim < 1 || n < 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(tables, pads, world);
  const int blocks = 32;
  if (dtype == kF32)
    dist_embed_gather_kernel<float><<<blocks, 256, 0, s>>>(pp, rank, world, idx, (float*)out, n, dim, num_embeddings, ctr, lbhost::status_word());
  else if (dtype == kBF16)
    dist_embed_gather_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(pp, rank, world, idx, (__nv_bfloat16*)out, n, dim, num_embeddings, ctr, lbhost::status_word());
  else
    dist_embed_gather_kernel<__half><<<blocks, 256, 0, s>>>(pp, rank, world, idx, (__half*)out, n, dim, num_embeddings, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

// table[owner(idx[s])][row(idx[s])] += scale * dy[s] for every s < n.
int lb_dist_embed_scatter(void* const* tables, void* const* pads, int rank, int world,
                          const long long* idx, const void* dy, long long n, int dim,
                          long long num_embeddings, float scale, int dtype, unsigned* ctr,
                          void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || dim < 1 || n < 0) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(tables, pads, world);
  const int blocks = 32;
  if (dtype == kF32)
    dist_embed_scatter_kernel<float><<<blocks, 256, 0, s>>>(pp, rank, world, idx, (const float*)dy, n, dim, num_embeddings, scale, ctr, lbhost::status_word());
  else if (dtype == kBF16)
    dist_embed_scatter_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(pp, rank, world, idx, (const __nv_bfloat16*)dy, n, dim, num_embeddings, scale, ctr, lbhost::status_word());
  else
    dist_embed_scatter_kernel<__half><<<blocks, 256, 0, s>>>(pp, rank, world, idx, (const __half*)dy, n, dim, num_embeddings, scale, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

// bufs: the receive buffers of the group's ranks; src: `count` slabs of slab_bytes bytes.
int lb_alltoall_slabs(void* const* bufs, void* const* pads, int rank, int world, const void* src,
                      long long count, long long slab_bytes, unsigned* ctr, void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || count < 0 || slab_bytes <= 0) return -1;
  if (slab_bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  for (int r = 0; r < world; ++r)
    if (reinterpret_cast<uintptr_t>(bufs[r]) & 15) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  // every rank launches the same number of blocks (they meet pairwise), whatever its count
  alltoall_slabs_kernel<<<kCommBlocks, 512, 0, s>>>(pp, rank, world, reinterpret_cast<const uint4*>(src),
                                                     count, slab_bytes / 16, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

// bufs: receive buffers of the group's ranks.  src: `rows` rows of row_bytes bytes (may be
// null when rows == 0: a rank that only receives still takes part in the rendezvous).
int lb_scatter_rows(void* const* bufs, void* const* pads, int rank, int world, const void* src,
                    const int* dst_rank, const int* dst_row, long long rows, long long row_bytes,
                    unsigned* ctr, void* stream_) {
  using namespace lb;
  if (world < 2 || world > kMaxRanks || rows < 0 || row_bytes <= 0) return -1;
  if (row_bytes % 16 || (reinterpret_cast<uintptr_t>(src) & 15)) return -2;
  for (int r = 0; r < world; ++r)
    if (reinterpret_cast<uintptr_t>(bufs[r]) & 15) return -2;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  scatter_rows_kernel<<<kCommBlocks, 512, 0, s>>>(pp, rank, world, reinterpret_cast<const uint4*>(src),
                                                   dst_rank, dst_row, rows, row_bytes / 16, ctr,
                                                   lbhost::status_word());
  return (int)cudaGetLastError();
}

int lb_group_barrier(void* const* bufs, void* const* pads, int rank, int world, int phase,
                     unsigned* ctr, void* stream_) {
  using namespace lb;
  if (world < 1 || world > kMaxRanks || phase < 0 || phase > 3) return -1;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream_);
  PeerPtrs pp = make_ptrs(bufs, pads, world);
  group_barrier_kernel<<<1, 32, 0, s>>>(pp, rank, world, phase, ctr, lbhost::status_word());
  return (int)cudaGetLastError();
}

}  // extern "C"
