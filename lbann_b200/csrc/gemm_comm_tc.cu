// tcgen05 GEMM fused with its collective over NVLink peer memory.
//
//   all-gather -> GEMM:   an operand is the concatenation, along its M (or N) dimension,
//       of one shard per rank living in symmetric memory.  The producer warp loads each
//       tile with TMA straight from the shard of the rank that owns it (a plain tiled
//       TMA load from a peer address - no multicast), so there is no all-gather pass and
//       no gathered copy: remote tiles stream in under the math of the tiles before them.
//       Tiles are walked starting at the local shard, which spreads the ranks' requests
//       over different peers.
//   GEMM -> reduce-scatter:   every rank multiplies its K slice; the epilogue adds each
//       finished tile, with fp32 vector atomics, into the output shard of the rank that
//       owns those rows (EpiParams::rs_*).  No partial-result buffer, no separate
//       reduction pass; the transfer of a tile overlaps the main loop of the next one.
//
// Ordering across ranks is the caller's job: shards must be complete (and reduce-scatter
// destinations zeroed) before the launch and read only after a barrier behind it; the
// symmetric-memory group provides both barriers.
//
// Stands in for the gather-then-GEMM and GEMM-then-allreduce sequences of the reference's
// sharded weights (src/weights/data_type_weights.cpp:456-462,
// include/lbann/optimizers/optimizer_impl.hpp:113-169) and of its model-parallel fully
// connected layer (src/layers/learning/fully_connected.cpp:638-808).
#include "tc_pipeline.cuh"

namespace lb {

// Staging of a sharded operand (mode "staged"): when a remote tile would be read by many
// output tiles, reading it through NVLink every time multiplies the traffic (peer memory is
// not cached in the local L2).  The last `helpers` CTAs of the grid therefore copy the
// remote shards ONCE into a local gathered buffer with untiled bulk copies (peer -> shared
// memory -> local memory, several 32 KB pieces in flight per CTA) and publish a flag per
// 128-row block; the multiplying CTAs walk the local shard's tiles first and wait (bounded)
// for the flag of a block before their first TMA load from it.
struct StageInfo {
  const void* shard_ptr[8];   // every rank's shard (peer addresses), rows x K, contiguous
  void* gathered;             // local [ranks * rows][K]
  uint32_t* flags;            // one per 128-row block of the gathered operand
  uint32_t epoch;             // value that marks "block present" for this launch
  int helpers;                // copying CTAs
  int block_bytes;            // 128 rows * K * 2
  int blocks_per_shard;
};

constexpr int kCopyPiece = 32 * 1024;
constexpr int kCopySlots = 6;

template <int BN_>
struct GemmCommPolicy {
  static constexpr int BN = BN_;
  using G = StageGeom<BN>;
  using HasHelpers = void;
  using HasEpilogue = void;

  struct Params {
    int M, N, K;
    int tiles_m, tiles_n, num_tiles, k_iters;
    int a_mn, b_mn, in_dtype;
    // the sharded operand: maps[r] describes rank r's shard, maps[8] the gathered buffer.
    // They live in the kernel parameters (the kernel takes them as __grid_constant__), where
    // the copy engine finds a descriptor faster than in global memory.
    alignas(64) CUtensorMap maps[9];
    int a_shards, a_rows;     // rows of M per shard (multiple of 128)
    int b_shards, b_rows;     // rows of N per shard (multiple of BN and of 128)
    int rank;
    int staged;               // 0: TMA reads peers directly, 1: A staged, 2: B staged
    StageInfo st;
    int* status;
    EpiParams epi;
  };
  struct Tile {
    int m0, n0;
  };

  __device__ static int helpers(const Params& p) { return p.staged ? p.st.helpers : 0; }

  // Reduce-scatter epilogue: the 32 x 32 block a warp reads from TMEM (one row per lane) is
  // turned through shared memory so that every store / reduction instruction of the warp
  // covers 128 contiguous bytes of ONE output row.  Over NVLink that is one transaction
  // where a row-per-lane float4 store makes thirty-two of 16 bytes.
  __device__ static void epilogue(uint32_t taddr, bool row_ok, long long row_off, int n0,
                                  int n_total, int row_index, const EpiParams& e, const Params& p) {
    if (e.rs_ranks == 0) {
      tc_epilogue_rows<BN>(TmemSrc{taddr}, row_ok, row_off, n0, n_total, row_index, e);
      return;
    }
    __shared__ __align__(16) float stg[4][32][36];   // row pitch 144 B: 16-byte aligned rows
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row_first = row_index - lane;           // first row of this warp's block
    const int r4 = lane >> 3, c4 = (lane & 7) * 4;    // lane -> (row within a group of 4, 4 columns)
#pragma unroll 1
    for (int c = 0; c < BN; c += 32) {
      if (n0 + c >= n_total) break;
      uint32_t r[32];
      __syncwarp();
      tmem_ld_32x32(taddr + c, r);
      tmem_ld_wait();
#pragma unroll
      for (int j = 0; j < 32; j += 4)
        *reinterpret_cast<float4*>(&stg[warp][lane][j]) =
            make_float4(__uint_as_float(r[j]) * e.alpha, __uint_as_float(r[j + 1]) * e.alpha,
                        __uint_as_float(r[j + 2]) * e.alpha, __uint_as_float(r[j + 3]) * e.alpha);
      __syncwarp();
      const int col = n0 + c + c4;
      const bool vec = col + 3 < n_total && (e.ldc & 3) == 0;
      // one instruction = 4 rows x 128 contiguous bytes
#pragma unroll 2
      for (int rr = 0; rr < 32; rr += 4) {
        const int m = row_first + rr + r4;
        if (m >= p.M || col >= n_total) continue;
        const int owner = m / e.rs_rows;
        float* dst = e.rs_ptr[owner] + (long long)(m - owner * e.rs_rows) * e.ldc + col;
        const float4 v = *reinterpret_cast<const float4*>(&stg[warp][rr + r4][c4]);
        if (vec && ((reinterpret_cast<uintptr_t>(dst) & 15) == 0)) {
          if (e.rs_store) *reinterpret_cast<float4*>(dst) = v;
          else atomicAdd(reinterpret_cast<float4*>(dst), v);
        } else {
          const float vv[4] = {v.x, v.y, v.z, v.w};
          for (int q = 0; q < 4; ++q) {
            if (col + q >= n_total) break;
            if (e.rs_store) dst[q] = vv[q];
            else atomicAdd(dst + q, vv[q]);
          }
        }
      }
    }
  }

  // ---- copying CTA: one thread drives a ring of bulk copies -----------------------------
  __device__ static void helper_cta(const Params& p, int index, int n, uint8_t* smem, int* status) {
    __shared__ uint64_t bar[kCopySlots];
    if (threadIdx.x != 0) return;
    const uint32_t base = (smem_u32(smem) + 127u) & ~127u;
    for (int s = 0; s < kCopySlots; ++s) mbar_init(smem_u32(&bar[s]), 1);
    mbar_fence_init();
    const StageInfo& st = p.st;
    const int shards = p.staged == 1 ? p.a_shards : p.b_shards;
    const int nb = st.blocks_per_shard;
    const int pieces = (st.block_bytes + kCopyPiece - 1) / kCopyPiece;
    int abort_flag = 0;
    uint32_t issued = 0, stored = 0;      // pieces loaded / stored so far (ring positions)
    // remote blocks in the order the multiplying CTAs reach them, dealt round-robin
    int i = 0;
    for (int sft = 1; sft < shards; ++sft) {
      const int r = (p.rank + sft) % shards;
      for (int blk = 0; blk < nb; ++blk, ++i) {
        if (i % n != index) continue;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(st.shard_ptr[r]) +
                             (long long)blk * st.block_bytes;
        uint8_t* dst = reinterpret_cast<uint8_t*>(st.gathered) +
                       ((long long)r * nb + blk) * st.block_bytes;
        int loaded = 0, done = 0;
        while (done < pieces) {
          // keep up to kCopySlots loads in flight
          while (loaded < pieces && issued - stored < (uint32_t)kCopySlots) {
            const uint32_t slot = issued % kCopySlots;
            if (issued >= (uint32_t)kCopySlots) bulk_wait_read<0>();   // the slot's last store has read it
            const int off = loaded * kCopyPiece;
            const uint32_t bytes = (uint32_t)min(kCopyPiece, st.block_bytes - off);
            mbar_expect_tx(smem_u32(&bar[slot]), bytes);
            bulk_load_1d(base + slot * kCopyPiece, src + off, bytes, smem_u32(&bar[slot]));
            ++issued;
            ++loaded;
          }
          const uint32_t slot = stored % kCopySlots;
          if (!mbar_wait_bounded(smem_u32(&bar[slot]), (stored / kCopySlots) & 1, &abort_flag)) {
            if (status) atomicCAS(status, 0, kTimeoutPeerFlag);
            // let the loads in flight land before shared memory is released
            for (uint32_t q = stored; q < issued; ++q)
              mbar_wait_budget_only(smem_u32(&bar[q % kCopySlots]), (q / kCopySlots) & 1);
            bulk_wait<0>();
            return;
          }
          const int off = done * kCopyPiece;
          const uint32_t bytes = (uint32_t)min(kCopyPiece, st.block_bytes - off);
          bulk_store_1d(dst + off, base + slot * kCopyPiece, bytes);
          bulk_commit();
          ++stored;
          ++done;
        }
        bulk_wait<0>();                       // the block is in local memory
        __threadfence();
        st_release_u32(st.flags + r * nb + blk, st.epoch);
      }
    }
  }

  __device__ static void wait_block(const Params& p, int blk) {
    const uint32_t* f = p.st.flags + blk;
    if (ld_acquire_u32(f) != p.st.epoch) {
      const uint64_t t0 = globaltimer_ns();
      uint32_t spins = 0;
      while (ld_acquire_u32(f) != p.st.epoch) {
        if ((++spins & 0xff) == 0 && globaltimer_ns() - t0 > LB_WAIT_BUDGET_NS) {
          if (p.status) atomicCAS(p.status, 0, kTimeoutPeerFlag);
          break;      // give up: the tile is computed from whatever is there, status says so
        }
      }
    }
    fence_proxy_async();   // the copies were made by the async proxy of another SM
  }

  __device__ static Tile decode(const Params& p, int t) {
    int mb, nb;
    if (p.a_shards > 1) {
      // shard-major: all tiles of the local shard first, then the next rank's, ...
      const int tps = p.a_rows / kBM;
      const int per_shard = tps * p.tiles_n;
      const int s = t / per_shard, r = t - s * per_shard;
      nb = r / tps;
      mb = ((p.rank + s) % p.a_shards) * tps + (r - nb * tps);
    } else if (p.b_shards > 1) {
      const int tps = p.b_rows / BN;
      const int per_shard = tps * p.tiles_m;
      const int s = t / per_shard, r = t - s * per_shard;
      const int nl = r / p.tiles_m;
      mb = r - nl * p.tiles_m;
      nb = ((p.rank + s) % p.b_shards) * tps + nl;
    } else {
      nb = t / p.tiles_m;
      mb = t - nb * p.tiles_m;
    }
    Tile tl;
    tl.m0 = mb * kBM;
    tl.n0 = nb * BN;
    return tl;
  }
  __device__ static uint32_t stage_bytes(const Params&, const Tile&, int) {
    return G::kStageBytes;
  }
  __device__ static void load(const Params& p, const Tile& tl, int k, uint32_t sA, uint32_t sB,
                              uint32_t bar, const CUtensorMap* tmA, const CUtensorMap* tmB,
                              int lane) {
    const int k0 = k * kBK;
    int m0 = tl.m0, n0 = tl.n0;
    bool a_wait = false, b_wait = false;
    if (p.a_shards > 1) {
      const int r = m0 / p.a_rows;
      if (p.staged == 1 && r != p.rank) {
        tmA = &p.maps[8];                 // gathered buffer, global row coordinates
        a_wait = k == 0;
      } else {
        tmA = &p.maps[r];
        m0 -= r * p.a_rows;
      }
    }
    if (p.b_shards > 1) {
      const int r = n0 / p.b_rows;
      if (p.staged == 2 && r != p.rank) {
        tmB = &p.maps[8];
        b_wait = k == 0;
      } else {
        tmB = &p.maps[r];
        n0 -= r * p.b_rows;
      }
    }
    const bool a_lane = p.a_mn ? lane < kBM / 64 : lane == 0;
    const bool b_lane = p.b_mn ? (lane >= 8 && lane < 8 + BN / 64) : lane == 8;
    if (a_lane) {
      if (a_wait) wait_block(p, tl.m0 / 128);
      if (!p.a_mn) tma_load_3d(sA, tmA, bar, k0, m0, 0);
      else tma_load_3d(sA + lane * 8192, tmA, bar, m0 + lane * 64, k0, 0);
    }
    if (b_lane) {
      if (b_wait)
        for (int q = 0; q < BN / 128 + (BN < 128 ? 1 : 0); ++q) wait_block(p, tl.n0 / 128 + q);
      if (!p.b_mn) tma_load_3d(sB, tmB, bar, k0, n0, 0);
      else tma_load_3d(sB + (lane - 8) * 8192, tmB, bar, n0 + (lane - 8) * 64, k0, 0);
    }
  }
  __device__ static uint32_t idesc(const Params& p) {
    return make_idesc_f16(p.in_dtype == kBF16 ? 1u : 0u, p.a_mn, p.b_mn, kBM, BN);
  }
  __device__ static void mma(const Params& p, int, uint32_t sA, uint32_t sB, uint32_t tmem_acc,
                             uint32_t idesc, bool first) {
#pragma unroll
    for (int kk = 0; kk < kBK / 16; ++kk) {
      const uint64_t ad = p.a_mn ? make_smem_desc(sA + kk * 2048, 8192, 1024, kLayoutSw128)
                                 : make_smem_desc(sA + kk * 32, 16, 1024, kLayoutSw128);
      const uint64_t bd = p.b_mn ? make_smem_desc(sB + kk * 2048, 8192, 1024, kLayoutSw128)
                                 : make_smem_desc(sB + kk * 32, 16, 1024, kLayoutSw128);
      umma_f16(tmem_acc, ad, bd, idesc, (first && kk == 0) ? 0u : 1u);
    }
  }
  __device__ static bool row_addr(const Params& p, const Tile& tl, int row, long long& off) {
    const int m = tl.m0 + row;
    off = (long long)m * p.epi.ldc;
    return m < p.M;
  }
  __device__ static int row_index(const Params&, const Tile& tl, int row) { return tl.m0 + row; }
  __device__ static int col0(const Params&, const Tile& tl) { return tl.n0; }
  __device__ static int ncols(const Params& p) { return p.N; }
};

template <int BN>
static int launch_gemm_comm(const CUtensorMap& tmA, const CUtensorMap& tmB,
                            typename GemmCommPolicy<BN>::Params p, cudaStream_t stream) {
  using P = GemmCommPolicy<BN>;
  using G = StageGeom<BN>;
  static bool configured = false;
  if (!configured) {
    cudaFuncSetAttribute(tc_persistent_kernel<P>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         G::kSmemBytes);
    configured = true;
  }
  p.tiles_m = (p.M + kBM - 1) / kBM;
  p.tiles_n = (p.N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_iters = (p.K + kBK - 1) / kBK;
  int grid = p.num_tiles < lbhost::sm_count() ? p.num_tiles : lbhost::sm_count();
  if (p.staged) {
    // helpers and multiplying CTAs wait on one another: all of them must be resident
    grid = lbhost::sm_count();
    if (p.st.helpers >= grid) return -1;
  }
  p.status = lbhost::status_word();
  tc_persistent_kernel<P><<<grid, tc_threads<P>(), G::kSmemBytes, stream>>>(tmA, tmB, p,
                                                                       lbhost::status_word());
  return (int)cudaGetLastError();
}

static bool encode_operand(CUtensorMap* tm, const void* base, int rows, int K, long long ld, int mn,
                           int in_dtype, int box_rows) {
  uint64_t dims[3], strides[2];
  uint32_t box[3];
  if (!mn) { dims[0] = K; dims[1] = rows; box[0] = 64; box[1] = box_rows; }
  else     { dims[0] = rows; dims[1] = K; box[0] = 64; box[1] = 64; }
  dims[2] = 1; box[2] = 1;
  strides[0] = (uint64_t)ld * 2;
  strides[1] = (uint64_t)ld * (mn ? K : rows) * 2;
  return lbhost::encode_tmap(tm, in_dtype, 3, base, dims, strides, box, nullptr, 128);
}

}  // namespace lb

namespace lb {
__global__ void rs_reduce_kernel(float4* __restrict__ out, const float4* __restrict__ slots,
                                 int nslots, long long slot4, long long n4) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4;
       i += (long long)gridDim.x * blockDim.x) {
    float4 a = out[i];
    for (int s = 0; s < nslots; ++s) {
      const float4 b = slots[s * slot4 + i];
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    out[i] = a;
  }
}
struct MapCacheEntry { void* dev; CUtensorMap maps[32]; };
static MapCacheEntry g_map_cache[8];
static int g_map_cache_next = 0;
}  // namespace lb

extern "C" {

// A tensor-map workspace was (re)allocated: forget what was uploaded to that address.
void lb_gemm_comm_forget(void* maps_dev) {
  for (int i = 0; i < 8; ++i)
    if (lb::g_map_cache[i].dev == maps_dev) lb::g_map_cache[i].dev = nullptr;
}

// C = alpha * A . B^T with optionally sharded operands and / or a reduce-scatter epilogue.
//   A: M x K (a_mn = 0: [M][K] pitch lda; 1: [K][M]), B: N x K likewise.
//   a_shard_ptrs: nullptr, or `ranks` device addresses (own + peers') of equally shaped
//       shards of a_rows rows each (M = ranks * a_rows, a_rows % 128 == 0); A is then ignored.
//   b_shard_ptrs / b_rows: the same for B along N (b_rows a multiple of the tile width).
//   maps_dev: device workspace of 32 * 128 bytes (tensor maps), needed with shards.
//   gathered / flags / epoch / helpers: staging of the sharded operand (see StageInfo):
//       `gathered` is a local [ranks * rows][K] buffer (K-major shards, pitch K), `flags`
//       one uint32 per 128 rows of it (never equal to `epoch` before the call), `helpers`
//       the number of copying CTAs.  gathered == nullptr: TMA reads the peers directly.
//   rs_ptrs: nullptr, or `ranks` fp32 output shards of rs_rows rows each, pitch ldc: the
//       result is ADDED there (fp32 atomics) instead of being stored to C (which may then be
//       nullptr).  rs_store = 1: plain stores instead - rs_ptrs[r] is then the slot that rank
//       r keeps for THIS rank's partial result (its own output shard for r == rank), and
//       lb_rs_reduce sums the slots after a rendezvous.
// Returns 0, a cudaError_t (> 0), or -1 for a bad argument.
int lb_gemm_comm_tc(const void* A, const void* B, void* C, int M, int N, int K, long long lda,
                    long long ldb, long long ldc, int a_mn, int b_mn, int in_dtype, int out_dtype,
                    float alpha, const void* const* a_shard_ptrs, int a_rows,
                    const void* const* b_shard_ptrs, int b_rows, int ranks, int rank,
                    void* maps_dev, void* gathered, unsigned int* flags, unsigned int epoch,
                    int helpers, float* const* rs_ptrs, int rs_rows, int rs_store,
                    void* stream_) {
  using namespace lb;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || ranks < 1 || ranks > 8 || rank < 0 || rank >= ranks) return -1;
  if ((lda % 8) || (ldb % 8)) return -1;
  if (a_shard_ptrs && b_shard_ptrs) return -1;
  int BN = N > 128 ? 256 : (N > 64 ? 128 : 64);
  if (b_shard_ptrs && b_rows % BN) BN = b_rows % 128 == 0 ? 128 : 64;
  if (a_shard_ptrs && (a_rows % kBM || a_rows * ranks != M)) return -1;
  if (b_shard_ptrs && (b_rows % BN || b_rows * ranks != N)) return -1;
  if (rs_ptrs && (rs_rows <= 0 || (long long)rs_rows * ranks < M)) return -1;
  int staged = 0;
  if (gathered && ranks > 1) {
    staged = a_shard_ptrs ? 1 : (b_shard_ptrs ? 2 : 0);
    if (!staged || !flags || helpers < 1) return -1;
    if (staged == 1 && (a_mn || lda != K)) return -1;             // contiguous K-major shards
    if (staged == 2 && (b_mn || ldb != K || b_rows % 128)) return -1;
    if (((long long)128 * K * 2) % 16) return -1;
  }

  CUtensorMap host_maps[32];
  memset(host_maps, 0, sizeof(host_maps));
  CUtensorMap tmA, tmB;
  for (int r = 0; r < ranks; ++r) {
    if (a_shard_ptrs &&
        !encode_operand(&host_maps[r], a_shard_ptrs[r], a_rows, K, lda, a_mn, in_dtype, 128))
      return -1;
    if (b_shard_ptrs &&
        !encode_operand(&host_maps[16 + r], b_shard_ptrs[r], b_rows, K, ldb, b_mn, in_dtype, BN))
      return -1;
  }
  if (staged == 1 && !encode_operand(&host_maps[8], gathered, M, K, K, 0, in_dtype, 128)) return -1;
  if (staged == 2 && !encode_operand(&host_maps[24], gathered, N, K, K, 0, in_dtype, BN)) return -1;
  if (!encode_operand(&tmA, a_shard_ptrs ? a_shard_ptrs[rank] : A, a_shard_ptrs ? a_rows : M, K,
                      lda, a_mn, in_dtype, 128))
    return -1;
  if (!encode_operand(&tmB, b_shard_ptrs ? b_shard_ptrs[rank] : B, b_shard_ptrs ? b_rows : N, K,
                      ldb, b_mn, in_dtype, BN))
    return -1;
  (void)maps_dev;   // kept in the signature; the maps travel as kernel parameters

#define LB_LAUNCH(BN_)                                                                \
  {                                                                                   \
    GemmCommPolicy<BN_>::Params p;                                                    \
    p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn; p.in_dtype = in_dtype;   \
    for (int r = 0; r < 9; ++r) p.maps[r] = host_maps[(b_shard_ptrs ? 16 : 0) + r];   \
    p.a_shards = a_shard_ptrs ? ranks : 0; p.a_rows = a_rows;                         \
    p.b_shards = b_shard_ptrs ? ranks : 0; p.b_rows = b_rows;                         \
    p.rank = rank; p.staged = staged;                                                 \
    memset(&p.st, 0, sizeof(p.st));                                                   \
    if (staged) {                                                                     \
      const void* const* sp = staged == 1 ? a_shard_ptrs : b_shard_ptrs;              \
      for (int r = 0; r < ranks; ++r) p.st.shard_ptr[r] = sp[r];                      \
      p.st.gathered = gathered; p.st.flags = flags; p.st.epoch = epoch;               \
      p.st.helpers = helpers; p.st.block_bytes = 128 * K * 2;                         \
      p.st.blocks_per_shard = (staged == 1 ? a_rows : b_rows) / 128;                  \
    }                                                                                 \
    p.epi.C = C; p.epi.bias = nullptr; p.epi.alpha = alpha; p.epi.beta = 0.f;         \
    p.epi.out_dtype = out_dtype; p.epi.bias_mode = 0; p.epi.act = 0;                  \
    p.epi.act_param = 0.f; p.epi.ldc = ldc;                                           \
    if (rs_ptrs) {                                                                    \
      p.epi.rs_ranks = ranks; p.epi.rs_rows = rs_rows; p.epi.rs_store = rs_store;     \
      for (int r = 0; r < ranks; ++r) p.epi.rs_ptr[r] = rs_ptrs[r];                   \
    }                                                                                 \
    return launch_gemm_comm<BN_>(tmA, tmB, p, stream);                                \
  }
  if (BN == 256) LB_LAUNCH(256)
  if (BN == 128) LB_LAUNCH(128)
  LB_LAUNCH(64)
#undef LB_LAUNCH
}

// out[i] += sum over s < nslots of slots[s * slot_elems + i]   (fp32, n elements, n % 4 == 0)
int lb_rs_reduce(float* out, const float* slots, int nslots, long long slot_elems, long long n,
                 void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  if (n <= 0 || (n % 4) || nslots < 0) return -1;
  const long long n4 = n / 4;
  int blocks = (int)((n4 + 255) / 256);
  const int cap = 8 * lbhost::sm_count();
  if (blocks > cap) blocks = cap;
  lb::rs_reduce_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<float4*>(out),
                                                   reinterpret_cast<const float4*>(slots), nslots,
                                                   slot_elems / 4, n4);
  return (int)cudaGetLastError();
}

}  // extern "C"
