// Shared device-side primitives for the sm_100a kernels of lbann_b200:
// mbarrier + TMA (cp.async.bulk.tensor) + tcgen05 (TMEM alloc / MMA / commit / ld)
// wrappers in inline PTX, bounded waits that report through a status word, and
// small numeric helpers.  Everything here is Blackwell-only (compute_100a).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace lb {

// ----------------------------------------------------------------------------
// Error / status codes written by kernels into the library status word.
// A kernel never traps: a wait that runs out records one of these and returns.
// ----------------------------------------------------------------------------
enum Status : int {
  kOk = 0,
  kTimeoutTmaFull = 1,    // consumer gave up waiting for a TMA stage to land
  kTimeoutStageEmpty = 2, // producer gave up waiting for a free stage
  kTimeoutTmemFull = 3,   // epilogue gave up waiting for the accumulator
  kTimeoutTmemEmpty = 4,  // MMA issuer gave up waiting for a drained accumulator
  kTimeoutPeerFlag = 5,   // a flag written by another rank did not arrive
  kBadArgument = 6,
};

// Wait budget for every spin in this library (nanoseconds of %globaltimer).
#ifndef LB_WAIT_BUDGET_NS
#define LB_WAIT_BUDGET_NS 2000000000ull
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(pred));
  return pred;
}

// ------------------------------- mbarrier -----------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, P;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}

// Bounded wait.  Returns true when the phase completed; false when the budget ran
// out or another role of this CTA already raised `*abort_flag` (shared memory).
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3ff) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > LB_WAIT_BUDGET_NS) return false;
    }
  }
}

// Same budget, but keeps waiting after the CTA-wide abort flag went up: used by the
// producer to let its own in-flight copies land before shared memory is released.
__device__ __forceinline__ bool mbar_wait_budget_only(uint32_t bar, uint32_t parity) {
  if (mbar_try_wait(bar, parity)) return true;
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0x3ff) == 0 && globaltimer_ns() - t0 > LB_WAIT_BUDGET_NS / 4) return false;
  }
}

// Budget of the waits on OTHER RANKS (rendezvous flags, halo arrival counters).  It can be
// changed at run time: the status allocation holds it as a 64-bit nanosecond count in bytes
// 8..15 (0 = the compile-time default), set with lb_set_wait_budget_ns.
__device__ __forceinline__ uint64_t peer_wait_budget_ns(const int* status) {
  if (!status) return LB_WAIT_BUDGET_NS;
  const uint64_t v = *reinterpret_cast<const volatile uint64_t*>(status + 2);
  return v ? v : LB_WAIT_BUDGET_NS;
}

__device__ __forceinline__ void raise_status(int* status, volatile int* abort_flag, int code) {
  *abort_flag = 1;
  if (status) atomicCAS(status, 0, code);
}

// ------------------------ untiled bulk copies (TMA, 1-D) and flags ----------------
// Addresses 16-byte aligned, sizes multiples of 16 bytes.
__device__ __forceinline__ void bulk_load_1d(uint32_t dst_smem, const void* src, uint32_t bytes,
                                             uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          dst_smem),
      "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void bulk_store_1d(void* dst, uint32_t src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(
                   reinterpret_cast<uint64_t>(dst)),
               "r"(src_smem), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_read() {   // sources of all but the last N groups read
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait() {        // all but the last N groups complete
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async;" ::: "memory");
}

// ----------------------------- shared-memory access ---------------------------
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr));
  return v;
}
__device__ __forceinline__ void sts128(uint32_t addr, uint4 v) {
  asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// --------------------------------- TMA --------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_load_5d(uint32_t dst, const CUtensorMap* m, uint32_t bar,
                                            int c0, int c1, int c2, int c3, int c4) {
  asm volatile(
      "cp.async.bulk.tensor.5d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%3, %4, %5, %6, %7}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4)
      : "memory");
}

// ------------------------------- tcgen05 ------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_result),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; 16-bit inputs, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// All MMAs issued so far by this thread arrive on `bar` when they retire.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
      : "memory");
}
// 32 lanes x 32 consecutive fp32 columns -> 32 registers per thread.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
        "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
        "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format, version 1).
//   K-major operand, 128-byte swizzle: rows are 128 B, groups of 8 rows are
//   `sbo_bytes` apart; LBO is unused by the hardware for this mode (set to 16 B).
//   MN-major operand, 128-byte swizzle: 64 contiguous MN elements per 128 B row,
//   8 K-rows per atom; atoms along MN are `lbo_bytes` apart, atoms along K are
//   `sbo_bytes` apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes,
                                                   uint32_t sbo_bytes, uint32_t layout_type) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version for Blackwell
  d |= static_cast<uint64_t>(layout_type & 7) << 61;
  return d;
}
constexpr uint32_t kLayoutSw128 = 2;
constexpr uint32_t kLayoutSw64 = 4;
constexpr uint32_t kLayoutSw32 = 6;

// ---------------------------------------------------------------------------------------
// Helpers for the single threads that drive a pipeline (TMA producer, MMA issuer).  One
// thread issues everything, so every instruction between two tcgen05.mma or two TMA boxes
// is on the critical path: an integer division by a run-time value costs it 100-150 cycles
// and a multiply-add chain per descriptor about as much as the MMA itself takes to execute
// (48 cycles at N = 64, 64 at N = 128, 128 at N = 256 for M = 128, K = 16).

// Division by a run-time constant as multiply-high: exact for n * d < 2^32.
struct FastDiv {
  uint32_t d, m;
  __host__ __device__ FastDiv() : d(1), m(0) {}
  __host__ explicit FastDiv(uint32_t divisor)
      : d(divisor ? divisor : 1u), m(divisor > 1 ? (uint32_t)(0x100000000ull / divisor) + 1u : 0u) {}
  __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : __umulhi(n, m); }
  __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
    q = div(n);
    r = n - q * d;
  }
};

// Position in a ring of `S` pipeline stages: stage index and the parity of its barrier.
struct RingPos {
  uint32_t s = 0, ph = 0;
  __device__ __forceinline__ void advance(uint32_t S) {
    if (++s == S) { s = 0; ph ^= 1u; }
  }
};

// tcgen05.mma without a memory clobber: for runs of MMAs between two barrier operations
// (which carry the clobber), so that the compiler keeps descriptors in registers.  The
// start-address field of a descriptor is its low 14 bits (address >> 4): operands of one
// shared-memory window differ in the low word only.
__device__ __forceinline__ void umma_f16_lo(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi,
                                            uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"
      "setp.ne.b32 p, %6, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n\t}" ::"r"(tmem_d),
      "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}

// Instruction descriptor for tcgen05.mma kind::f16 with fp32 accumulation.
//   fmt: 0 = fp16 inputs, 1 = bf16 inputs.  M is 128 here; N a multiple of 16.
__host__ __device__ __forceinline__ uint32_t make_idesc_f16(uint32_t fmt, uint32_t a_mn,
                                                            uint32_t b_mn, uint32_t M,
                                                            uint32_t N) {
  uint32_t d = 0;
  d |= 1u << 4;            // accumulator format: fp32
  d |= (fmt & 7u) << 7;    // A format
  d |= (fmt & 7u) << 10;   // B format
  d |= (a_mn & 1u) << 15;  // A major: 0 = K, 1 = MN
  d |= (b_mn & 1u) << 16;  // B major
  d |= ((N >> 3) & 0x3Fu) << 17;
  d |= ((M >> 4) & 0x1Fu) << 24;
  return d;
}

// ------------------------------- numerics -----------------------------------
enum Act : int { kActNone = 0, kActRelu = 1, kActLeaky = 2, kActGelu = 3, kActTanh = 4,
                 kActSigmoid = 5 };

__device__ __forceinline__ float apply_act(float x, int act, float p) {
  switch (act) {
    case kActRelu: return x > 0.f ? x : 0.f;
    case kActLeaky: return x > 0.f ? x : p * x;
    case kActGelu: return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
    case kActTanh: return tanhf(x);
    case kActSigmoid: return 1.f / (1.f + __expf(-x));
    default: return x;
  }
}

// kI64 is only used for tensor maps that view 16-bit data as 8-byte units (long rows).
enum DType : int { kF16 = 0, kBF16 = 1, kF32 = 2, kI64 = 3 };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ uint32_t pack2(float a, float b, int dtype) {
  if (dtype == kBF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float load_as_f32(const void* p, long long i, int dtype) {
  if (dtype == kF32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == kBF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(reinterpret_cast<const __half*>(p)[i]);
}
__device__ __forceinline__ void store_from_f32(void* p, long long i, float v, int dtype) {
  if (dtype == kF32) reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == kBF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace lb

// ----------------------------- host-side helpers ----------------------------
namespace lbhost {

// The device status word shared by every kernel of the library (one per device).
int* status_word();
// Reads and clears the status word (synchronises the stream first).
int consume_status(cudaStream_t stream);

// cuTensorMapEncodeTiled through the runtime's driver entry point (no libcuda link).
// dims/strides are innermost first; strides are in bytes and skip the innermost dim.
bool encode_tmap(CUtensorMap* out, int dtype, int rank, const void* base, const uint64_t* dims,
                 const uint64_t* strides_bytes, const uint32_t* box, const uint32_t* elem_strides,
                 int swizzle_bytes /*0,32,64,128*/);

int sm_count();

// Scratch memory that the caller lends to the NEXT tensor-core launch of this thread for a
// split of the reduction (fp32 partial tiles).  plan_splitk takes the offer (it holds for one launch only) and returns the
// number of splits: 1 when nothing was offered or the problem fills the GPU as it is.
struct SplitKOffer {
  float* ws = nullptr;
  long long ws_bytes = 0;
};
SplitKOffer take_splitk_offer();
int plan_splitk(const SplitKOffer& o, int num_tiles, int k_iters, int bn);

}  // namespace lbhost
