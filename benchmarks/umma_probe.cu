// Probe: how fast one thread can issue tcgen05.mma (M = 128, K = 16, 16-bit inputs) and how fast
// the tensor core executes them, on every SM at once.
//
//   nvcc -gencode arch=compute_100a,code=sm_100a -O3 -std=c++17 -I lbann_b200/csrc \
//        -o umma_probe benchmarks/umma_probe.cu lbann_b200/csrc/host_runtime.cu && ./umma_probe
//
// Cases: a 3x3x3 filter walked over a halo slab (the instruction stream of the halo-slab
// convolution) with the tap loops rolled (run-time bounds) or straight-line (template
// constants); operands repeated or different for every instruction; un-swizzled operand
// layouts of the first-layer kernels; bulk copies landing in other stages meanwhile.
// Every wait is bounded (common.cuh); nothing here can hang.
#include "common.cuh"
#include <cstdio>
#include <vector>
using namespace lb;
constexpr uint32_t kLayoutNone = 0;

struct Cfg { int N, Cb, distinct_b, walk_a, n_tiles, copy_bytes_per_mma, taps = 3; };

template <int KSTEPS, bool ROLLED>
__global__ void __launch_bounds__(128, 1) slab_stream(Cfg c, const uint8_t* src, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar, cbar[2];
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  __shared__ volatile int stop;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  for (int i = threadIdx.x; i < 220 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem_raw)[i] = 0;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);
    mbar_init(smem_u32(&cbar[0]), 1);
    mbar_init(smem_u32(&cbar[1]), 1);
    abort_flag = 0; stop = 0; mbar_fence_init();
  }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tb = tmem_base_s;
  // filter at base (<= 112 KB), slab of 5 x 66 rows behind it, two 16 KB copy stages at the end
  const uint32_t filter = base, slab = base + 112 * 1024, ring = base + 176 * 1024;
  if (threadIdx.x == 0) {
    const uint32_t row_bytes = c.Cb * 2;
    const uint32_t lay = c.Cb == 64 ? kLayoutSw128 : (c.Cb == 32 ? kLayoutSw64 : kLayoutSw32);
    const uint32_t idesc = make_idesc_f16(0, 0, 0, 128, c.N);
    const uint64_t desc0 = make_smem_desc(0, 16, 8 * row_bytes, lay);
    const uint32_t d_lo = (uint32_t)desc0, d_hi = (uint32_t)(desc0 >> 32);
    const uint32_t tap_step = c.distinct_b ? (c.N * row_bytes) >> 4 : 0;
    const uint32_t pix_step = c.walk_a ? row_bytes >> 4 : 0, line_step = c.walk_a ? (66 * row_bytes) >> 4 : 0;
    const int kh = ROLLED ? c.taps : 3, kw = kh;                          // a run-time 3 when rolled
    const int ks = ROLLED ? c.Cb / 16 : KSTEPS;
    long long t0 = clock64(), n = 0;
    for (int t = 0; t < c.n_tiles; ++t) {
      uint32_t accum = 0, bd = d_lo + (filter >> 4);
      for (int a = 0; a < 3; ++a) {
        uint32_t a_line = d_lo + (slab >> 4);
        if (ROLLED) {
          for (int b = 0; b < kh; ++b, a_line += line_step) {
            uint32_t ad = a_line;
            for (int cc = 0; cc < kw; ++cc, ad += pix_step, bd += tap_step)
              for (int kk = 0; kk < ks; ++kk) {
                umma_f16_lo(tb, ad + 2 * kk, d_hi, bd + 2 * kk, d_hi, idesc, accum);
                accum = 1; ++n;
              }
          }
        } else {
#pragma unroll
          for (int b = 0; b < 3; ++b) {
#pragma unroll
            for (int cc = 0; cc < 3; ++cc) {
#pragma unroll
              for (int kk = 0; kk < KSTEPS; ++kk) {
                umma_f16_lo(tb, a_line + b * line_step + cc * pix_step + 2 * kk, d_hi,
                            bd + (b * 3 + cc) * tap_step + 2 * kk, d_hi, idesc, accum);
                accum = 1; ++n;
              }
            }
          }
          bd += 9 * tap_step;
        }
      }
    }
    umma_commit(smem_u32(&bar));
    const bool ok = mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag);
    const long long t2 = clock64();
    stop = 1;
    out[blockIdx.x * 4 + 0] = t2 - t0; out[blockIdx.x * 4 + 1] = n; out[blockIdx.x * 4 + 2] = ok;
  } else if (threadIdx.x == 32 && c.copy_bytes_per_mma > 0) {
    // the copy engine writes 16 KB stages next to the operands, as a TMA producer would
    const uint8_t* s = src + (size_t)blockIdx.x * (1 << 20);
    const long long want = (long long)c.copy_bytes_per_mma * c.n_tiles * 27 * (c.Cb / 16);
    long long copied = 0;
    uint32_t it = 0;
    while (copied < want && !stop) {
      const uint32_t st = it & 1, ph = (it >> 1) & 1;
      if (it >= 2 && !mbar_wait_bounded(smem_u32(&cbar[st]), ph ^ 1, &abort_flag)) break;
      mbar_expect_tx(smem_u32(&cbar[st]), 16384);
      bulk_load_1d(ring + st * 16384, s + (it & 31) * 16384, 16384, smem_u32(&cbar[st]));
      copied += 16384; ++it;
    }
    for (uint32_t j = 0; j < (it < 2 ? it : 2); ++j) {
      const uint32_t q = it - 1 - j;
      mbar_wait_budget_only(smem_u32(&cbar[q & 1]), (q >> 1) & 1);
    }
    out[blockIdx.x * 4 + 3] = copied;
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

struct Lay { int N; uint32_t a_lbo, a_sbo, a_lay, a_step, b_lbo, b_sbo, b_lay, b_step; int a_mn, b_mn; };

__global__ void __launch_bounds__(128, 1) layout_run(Lay c, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_s;
  __shared__ int abort_flag;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  for (int i = threadIdx.x; i < 200 * 1024 / 4; i += blockDim.x) ((uint32_t*)smem_raw)[i] = 0;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_flag = 0; mbar_fence_init(); }
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base_s), 512); tmem_relinquish(); }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tb = tmem_base_s;
  if (threadIdx.x == 0) {
    const uint32_t idesc = make_idesc_f16(0, c.a_mn, c.b_mn, 128, c.N);
    const uint64_t da = make_smem_desc(base, c.a_lbo, c.a_sbo, c.a_lay);
    const uint64_t db = make_smem_desc(base + 96 * 1024, c.b_lbo, c.b_sbo, c.b_lay);
    const uint32_t alo = (uint32_t)da, ahi = (uint32_t)(da >> 32), blo = (uint32_t)db, bhi = (uint32_t)(db >> 32);
    long long t0 = clock64(), n = 0;
    for (int t = 0; t < 256; ++t) {
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        umma_f16_lo(tb, alo + (kk & 3) * (c.a_step >> 4), ahi, blo + (kk & 3) * (c.b_step >> 4), bhi, idesc, kk ? 1u : 0u);
        ++n;
      }
    }
    umma_commit(smem_u32(&bar));
    const bool ok = mbar_wait_bounded(smem_u32(&bar), 0, &abort_flag);
    out[blockIdx.x * 4 + 0] = clock64() - t0; out[blockIdx.x * 4 + 1] = n; out[blockIdx.x * 4 + 2] = ok;
  }
  tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tb, 512); }
}

template <class F>
static int report(const char* name, long long* d, F launch) {
  cudaMemset(d, 0, 148 * 4 * 8);
  launch();
  const cudaError_t e = cudaDeviceSynchronize();
  std::vector<long long> h(148 * 4);
  cudaMemcpy(h.data(), d, 148 * 4 * 8, cudaMemcpyDeviceToHost);
  double sum = 0, copied = 0; int oks = 0;
  for (int b = 0; b < 148; ++b) {
    sum += (double)h[b * 4] / (double)(h[b * 4 + 1] ? h[b * 4 + 1] : 1);
    copied += (double)h[b * 4 + 3] / (double)(h[b * 4 + 1] ? h[b * 4 + 1] : 1);
    oks += (int)h[b * 4 + 2];
  }
  printf("%-64s %6.1f cycles/mma  copied %5.0f B/mma  ok=%d/148 %s\n", name, sum / 148, copied / 148, oks,
         e == cudaSuccess ? "" : cudaGetErrorString(e));
  return e == cudaSuccess ? 0 : 1;
}

int main() {
  long long* d; cudaMalloc(&d, 148 * 4 * 8);
  uint8_t* src; cudaMalloc(&src, 148ull << 20); cudaMemset(src, 1, 148ull << 20);
  const int smem = 222 * 1024;
#define SETUP(K, R) cudaFuncSetAttribute(slab_stream<K, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)
  SETUP(1, false); SETUP(2, false); SETUP(4, false); SETUP(1, true);
  cudaFuncSetAttribute(layout_run, cudaFuncAttributeMaxDynamicSharedMemorySize, 202 * 1024);
  int rc = 0;
  struct Named { const char* name; Cfg c; };
  const std::vector<Named> cases = {
      {"N=256 Cb=64", {256, 64, 0, 1, 32, 0}},
      {"N=128 Cb=64", {128, 64, 0, 1, 64, 0}},
      {"N=64  Cb=64", {64, 64, 1, 1, 64, 0}},
      {"N=64  Cb=32 (conv 32->64 forward)", {64, 32, 1, 1, 64, 0}},
      {"N=64  Cb=32, same operands every time", {64, 32, 0, 0, 64, 0}},
      {"N=32  Cb=64 (conv 64->32 data gradient)", {32, 64, 1, 1, 64, 0}},
      {"N=32  Cb=16", {32, 16, 1, 1, 64, 0}},
      {"N=128 Cb=64 + 8 KB of bulk copies per mma", {128, 64, 0, 1, 64, 8192}},
      {"N=256 Cb=64 + 12 KB of bulk copies per mma", {256, 64, 0, 1, 32, 12288}},
  };
  for (const auto& nc : cases) {
    char name[160];
    snprintf(name, sizeof(name), "straight-line  %s", nc.name);
    rc |= report(name, d, [&] {
      if (nc.c.Cb == 64) slab_stream<4, false><<<148, 128, smem>>>(nc.c, src, d);
      else if (nc.c.Cb == 32) slab_stream<2, false><<<148, 128, smem>>>(nc.c, src, d);
      else slab_stream<1, false><<<148, 128, smem>>>(nc.c, src, d);
    });
    if (nc.c.copy_bytes_per_mma) continue;
    snprintf(name, sizeof(name), "rolled loops   %s", nc.name);
    rc |= report(name, d, [&] { slab_stream<1, true><<<148, 128, smem>>>(nc.c, src, d); });
  }
  struct NamedLay { const char* name; Lay c; };
  const std::vector<NamedLay> lays = {
      {"first-layer forward: A none(128, 2048), B none(512, 128), N=32", {32, 128, 2048, kLayoutNone, 256, 512, 128, kLayoutNone, 1024, 0, 0}},
      {"same shape, both 128-byte swizzle K-major", {32, 16, 1024, kLayoutSw128, 32, 16, 1024, kLayoutSw128, 32, 0, 0}},
      {"first-layer wgrad: A MN none(2048, 128), B MN sw64, N=32", {32, 2048, 128, kLayoutNone, 4096, 8192, 512, kLayoutSw64, 1024, 1, 1}},
      {"MN-major both 128-byte swizzle, N=128", {128, 8192, 1024, kLayoutSw128, 2048, 8192, 1024, kLayoutSw128, 2048, 1, 1}},
      {"MN-major both 128-byte swizzle, N=256", {256, 8192, 1024, kLayoutSw128, 2048, 8192, 1024, kLayoutSw128, 2048, 1, 1}},
  };
  for (const auto& nl : lays) rc |= report(nl.name, d, [&] { layout_run<<<148, 128, 202 * 1024>>>(nl.c, d); });
  return rc;
}
