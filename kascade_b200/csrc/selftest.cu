// Self-test of the tensor-core conventions the prefill kernels rely on: four 128x128x128 fp16
// products on one CTA, through (0) A and B K-major from shared memory, (1) B MN-major, (2) A from
// tensor memory with B K-major, (3) A from tensor memory with B MN-major.  A host-side comparison
// with a plain matrix product tells whether the descriptor encodings in umma.cuh match the hardware.
#include "common.cuh"
#include "umma.cuh"

namespace kb200 {

constexpr int kSelfSmem = 2 * 32768 + 1024;   // two 128x128 fp16 row tiles + alignment slack

__global__ void __launch_bounds__(128, 1)
selftest_umma_kernel(const __half* __restrict__ a, const __half* __restrict__ b, float* __restrict__ out,
                     int32_t* __restrict__ status) {
  using namespace umma;
  extern __shared__ uint8_t smem_raw[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base_sh;
  __shared__ int give_up;
  const int tid = threadIdx.x, warp = tid >> 5;
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* As = smem;
  uint8_t* Bs = smem + 32768;

  if (tid == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
    give_up = 0;
  }
  // row r of a / b -> row tile (16 chunks of 16 bytes)
  for (int i = tid; i < 128 * 16; i += 128) {
    int r = i >> 4, c = i & 15;
    *reinterpret_cast<uint4*>(As + tile_off(r, c, 128)) = *reinterpret_cast<const uint4*>(a + r * 128 + c * 8);
    *reinterpret_cast<uint4*>(Bs + tile_off(r, c, 128)) = *reinterpret_cast<const uint4*>(b + r * 128 + c * 8);
  }
  fence_proxy_async_smem();
  if (warp == 0) {
    tmem_alloc(&tmem_base_sh, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_base_sh;
  const uint32_t t_d = tmem;            // accumulator: columns 0..127
  const uint32_t t_a = tmem + 128;      // fp16 copy of `a`: columns 128..191
  const uint32_t a_s = smem_addr(As), b_s = smem_addr(Bs);

  // tensor-memory copy of a: thread = row, 32-bit column c holds elements 2c, 2c+1
  {
    const uint32_t* arow = reinterpret_cast<const uint32_t*>(a + tid * 128);
    uint32_t regs[32];
#pragma unroll
    for (int part = 0; part < 2; ++part) {
#pragma unroll
      for (int i = 0; i < 32; ++i) regs[i] = arow[part * 32 + i];
      tmem_st32(tmem_lane_base(t_a, warp) + part * 32, regs);
    }
    tmem_wait_st();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();

#pragma unroll 1
  for (int test = 0; test < 4; ++test) {
    const bool a_tmem = test >= 2, b_mn = test & 1;
    if (tid == 0) {
      const uint32_t idesc = idesc_f16(128, 128, 0, b_mn ? 1 : 0);
#pragma unroll 1
      for (int ks = 0; ks < 8; ++ks) {
        const uint32_t bd = b_mn ? desc_lo(b_s + ks * 2048, 16384)
                                 : desc_lo(b_s + (ks >> 2) * 16384 + (ks & 3) * 32, 16);
        if (a_tmem) {
          mma_ts_lo(t_d, t_a + ks * 8, bd, idesc, ks > 0);
        } else {
          const uint32_t ad = desc_lo(a_s + (ks >> 2) * 16384 + (ks & 3) * 32, 16);
          mma_ss_lo(t_d, ad, bd, idesc, ks > 0);
        }
      }
      mma_commit(&bar);
    }
    bool ok = mbar_wait(&bar, test & 1, &give_up, test + 1);
    tc_fence_after();
    if (ok) {
#pragma unroll 1
      for (int part = 0; part < 4; ++part) {
        uint32_t regs[32];
        tmem_ld32(tmem_lane_base(t_d, warp) + part * 32, regs);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i)
          out[(test * 128 + tid) * 128 + part * 32 + i] = __uint_as_float(regs[i]);
      }
    }
    if (tid == 0) status[test] = ok ? 0 : 1;
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (give_up) break;
  }
  __syncthreads();
  if (warp == 0) tmem_dealloc(tmem, 256);
}

int init_selftest() {
  KB_CUDA(cudaFuncSetAttribute(selftest_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelfSmem));
  return 0;
}

}  // namespace kb200

extern "C" int kb200_selftest_umma(const void* a, const void* b, float* out, int32_t* status, void* stream) {
  using namespace kb200;
  KB_ENTRY(a, "selftest_umma: a");
  KB_REQUIRE(a && b && out && status, "selftest_umma: null pointer");
  KB_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(b) & 15) == 0,
             "selftest_umma: inputs must be 16-byte aligned");
  selftest_umma_kernel<<<1, 128, kSelfSmem, (cudaStream_t)stream>>>(
      static_cast<const __half*>(a), static_cast<const __half*>(b), out, status);
  KB_CHECK_LAUNCH("selftest_umma_kernel");
  return 0;
}
