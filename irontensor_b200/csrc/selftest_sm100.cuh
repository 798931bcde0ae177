// Self-test kernels: one 128x128x128 bf16 MMA through each operand path the attention kernels
// use (so a wrong shared-memory or instruction descriptor shows up in isolation), and a kernel
// whose only job is to let a bounded barrier wait run out.
#pragma once
#include "sm100_ptx.cuh"

namespace it {

// VARIANT 0: A K-major smem (TMA), B K-major smem (TMA)
// VARIANT 1: A in TMEM,            B N-major smem (TMA)
// VARIANT 2: A K-major smem written by threads, B N-major smem (TMA)
// VARIANT 3: A M-major smem written by threads, B N-major smem (TMA)
template <int VARIANT>
__global__ void __launch_bounds__(128, 1)
umma_selftest_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __nv_bfloat16* __restrict__ a, float* __restrict__ out, int* status) {
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];
  constexpr int BLOCK_BYTES = 128 * 128;
  uint8_t* sA = smem;
  uint8_t* sB = smem + 2 * BLOCK_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 4 * BLOCK_BYTES);
  uint64_t* load_full = bars;
  uint64_t* mma_done = bars + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  if (tid == 0) {
    *abort_flag = 0;
    if (smem_addr(smem) & 1023u) {
      *abort_flag = 1;
      atomicCAS(status, 0, DEV_ERR_SMEM_ALIGN);
    }
    mbar_init(load_full, 1);
    mbar_init(mma_done, 1);
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 0) {
    tmem_alloc(tmem_slot, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(warp * 32) << 16);
  bool ok = (*abort_flag == 0);

  if (ok) {
    if (tid == 0) {
      const uint32_t bytes = (VARIANT == 0 ? 4 : 2) * BLOCK_BYTES;
      mbar_arrive_expect_tx(load_full, bytes);
      for (int b = 0; b < 2; ++b) {
        if (VARIANT == 0) tma_load_4d(sA + b * BLOCK_BYTES, &tmap_a, load_full, b * 64, 0, 0, 0);
        tma_load_4d(sB + b * BLOCK_BYTES, &tmap_b, load_full, b * 64, 0, 0, 0);
      }
    }
    if (VARIANT == 1) {   // row `tid` of A, packed bf16 pairs, into TMEM columns [128,192)
      const uint32_t* arow = reinterpret_cast<const uint32_t*>(a + tid * 128);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) pk[i] = arow[c * 16 + i];
        tmem_st_x16(t_lane + 128 + c * 16, pk);
      }
      tmem_wait_st();
      tc_fence_before();
    } else if (VARIANT == 2) {   // K-major: smem row = m, 64 k per 128-byte row, two k blocks
      const uint4* arow = reinterpret_cast<const uint4*>(a + tid * 128);
#pragma unroll
      for (int c = 0; c < 16; ++c)
        *reinterpret_cast<uint4*>(sA + (c >> 3) * BLOCK_BYTES + tid * 128 + (((c & 7) ^ (tid & 7)) << 4)) = arow[c];
      fence_proxy_async_smem();
    } else if (VARIANT == 3) {   // M-major: smem row = k (this thread), 64 m per row, two m blocks
      const uint16_t* a16 = reinterpret_cast<const uint16_t*>(a);
#pragma unroll 1
      for (int c = 0; c < 16; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const uint32_t lo = a16[(8 * c + 2 * e) * 128 + tid];
          const uint32_t hi = a16[(8 * c + 2 * e + 1) * 128 + tid];
          w[e] = lo | (hi << 16);
        }
        *reinterpret_cast<uint4*>(sA + (c >> 3) * BLOCK_BYTES + tid * 128 + (((c & 7) ^ (tid & 7)) << 4)) =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
      fence_proxy_async_smem();
    }
  }
  __syncthreads();
  if (ok && tid == 0) {
    ok = mbar_wait(load_full, 0, abort_flag, status, DEV_ERR_TIMEOUT_LOAD);
    if (ok) {
      tc_fence_after();
      const uint32_t a_addr = smem_addr(sA), b_addr = smem_addr(sB);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint32_t koff = (kk >> 2) * BLOCK_BYTES + (kk & 3) * 32;
        if (VARIANT == 0) {
          umma_ss(tmem_base, sdesc_advance(make_sdesc(a_addr, 16, 1024), koff),
                  sdesc_advance(make_sdesc(b_addr, 16, 1024), koff), make_idesc(128, 128, false, false), kk > 0);
        } else if (VARIANT == 1) {
          umma_ts(tmem_base, tmem_base + 128 + kk * 8, sdesc_advance(make_sdesc(b_addr, BLOCK_BYTES, 1024), kk * 2048),
                  make_idesc(128, 128, false, true), kk > 0);
        } else if (VARIANT == 2) {
          umma_ss(tmem_base, sdesc_advance(make_sdesc(a_addr, 16, 1024), koff),
                  sdesc_advance(make_sdesc(b_addr, BLOCK_BYTES, 1024), kk * 2048),
                  make_idesc(128, 128, false, true), kk > 0);
        } else {
          umma_ss(tmem_base, sdesc_advance(make_sdesc(a_addr, BLOCK_BYTES, 1024), kk * 2048),
                  sdesc_advance(make_sdesc(b_addr, BLOCK_BYTES, 1024), kk * 2048),
                  make_idesc(128, 128, true, true), kk > 0);
        }
      }
      umma_commit(mma_done);
    }
  }
  __syncwarp();
  ok = mbar_wait(mma_done, 0, abort_flag, status, DEV_ERR_TIMEOUT_MMA);
  ok = __all_sync(0xffffffffu, ok);
  if (ok) {
    tc_fence_after();
    uint32_t r[32];
#pragma unroll 1
    for (int c = 0; c < 4; ++c) {
      tmem_ld_x32(t_lane + c * 32, r);
      tmem_wait_ld();
#pragma unroll
      for (int i = 0; i < 32; ++i) out[tid * 128 + c * 32 + i] = __uint_as_float(r[i]);
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    if (*abort_flag)
      for (int i = 0; i < 50; ++i) __nanosleep(20000);
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}

// Waits on a barrier that nothing ever arrives on; the wait gives up after `limit_ns`.
__global__ void wait_timeout_selftest_kernel(int* status, unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    ptx::mbar_init(&bar, 1);
    ptx::fence_mbar_init();
  }
  __syncthreads();
  ptx::mbar_wait(&bar, 0, &abort_flag, status, DEV_ERR_TIMEOUT_TEST, limit_ns);
}

}  // namespace it
