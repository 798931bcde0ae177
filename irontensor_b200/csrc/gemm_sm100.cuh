// bf16 GEMMs for the projections around attention on sm_100a: C = A * B^T, C = A * B, C = A^T * B.
//
// Replaces the reference's linear_forward / linear_backward (src/train/helpers.rs:48-76:
// y = x W^T through matmul_mps_nt, dx = dy W through matmul, dW = dy^T x through matmul_mps_tn; all on
// MPS in fp32, src/ops/mps_gemm.rs) for bf16 tensors: row-major operands as they lie in memory, the
// three transposition cases as descriptor bits (which index is contiguous in shared memory), fp32
// accumulation in TMEM, bf16 or fp32 result.
//   LAYOUT 0 (NT): A [M,K], B [N,K]   -> both K-major           y  = x W^T
//   LAYOUT 1 (NN): A [M,K], B [K,N]   -> A K-major, B N-major   dx = dy W
//   LAYOUT 2 (TN): A [K,M], B [K,N]   -> A M-major, B N-major   dW = dy^T x
// Persistent kernel, one CTA per SM, tiles of 128 x 256 handed out round-robin in an order that keeps the
// tiles of the CTAs running at one time close together (gemm_tile_coords):
//   warp 0     : TMA producer, a four-stage ring of (A 128x64, B 256x64) blocks, 128-byte swizzle
//   warp 1     : MMA issuer, tcgen05.mma 128x256x16, two accumulators of 256 TMEM columns so that the
//                next tile's MMAs run while the previous tile is stored
//   warp 2     : TMEM allocation / release
//   warps 4-7  : epilogue, a thread per row: TMEM -> registers -> bf16/fp32 -> global
// K and the row pitches must be multiples of 8 elements (16-byte rows for TMA); M, N, K are
// otherwise free (edges are zero-filled on load and masked on store).
#pragma once
#include "rope.cuh"
#include "sm100_ptx.cuh"

namespace it {

struct GemmTraits {
  static constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4;
  static constexpr int A_BYTES = BM * BK * 2;      // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;      // 32 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int OUT_BYTES = BM * 128;       // reduce-scatter epilogue: staging of 128 rows x 64 bf16 columns, two of them
  static constexpr int SMEM_OUT = STAGES * STAGE_BYTES;
  static constexpr int SMEM_BAR = SMEM_OUT + 2 * OUT_BYTES;
  static constexpr int NUM_BARS = 2 * STAGES + 4 + 4;
  static constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = SMEM_MISC + 16;
  static constexpr int THREADS = 256;
  static constexpr uint32_t TMEM_COLS = 512;
};

struct GemmParams {
  void* c;            // [M, N] row-major, bf16 or fp32
  long long ldc;      // elements between rows of C
  int M, N, K;
  int c_is_f32;
  int* status;
  // QKV epilogue (gemm_bf16_sm100_kernel<0, true>): the N columns are [heads*D of Q | kv_heads*D of K | kv_heads*D
  // of V]; row r is token (batch, r % seq).  Q and K columns are rotated by the token's position and the three
  // ranges are stored to q [M, heads, D], k and v [M, kv_heads, D].
  __nv_bfloat16 *q, *k, *v;
  int seq, heads, kv_heads, head_dim;
  long long ld_q, ld_kv;      // elements between the rows (tokens) of q and of k / v: heads*D and kv_heads*D when the three are
                              // separate tensors, (heads + 2 kv_heads)*D when they are column ranges of one packed buffer
  const float2* rope_table;   // [seq][head_dim / 2] (cos, sin), or null: no rotation
  // Reduce-scatter epilogue (gemm_bf16_sm100_kernel<.., .., true>): row block [r * rs_rows, (r + 1) * rs_rows) of the
  // product is ADDED into rank r's copy of C, so that after every rank's GEMM rank r holds the sum over ranks of its
  // row block.  rs_rows is a multiple of the tile height, so a tile has one owner.
  int rs_world;
  int rs_rows;
};

// Tensor maps of every rank's copy of C ([n, width] bf16, boxes of 64 columns x 128 rows) for the reduce-scatter
// epilogue: this GPU's own memory or a peer's, mapped into this process.
struct GemmScatterMaps {
  CUtensorMap c_of_rank[8];
};

// Tile index -> tile coordinates.  Tiles are numbered in groups of 16 rows of tiles: within a group the M
// index runs fastest, then N.  The CTAs running at one time hold consecutive numbers, i.e. a block of
// about 16 x 9 tiles, so each A and B tile they stream is shared by many of them while it sits in L2
// (with M simply running fastest over the whole matrix, A was re-read from DRAM once per column of tiles:
// 2.4 GB of DRAM reads for 0.16 GB of operands on 32768 x 2048 x 6144).
__device__ __forceinline__ void gemm_tile_coords(int tile, int tiles_m, int tiles_n, int* tm, int* tn) {
  constexpr int GROUP_M = 16;
  const int per_group = GROUP_M * tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int gm = min(GROUP_M, tiles_m - first_m);
  const int in_group = tile - group * per_group;
  *tm = first_m + in_group % gm;
  *tn = in_group / gm;
}

// QKV = true (layout 0 only) is the fused Q/K/V projection: one GEMM over the stacked weights
// [Wq; Wk; Wv] (the reference runs three linear_forward calls on the same input and then rope() twice:
// src/train/forward.rs:101-103,111-112) whose epilogue applies the rotary embedding to the Q and K
// columns - a rotation pair is two neighbouring accumulator registers of the thread that owns the token's
// row; cosines and sines come from a table built once per call - and writes q_rope, k_rope and v in the [batch, seq, heads, head_dim] layout attention reads.
// RS = true is the GEMM that does its own reduce-scatter: the epilogue warps round each 128 x 64 piece of a finished
// tile to bf16 into a swizzled staging buffer, and one thread (warp 3) adds it into the copy of C of the rank that
// owns those rows with a TMA reduce-add -- whole 128-byte lines, over NVLink when the owner is a peer -- while the
// tensor core is already on the next tile.
template <int LAYOUT, bool QKV = false, bool RS = false>
__global__ void __launch_bounds__(256, 1)
gemm_bf16_sm100_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                       const GemmParams prm, const __grid_constant__ GemmScatterMaps rs_maps) {
  using T = GemmTraits;
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::SMEM_BAR);
  uint64_t* full = bars;                    // [STAGES] operands landed
  uint64_t* empty = full + T::STAGES;       // [STAGES] MMAs that read the stage are complete
  uint64_t* acc_full = empty + T::STAGES;   // [2] a tile's accumulator is complete
  uint64_t* acc_empty = acc_full + 2;       // [2] the epilogue has read it (128 arrivals)
  uint64_t* out_full = acc_empty + 2;       // [2] a staging buffer holds a piece (128 arrivals)
  uint64_t* out_free = out_full + 2;        // [2] the reduce-add has read it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + T::SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_m = (prm.M + T::BM - 1) / T::BM, tiles_n = (prm.N + T::BN - 1) / T::BN;
  const int n_tiles = tiles_m * tiles_n;
  const int n_kb = (prm.K + T::BK - 1) / T::BK;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if (smem_addr(smem) & 1023u) {
      *abort_flag = 1;
      atomicCAS(prm.status, 0, DEV_ERR_SMEM_ALIGN);
    }
    if (*reinterpret_cast<volatile int*>(prm.status) != 0) *abort_flag = 1;
    for (int i = 0; i < T::STAGES; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&acc_full[i], 1);
      mbar_init(&acc_empty[i], 128);
      mbar_init(&out_full[i], 128);
      mbar_init(&out_free[i], 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const bool run = (*abort_flag == 0) && n_kb > 0;

  if (!run) {
    // nothing to do
  } else if (warp == 0) {
    if (lane == 0) {
      prefetch_tensormap(&tmap_a);
      prefetch_tensormap(&tmap_b);
      int it = 0;   // stage use counter
      for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
        int tm, tn;
        gemm_tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        const int m0 = tm * T::BM, n0 = tn * T::BN;
        bool ok = true;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int st = it % T::STAGES;
          const uint32_t ph = (it / T::STAGES) & 1;
          ok = mbar_wait(&empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY);
          if (!ok) break;
          uint8_t* sa = smem + st * T::STAGE_BYTES;
          uint8_t* sb = sa + T::A_BYTES;
          mbar_arrive_expect_tx(&full[st], T::STAGE_BYTES);
          const int k0 = kb * T::BK;
          if (LAYOUT == 2) {   // A [K,M]: 64 K-rows of M, two 64-wide M blocks
            tma_load_4d(sa, &tmap_a, &full[st], m0, k0, 0, 0);
            tma_load_4d(sa + T::A_BYTES / 2, &tmap_a, &full[st], m0 + 64, k0, 0, 0);
          } else {             // A [M,K]: 128 rows of 64 K
            tma_load_4d(sa, &tmap_a, &full[st], k0, m0, 0, 0);
          }
          if (LAYOUT == 0) {   // B [N,K]: 256 rows of 64 K
            tma_load_4d(sb, &tmap_b, &full[st], k0, n0, 0, 0);
          } else {             // B [K,N]: 64 K-rows of N, four 64-wide N blocks
#pragma unroll
            for (int b = 0; b < 4; ++b) tma_load_4d(sb + b * (T::B_BYTES / 4), &tmap_b, &full[st], n0 + b * 64, k0, 0, 0);
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t IDESC = make_idesc(T::BM, T::BN, LAYOUT == 2, LAYOUT != 0);
      int it = 0, t = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
        const int buf = t & 1;
        ok = mbar_wait(&acc_empty[buf], ((t >> 1) & 1) ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
        if (!ok) break;
        tc_fence_after();
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          const int st = it % T::STAGES;
          ok = mbar_wait(&full[st], (it / T::STAGES) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a_addr = smem_addr(smem + st * T::STAGE_BYTES), b_addr = a_addr + T::A_BYTES;
          // K-major: 8-row groups 1024 bytes apart, a K step of 16 is 32 bytes along the row.
          // MN-major: the next 64 M/N elements one block further, a K step of 16 rows is 2048 bytes.
          const uint64_t da = (LAYOUT == 2) ? make_sdesc(a_addr, T::A_BYTES / 2, 1024) : make_sdesc(a_addr, 16, 1024);
          const uint64_t db = (LAYOUT == 0) ? make_sdesc(b_addr, 16, 1024) : make_sdesc(b_addr, T::B_BYTES / 4, 1024);
#pragma unroll
          for (int kk = 0; kk < T::BK / 16; ++kk)
            umma_ss(tmem_base + buf * T::BN, sdesc_advance(da, (LAYOUT == 2) ? kk * 2048 : kk * 32),
                    sdesc_advance(db, (LAYOUT == 0) ? kk * 32 : kk * 2048), IDESC, (kb > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&empty[st]);
        }
        if (ok) umma_commit(&acc_full[buf]);
      }
    }
  } else if (warp == 3) {
    if (RS && lane == 0) {
      // reduce-add issuer: pieces in the order the epilogue produces them
      int g = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        int tm, tn;
        gemm_tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
        const int m0 = tm * T::BM, n0 = tn * T::BN;
        const CUtensorMap* map = &rs_maps.c_of_rank[min(m0 / prm.rs_rows, prm.rs_world - 1)];
        for (int c = 0; c < T::BN / 64; ++c) {
          if (n0 + c * 64 >= prm.N) break;        // the epilogue produces no piece past the last column
          const int buf = g & 1;
          ok = mbar_wait(&out_full[buf], static_cast<uint32_t>(g >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tma_reduce_add_4d(map, smem + T::SMEM_OUT + buf * T::OUT_BYTES, n0 + c * 64, m0, 0, 0);
          bulk_commit_group();
          if (g >= 1) {   // the previous piece's reduce has read the other buffer: hand it back
            bulk_wait_group_read<1>();
            mbar_arrive(&out_free[buf ^ 1]);
          }
          ++g;
        }
      }
      bulk_wait_group_all();   // the adds have been performed, at the peers too, before the kernel ends
    }
  } else if (warp >= 4) {
    const int row_in_tile = (warp & 3) * 32 + lane;
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16);
    int t = 0;
    int rs_g = 0;   // staged pieces so far (reduce-scatter epilogue)
    bool ok = true;
    uint32_t r[32];
    for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++t) {
      const int buf = t & 1;
      int tm, tn;
      gemm_tile_coords(tile, tiles_m, tiles_n, &tm, &tn);
      const int m0 = tm * T::BM, n0 = tn * T::BN;
      ok = mbar_wait(&acc_full[buf], (t >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m0 + row_in_tile;
      if constexpr (RS) {
        // 64 columns at a time: this thread's row of the piece is 128 bytes of the staging buffer (128-byte swizzle, the
        // layout the tensor map of C expects); rows past M and columns past N are dropped by the reduce-add
        const int swz = row_in_tile & 7;
#pragma unroll 1
        for (int c = 0; c < T::BN / 64; ++c) {
          if (n0 + c * 64 >= prm.N) break;
          const int obuf = rs_g & 1;
          ok = mbar_wait(&out_free[obuf], ((static_cast<uint32_t>(rs_g) >> 1) & 1) ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          uint8_t* dst = smem + T::SMEM_OUT + obuf * T::OUT_BYTES + row_in_tile * 128;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            tmem_ld_x32(t_lane + buf * T::BN + c * 64 + h * 32, r);
            tmem_wait_ld();
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              w.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              w.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              w.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + (((h * 4 + v) ^ swz) << 4)) = w;
            }
          }
          fence_proxy_async_smem();
          mbar_arrive(&out_full[obuf]);
          ++rs_g;
        }
        if (!ok) break;
      } else {
#pragma unroll 1
      for (int c = 0; c < T::BN / 32; ++c) {
        tmem_ld_x32(t_lane + buf * T::BN + c * 32, r);
        tmem_wait_ld();
        const int col = n0 + c * 32;
        if (QKV) {
          if (row < prm.M && col < prm.N) {   // head_dim is a multiple of 32: a chunk lies inside one head of one tensor
            const int hd_total = prm.heads * prm.head_dim, kv_total = prm.kv_heads * prm.head_dim;
            __nv_bfloat16* dst;
            int d0;
            bool rotate = true;
            if (col < hd_total) {
              d0 = col % prm.head_dim;
              dst = prm.q + static_cast<long long>(row) * prm.ld_q + col;
            } else if (col < hd_total + kv_total) {
              const int cc = col - hd_total;
              d0 = cc % prm.head_dim;
              dst = prm.k + static_cast<long long>(row) * prm.ld_kv + cc;
            } else {
              const int cc = col - hd_total - kv_total;
              d0 = cc % prm.head_dim;
              dst = prm.v + static_cast<long long>(row) * prm.ld_kv + cc;
              rotate = false;
            }
            if (rotate && prm.rope_table != nullptr) {
              // 16 (cos, sin) pairs of this token's position: 128 contiguous bytes of the table
              const float4* tab = reinterpret_cast<const float4*>(prm.rope_table + static_cast<size_t>(row % prm.seq) * (prm.head_dim >> 1) +
                                                                  (d0 >> 1));
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                const float4 cs = __ldg(tab + i);   // (cos, sin) of pairs 2i and 2i+1
                const float a0 = __uint_as_float(r[4 * i]), a1 = __uint_as_float(r[4 * i + 1]);
                const float b0 = __uint_as_float(r[4 * i + 2]), b1 = __uint_as_float(r[4 * i + 3]);
                r[4 * i] = __float_as_uint(a0 * cs.x - a1 * cs.y);
                r[4 * i + 1] = __float_as_uint(a0 * cs.y + a1 * cs.x);
                r[4 * i + 2] = __float_as_uint(b0 * cs.z - b1 * cs.w);
                r[4 * i + 3] = __float_as_uint(b0 * cs.w + b1 * cs.z);
              }
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 w;
              w.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
              w.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
              w.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
              w.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
              *reinterpret_cast<uint4*>(dst + v * 8) = w;
            }
          }
        } else if (row < prm.M && col < prm.N) {
          if (prm.c_is_f32) {
            float* dst = static_cast<float*>(prm.c) + static_cast<long long>(row) * prm.ldc + col;
            if (col + 32 <= prm.N && (prm.ldc & 3) == 0) {
#pragma unroll
              for (int v = 0; v < 8; ++v)
                *reinterpret_cast<uint4*>(dst + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col + i < prm.N) dst[i] = __uint_as_float(r[i]);
            }
          } else {
            __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(prm.c) + static_cast<long long>(row) * prm.ldc + col;
            if (col + 32 <= prm.N && (prm.ldc & 7) == 0) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                uint4 w;
                w.x = pack_bf16(__uint_as_float(r[v * 8 + 0]), __uint_as_float(r[v * 8 + 1]));
                w.y = pack_bf16(__uint_as_float(r[v * 8 + 2]), __uint_as_float(r[v * 8 + 3]));
                w.z = pack_bf16(__uint_as_float(r[v * 8 + 4]), __uint_as_float(r[v * 8 + 5]));
                w.w = pack_bf16(__uint_as_float(r[v * 8 + 6]), __uint_as_float(r[v * 8 + 7]));
                *reinterpret_cast<uint4*>(dst + v * 8) = w;
              }
            } else {
#pragma unroll
              for (int i = 0; i < 32; ++i)
                if (col + i < prm.N) dst[i] = __float2bfloat16_rn(__uint_as_float(r[i]));
            }
          }
        }
      }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[buf]);
    }
  }

  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*abort_flag)
      for (int i = 0; i < 50; ++i) __nanosleep(20000);
    tc_fence_after();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace it
