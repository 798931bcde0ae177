// Causal / full scaled-dot-product attention forward for bf16 inputs on sm_100a, long sequences:
// one query tile per CTA, the two softmax groups alternating over KEY tiles.
//
// Replaces, for bf16 tensors, the reference project's forward kernels
// (src/shaders/flash_attention.metal:45-163 online softmax; :167-223 exact softmax) and adds the
// per-row log-sum-exp output the fused backward needs.  The launcher picks this kernel for head_dim 128
// and 5120 keys or more; fa_fwd_sm100.cuh (two query tiles per CTA) covers the rest.
//
// One CTA owns one 128-row query tile of one (batch, head) slice and walks its key tiles once:
//   warp 0      : TMA producer  - the Q tile once, then a ring of K tiles (128-byte swizzle)
//   warp 3      : TMA producer  - a ring of V tiles
//   warp 1      : MMA issuer    - S(j) = Q K(j)^T into one of two S buffers (tcgen05, accumulators in TMEM)
//   warp 2      : MMA issuer    - O += P(j) V(j); TMEM allocation / release
//   warps 4-7   : softmax of the even key tiles (one thread per query row)
//   warps 8-11  : softmax of the odd key tiles (the thread with the same lane owns the same row)
// S(j) and P(j) have TMEM columns of their own, so S(j+2) is issued as soon as S(j) sits in the
// registers of its softmax group and never waits for P(j) V(j); the two MMA streams have no order
// between them and each has its own issuing thread, so one stream's barrier waits hide behind the
// other's bursts (the queue in front of the tensor core holds only a few hundred cycles of work, and
// with a single issuing thread every wait was a gap).  Q is copied into TMEM once and is the A operand
// of every S MMA from there: with one query tile per CTA the K/V tiles are not shared between query
// tiles, and re-reading Q from shared memory for each key tile made shared memory the bound.
// The exponentials of two consecutive key tiles overlap.  The only thing the two softmax groups hand
// each other is the per-row reference maximum (shared memory, one small barrier per warp): group A
// needs it after group B's max pass, not after its exponentials.
// Softmax runs in the exp2 domain with 1/sqrt(D)*log2(e) folded into one FMA; the reference maximum
// is only raised (and O rescaled in TMEM) when it would grow by more than 2^8.  Each group keeps its
// own partial row sum relative to the reference it last used; the two are brought to the final
// reference and added at the end.  P(j) is packed in place over the row's registers and stored to the
// one P buffer when P(j-1) V(j-1) has read it, which by then has long happened.
// Causal: key tiles above the diagonal are never loaded; only the diagonal tile is masked.
// TMEM columns (512 allocated): S buffers [0,128) [128,256), O [256,256+D), P [256+D,256+D+64) and
// Q [256+D+64,256+D+64+D/2) as packed bf16.
#pragma once
#include "fa_fwd_sm100.cuh"   // FwdParams
#include "sm100_ptx.cuh"

namespace it {

template <int D>
struct FwdPPTraits {
  static constexpr int BM = 128;            // query rows per tile
  static constexpr int BN = 128;            // keys per tile
  static constexpr int QT_PER_CTA = 1;      // query tiles per CTA
  static constexpr int STAGES = (D == 128) ? 3 : 4;       // K ring and V ring, each
  static constexpr int TILE_BYTES = BM * D * 2;          // one Q, K or V tile
  static constexpr int BLOCK_BYTES = 128 * 128;          // one [128 x 64] bf16 swizzled block
  static constexpr int NBLK = D / 64;                    // 64-column blocks per tile
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_K = SMEM_Q + TILE_BYTES;
  static constexpr int SMEM_V = SMEM_K + STAGES * TILE_BYTES;
  static constexpr int SMEM_MREF = SMEM_V + STAGES * TILE_BYTES;   // [128] fp32 reference maxima
  static constexpr int SMEM_LPART = SMEM_MREF + 512;               // [2][128] fp32 partial row sums
  static constexpr int SMEM_BAR = SMEM_LPART + 1024;
  static constexpr int NUM_BARS = 1 + 4 * STAGES + 2 + 2 + 8 + 1 + 1;
  static constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = SMEM_MISC + 16;
  static constexpr int THREADS = 384;
  static constexpr uint32_t TMEM_COLS = 512;
  static constexpr uint32_t COL_S = 0, COL_O = 256, COL_P = 256 + D, COL_Q = 256 + D + 64;
};


// DECODE = true is the same pipeline for one new token per sequence against a key/value cache
// (fa_decode.cuh describes the op): the rows of the query tile are the query HEADS of one K/V head's
// group (rows past the group are zero-filled by TMA and never stored), prm.S is the number of valid
// cache positions, a CTA takes one split of the key tiles of one (batch, K/V head) and leaves either
// the final output (one split) or an unnormalised partial output with its reference maximum and row
// sum for fa_decode_merge_kernel.  The cache is streamed by TMA through the same K and V rings, so
// the op runs at the rate the memory system delivers tiles, not at the rate CUDA cores can issue loads.
template <int D, bool DECODE = false>
__global__ void __launch_bounds__(384, 1)
fa_fwd_pp_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FwdParams prm) {
  using T = FwdPPTraits<D>;
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::SMEM_BAR);
  uint64_t* q_full = bars;                        // [1]
  uint64_t* k_full = q_full + 1;                  // [STAGES]
  uint64_t* k_empty = k_full + T::STAGES;
  uint64_t* v_full = k_empty + T::STAGES;
  uint64_t* v_empty = v_full + T::STAGES;
  // k_empty[j % STAGES] doubles as "S(j) complete" and v_empty[j % STAGES] as "P(j) V(j) complete" for the
  // softmax groups: one commit per MMA burst keeps the issuing thread's time between bursts short (the
  // queue in front of the tensor core holds only a few hundred cycles of work).
  uint64_t* s_free = v_empty + T::STAGES;         // [2] S(j) read into registers (128 arrivals)
  uint64_t* p_full = s_free + 2;                  // [2] P(j) written (128 arrivals)
  uint64_t* m_pub = p_full + 2;                   // [2][4] reference maxima of tile j published (32 arrivals)
  uint64_t* l_bar = m_pub + 8;                    // [1] partial row sums exchanged (256 arrivals)
  uint64_t* q_tmem = l_bar + 1;                   // [1] Q copied into TMEM (256 arrivals)
  float* m_ref = reinterpret_cast<float*>(smem + T::SMEM_MREF);
  float* l_part = reinterpret_cast<float*>(smem + T::SMEM_LPART);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + T::SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 4);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = prm.S;
  const int n_kv_total = (S + T::BN - 1) / T::BN;
  const int n_qt = (S + T::BM - 1) / T::BM;
  // Head-major order: the CTAs resident at one time belong to a few (batch, head) slices, so the K/V
  // tiles they all stream stay in L2.  Within a slice the last query tiles (most keys) go first.
  int bh, qt, hd, bt, hkv, nkv, j0 = 0;   // j0: first key tile of this CTA (decode splits)
  if (DECODE) {
    const int kv_heads = prm.st.heads / prm.kv_group;
    const int bkv = static_cast<int>(blockIdx.x) / prm.dec_n_splits;   // batch * kv_heads + kv_head
    const int sp = static_cast<int>(blockIdx.x) % prm.dec_n_splits;
    hkv = bkv % kv_heads;
    bt = bkv / kv_heads;
    hd = hkv;                      // the query tensor map is [D, group, kv_heads, batch]
    qt = 0;
    bh = bt * prm.st.heads + hkv * prm.kv_group;   // first query slice of the group
    j0 = sp * prm.dec_tiles_per_split;
    nkv = max(0, min(prm.dec_tiles_per_split, n_kv_total - j0));
  } else {
    // Slice after slice, except that the last eight slices are taken together, heaviest query tiles of
    // all eight first (tail_grouped_order): otherwise the last slice's 64-tile CTA runs almost alone
    // (3 % of a 64-slice launch, 28 % of the 8-slice launch one of eight GPUs gets).
    int rank;
    tail_grouped_order(static_cast<int>(blockIdx.x), n_qt, static_cast<int>(gridDim.x) / n_qt, &bh, &rank);
    qt = n_qt - 1 - rank;
    hd = bh % prm.st.heads;   // TMA coordinates of the slice
    bt = bh / prm.st.heads;
    hkv = hd / prm.kv_group;  // the K/V head this query head reads
    nkv = prm.causal ? min(qt + 1, n_kv_total) : n_kv_total;
  }

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if (smem_addr(smem) & 1023u) {
      *abort_flag = 1;
      atomicCAS(prm.status, 0, DEV_ERR_SMEM_ALIGN);
    }
    // An earlier CTA of this (or a previous) launch gave up on a wait: do not start, so that a
    // launch that cannot make progress drains quickly instead of timing out CTA by CTA.
    if (*reinterpret_cast<volatile int*>(prm.status) != 0) *abort_flag = 1;
    mbar_init(q_full, 1);
    mbar_init(l_bar, 256);
    mbar_init(q_tmem, 256);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_free[i], 128);
      mbar_init(&p_full[i], 128);
    }
    for (int i = 0; i < 8; ++i) mbar_init(&m_pub[i], 32);
    for (int i = 0; i < T::STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  // The query tile and the first K and V tiles go out before the CTA-wide set-up (tensor-memory allocation, barrier,
  // register hand-over), so their round trip to memory runs under it.  Nothing is loaded into a CTA that will not run.
  if (threadIdx.x == 0 && *abort_flag == 0 && nkv > 0) {
    grid_dep_wait();   // the inputs may be what the kernel in front of this one wrote (no-op unless launched as its dependent)
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
    mbar_arrive_expect_tx(q_full, T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_Q + b * T::BLOCK_BYTES, &tmap_q, q_full, b * 64, qt * T::BM, hd, bt);
    mbar_arrive_expect_tx(&k_full[0], T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_K + b * T::BLOCK_BYTES, &tmap_k, &k_full[0], b * 64, j0 * T::BN, hkv, bt);
    mbar_arrive_expect_tx(&v_full[0], T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_V + b * T::BLOCK_BYTES, &tmap_v, &v_full[0], b * 64, j0 * T::BN, hkv, bt);
  }
  if (warp == 2) {
    tmem_alloc(tmem_slot, T::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  grid_dep_wait();     // (thread 0 has been through it; the others write outputs the kernel in front may still read)
  grid_dep_launch();   // a dependent launch behind this kernel (the backward's prepare pass) may be set up meanwhile
  const uint32_t tmem_base = *tmem_slot;
  const bool bad_start = (*abort_flag != 0) || nkv <= 0;   // an empty split (the launcher makes none) must not wait

  // Register budget: the control warpgroup keeps 80 per thread, the two softmax warpgroups take
  // 208 each so that a whole 128-column row of S stays in registers (128*80 + 256*208 = 63488).
  static_assert(128 * 80 + 256 * 208 <= 384 * 168, "setmaxnreg budget exceeds the registers the CTA is launched with");
  if (warp < 4) {
    setmaxnreg_dec<80>();
    if (bad_start) {
      // nothing to do
    } else if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      // (the query tile and K tile 0 were issued by this thread before the set-up barrier)
      if (lane == 0) {
        for (int i = 1; i < nkv; ++i) {
          const int st = i % T::STAGES;
          const uint32_t ph = (i / T::STAGES) & 1;
          if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) break;
          mbar_arrive_expect_tx(&k_full[st], T::TILE_BYTES);
          for (int b = 0; b < T::NBLK; ++b)
            tma_load_4d(smem + T::SMEM_K + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_k, &k_full[st], b * 64,
                        (j0 + i) * T::BN, hkv, bt);
        }
      }
    } else if (warp == 3) {
      // ------------------------------------------------------------ TMA producer for V: a ring of its own,
      // because K runs two tiles ahead of V (S(j+2) is issued while P(j) is still being computed) and a
      // wait for a free V stage must not hold back the next K tile.
      // (V tile 0 was issued by thread 0 before the set-up barrier)
      if (lane == 0) {
        for (int i = 1; i < nkv; ++i) {
          const int st = i % T::STAGES;
          const uint32_t ph = (i / T::STAGES) & 1;
          if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) break;
          mbar_arrive_expect_tx(&v_full[st], T::TILE_BYTES);
          for (int b = 0; b < T::NBLK; ++b)
            tma_load_4d(smem + T::SMEM_V + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_v, &v_full[st], b * 64,
                        (j0 + i) * T::BN, hkv, bt);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer for S = Q K^T (one thread)
      // The two MMA streams have no ordering between them (S and P have separate TMEM columns), so each
      // has its own issuing thread: while one sits in a barrier wait the other keeps the tensor core fed.
      if (lane == 0) {
        constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
        const uint32_t k_addr = smem_addr(smem + T::SMEM_K);
        auto issue_s = [&](int j) {   // S(j) = Q * K(j)^T into S buffer j&1: Q from TMEM, K K-major from shared memory
          const int st = j % T::STAGES;
          const uint64_t dk = make_sdesc(k_addr + st * T::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * T::BLOCK_BYTES + (kk & 3) * 32;
            umma_ts(tmem_base + T::COL_S + (j & 1) * 128, tmem_base + T::COL_Q + kk * 8, sdesc_advance(dk, off), IDESC_S,
                    kk > 0);
          }
          umma_commit(&k_empty[st]);
        };
        bool ok = mbar_wait(q_tmem, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
        for (int j = 0; j < nkv && ok; ++j) {
          if (j < 2) {
            ok = mbar_wait(&k_full[j], 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
          } else {   // K(j) has landed and S(j-2) sits in the registers of its softmax group
            ok = mbar_wait(&k_full[j % T::STAGES], (j / T::STAGES) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD) &&
                 mbar_wait(&s_free[j & 1], ((j - 2) >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
          }
          if (!ok) break;
          tc_fence_after();
          issue_s(j);
        }
      }
    } else if (warp == 2) {
      // ------------------------------------------------------------ MMA issuer for O += P V (one thread)
      if (lane == 0) {
        constexpr uint32_t IDESC_PV = make_idesc(128, D, false, true);
        const uint32_t v_addr = smem_addr(smem + T::SMEM_V);
        bool ok = true;
        for (int j = 0; j < nkv && ok; ++j) {
          const int st = j % T::STAGES;
          ok = mbar_wait(&v_full[st], (j / T::STAGES) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD) &&
               mbar_wait(&p_full[j & 1], (j >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
          if (!ok) break;
          tc_fence_after();
          const uint64_t dv = make_sdesc(v_addr + st * T::TILE_BYTES, T::BLOCK_BYTES, 1024);   // V N-major
#pragma unroll
          for (int kk = 0; kk < T::BN / 16; ++kk)
            umma_ts(tmem_base + T::COL_O, tmem_base + T::COL_P + kk * 8, sdesc_advance(dv, kk * 2048),
                    IDESC_PV, (j > 0 || kk > 0) ? 1u : 0u);
          umma_commit(&v_empty[st]);
        }
      }
    }
  } else {
    setmaxnreg_inc<208>();
    // ------------------------------------------------------------ softmax + epilogue
    const int w = (warp - 4) >> 2;       // 0: even key tiles, 1: odd key tiles
    const int wq = warp & 3;             // TMEM lane quarter of this warp
    if (!bad_start) {
      const int lane_base = wq * 32;
      const int row = lane_base + lane;
      const int q_row = qt * T::BM + row;
      const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(lane_base) << 16);
      const uint32_t t_s = t_lane + T::COL_S + w * 128;
      const uint32_t t_o = t_lane + T::COL_O;
      const uint32_t t_p = t_lane + T::COL_P;
      const float sl2 = prm.scale_log2;
      const int k_limit = (!DECODE && prm.causal) ? min(S - 1, q_row) : (S - 1);   // last visible key index
      float m_used = -INFINITY;   // the reference this group's partial sum is relative to
      float l_sum = 0.f;
      bool ok = true;
      uint32_t r[128];   // this thread's row of S
      // Q goes into TMEM once (as the A operand of every S MMA it is then not re-read from shared memory
      // for each key tile, which was a third of the kernel's shared-memory traffic).  Each thread copies
      // its row: this group the 64-column blocks w, w+2, ...
      ok = mbar_wait(q_full, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
      ok = __all_sync(0xffffffffu, ok);
      if (ok) {
        for (int b = w; b < T::NBLK; b += 2) {
          const uint8_t* qrow = smem + T::SMEM_Q + b * T::BLOCK_BYTES + row * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            const uint4 x = *reinterpret_cast<const uint4*>(qrow + ((c ^ (row & 7)) << 4));
            r[c * 4 + 0] = x.x;
            r[c * 4 + 1] = x.y;
            r[c * 4 + 2] = x.z;
            r[c * 4 + 3] = x.w;
          }
          tmem_st_x32(t_lane + T::COL_Q + b * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        }
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(q_tmem);
      }
      for (int j = w; ok && j < nkv; j += 2) {
        ok = mbar_wait(&k_empty[j % T::STAGES], (j / T::STAGES) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);   // S(j)
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        // the whole row in one go: four loads in flight, one wait
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        // Probe the barrier needed after the max pass now: its shared-memory round trip (slow while the
        // tensor core streams operands) then overlaps the loads and the max pass.
        const bool m_ready = (j > 0) && mbar_test_wait(&m_pub[((j - 1) & 1) * 4 + wq], ((j - 1) >> 1) & 1);
        tmem_wait_ld();
        tc_fence_before();
        mbar_arrive(&s_free[w]);   // the S buffer may take S(j+2)
        if ((!DECODE && prm.causal && j == qt) || ((j0 + j + 1) * T::BN > S)) {   // diagonal or ragged last tile
          const int vis = k_limit - (j0 + j) * T::BN;   // columns 0..vis are visible
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i > vis) r[i] = 0xFF800000u;     // -inf: drops out of the max, exp2 gives 0
        }
        float mx0 = __uint_as_float(r[0]), mx1 = __uint_as_float(r[1]), mx2 = __uint_as_float(r[2]),
              mx3 = __uint_as_float(r[3]);
#pragma unroll
        for (int i = 4; i < 124; i += 8) {   // three-input max: two new values per instruction
          mx0 = fmax3(mx0, __uint_as_float(r[i]), __uint_as_float(r[i + 1]));
          mx1 = fmax3(mx1, __uint_as_float(r[i + 2]), __uint_as_float(r[i + 3]));
          mx2 = fmax3(mx2, __uint_as_float(r[i + 4]), __uint_as_float(r[i + 5]));
          mx3 = fmax3(mx3, __uint_as_float(r[i + 6]), __uint_as_float(r[i + 7]));
        }
        mx0 = fmax3(mx0, __uint_as_float(r[124]), __uint_as_float(r[125]));
        mx1 = fmax3(mx1, __uint_as_float(r[126]), __uint_as_float(r[127]));
        const float m_new = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * sl2;
        float m_next;
        if (j == 0) {
          m_next = m_new;
        } else {
          // the reference after tile j-1, published by the other group after its max pass
          if (!__all_sync(0xffffffffu, m_ready)) {
            ok = mbar_wait(&m_pub[((j - 1) & 1) * 4 + wq], ((j - 1) >> 1) & 1, abort_flag, prm.status,
                           DEV_ERR_TIMEOUT_SOFTMAX);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          const float m_cur = m_ref[row];
          m_next = m_cur;
          const bool grow = m_new > m_cur + 8.0f;
          if (__any_sync(0xffffffffu, grow)) {   // rare: raise the reference and rescale O in TMEM
            m_next = fmaxf(m_cur, m_new);
            const float f = ex2(m_cur - m_next);
            // O holds tiles 0..j-1 once P(j-1) V(j-1) is complete; P(j) V(j) cannot start before this
            // group has written P(j).
            ok = mbar_wait(&v_empty[(j - 1) % T::STAGES], ((j - 1) / T::STAGES) & 1, abort_flag, prm.status,
                           DEV_ERR_TIMEOUT_MMA);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            uint32_t tmp[16];
#pragma unroll 1
            for (int c = 0; c < D / 16; ++c) {
              tmem_ld_x16(t_o + c * 16, tmp);
              tmem_wait_ld();
#pragma unroll
              for (int i = 0; i < 16; ++i) tmp[i] = __float_as_uint(__uint_as_float(tmp[i]) * f);
              tmem_st_x16(t_o + c * 16, tmp);
            }
            tmem_wait_st();
          }
        }
        if (m_used != m_next) l_sum *= ex2(m_used - m_next);   // -inf on this group's first tile: l_sum is 0
        m_used = m_next;
        m_ref[row] = m_next;
        mbar_arrive(&m_pub[w * 4 + wq]);
        // the one P buffer: P(j-1) V(j-1) must have read it before P(j) goes in; probed here, needed after the exponentials
        const bool p_free = (j == 0) || mbar_test_wait(&v_empty[(j - 1) % T::STAGES], ((j - 1) / T::STAGES) & 1);
        // P = 2^(s*scale - m), packed bf16 in place over the row's registers
        const float neg_m = -m_used;
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
#pragma unroll
          for (int i = 0; i < 32; i += 4) {
            const float p0 = ex2(fmaf(__uint_as_float(r[c * 32 + i + 0]), sl2, neg_m));
            const float p1 = ex2(fmaf(__uint_as_float(r[c * 32 + i + 1]), sl2, neg_m));
            const float p2 = ex2(fmaf(__uint_as_float(r[c * 32 + i + 2]), sl2, neg_m));
            const float p3 = ex2(fmaf(__uint_as_float(r[c * 32 + i + 3]), sl2, neg_m));
            l0 += p0;
            l1 += p1;
            l2 += p2;
            l3 += p3;
            r[c * 16 + (i >> 1)] = pack_bf16(p0, p1);       // words [16c, 16c+16) were consumed by chunk c/2
            r[c * 16 + (i >> 1) + 1] = pack_bf16(p2, p3);
          }
        }
        l_sum += (l0 + l1) + (l2 + l3);
        if (!__all_sync(0xffffffffu, p_free)) {
          ok = mbar_wait(&v_empty[(j - 1) % T::STAGES], ((j - 1) / T::STAGES) & 1, abort_flag, prm.status,
                         DEV_ERR_TIMEOUT_MMA);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
        }
        tc_fence_after();
        tmem_st_x32(t_p, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
        tmem_st_x32(t_p + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[w]);
      }
      // ---- both partial sums relative to the final reference, added; then each group stores half the columns
      float m_fin = m_used;
      const int w_last = (nkv - 1) & 1;
      if (ok && w != w_last) {
        ok = mbar_wait(&m_pub[w_last * 4 + wq], ((nkv - 1) >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) m_fin = m_ref[row];
      }
      if (ok) {
        if (m_used != m_fin) l_sum *= ex2(m_used - m_fin);
        l_part[w * 128 + row] = l_sum;
        mbar_arrive(l_bar);
        ok = mbar_wait(l_bar, 0, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok) {
        ok = mbar_wait(&v_empty[(nkv - 1) % T::STAGES], ((nkv - 1) / T::STAGES) & 1, abort_flag, prm.status,
                       DEV_ERR_TIMEOUT_MMA);   // last P V complete
        ok = __all_sync(0xffffffffu, ok);
      }
      if (ok && DECODE) {
        // rows are the query heads of the group; this group stores half of the columns of each
        tc_fence_after();
        const float l_tot = l_part[row] + l_part[128 + row];
        constexpr int HC = D / 2;
#pragma unroll
        for (int c = 0; c < HC / 32; ++c)
          tmem_ld_x32(t_o + w * HC + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_wait_ld();
        if (row < prm.kv_group) {
          const size_t slice = static_cast<size_t>(bh) + row;
          if (prm.dec_n_splits == 1) {
            const float inv_l = 1.0f / l_tot;
            __nv_bfloat16* orow = prm.o + slice * D + w * HC;
#pragma unroll
            for (int v = 0; v < HC / 8; ++v) {
              uint4 o4;
              o4.x = pack_bf16(__uint_as_float(r[v * 8 + 0]) * inv_l, __uint_as_float(r[v * 8 + 1]) * inv_l);
              o4.y = pack_bf16(__uint_as_float(r[v * 8 + 2]) * inv_l, __uint_as_float(r[v * 8 + 3]) * inv_l);
              o4.z = pack_bf16(__uint_as_float(r[v * 8 + 4]) * inv_l, __uint_as_float(r[v * 8 + 5]) * inv_l);
              o4.w = pack_bf16(__uint_as_float(r[v * 8 + 6]) * inv_l, __uint_as_float(r[v * 8 + 7]) * inv_l);
              *reinterpret_cast<uint4*>(orow + v * 8) = o4;
            }
            if (w == 0 && prm.lse != nullptr) prm.lse[slice] = (m_fin + lg2(l_tot)) * 0.6931471805599453f;
          } else {
            const int sp = static_cast<int>(blockIdx.x) % prm.dec_n_splits;
            float* prow = prm.dec_part_o + (slice * prm.dec_n_splits + sp) * D + w * HC;
#pragma unroll
            for (int v = 0; v < HC / 4; ++v)
              *reinterpret_cast<uint4*>(prow + v * 4) = make_uint4(r[v * 4], r[v * 4 + 1], r[v * 4 + 2], r[v * 4 + 3]);
            if (w == 0) {
              prm.dec_part_ml[(slice * prm.dec_n_splits + sp) * 2] = m_fin;
              prm.dec_part_ml[(slice * prm.dec_n_splits + sp) * 2 + 1] = l_tot;
            }
          }
        }
      } else if (ok) {
        tc_fence_after();
        const float l_tot = l_part[row] + l_part[128 + row];
        const float inv_l = 1.0f / l_tot;
        constexpr int HC = D / 2;   // columns per group
        __nv_bfloat16* orow = prm.o + prm.st.slice(bh) + static_cast<long long>(q_row) * prm.st.row + w * HC;
#pragma unroll
        for (int c = 0; c < HC / 32; ++c)
          tmem_ld_x32(t_o + w * HC + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_wait_ld();
        if (q_row < S) {
#pragma unroll
          for (int v = 0; v < HC / 8; ++v) {
            uint4 o4;
            o4.x = pack_bf16(__uint_as_float(r[v * 8 + 0]) * inv_l, __uint_as_float(r[v * 8 + 1]) * inv_l);
            o4.y = pack_bf16(__uint_as_float(r[v * 8 + 2]) * inv_l, __uint_as_float(r[v * 8 + 3]) * inv_l);
            o4.z = pack_bf16(__uint_as_float(r[v * 8 + 4]) * inv_l, __uint_as_float(r[v * 8 + 5]) * inv_l);
            o4.w = pack_bf16(__uint_as_float(r[v * 8 + 6]) * inv_l, __uint_as_float(r[v * 8 + 7]) * inv_l);
            *reinterpret_cast<uint4*>(orow + v * 8) = o4;
          }
          if (w == 0 && prm.lse != nullptr)
            prm.lse[static_cast<size_t>(bh) * S + q_row] = (m_fin + lg2(l_tot)) * 0.6931471805599453f;
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    if (*abort_flag) {
      // Let any TMA copy or MMA still in flight land before the CTA's memory goes away.
      for (int i = 0; i < 50; ++i) __nanosleep(20000);
    }
    tc_fence_after();
    tmem_dealloc(tmem_base, T::TMEM_COLS);
  }
}

}  // namespace it
