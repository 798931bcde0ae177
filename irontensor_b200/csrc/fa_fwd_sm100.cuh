// Causal / full scaled-dot-product attention forward for bf16 inputs on sm_100a: two query tiles per
// CTA sharing each K/V tile.  The launcher uses it for head_dim 64 and for sequences below 5120 keys
// (fa_fwd_pp_sm100.cuh takes head_dim 128 from 5120 keys on).
//
// Replaces, for bf16 tensors with head_dim 64 or 128, the reference project's forward kernels
// (src/shaders/flash_attention.metal:45-163 online softmax; :167-223 exact softmax) and adds the
// per-row log-sum-exp output the fused backward needs.
//
// One CTA owns two consecutive 128-row query tiles of one (batch, head) slice and walks the key
// tiles once, feeding both:
//   warp 0      : TMA producer  - Q tiles once, then a ring of K and V tiles (128-byte swizzle)
//   warp 1      : MMA issuer    - S_t = Q_t K^T and O_t += P_t V on tcgen05, accumulators in TMEM
//   warp 2      : TMEM allocation / release
//   warps 4-7   : softmax for query tile 0 (one thread per query row)
//   warps 8-11  : softmax for query tile 1
// While one softmax group works on its S tile the tensor core runs the other tile's MMAs.
// Softmax runs in the exp2 domain with 1/sqrt(D)*log2(e) folded into one FMA; the running max is
// only raised (and O rescaled in TMEM) when it would grow by more than 2^8, which keeps rescales
// rare without loss of accuracy (fp32 accumulators hold the extra range).  P is written back over
// S in TMEM as packed bf16 and consumed from there as the A operand of the P*V MMA.
// Causal: key tiles above the diagonal are never loaded; only the diagonal tile is masked.
// TMEM columns (512 allocated): S0 [0,128) S1 [128,256) O0 [256,256+D) O1 [256+D,256+2D).
#pragma once
#include "sm100_ptx.cuh"

namespace it {

template <int D>
struct FwdTraits {
  static constexpr int BM = 128;            // query rows per tile
  static constexpr int BN = 128;            // keys per tile
  static constexpr int QT_PER_CTA = 2;      // query tiles per CTA
  static constexpr int STAGES = (D == 128) ? 2 : 4;
  static constexpr int TILE_BYTES = BM * D * 2;          // one Q, K or V tile
  static constexpr int BLOCK_BYTES = 128 * 128;          // one [128 x 64] bf16 swizzled block
  static constexpr int NBLK = D / 64;                    // 64-column blocks per tile
  static constexpr int SMEM_Q = 0;
  static constexpr int SMEM_K = SMEM_Q + 2 * TILE_BYTES;
  static constexpr int SMEM_V = SMEM_K + STAGES * TILE_BYTES;
  static constexpr int SMEM_BAR = SMEM_V + STAGES * TILE_BYTES;
  static constexpr int NUM_BARS = 4 + 4 * STAGES + 6 + 4;
  static constexpr int SMEM_MISC = SMEM_BAR + NUM_BARS * 8;
  static constexpr int SMEM_BYTES = SMEM_MISC + 16;
  static constexpr int THREADS = 384;
  static constexpr uint32_t TMEM_COLS = 512;
};

struct FwdParams {
  ptx::TensorStrides st; // layout of q, k, v and o
  __nv_bfloat16* o;     // output, same layout as the inputs
  float* lse;           // [BH, S] or null
  int* status;          // device status word
  int S;
  int BH;
  int causal;
  float scale_log2;     // 1/sqrt(D) * log2(e)
  int kv_group;         // query heads per K/V head (grouped-query attention; 1 otherwise)
  int group_slices;     // fa_fwd_sm100_kernel: slices per group of its work-item order
  int* work_counter;    // fa_fwd_sm100_kernel: zeroed before the launch when the grid is smaller than the number of work items, else null
  // decode instantiation of the long-sequence kernel only (one new token against a key/value cache):
  int dec_tiles_per_split;   // key tiles per CTA
  int dec_n_splits;
  float* dec_part_o;    // [B*H, n_splits, D] unnormalised partial outputs (n_splits > 1)
  float* dec_part_ml;   // [B*H, n_splits, 2] reference maximum (log2 domain) and row sum of each split
};

template <int D>
__global__ void __launch_bounds__(384, 1)
fa_fwd_sm100_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, const FwdParams prm) {
  using T = FwdTraits<D>;
  using namespace ptx;
  extern __shared__ __align__(1024) uint8_t smem[];

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + T::SMEM_BAR);
  uint64_t* q_full = bars;                        // [2]
  uint64_t* q_empty = q_full + 2;                 // [2] every S MMA of the work item that reads Q_t has completed
  uint64_t* k_full = q_empty + 2;                 // [STAGES]
  uint64_t* k_empty = k_full + T::STAGES;
  uint64_t* v_full = k_empty + T::STAGES;
  uint64_t* v_empty = v_full + T::STAGES;
  uint64_t* s_full = v_empty + T::STAGES;         // [2]
  uint64_t* p_full = s_full + 2;                  // [2]
  uint64_t* o_done = p_full + 2;                  // [2]
  uint64_t* sched_full = o_done + 2;              // [2] item index written (1 arrival)
  uint64_t* sched_empty = sched_full + 2;         // [2] every role is through with the item (producer, MMA thread, 8 softmax warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + T::SMEM_MISC);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 4);
  volatile int* sched_item = reinterpret_cast<volatile int*>(smem + T::SMEM_MISC + 8);   // [2] item index, -1: no more

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int S = prm.S;
  const int n_kv_total = (S + T::BN - 1) / T::BN;
  const int n_pairs = (S + 2 * T::BM - 1) / (2 * T::BM);
  // Work items are (slice, pair of query tiles).  The grid is at most one CTA per SM and a CTA walks items in a loop
  // in which every role runs ahead on its own: the producer fetches the next item's Q and first K/V tiles while the
  // current item's last tiles are in the softmax, and the MMA thread issues the next item's first S tiles right
  // behind the current item's last P V, so that a CTA pays set-up, first-load latency and tear-down once and not
  // once per item (at a thousand keys an item is a handful of tiles long and they were a quarter of its life).
  // Item order: slices in groups chosen by the launcher (a bound on the K and V bytes in work at once); within a group the pairs with the most key
  // tiles first, all slices of the group for one pair, then the next pair.  A CTA's first item is its own index;
  // the following ones it draws from a counter in global memory (warp 3), one item ahead of the softmax groups, and
  // hands to the other roles through a two-slot ring in shared memory: the lightest items come last, so the CTAs
  // finish within about one small item of each other whatever the mix.
  const int n_items = prm.BH * n_pairs;
  const int G = static_cast<int>(gridDim.x);
  struct Item {
    int bh, pair, hd, bt, hkv, n_kv[2], n_iter;
  };
  auto decode = [&](int idx, Item& it) {
    const int per_group = n_pairs * prm.group_slices;
    const int g = idx / per_group, r = idx - g * per_group;
    const int gs = min(prm.group_slices, prm.BH - g * prm.group_slices);
    it.pair = n_pairs - 1 - r / gs;
    it.bh = g * prm.group_slices + r % gs;
    it.hd = it.bh % prm.st.heads;   // TMA coordinates of the slice
    it.bt = it.bh / prm.st.heads;
    it.hkv = it.hd / prm.kv_group;  // the K/V head this query head reads
#pragma unroll
    for (int t = 0; t < 2; ++t) {
      const int qt = 2 * it.pair + t;
      it.n_kv[t] = (qt * T::BM < S) ? (prm.causal ? min(qt + 1, n_kv_total) : n_kv_total) : 0;
    }
    it.n_iter = max(it.n_kv[0], it.n_kv[1]);
  };
  // The n-th item of this CTA, as the roles other than the scheduler see it: 1 = there is one, 0 = no more, -1 = gave up.
  auto fetch = [&](uint32_t n, Item& it) -> int {
    if (prm.work_counter == nullptr) {   // one item per CTA (a launch no larger than the GPU): nothing to wait for
      if (n > 0) return 0;
      decode(static_cast<int>(blockIdx.x), it);
      return 1;
    }
    if (!mbar_wait(&sched_full[n & 1], (n >> 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) return -1;
    const int idx = sched_item[n & 1];
    if (idx < 0) return 0;
    decode(idx, it);
    return 1;
  };

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    if (smem_addr(smem) & 1023u) {
      *abort_flag = 1;
      atomicCAS(prm.status, 0, DEV_ERR_SMEM_ALIGN);
    }
    // An earlier CTA of this (or a previous) launch gave up on a wait: do not start, so that a
    // launch that cannot make progress drains quickly instead of timing out CTA by CTA.
    if (*reinterpret_cast<volatile int*>(prm.status) != 0) *abort_flag = 1;
    for (int i = 0; i < 2; ++i) {
      mbar_init(&q_full[i], 1);
      mbar_init(&q_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
      mbar_init(&o_done[i], 1);
      mbar_init(&sched_full[i], 1);
      mbar_init(&sched_empty[i], 10);
    }
    for (int i = 0; i < T::STAGES; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
    }
    fence_mbar_init();
    fence_proxy_async_smem();
  }
  // Key/value tile j of an item into ring slot g (g counts the tiles of all items of this CTA; producer thread only).
  auto load_kv = [&](uint32_t g, int j, const Item& it) -> bool {
    const int st = static_cast<int>(g % T::STAGES);
    const uint32_t ph = (g / T::STAGES) & 1;
    if (!mbar_wait(&k_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) return false;
    mbar_arrive_expect_tx(&k_full[st], T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_K + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_k, &k_full[st], b * 64, j * T::BN, it.hkv,
                  it.bt);
    if (!mbar_wait(&v_empty[st], ph ^ 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) return false;
    mbar_arrive_expect_tx(&v_full[st], T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_V + st * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_v, &v_full[st], b * 64, j * T::BN, it.hkv,
                  it.bt);
    return true;
  };
  auto load_q = [&](int t, const Item& it) {
    mbar_arrive_expect_tx(&q_full[t], T::TILE_BYTES);
    for (int b = 0; b < T::NBLK; ++b)
      tma_load_4d(smem + T::SMEM_Q + t * T::TILE_BYTES + b * T::BLOCK_BYTES, &tmap_q, &q_full[t], b * 64,
                  (2 * it.pair + t) * T::BM, it.hd, it.bt);
  };
  // The first item's query tiles and first key/value tile go out before the CTA-wide set-up (tensor-memory allocation,
  // barrier, register hand-over), so their round trip to memory runs under it.  Nothing is loaded into a CTA that
  // will not run.
  if (threadIdx.x == 0 && *abort_flag == 0) {
    grid_dep_wait();   // the inputs may be what the kernel in front of this one wrote (no-op unless launched as its dependent)
    prefetch_tensormap(&tmap_q);
    prefetch_tensormap(&tmap_k);
    prefetch_tensormap(&tmap_v);
    Item it;
    decode(static_cast<int>(blockIdx.x), it);
    for (int t = 0; t < 2; ++t)
      if (it.n_kv[t] > 0) load_q(t, it);
    if (it.n_iter > 0) load_kv(0, 0, it);
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
  const bool bad_start = (*abort_flag != 0);

  // Register budget: the control warpgroup keeps 88 per thread, the two softmax warpgroups take 208 each so that a
  // whole 128-column row of S stays in registers.  The CTA owns what it was launched with, 384 threads x 168 registers;
  // a request beyond that would leave setmaxnreg.inc waiting for registers that never come.
  constexpr int REGS_CTRL = 88, REGS_SOFTMAX = 208;
  static_assert(128 * REGS_CTRL + 256 * REGS_SOFTMAX <= 384 * 168, "setmaxnreg budget exceeds the CTA's registers");
  if (warp < 4) {
    setmaxnreg_dec<REGS_CTRL>();
    if (bad_start) {
      // nothing to do
    } else if (warp == 0) {
      // ------------------------------------------------------------ TMA producer
      // (the first item's query tiles and key/value tile 0 were issued by this thread before the set-up barrier)
      if (lane == 0) {
        uint32_t g = 0;               // key/value tiles issued so far
        uint32_t q_uses[2] = {0, 0};  // items so far that had query tile t
        bool ok = true;
        Item it;
        for (uint32_t k = 0; ok && fetch(k, it) == 1; ++k) {
          for (int t = 0; t < 2 && ok; ++t) {
            if (it.n_kv[t] == 0) continue;
            if (k > 0) {
              // the buffer's previous tile has been read by its last S MMA
              ok = mbar_wait(&q_empty[t], (q_uses[t] - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY);
              if (ok) load_q(t, it);
            }
            ++q_uses[t];
          }
          for (int j = 0; j < it.n_iter && ok; ++j, ++g)
            if (k > 0 || j > 0) ok = load_kv(g, j, it);
          mbar_arrive(&sched_empty[k & 1]);
        }
      }
    } else if (warp == 1) {
      // ------------------------------------------------------------ MMA issuer (one thread)
      if (lane == 0) {
        constexpr uint32_t IDESC_S = make_idesc(128, 128, false, false);
        constexpr uint32_t IDESC_PV = make_idesc(128, D, false, true);
        const uint32_t q_addr = smem_addr(smem + T::SMEM_Q);
        const uint32_t k_addr = smem_addr(smem + T::SMEM_K);
        const uint32_t v_addr = smem_addr(smem + T::SMEM_V);
        auto issue_s = [&](int t, int st) {   // S_t = Q_t * K_st^T, K-major operands
          const uint64_t dq = make_sdesc(q_addr + t * T::TILE_BYTES, 16, 1024);
          const uint64_t dk = make_sdesc(k_addr + st * T::TILE_BYTES, 16, 1024);
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * T::BLOCK_BYTES + (kk & 3) * 32;
            umma_ss(tmem_base + t * 128, sdesc_advance(dq, off), sdesc_advance(dk, off), IDESC_S, kk > 0);
          }
          umma_commit(&s_full[t]);
        };
        auto issue_pv = [&](int t, int st, bool first) {   // O_t += P_t * V_st, P from TMEM, V N-major
          const uint64_t dv = make_sdesc(v_addr + st * T::TILE_BYTES, T::BLOCK_BYTES, 1024);
#pragma unroll
          for (int kk = 0; kk < T::BN / 16; ++kk)
            umma_ts(tmem_base + 256 + t * D, tmem_base + t * 128 + kk * 8, sdesc_advance(dv, kk * 2048), IDESC_PV,
                    (!first || kk > 0) ? 1u : 0u);
        };
        bool ok = true;
        uint32_t g0 = 0;               // ring slot counter of the current item's key tile 0
        uint32_t q_uses[2] = {0, 0};   // items before the current one that had query tile t
        uint32_t pv_cnt[2] = {0, 0};   // P tiles consumed so far
        // S_t(0) of an item: issued behind the previous item's last P V (the tensor core runs its MMAs in issue
        // order, so S_t may overwrite the P_t that P V still reads), ahead of that item's epilogue.
        auto first_s = [&](const Item& it, uint32_t g) -> bool {
          const int st = static_cast<int>(g % T::STAGES);
          if (!mbar_wait(&k_full[st], (g / T::STAGES) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD)) return false;
          for (int t = 0; t < 2; ++t) {
            if (it.n_kv[t] == 0) continue;
            if (!mbar_wait(&q_full[t], q_uses[t] & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD)) return false;
            tc_fence_after();
            issue_s(t, st);
            if (it.n_kv[t] == 1) umma_commit(&q_empty[t]);
          }
          umma_commit(&k_empty[st]);
          return true;
        };
        Item it;
        bool have = fetch(0, it) == 1;
        if (have) ok = first_s(it, g0);
        for (uint32_t k = 0; have && ok; ++k) {
          for (int j = 0; j < it.n_iter && ok; ++j) {
            const uint32_t g = g0 + j;
            const int st = static_cast<int>(g % T::STAGES);
            const uint32_t ph = (g / T::STAGES) & 1;
            const int st_n = static_cast<int>((g + 1) % T::STAGES);
            const uint32_t ph_n = ((g + 1) / T::STAGES) & 1;
            const bool have_next = (j + 1 < it.n_iter);
            if (have_next) ok = mbar_wait(&k_full[st_n], ph_n, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
            if (!ok) break;
            ok = mbar_wait(&v_full[st], ph, abort_flag, prm.status, DEV_ERR_TIMEOUT_LOAD);
            if (!ok) break;
            for (int t = 0; t < 2; ++t) {
              if (j >= it.n_kv[t]) continue;
              ok = mbar_wait(&p_full[t], pv_cnt[t] & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_SOFTMAX);
              if (!ok) break;
              ++pv_cnt[t];
              tc_fence_after();
              issue_pv(t, st, j == 0);
              if (j == it.n_kv[t] - 1) umma_commit(&o_done[t]);
              if (j + 1 < it.n_kv[t]) {
                issue_s(t, st_n);
                if (j + 2 == it.n_kv[t]) umma_commit(&q_empty[t]);   // that was the item's last read of Q_t
              }
            }
            if (!ok) break;
            umma_commit(&v_empty[st]);
            if (have_next) umma_commit(&k_empty[st_n]);
          }
          if (!ok) break;
          g0 += it.n_iter;
          for (int t = 0; t < 2; ++t) q_uses[t] += (it.n_kv[t] > 0) ? 1u : 0u;
          mbar_arrive(&sched_empty[k & 1]);
          have = fetch(k + 1, it) == 1;
          if (have) ok = first_s(it, g0);
        }
      }
    } else if (warp == 3) {
      // ------------------------------------------------------------ work-item scheduler (one thread)
      if (lane == 0 && prm.work_counter != nullptr) {
        for (uint32_t n = 0;; ++n) {
          // the slot's previous item (n - 2) has been released by every role
          if (n >= 2 && !mbar_wait(&sched_empty[n & 1], ((n >> 1) - 1) & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_EMPTY)) break;
          int idx = static_cast<int>(blockIdx.x);
          if (n > 0) {
            idx = G + atomicAdd(prm.work_counter, 1);
            if (idx >= n_items) idx = -1;
          }
          sched_item[n & 1] = idx;
          mbar_arrive(&sched_full[n & 1]);
          if (idx < 0) break;
        }
      }
    }
  } else {
    setmaxnreg_inc<REGS_SOFTMAX>();
    // ------------------------------------------------------------ softmax + epilogue
    const int t = (warp - 4) >> 2;
    const int lane_base = (warp & 3) * 32;
    const uint32_t t_s = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + t * 128;
    const uint32_t t_o = tmem_base + (static_cast<uint32_t>(lane_base) << 16) + 256 + t * D;
    const float sl2 = prm.scale_log2;
    uint32_t s_seen = 0;   // S tiles of this group consumed so far
    uint32_t items = 0;    // items so far that had this group's query tile
    bool ok = !bad_start;
    Item it;
    for (uint32_t k = 0; ok; ++k) {
      const int got = fetch(k, it);
      if (__any_sync(0xffffffffu, got != 1)) break;
      const int nkv = it.n_kv[t];
      if (nkv == 0) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&sched_empty[k & 1]);
        continue;
      }
      const int qt = 2 * it.pair + t;
      const int q_row = qt * T::BM + lane_base + lane;
      const int k_limit = prm.causal ? min(S - 1, q_row) : (S - 1);   // last visible key index
      float m_used = -INFINITY;
      float l_sum = 0.f;
      uint32_t r[128];   // this thread's row of S
      for (int j = 0; j < nkv; ++j) {
        ok = mbar_wait(&s_full[t], s_seen & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ++s_seen;
        tc_fence_after();
        // the whole row in one go: four loads in flight, one wait
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_x32(t_s + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
        tmem_wait_ld();
        if ((prm.causal && j == qt) || ((j + 1) * T::BN > S)) {   // diagonal or ragged last tile
          const int vis = k_limit - j * T::BN;   // columns 0..vis are visible
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
        if (j == 0) {
          m_used = m_new;
        } else {
          const bool grow = m_new > m_used + 8.0f;
          if (__any_sync(0xffffffffu, grow)) {   // rare: raise the reference and rescale O in TMEM
            const float m_next = fmaxf(m_used, m_new);
            const float f = ex2(m_used - m_next);
            l_sum *= f;
            m_used = m_next;
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
        // P = 2^(s*scale - m), packed bf16, written over S 32 keys at a time
        const float neg_m = -m_used;
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
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
            pk[(i >> 1)] = pack_bf16(p0, p1);
            pk[(i >> 1) + 1] = pack_bf16(p2, p3);
          }
          tmem_st_x16(t_s + c * 16, pk);
        }
        l_sum += (l0 + l1) + (l2 + l3);
        tmem_wait_st();
        tc_fence_before();
        mbar_arrive(&p_full[t]);
      }
      if (ok) {
        ok = mbar_wait(&o_done[t], items & 1, abort_flag, prm.status, DEV_ERR_TIMEOUT_MMA);
        ok = __all_sync(0xffffffffu, ok);
      }
      if (!ok) break;
      ++items;
      // The next item's first P V overwrites O_t; it is issued after this group's next arrival on p_full, which
      // comes after these loads in program order.
      tc_fence_after();
      const float inv_l = 1.0f / l_sum;
      __nv_bfloat16* orow = prm.o + prm.st.slice(it.bh) + static_cast<long long>(q_row) * prm.st.row;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) tmem_ld_x32(t_o + c * 32, *reinterpret_cast<uint32_t(*)[32]>(&r[c * 32]));
      tmem_wait_ld();
      if (q_row < S) {
#pragma unroll
        for (int v = 0; v < D / 8; ++v) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(r[v * 8 + 0]) * inv_l, __uint_as_float(r[v * 8 + 1]) * inv_l);
          w.y = pack_bf16(__uint_as_float(r[v * 8 + 2]) * inv_l, __uint_as_float(r[v * 8 + 3]) * inv_l);
          w.z = pack_bf16(__uint_as_float(r[v * 8 + 4]) * inv_l, __uint_as_float(r[v * 8 + 5]) * inv_l);
          w.w = pack_bf16(__uint_as_float(r[v * 8 + 6]) * inv_l, __uint_as_float(r[v * 8 + 7]) * inv_l);
          *reinterpret_cast<uint4*>(orow + v * 8) = w;
        }
        if (prm.lse != nullptr)
          prm.lse[static_cast<size_t>(it.bh) * S + q_row] = (m_used + lg2(l_sum)) * 0.6931471805599453f;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&sched_empty[k & 1]);
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
