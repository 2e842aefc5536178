// Attention forward on the 5th-generation tensor cores for head_dim 64, bf16.
//
// Persistent kernel, one CTA per SM. A work item is a PAIR of adjacent 128-row query tiles (lo and
// hi) of one (batch, head); both tiles are multiplied against the same stream of 128-key K/V
// tiles, so every K/V byte staged in shared memory feeds two query tiles. The work of an item is a
// sequence of UNITS (query tile, key tile j): lo_0 hi_0 lo_1 hi_1 ... Two softmax GROUPS of four
// warps each own one query tile of the item (and swap tiles from item to item: under a causal
// mask the hi tile has one key tile more, and a fixed assignment would leave one group idle for
// a unit in every item). Per group g, tensor memory holds a 128-column score buffer S_g, a
// 64-column probability buffer P_g (bf16 pairs) and a 64-column output accumulator O_g:
// 2 * (128 + 64 + 64) = 512 columns.
//   warp 0      TMA producer: Q_lo and Q_hi of the item (double buffered, so the next item's
//               queries land while this one computes), then K_j / V_j into a 4-deep ring.
//   warps 1, 2  MMA issuers, one per softmax group (converged warp, one elected lane). For the
//               group's unit k: S_g = Q K_j^T as soon as the group has pulled the scores of unit
//               k - 1 out of S_g (s_free) -- that is at the START of the group's work on unit
//               k - 1, so the next scores are complete long before they are asked for; and
//               O_g (+)= P_g V_j with P_g read from TENSOR MEMORY as the A operand as soon as the
//               group has published P_g (p_full), committing pv_done (P_g free, O_g current). A
//               K/V ring slot or Q buffer is released when both warps have passed it.
//   warps 4-7   softmax group 0, warps 8-11 group 1 (warp 3 idle): ONE thread per query row, 128
//               scores per unit. Each thread pulls its row of S out of TMEM and releases the score
//               buffer, takes the row maximum, computes P = exp2(s * scale * log2 e - m) (packed
//               f32x2 FMA + ex2.approx), rounds P to bf16 and stores it into P_g with tcgen05.st --
//               no shared-memory round trip and no proxy fence between the softmax and the second
//               MMA. O is rescaled in TMEM lazily: the reference maximum follows the true maximum
//               only when it is more than 8 (a factor 256) behind, which in practice means during
//               the first tile only. The same threads divide by the row sum and write O and the
//               natural-log LSE; that epilogue is deferred into the first unit of the group's
//               next item, by which time the last P V has long finished.
// The two groups never wait for each other: every barrier of a group is a ping-pong between the
// group and its issuing warp. The kernel is bound by the MUFU pipe (one ex2 per score, 16 per clock and SM,
// against 8192 tensor flops per clock); the two softmax warps of an SM sub-partition keep it busy
// while each other loads scores and takes maxima.
// The 12 warps re-balance the register file with setmaxnreg: a thread that holds a 128-score row
// needs ~200 registers, the producer and issuer warps few.
//
// Work items are ordered for L2: (batch, head) pairs are taken in groups whose K and V together
// fit a fixed L2 budget, and inside a group the query-tile pairs are walked heaviest first (the
// causal mask makes late query tiles the longest). With one CTA per pair of a group, a CTA walks
// all the query tiles of "its" (batch, head) back to back and K/V are fetched from HBM once.
//
// Numerics: scores scaled by scale*log2(e), P = exp2(s - m), masked scores are -inf, P is rounded
// to bf16 before the second MMA, O is divided by the fp32 row sum once at the end, and the
// natural-log LSE is (m + log2(l)) * ln 2.
#include "ptx.cuh"
#include "sdpa_internal.cuh"
#include "tma.cuh"

#include <cstdlib>

namespace b200 {
namespace {

constexpr int BM = 128;   // query rows per tile; a work item has two tiles
constexpr int BN = 128;   // keys per tile
constexpr int D = 64;     // head_dim
constexpr int kStages = 4;
constexpr int kSoftmaxWarps = 8;  // four per group
constexpr int kThreads = 128 + kSoftmaxWarps * 32;  // warp group 0: TMA warp, two MMA warps, one idle warp
// Registers per thread after the warp groups re-balance the register file (setmaxnreg): the 12
// warps start with kRegsAtLaunch each (what __launch_bounds__(384, 1) gives); the producer/issuer
// group hands most of its share to the softmax groups. The CTA's register pool is what it was
// launched with, so the three groups together must not ask for more than 3 * kRegsAtLaunch: a
// request beyond the pool blocks for ever.
constexpr int kRegsAtLaunch = 168;
constexpr int kRegsControl = 72, kRegsSoftmax = 216;
static_assert(kRegsControl + 2 * kRegsSoftmax <= 3 * kRegsAtLaunch, "setmaxnreg requests exceed the CTA's register pool");
constexpr int TILE_BYTES = 128 * D * 2;  // 16 KiB: one Q, K or V tile
constexpr int kTmemCols = 512;
// tensor memory columns of group g: S at 128 g, P at 256 + 64 g, O at 384 + 64 g
constexpr int TMEM_S = 0, TMEM_P = 256, TMEM_O = 384;

constexpr int SMEM_Q = 0;                                // [2 buffers][tile lo, tile hi]
constexpr int SMEM_K = SMEM_Q + 4 * TILE_BYTES;
constexpr int SMEM_V = SMEM_K + kStages * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_V + kStages * TILE_BYTES;
// barriers: q_full[2], q_empty[2], kv_full[kStages], kv_empty[kStages], and per group s_full,
// s_free, p_full, pv_done
constexpr int kNumBars = 4 + 2 * kStages + 8;
constexpr int SMEM_MISC = SMEM_BAR + kNumBars * 8;
constexpr int SMEM_BYTES = SMEM_MISC + 16 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of one SM exceeded");

constexpr int64_t kL2GroupBytes = 48ll << 20;  // K+V bytes of one group of (batch, head) pairs

struct Params {
  __nv_bfloat16* o;
  float* lse;
  uint32_t heads;
  int32_t q_len, kv_len;
  int64_t os_b, os_h, os_t;
  float scale_log2;  // scale * log2(e)
  int causal;
  uint32_t q_pairs;    // pairs of query tiles per (batch, head)
  uint32_t bh;         // batch * heads
  uint32_t group;      // (batch, head) pairs per L2 group
  uint32_t num_items;  // q_pairs * bh
  int q_heads_inner, k_heads_inner, v_heads_inner;  // tensor map dim order is (d, head, pos, batch)
  unsigned int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

#ifdef B200_SDPA_PROBE
// Development build only: per-CTA cycle counters of the roles, read back by b200_debug_sdpa_probe.
__device__ unsigned long long g_probe[160][48];
#define PROBE_DECL(n) long long n = 0
#define PROBE_T0(t) const long long t = clock64()
#define PROBE_ADD(n, t) n += clock64() - t
#else
#define PROBE_DECL(n)
#define PROBE_T0(t)
#define PROBE_ADD(n, t)
#endif

// The issuing warps' long waits (for the softmax group to hand over S or P: most of a unit's time)
// back off between polls, so that the polling does not take issue slots from the softmax warps that
// share their SM sub-partitions.
#define ISSUER_WAIT ptx::mbar_wait_relaxed

struct Item {
  int32_t q0;      // first query row of tile A; tile B starts at q0 + BM
  int32_t b, h;
  int n_a, n_b;    // key tiles tile A / tile B attend to (n_b == 0: no tile B)
  int n;           // key tiles of the item: max(n_a, n_b)
};

__device__ __forceinline__ int key_tiles(int32_t q0, const Params& p) {
  int32_t last_key = p.kv_len;  // exclusive
  if (p.causal) {
    const int32_t lim = q0 + BM;  // rows q0..q0+127 see keys <= row
    if (lim < last_key) last_key = lim;
  }
  return (last_key + BN - 1) / BN;
}

// Work item w -> (query-tile pair, batch, head): groups of p.group (batch, head) pairs, inside a
// group the last (heaviest) query-tile pair of every member first. 32-bit arithmetic throughout
// (the host refuses problems whose item count does not fit): the issuing warps decode an item
// per cursor and 64-bit divisions there were a measurable share of their time.
__device__ __forceinline__ Item decode_item(uint32_t w, const Params& p) {
  Item it;
  const uint32_t per_group = p.group * p.q_pairs;
  const uint32_t g = w / per_group;
  const uint32_t r = w - g * per_group;
  const uint32_t first = g * p.group;
  const uint32_t members = (p.bh - first < p.group) ? p.bh - first : p.group;
  const uint32_t rq = r / members;
  const uint32_t bh = first + (r - rq * members);
  it.b = (int32_t)(bh / p.heads);
  it.h = (int32_t)(bh - (uint32_t)it.b * p.heads);
  it.q0 = (int32_t)(p.q_pairs - 1 - rq) * (2 * BM);
  it.n_a = key_tiles(it.q0, p);
  it.n_b = (it.q0 + BM < p.q_len) ? key_tiles(it.q0 + BM, p) : 0;
  it.n = it.n_a > it.n_b ? it.n_a : it.n_b;
  return it;
}

__global__ void __launch_bounds__(kThreads, 1)
sdpa_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t base = ptx::smem_u32(smem);
  const uint32_t q_smem = base + SMEM_Q, k_smem = base + SMEM_K, v_smem = base + SMEM_V;
  const uint32_t bar = base + SMEM_BAR;
  auto q_full = [&](int b) { return bar + 8u * b; };
  auto q_empty = [&](int b) { return bar + 8u * (2 + b); };
  auto kv_full = [&](int s) { return bar + 8u * (4 + s); };
  auto kv_empty = [&](int s) { return bar + 8u * (4 + kStages + s); };
  // Per softmax group g, each a strict ping-pong between the group and one issuing warp, so the
  // n-th use of a barrier is waited for with parity n & 1 and no waiter can fall a phase behind:
  auto s_full = [&](int g) { return bar + 8u * (4 + 2 * kStages + g); };       // scores of the group's next unit are in S_g
  auto s_free = [&](int g) { return bar + 8u * (4 + 2 * kStages + 2 + g); };   // the group has read S_g
  auto p_full = [&](int g) { return bar + 8u * (4 + 2 * kStages + 4 + g); };   // the group has written P_g
  auto pv_done = [&](int g) { return bar + 8u * (4 + 2 * kStages + 6 + g); };  // P_g V has completed: P_g free, O_g current
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + SMEM_MISC);
  volatile uint32_t* tmem_holder = misc;
  volatile uint32_t* abort_flag = misc + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(q_full(b), 1);
      ptx::mbar_init(q_empty(b), 2);  // both issuing warps have left the item
      ptx::mbar_init(s_full(b), 1);
      ptx::mbar_init(s_free(b), kSoftmaxWarps / 2);  // one arrival per warp of the group
      ptx::mbar_init(p_full(b), kSoftmaxWarps / 2);
      ptx::mbar_init(pv_done(b), 1);
    }
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(kv_full(s), 1);
      ptx::mbar_init(kv_empty(s), 2);  // both issuing warps have passed the key tile
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;

  // Each role re-sizes its register allocation at the top of its own branch (every warp of a warp
  // group executes the same request), so that the compiler allocates each branch for its own size.
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      uint32_t items = 0;
      bool ok = true;
      for (uint32_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++items) {
        const Item it = decode_item(w, p);
        const int qb = items & 1;
        // this Q buffer is free once the score MMAs of the item before the previous one have read it
        if (!ptx::mbar_wait_relaxed(q_empty(qb), ((items >> 1) & 1) ^ 1, abort_flag)) break;
        const uint32_t qa = q_smem + qb * 2 * TILE_BYTES;
        ptx::mbar_arrive_expect_tx(q_full(qb), (it.n_b > 0 ? 2 : 1) * TILE_BYTES);
        for (int x = 0; x < (it.n_b > 0 ? 2 : 1); ++x) {
          const int32_t q0 = it.q0 + x * BM;
          if (p.q_heads_inner) ptx::tma_load_4d(qa + x * TILE_BYTES, &tmap_q, q_full(qb), 0, it.h, q0, it.b);
          else ptx::tma_load_4d(qa + x * TILE_BYTES, &tmap_q, q_full(qb), 0, q0, it.h, it.b);
        }
        for (int j = 0; j < it.n; ++j) {
          const int32_t kv0 = j * BN;
          if (!ptx::mbar_wait_relaxed(kv_empty(s), phase ^ 1, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(kv_full(s), 2 * TILE_BYTES);  // K and V of the tile on one barrier
          if (p.k_heads_inner) ptx::tma_load_4d(k_smem + s * TILE_BYTES, &tmap_k, kv_full(s), 0, it.h, kv0, it.b);
          else ptx::tma_load_4d(k_smem + s * TILE_BYTES, &tmap_k, kv_full(s), 0, kv0, it.h, it.b);
          if (p.v_heads_inner) ptx::tma_load_4d(v_smem + s * TILE_BYTES, &tmap_v, kv_full(s), 0, it.h, kv0, it.b);
          else ptx::tma_load_4d(v_smem + s * TILE_BYTES, &tmap_v, kv_full(s), 0, kv0, it.h, it.b);
          if (++s == kStages) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issuers: warp 1 for softmax group 0, warp 2 for group 1 ----------------
    // Each warp walks the units of ITS group converged (addresses and descriptors are then
    // warp-uniform values) and one elected lane, the same on every election, issues the MMAs and
    // the commits that track them. Per unit k of the group the warp alternates between two
    // events that the group produces in this order: "scores of unit k read" (s_free) -> issue the
    // score MMA of unit k + 1; "P of unit k written" (p_full) -> issue P V of unit k. The two
    // groups' streams share nothing but the read-only Q and K/V tiles, so the warps never wait for
    // each other; a ring slot (a Q buffer) is released when BOTH warps have passed it.
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));
    const int g = warp - 1;
    const uint32_t bar_s_full = s_full(g), bar_s_free = s_free(g), bar_p_full = p_full(g), bar_pv_done = pv_done(g);
    struct Cursor {
      uint32_t w;       // work item
      Item it;
      int j;            // key tile
      int x, n_mine;    // the group's query tile in this item (0 = lo, 1 = hi) and its number of key tiles
      int slot;         // K/V ring slot of key tile j
      uint32_t phase;   // ring phase of that slot
      uint32_t items;   // items of this CTA before this one
      bool valid;
    };
    auto start_item = [&](Cursor& c) {
      c.valid = c.w < p.num_items;
      c.j = 0;
      if (c.valid) {
        c.it = decode_item(c.w, p);
        c.x = g ^ (int)(c.items & 1);  // the groups swap query tiles every item
        c.n_mine = c.x ? c.it.n_b : c.it.n_a;
      }
    };
    auto next_tile = [&](Cursor& c) {
      ++c.j;
      if (++c.slot == kStages) { c.slot = 0; c.phase ^= 1; }
      if (c.j < c.it.n) return;
      c.w += gridDim.x;
      ++c.items;
      start_item(c);
    };
    Cursor qk;
    qk.w = blockIdx.x; qk.slot = 0; qk.phase = 0; qk.items = 0;
    start_item(qk);
    Cursor pv = qk;
    uint32_t k_qk = 0, k_pv = 0;  // units of the group whose score MMA / P V has been issued
    constexpr uint32_t idesc_qk = ptx::idesc_bf16_f32(BM, BN, 0, 0);
    constexpr uint32_t idesc_pv = ptx::idesc_bf16_f32(BM, D, 0, 1);
    PROBE_DECL(c_wait_a); PROBE_DECL(c_wait_b); PROBE_DECL(c_issue); PROBE_DECL(c_wait_p); PROBE_DECL(c_issue_pv);
    PROBE_T0(t_mma_start);

    // Score MMA of the group's next unit: S_g = Q_x K_j^T. Key tiles the group's query tile does
    // not attend to are passed over; leaving an item releases its Q buffer.
    auto issue_next_qk = [&]() -> bool {
      while (qk.valid && qk.j >= qk.n_mine) {
        // An item in which the group has no query tile still takes part in releasing the Q buffer;
        // seeing the item's Q land first keeps this arrival inside the buffer's current round.
        if (qk.j == 0 && !__all_sync(0xffffffffu, ptx::mbar_wait(q_full(qk.items & 1), (qk.items >> 1) & 1, abort_flag)))
          return false;
        if (qk.j + 1 >= qk.it.n && ptx::elect_one()) ptx::tc_commit(q_empty(qk.items & 1));
        __syncwarp();
        next_tile(qk);
      }
      if (!qk.valid) return true;
      const int qb = qk.items & 1;
      PROBE_T0(t0);
      // the group must have pulled its previous scores out of S_g
      bool go = k_qk == 0 || ISSUER_WAIT(bar_s_free, (k_qk - 1) & 1, abort_flag);
      PROBE_ADD(c_wait_a, t0);
      PROBE_T0(t1);
      if (qk.j == 0) go = go && ptx::mbar_wait(q_full(qb), (qk.items >> 1) & 1, abort_flag);
      go = go && ptx::mbar_wait(kv_full(qk.slot), qk.phase, abort_flag);  // K and V of the tile
      if (!__all_sync(0xffffffffu, go)) return false;
      ptx::tc_fence_after_sync();
      PROBE_ADD(c_wait_b, t1);
      PROBE_T0(t2);
      const uint32_t d_tmem = tmem + TMEM_S + g * 128;
      const uint32_t qx = q_smem + (qb * 2 + qk.x) * TILE_BYTES;
      const uint32_t kb = k_smem + qk.slot * TILE_BYTES;
      if (ptx::elect_one()) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint64_t a_desc = ptx::smem_desc_sw128(qx + kk * 32, 0, 1024);
          const uint64_t b_desc = ptx::smem_desc_sw128(kb + kk * 32, 0, 1024);
          ptx::mma_f16_ss(d_tmem, a_desc, b_desc, idesc_qk, kk > 0 ? 1u : 0u);
        }
        ptx::tc_commit(bar_s_full);
        if (qk.j + 1 >= qk.it.n) ptx::tc_commit(q_empty(qb));  // last key tile of the item
      }
      __syncwarp();
      PROBE_ADD(c_issue, t2);
      ++k_qk;
      next_tile(qk);
      return true;
    };

    bool ok = issue_next_qk();
    while (ok && pv.valid) {
      if (pv.j < pv.n_mine) {
        // scores of unit k + 1 first (the group released S_g at the start of unit k), then P V of unit k
        if (!issue_next_qk()) break;
        PROBE_T0(t0);
        if (!__all_sync(0xffffffffu, ISSUER_WAIT(bar_p_full, k_pv & 1, abort_flag))) break;
        ptx::tc_fence_after_sync();
        PROBE_ADD(c_wait_p, t0);
        PROBE_T0(t2);
        // O_g (+)= P_g V_j: eight k-steps of 16 keys; P_g holds two bf16 per column, V is [keys][d]
        // with d contiguous: MN-major B, 16 keys = two 8-row groups of 1 KiB
        const uint32_t d_tmem = tmem + TMEM_O + g * 64;
        const uint32_t a_tmem = tmem + TMEM_P + g * 64;
        const uint32_t vb = v_smem + pv.slot * TILE_BYTES;  // landed together with K, which fed this unit's scores
        if (ptx::elect_one()) {
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            const uint64_t b_desc = ptx::smem_desc_sw128(vb + kk * 2048, 0, 1024);
            ptx::mma_f16_ts(d_tmem, a_tmem + kk * 8, b_desc, idesc_pv, (pv.j > 0 || kk > 0) ? 1u : 0u);
          }
          ptx::tc_commit(bar_pv_done);
          ptx::tc_commit(kv_empty(pv.slot));  // this group is done with K_j and V_j
        }
        __syncwarp();
        PROBE_ADD(c_issue_pv, t2);
        ++k_pv;
      } else {
        // A key tile only the other group's query tile attends to: this warp still takes part in
        // releasing the ring slot; seeing the tile land first keeps the arrival inside the slot's
        // current round however far this warp runs ahead of the other.
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(kv_full(pv.slot), pv.phase, abort_flag))) break;
        if (ptx::elect_one()) ptx::tc_commit(kv_empty(pv.slot));
        __syncwarp();
      }
      next_tile(pv);
    }
#ifdef B200_SDPA_PROBE
    if (lane == 0) {
      unsigned long long* o = g_probe[blockIdx.x] + 16 * g;
      o[0] = clock64() - t_mma_start; o[1] = k_pv; o[2] = c_wait_a; o[3] = c_wait_b; o[4] = c_issue; o[5] = c_wait_p; o[6] = c_issue_pv;
    }
#endif
  } else if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsControl));  // idle warp of group 0
  } else {
    // ---------------- softmax + output: warps 4-7 group 0, warps 8-11 group 1 ----------------
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsSoftmax));
    const int grp = (warp - 4) >> 2;
    const int quad = warp & 3;               // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;          // row inside the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t s_addr = tmem + TMEM_S + grp * 128 + lane_addr;
    const uint32_t p_addr = tmem + TMEM_P + grp * 64 + lane_addr;
    const uint32_t o_addr = tmem + TMEM_O + grp * 64 + lane_addr;
    const uint32_t bar_s_full = s_full(grp), bar_s_free = s_free(grp), bar_p_full = p_full(grp), bar_pv_done = pv_done(grp);
    const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
    uint32_t k = 0;       // units this group has processed
    uint32_t items = 0;   // items of this CTA before the current one
    bool ok = true;
    // Epilogue of the previous item, deferred (see below).
    bool pending = false;
    float pend_l = 0.0f, pend_m = 0.0f;
    __nv_bfloat16* pend_o = nullptr;  // this row's output, nullptr for rows past q_len
    float* pend_lse = nullptr;
    PROBE_DECL(c_wait_s); PROBE_DECL(c_ld); PROBE_DECL(c_max); PROBE_DECL(c_exp); PROBE_DECL(c_pub); PROBE_DECL(c_epi);
    PROBE_DECL(c_wait_pv);
    PROBE_T0(t_sm_start);

    // O / l and the LSE of this row for the pending item; its last P V has been waited for.
    auto epilogue = [&]() {
      const float inv = 1.0f / pend_l;  // l == 0 (no visible key) gives NaN like torch
#pragma unroll
      for (int hcol = 0; hcol < 2; ++hcol) {
        uint32_t o[32];
        ptx::tmem_ld_32x32b_x32(o_addr + hcol * 32, o);
        ptx::tmem_ld_wait();
        if (pend_o != nullptr) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 t;
            t.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
            t.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
            t.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
            t.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
            reinterpret_cast<uint4*>(pend_o)[hcol * 4 + c] = t;
          }
        }
      }
      if (pend_lse != nullptr) *pend_lse = (pend_m + log2f(pend_l)) * 0.6931471805599453f;
      pending = false;
    };

    for (uint32_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++items) {
      const Item it = decode_item(w, p);
      const int x = grp ^ (int)(items & 1);  // the groups swap query tiles every item
      const int n_mine = x ? it.n_b : it.n_a;
      if (n_mine == 0) continue;
      const int32_t q0 = it.q0 + x * BM;
      const int32_t row = q0 + r;
      float m_ref = -INFINITY;  // maximum this row's P and O are relative to (log2 domain)
      float l = 0.0f;
      for (int j = 0; j < n_mine; ++j, ++k) {
        // wait results are made warp-uniform: the TMEM loads and votes below need the whole warp
        PROBE_T0(t0);
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar_s_full, k & 1, abort_flag))) { ok = false; break; }
        ptx::tc_fence_after_sync();
        PROBE_ADD(c_wait_s, t0);
        PROBE_T0(t1);
        uint32_t s[BN];
#pragma unroll
        for (int c = 0; c < BN / 32; ++c)
          ptx::tmem_ld_32x32b_x32(s_addr + c * 32, reinterpret_cast<uint32_t(&)[32]>(s[c * 32]));
        ptx::tmem_ld_wait();
        // the scores are in registers: the score buffer can take the group's next unit right away
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_s_free);
        PROBE_ADD(c_ld, t1);
        PROBE_T0(t2);

        const int32_t kv0 = j * BN;
        const bool need_mask = (p.causal && kv0 + BN - 1 > q0) || (kv0 + BN > p.kv_len);
        if (need_mask) {
          int32_t lim = p.kv_len - kv0;  // keys [kv0, kv0 + lim) of the tile are visible to this row
          if (p.causal && row - kv0 + 1 < lim) lim = row - kv0 + 1;
          const int visible = lim < 0 ? 0 : (lim > BN ? BN : lim);
#pragma unroll
          for (int c = 0; c < BN; ++c)
            if (c >= visible) s[c] = 0xff800000u;  // -inf
        }
        // maximum of the raw scores, four independent chains of three-input max (scale > 0, so the
        // scaled maximum is the maximum scaled)
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < BN; c += 8) {
#pragma unroll
          for (int u4 = 0; u4 < 4; ++u4)
            mx[u4] = ptx::max3(mx[u4], __uint_as_float(s[c + 2 * u4]), __uint_as_float(s[c + 2 * u4 + 1]));
        }
        const float tile_max = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3])) * p.scale_log2;
        // lazy rescale: follow the true maximum only when it ran away by more than 2^8
        float alpha = 1.0f;
        if (tile_max > m_ref + 8.0f) {
          alpha = ex2(m_ref - tile_max);  // m_ref == -inf so far: alpha = 0
          m_ref = tile_max;
          l *= alpha;
        }
        const float neg_m = (m_ref == -INFINITY) ? 0.0f : -m_ref;
        const float2 negm2 = make_float2(neg_m, neg_m);
        PROBE_ADD(c_max, t2);
        float2 sum2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for (int q = 0; q < BN / 32; ++q) {
          PROBE_T0(t3);
          uint32_t packed[16];
#pragma unroll
          for (int c = 0; c < 32; c += 2) {
            // p = exp2(s * scale * log2e - m): one packed FMA for two scores, then two MUFU ops
            const float2 s2 = make_float2(__uint_as_float(s[q * 32 + c]), __uint_as_float(s[q * 32 + c + 1]));
            const float2 e2 = __ffma2_rn(s2, scale2, negm2);
            const float2 p2 = make_float2(ex2(e2.x), ex2(e2.y));
            sum2[(c >> 1) & 1] = __fadd2_rn(sum2[(c >> 1) & 1], p2);
            packed[c >> 1] = pack_bf16x2(p2.x, p2.y);
          }
          PROBE_ADD(c_exp, t3);
          if (q == 0 && k > 0) {
            // Before the first store into P_g: the group's previous P V must have completed (it
            // reads P_g and, for the epilogue and the rescale below, it must have landed in O_g).
            // It was published a quarter of a unit of softmax work ago, so this rarely waits.
            PROBE_T0(t4);
            if (!__all_sync(0xffffffffu, ptx::mbar_wait(bar_pv_done, (k - 1) & 1, abort_flag))) { ok = false; break; }
            ptx::tc_fence_after_sync();
            PROBE_ADD(c_wait_pv, t4);
            // The previous item's epilogue runs here, inside the first unit of this item: its
            // last P V has had time to finish, and O_g cannot be overwritten before it has been
            // read because the P V that restarts it needs the P published below.
            if (pending) {
              PROBE_T0(t5);
              epilogue();
              PROBE_ADD(c_epi, t5);
            }
            // this row's accumulator is rescaled in place (rare)
            if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll
              for (int hcol = 0; hcol < 2; ++hcol) {
                uint32_t o[32];
                ptx::tmem_ld_32x32b_x32(o_addr + hcol * 32, o);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
                ptx::tmem_st_32x32b_x32(o_addr + hcol * 32, o);
              }
            }
          }
          // keys 32q .. 32q+31 of this row: columns 16q .. 16q+15 of the A operand
          ptx::tmem_st_32x32b_x16(p_addr + q * 16, packed);
        }
        if (!ok) break;
        l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);
        PROBE_T0(t6);
        ptx::tmem_st_wait();
        // orders the TMEM stores (and the epilogue's loads) before the arrival
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(bar_p_full);
        PROBE_ADD(c_pub, t6);
      }
      if (!ok) break;
      pending = true;
      pend_l = l;
      pend_m = m_ref;
      const bool live = row < p.q_len;
      pend_o = live ? p.o + (int64_t)it.b * p.os_b + (int64_t)it.h * p.os_h + (int64_t)row * p.os_t : nullptr;
      pend_lse = (live && p.lse != nullptr) ? p.lse + ((int64_t)it.b * p.heads + it.h) * (int64_t)p.q_len + row : nullptr;
    }
    if (ok && pending) {
      // k >= 1 here; the last P V of the last item
      if (__all_sync(0xffffffffu, ptx::mbar_wait(bar_pv_done, (k - 1) & 1, abort_flag))) {
        ptx::tc_fence_after_sync();
        epilogue();
      }
    }
#ifdef B200_SDPA_PROBE
    if (lane == 0 && quad == 0) {
      unsigned long long* o = g_probe[blockIdx.x] + 32 + 8 * grp;
      o[0] = clock64() - t_sm_start; o[1] = c_wait_s; o[2] = c_ld; o[3] = c_max; o[4] = c_exp; o[5] = c_pub; o[6] = c_epi; o[7] = c_wait_pv;
    }
#endif
  }

  // ---------------- teardown ----------------
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0) atomicOr(p.status, STATUS_SDPA_TIMEOUT);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    ptx::tmem_dealloc(tmem, kTmemCols);
  }
}

// Byte strides of the (position, head, batch) dims with legal stand-ins for size-1 dims.
void byte_strides(const int64_t* s, int64_t batch, int64_t heads, int64_t len, uint64_t* st, uint64_t* sh,
                  uint64_t* sb) {
  *st = (uint64_t)(len > 1 ? s[2] : D) * 2;
  *sh = heads > 1 ? (uint64_t)s[1] * 2 : *st * (uint64_t)(len > 0 ? len : 1);
  const uint64_t big = (*st * (uint64_t)len > *sh * (uint64_t)heads) ? *st * (uint64_t)len : *sh * (uint64_t)heads;
  *sb = batch > 1 ? (uint64_t)s[0] * 2 : big;
}

// Tensor map over [batch, heads, len, 64] with boxes of 128 positions. Dims are listed innermost
// first with ascending strides: (d, pos, head, batch) for a [B, H, T, D]-contiguous tensor,
// (d, head, pos, batch) for views of a [B, T, H*D] projection. *heads_inner tells the kernel which
// coordinate order to use.
int32_t make_map(CUtensorMap* map, const void* ptr, int64_t batch, int64_t heads, int64_t len,
                 const int64_t* strides, int* heads_inner) {
  uint64_t st, sh, sb;
  byte_strides(strides, batch, heads, len, &st, &sh, &sb);
  *heads_inner = sh < st ? 1 : 0;
  if (*heads_inner) {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)len, (uint64_t)batch};
    const uint64_t str[3] = {sh, st, sb};
    const uint32_t box[4] = {(uint32_t)D, 1, 128, 1};
    return encode_tensor_map(map, B200_BF16, 4, ptr, dims, str, box, true);
  }
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)len, (uint64_t)heads, (uint64_t)batch};
  const uint64_t str[3] = {st, sh, sb};
  const uint32_t box[4] = {(uint32_t)D, 128, 1, 1};
  return encode_tensor_map(map, B200_BF16, 4, ptr, dims, str, box, true);
}

bool strides_ok(const int64_t* s, int64_t batch, int64_t heads, int64_t len) {
  if (len > 1 && (s[2] % 8 != 0 || s[2] < D)) return false;
  if (heads > 1 && (s[1] % 8 != 0 || s[1] < D)) return false;
  if (batch > 1 && (s[0] % 8 != 0 || s[0] < D)) return false;
  uint64_t st, sh, sb;
  byte_strides(s, batch, heads, len, &st, &sh, &sb);
  if (sb < st || sb < sh) return false;  // batch must be the outermost dim
  return true;
}

}  // namespace

const char* sdpa_tcgen05_ineligible(const b200_sdpa_args& a) {
  if (a.dtype != B200_BF16) return "tensors are not bf16";
  if (a.head_dim != D) return "head_dim is not 64";
  if (a.kv_len == 0) return "kv_len is zero";
  if (!(a.scale > 0.0f)) return "scale is not positive";
  if (!aligned_to(a.q, 16) || !aligned_to(a.k, 16) || !aligned_to(a.v, 16) || !aligned_to(a.o, 16))
    return "pointer not 16-byte aligned";
  if (!strides_ok(a.q_strides, a.batch, a.heads, a.q_len) || !strides_ok(a.k_strides, a.batch, a.heads, a.kv_len) ||
      !strides_ok(a.v_strides, a.batch, a.heads, a.kv_len))
    return "stride not a multiple of 16 bytes";
  if (a.o_strides[2] % 8 != 0 || a.o_strides[1] % 8 != 0 || a.o_strides[0] % 8 != 0)
    return "output stride not a multiple of 16 bytes";
  if (a.q_len > INT32_MAX - 512 || a.kv_len > INT32_MAX - 512) return "sequence too long";
  if (a.batch * a.heads > (1ll << 30) || (a.batch * a.heads) * ((a.q_len + 255) / 256) > (1ll << 30))
    return "too many (batch, head, query tile) work items";
  return nullptr;
}

int32_t launch_sdpa_tcgen05(const b200_sdpa_args& a, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  Params p;
  int32_t st = make_map(&mq, a.q, a.batch, a.heads, a.q_len, a.q_strides, &p.q_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mk, a.k, a.batch, a.heads, a.kv_len, a.k_strides, &p.k_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mv, a.v, a.batch, a.heads, a.kv_len, a.v_strides, &p.v_heads_inner);
  if (st != B200_OK) return st;

  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.lse = a.lse;
  p.heads = (uint32_t)a.heads; p.q_len = (int32_t)a.q_len; p.kv_len = (int32_t)a.kv_len;
  p.os_b = a.o_strides[0]; p.os_h = a.o_strides[1]; p.os_t = a.o_strides[2];
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.causal = a.causal;
  p.q_pairs = (uint32_t)((a.q_len + 2 * BM - 1) / (2 * BM));
  p.bh = (uint32_t)(a.batch * a.heads);
  p.num_items = p.q_pairs * p.bh;  // fits: checked by sdpa_tcgen05_ineligible
  p.status = device_status_ptr();
  B200_REQUIRE(p.status != nullptr, B200_ERR_CUDA, "sdpa(tcgen05): device status word unavailable");

  static thread_local bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(sdpa_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "sdpa(tcgen05): cannot opt in to %d bytes of shared memory: %s", SMEM_BYTES,
                cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int64_t slots = sm_count();  // one resident CTA per SM
  const int64_t grid = (int64_t)p.num_items < slots ? (int64_t)p.num_items : slots;
  // (batch, head) pairs per L2 group: as many as keep a group's K and V inside the budget, a whole
  // number of "one pair per CTA" rounds when there are that many
  const int64_t kv_bytes = 2 * a.kv_len * D * 2;
  int64_t group = kL2GroupBytes / (kv_bytes > 0 ? kv_bytes : 1);
  if (group < 1) group = 1;
  if (group >= (int64_t)p.bh) group = p.bh;
  else if (group >= grid) group = group / grid * grid;
  p.group = (uint32_t)group;
  sdpa_tcgen05_kernel<<<(unsigned)grid, kThreads, SMEM_BYTES, stream>>>(mq, mk, mv, p);
  B200_CHECK_LAUNCH("sdpa(tcgen05)");
  return B200_OK;
}

#ifdef B200_SDPA_PROBE
extern "C" B200_API int32_t b200_debug_sdpa_probe(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_probe, sizeof(g_probe)) == cudaSuccess ? 0 : -5;
}
#endif

}  // namespace b200
