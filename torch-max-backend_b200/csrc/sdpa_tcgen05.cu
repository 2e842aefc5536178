// Attention forward on the 5th-generation tensor cores for head_dim 64, bf16.
//
// Persistent kernel: two CTAs per SM, each looping over work items (128 query rows of one
// (batch, head)), heaviest items first. Inside a CTA:
//   warp 0      TMA producer: Q of the item, then its K_j / V_j tiles (64 keys) into two 3-deep
//               rings (128-byte swizzle). The rings keep streaming across item boundaries.
//   warp 1      MMA issuer: S = Q K_j^T into one of two TMEM score buffers and O += P_j V_j into
//               the TMEM output accumulators. The score stream runs one tile ahead of the P V
//               stream, also across item boundaries. Every barrier wait and every MMA/commit
//               costs this one thread a few hundred cycles, so the protocol is kept minimal: one
//               "K and V landed" barrier per ring slot, and buffer reuse is implied by program
//               order (a commit covers every MMA issued before it) instead of extra barriers.
//   warps 2-9   softmax, two threads per query row: the "a" thread (warps 2-5) owns keys 0-31 of
//               every tile, the "b" thread (warps 6-9) keys 32-63. Each runs its own online
//               softmax (exp2 domain, fp32 running maximum and sum) and owns its own output
//               accumulator in TMEM (O_a += P[:, :32] V[:32], O_b += P[:, 32:] V[32:]), so the
//               two never synchronise inside the key loop; the a thread merges the two partial
//               results once per item: O = (O_a 2^(m_a-m) + O_b 2^(m_b-m)) / (l_a 2^(m_a-m) +
//               l_b 2^(m_b-m)). P (rounded to bf16) goes into one of two shared-memory buffers as
//               the K-major A operand of the second MMA, so the softmax of tile j+1 does not wait
//               for P_j V_j. O is rescaled in TMEM lazily: the reference maximum only follows the
//               true maximum when it is more than 8 (a factor 256) behind, which keeps P inside
//               bf16/fp32 range and skips most TMEM round trips.
// Two CTAs fit on one SM (97 KB of shared memory and 256 TMEM columns each): 16 softmax warps per
// SM hide each other's dependency stalls, and one CTA's MMAs run under the other's softmax.
//
// Numerics: scores scaled by scale*log2(e), P = exp2(s - m), masked scores are -inf, P is rounded
// to bf16 before the second MMA, O is divided by the fp32 row sum once at the end, and the
// natural-log LSE is (m + log2(l)) * ln 2.
#include "ptx.cuh"
#include "sdpa_internal.cuh"
#include "tma.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;   // query rows per work item
constexpr int BN = 64;    // keys per tile
constexpr int D = 64;     // head_dim
constexpr int kStages = 3;
constexpr int kSoftmaxWarps = 8;
constexpr int kThreads = 64 + kSoftmaxWarps * 32;
constexpr int Q_BYTES = BM * D * 2;     // 16 KiB
constexpr int KV_BYTES = BN * D * 2;    // 8 KiB
constexpr int P_BYTES = BM * BN * 2;    // 16 KiB
constexpr int kTmemCols = 256;
constexpr int TMEM_S0 = 0, TMEM_S1 = 64, TMEM_OA = 128, TMEM_OB = 192;

constexpr int SMEM_Q = 0;
constexpr int SMEM_K = SMEM_Q + Q_BYTES;
constexpr int SMEM_V = SMEM_K + kStages * KV_BYTES;
constexpr int SMEM_P = SMEM_V + kStages * KV_BYTES;
constexpr int SMEM_STATS = SMEM_P + 2 * P_BYTES;  // (m_b, l_b) per row, handed from b to a threads
constexpr int SMEM_BAR = SMEM_STATS + BM * 8;
// barriers: q_full, q_empty, kv_full[3], kv_empty[3], (6 unused), s_full[2], (2 unused),
//           p_full[2], pv_done[2], stat_full, stat_empty
constexpr int kNumBars = 2 + 4 * kStages + 8 + 2;
constexpr int SMEM_MISC = SMEM_BAR + kNumBars * 8;
constexpr int SMEM_BYTES = SMEM_MISC + 16 + 1024;

struct Params {
  __nv_bfloat16* o;
  float* lse;
  int64_t heads, q_len, kv_len;
  int64_t os_b, os_h, os_t;
  float scale_log2;  // scale * log2(e)
  int causal;
  int q_tiles;
  int64_t bh;          // batch * heads
  int64_t num_items;   // q_tiles * bh
  int q_heads_inner, k_heads_inner, v_heads_inner;  // tensor map dim order is (d, head, pos, batch)
  unsigned int* status;
};

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Work item -> (query tile, batch, head). Items are ordered heaviest first: all (batch, head)
// pairs of the last query tile, then of the one before, ...
struct Item {
  int64_t q0;
  int32_t b, h;
  int n_tiles;
};

__device__ __forceinline__ Item decode_item(int64_t w, const Params& p) {
  Item it;
  const int q_tile = p.q_tiles - 1 - (int)(w / p.bh);
  const int64_t bh = w % p.bh;
  it.b = (int32_t)(bh / p.heads);
  it.h = (int32_t)(bh % p.heads);
  it.q0 = (int64_t)q_tile * BM;
  int64_t last_key = p.kv_len;  // exclusive
  if (p.causal) {
    const int64_t lim = it.q0 + BM;  // rows q0..q0+127 see keys <= row
    if (lim < last_key) last_key = lim;
  }
  it.n_tiles = (int)((last_key + BN - 1) / BN);
  return it;
}

__global__ void __launch_bounds__(kThreads, 2)
sdpa_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                    const __grid_constant__ CUtensorMap tmap_v, Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t base = ptx::smem_u32(smem);
  const uint32_t q_smem = base + SMEM_Q, k_smem = base + SMEM_K, v_smem = base + SMEM_V, p_smem = base + SMEM_P;
  const uint32_t bar = base + SMEM_BAR;
  const uint32_t q_full = bar, q_empty = bar + 8;
  auto kv_full = [&](int s) { return bar + 8u * (2 + s); };
  auto kv_empty = [&](int s) { return bar + 8u * (2 + kStages + s); };
  auto s_full = [&](int b) { return bar + 8u * (2 + 4 * kStages + b); };
  auto p_full = [&](int b) { return bar + 8u * (2 + 4 * kStages + 4 + b); };
  auto pv_done = [&](int b) { return bar + 8u * (2 + 4 * kStages + 6 + b); };
  const uint32_t stat_full = bar + 8u * (2 + 4 * kStages + 8), stat_empty = bar + 8u * (2 + 4 * kStages + 9);
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + SMEM_MISC);
  volatile uint32_t* tmem_holder = misc;
  volatile uint32_t* abort_flag = misc + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    ptx::mbar_init(q_full, 1);
    ptx::mbar_init(q_empty, 1);
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(kv_full(s), 1);
      ptx::mbar_init(kv_empty(s), 1);
    }
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(s_full(i), 1);
      // one arrival per softmax warp (lane 0 after a warp sync): 128 single-thread arrivals on
      // one barrier serialise in shared memory and were a large part of the per-tile latency
      ptx::mbar_init(p_full(i), kSoftmaxWarps);
      ptx::mbar_init(pv_done(i), 1);
    }
    ptx::mbar_init(stat_full, kSoftmaxWarps / 2);
    ptx::mbar_init(stat_empty, kSoftmaxWarps / 2);
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

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      uint32_t item_count = 0;
      bool ok = true;
      for (int64_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++item_count) {
        const Item it = decode_item(w, p);
        // Q buffer is free once the previous item's last score MMA has read it
        if (!ptx::mbar_wait_relaxed(q_empty, (item_count & 1) ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(q_full, Q_BYTES);
        if (p.q_heads_inner) ptx::tma_load_4d(q_smem, &tmap_q, q_full, 0, it.h, (int32_t)it.q0, it.b);
        else ptx::tma_load_4d(q_smem, &tmap_q, q_full, 0, (int32_t)it.q0, it.h, it.b);
        for (int j = 0; j < it.n_tiles; ++j) {
          const int32_t kv0 = j * BN;
          if (!ptx::mbar_wait_relaxed(kv_empty(s), phase ^ 1, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(kv_full(s), 2 * KV_BYTES);  // K and V of the tile on one barrier
          if (p.k_heads_inner) ptx::tma_load_4d(k_smem + s * KV_BYTES, &tmap_k, kv_full(s), 0, it.h, kv0, it.b);
          else ptx::tma_load_4d(k_smem + s * KV_BYTES, &tmap_k, kv_full(s), 0, kv0, it.h, it.b);
          if (p.v_heads_inner) ptx::tma_load_4d(v_smem + s * KV_BYTES, &tmap_v, kv_full(s), 0, it.h, kv0, it.b);
          else ptx::tma_load_4d(v_smem + s * KV_BYTES, &tmap_v, kv_full(s), 0, kv0, it.h, it.b);
          if (++s == kStages) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop converged (addresses and descriptors are then warp-uniform
    // values) and one elected lane, the same on every election, issues the MMAs and the commits
    // that track them.
    {
      constexpr uint32_t idesc_qk = ptx::idesc_bf16_f32(BM, BN, 0, 0);
      constexpr uint32_t idesc_pv = ptx::idesc_bf16_f32(BM, D, 0, 1);
      // Two cursors over the same sequence of (item, tile) pairs: the score stream (qk_*) runs
      // one tile ahead of the P V stream (pv_*). g counts tiles over the CTA's whole life; tile g
      // uses score buffer g & 1, P buffer g & 1 and K/V ring slot g % kStages.
      //
      // Reuse without extra barriers, from the issuing lane's program order
      //   ... PV(g-2), QK(g), wait p_full(g-1), PV(g-1), QK(g+1), ...
      //  * score buffer of QK(g+1) held S(g-1): p_full(g-1) was waited for just before, and the
      //    softmax warps publish P only after pulling S out of TMEM;
      //  * P buffer g & 1 is rewritten by the softmax of tile g after it has seen s_full(g); that
      //    commit was issued after PV(g-2), and a commit covers every MMA issued before it.
      int64_t qk_w = blockIdx.x, pv_w = blockIdx.x;
      int qk_j = 0, pv_j = 0;
      int qk_n = qk_w < p.num_items ? decode_item(qk_w, p).n_tiles : 0;
      int pv_n = qk_n;
      uint32_t qk_g = 0, pv_g = 0, qk_items = 0;
      int qk_slot = 0, pv_slot = 0;
      uint32_t qk_phase = 0;
      bool ok = true;

      auto issue_qk = [&]() -> bool {
        bool landed = true;
        if (qk_j == 0) landed = ptx::mbar_wait(q_full, qk_items & 1, abort_flag);
        landed = landed && ptx::mbar_wait(kv_full(qk_slot), qk_phase, abort_flag);  // K and V of the tile
        if (!__all_sync(0xffffffffu, landed)) return false;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem + ((qk_g & 1) ? TMEM_S1 : TMEM_S0);
        const uint32_t kb = k_smem + qk_slot * KV_BYTES;
        const bool last_of_item = qk_j + 1 == qk_n;
        if (ptx::elect_one()) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint64_t a_desc = ptx::smem_desc_sw128(q_smem + k * 32, 0, 1024);
            const uint64_t b_desc = ptx::smem_desc_sw128(kb + k * 32, 0, 1024);
            ptx::mma_f16_ss(d_tmem, a_desc, b_desc, idesc_qk, k > 0 ? 1u : 0u);
          }
          ptx::tc_commit(s_full(qk_g & 1));
          if (last_of_item) ptx::tc_commit(q_empty);  // last score MMA of the item: Q may be overwritten
        }
        __syncwarp();
        if (++qk_slot == kStages) { qk_slot = 0; qk_phase ^= 1; }
        ++qk_g;
        if (last_of_item) {
          ++qk_items;
          qk_j = 0;
          qk_w += gridDim.x;
          qk_n = qk_w < p.num_items ? decode_item(qk_w, p).n_tiles : 0;
        } else {
          ++qk_j;
        }
        return true;
      };

      if (qk_n > 0) ok = issue_qk();
      while (ok && pv_w < p.num_items) {
        if (qk_w < p.num_items) {
          ok = issue_qk();
          if (!ok) break;
        }
        const int pbuf = pv_g & 1;
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(p_full(pbuf), (pv_g >> 1) & 1, abort_flag))) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t vb = v_smem + pv_slot * KV_BYTES;  // landed together with K (seen at QK time)
        const uint32_t pb = p_smem + pbuf * P_BYTES;
        if (ptx::elect_one()) {
#pragma unroll
          for (int k = 0; k < BN / 16; ++k) {
            const uint64_t a_desc = ptx::smem_desc_sw128(pb + k * 32, 0, 1024);
            // V tile is [keys][d] with d contiguous: MN-major B, 16 keys = two 8-row groups of 1 KiB
            const uint64_t b_desc = ptx::smem_desc_sw128(vb + k * 2048, 0, 1024);
            // keys 0-31 accumulate into O_a, keys 32-63 into O_b (independent softmax streams)
            const int first = (k == 0 || k == 2);
            ptx::mma_f16_ss(tmem + (k < 2 ? TMEM_OA : TMEM_OB), a_desc, b_desc, idesc_pv,
                            (pv_j > 0 || !first) ? 1u : 0u);
          }
          ptx::tc_commit(kv_empty(pv_slot));  // frees K and V of the tile
          ptx::tc_commit(pv_done(pbuf));
        }
        __syncwarp();
        if (++pv_slot == kStages) pv_slot = 0;
        ++pv_g;
        if (++pv_j == pv_n) {
          pv_j = 0;
          pv_w += gridDim.x;
          pv_n = pv_w < p.num_items ? decode_item(pv_w, p).n_tiles : 0;
        }
      }
    }
  } else {
    // ---------------- softmax + output (warps 2..9), two threads per query row ----------------
    const int quad = warp & 3;
    const int hf = (warp - 2) >> 2;          // 0: keys 0-31 of every tile ("a"), 1: keys 32-63 ("b")
    const int r = quad * 32 + lane;          // row inside the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    const uint32_t o_mine = tmem + (hf ? TMEM_OB : TMEM_OA) + lane_addr;
    float* stats = reinterpret_cast<float*>(smem + SMEM_STATS);
    uint32_t g = 0;      // tiles processed by this CTA so far
    uint32_t items = 0;  // items processed by this CTA so far
    bool ok = true;
    for (int64_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++items) {
      const Item it = decode_item(w, p);
      const int64_t row = it.q0 + r;
      float m_ref = -INFINITY;  // maximum this thread's P / O are relative to (log2 domain)
      float l = 0.0f;
      for (int j = 0; j < it.n_tiles; ++j, ++g) {
        const int buf = g & 1;
        // wait results are made warp-uniform: the TMEM loads and votes below need the whole warp
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(s_full(buf), (g >> 1) & 1, abort_flag))) { ok = false; break; }
        ptx::tc_fence_after_sync();
        uint32_t raw[32];
        ptx::tmem_ld_32x32b_x32(tmem + (buf ? TMEM_S1 : TMEM_S0) + hf * 32 + lane_addr, raw);
        ptx::tmem_ld_wait();

        const int64_t kv0 = (int64_t)j * BN + hf * 32;  // first key of this thread's half
        const bool need_mask = (p.causal && kv0 + 31 > it.q0) || (kv0 + 32 > p.kv_len);
        if (need_mask) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int64_t key = kv0 + c;
            if (key >= p.kv_len || (p.causal && key > row)) raw[c] = 0xff800000u;  // -inf
          }
        }
        // maximum of the raw scores, four independent chains (scale > 0, so the scaled maximum
        // is the maximum scaled)
        float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx[u] = fmaxf(mx[u], fmaxf(__uint_as_float(raw[c + 2 * u]), __uint_as_float(raw[c + 2 * u + 1])));
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
        const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
        const float2 negm2 = make_float2(neg_m, neg_m);
        uint32_t packed[16];
        float2 sum2[2] = {make_float2(0.0f, 0.0f), make_float2(0.0f, 0.0f)};
#pragma unroll
        for (int c = 0; c < 32; c += 2) {
          // p = exp2(s * scale * log2e - m): one packed FMA for two scores, then two MUFU ops
          const float2 s2 = make_float2(__uint_as_float(raw[c]), __uint_as_float(raw[c + 1]));
          const float2 e2 = __ffma2_rn(s2, scale2, negm2);
          const float2 p2 = make_float2(ex2(e2.x), ex2(e2.y));
          sum2[(c >> 1) & 1] = __fadd2_rn(sum2[(c >> 1) & 1], p2);
          packed[c >> 1] = pack_bf16x2(p2.x, p2.y);
        }
        l += (sum2[0].x + sum2[0].y) + (sum2[1].x + sum2[1].y);

        // this thread's accumulator may only be rescaled once the previous P V has landed in it
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(pv_done((g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag))) { ok = false; break; }
          ptx::tc_fence_after_sync();
#pragma unroll
          for (int hcol = 0; hcol < 2; ++hcol) {
            uint32_t o[32];
            ptx::tmem_ld_32x32b_x32(o_mine + hcol * 32, o);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) o[c] = __float_as_uint(__uint_as_float(o[c]) * alpha);
            ptx::tmem_st_32x32b_x32(o_mine + hcol * 32, o);
          }
          ptx::tmem_st_wait();
        }
        // P buffer `buf` was last read by the P V of tile g-2, which had completed before s_full(g)
        // could arrive (see the MMA issuer), so it can be rewritten without another wait.
        // P row r: this thread's 32 bf16 are 16-byte chunks 4*hf .. 4*hf+3 of the 128-byte row,
        // 128-byte swizzle: chunk index XOR (row mod 8)
        {
          uint8_t* prow = smem + SMEM_P + buf * P_BYTES + r * 128;
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 v4 = make_uint4(packed[4 * c], packed[4 * c + 1], packed[4 * c + 2], packed[4 * c + 3]);
            *reinterpret_cast<uint4*>(prow + (((hf * 4 + c) ^ (r & 7)) << 4)) = v4;
          }
        }
        ptx::fence_proxy_async_smem();  // every writer: its P stores become visible to the MMA
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(p_full(buf));
      }
      if (!ok) break;

      // ---- item epilogue ----
      if (hf == 1) {
        // b threads hand (m_b, l_b) to the a thread of the same row and move on
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(stat_empty, (items & 1) ^ 1, abort_flag))) { ok = false; break; }
        stats[2 * r] = m_ref;
        stats[2 * r + 1] = l;
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(stat_full);  // mbarrier arrive has release semantics
        continue;
      }
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(stat_full, items & 1, abort_flag))) { ok = false; break; }
      const float m_b = stats[2 * r], l_b = stats[2 * r + 1];
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(stat_empty);
      // both accumulators are complete once the last P V of the item is
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(pv_done((g - 1) & 1), ((g - 1) >> 1) & 1, abort_flag))) { ok = false; break; }
      ptx::tc_fence_after_sync();
      const float m_all = fmaxf(m_ref, m_b);
      const float wa = (m_ref == -INFINITY) ? 0.0f : ex2(m_ref - m_all);
      const float wb = (m_b == -INFINITY) ? 0.0f : ex2(m_b - m_all);
      const float l_all = l * wa + l_b * wb;
      const float inv = 1.0f / l_all;  // l_all == 0 (no visible key) gives NaN like torch
      const float fa = wa * inv, fb = wb * inv;
      __nv_bfloat16* orow = p.o + it.b * p.os_b + it.h * p.os_h + row * p.os_t;
#pragma unroll
      for (int hcol = 0; hcol < 2; ++hcol) {
        uint32_t oa[32], ob[32];
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_OA + lane_addr + hcol * 32, oa);
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_OB + lane_addr + hcol * 32, ob);
        ptx::tmem_ld_wait();
        if (row < p.q_len) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            float v[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              v[e] = __uint_as_float(oa[8 * c + e]) * fa + __uint_as_float(ob[8 * c + e]) * fb;
            uint4 t;
            t.x = pack_bf16x2(v[0], v[1]);
            t.y = pack_bf16x2(v[2], v[3]);
            t.z = pack_bf16x2(v[4], v[5]);
            t.w = pack_bf16x2(v[6], v[7]);
            reinterpret_cast<uint4*>(orow)[hcol * 4 + c] = t;
          }
        }
      }
      ptx::tc_fence_before_sync();
      if (row < p.q_len && p.lse != nullptr)
        p.lse[((int64_t)it.b * p.heads + it.h) * p.q_len + row] = (m_all + log2f(l_all)) * 0.6931471805599453f;
    }
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

// Tensor map over [batch, heads, len, 64]. Dims are listed innermost first with ascending
// strides: (d, pos, head, batch) for a [B, H, T, D]-contiguous tensor, (d, head, pos, batch) for
// views of a [B, T, H*D] projection. *heads_inner tells the kernel which coordinate order to use.
int32_t make_map(CUtensorMap* map, const void* ptr, int64_t batch, int64_t heads, int64_t len,
                 const int64_t* strides, int rows_per_box, int* heads_inner) {
  uint64_t st, sh, sb;
  byte_strides(strides, batch, heads, len, &st, &sh, &sb);
  *heads_inner = sh < st ? 1 : 0;
  if (*heads_inner) {
    const uint64_t dims[4] = {(uint64_t)D, (uint64_t)heads, (uint64_t)len, (uint64_t)batch};
    const uint64_t str[3] = {sh, st, sb};
    const uint32_t box[4] = {(uint32_t)D, 1, (uint32_t)rows_per_box, 1};
    return encode_tensor_map(map, B200_BF16, 4, ptr, dims, str, box, true);
  }
  const uint64_t dims[4] = {(uint64_t)D, (uint64_t)len, (uint64_t)heads, (uint64_t)batch};
  const uint64_t str[3] = {st, sh, sb};
  const uint32_t box[4] = {(uint32_t)D, (uint32_t)rows_per_box, 1, 1};
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
  if (a.q_len > INT32_MAX - 256 || a.kv_len > INT32_MAX - 256) return "sequence too long";
  return nullptr;
}

int32_t launch_sdpa_tcgen05(const b200_sdpa_args& a, cudaStream_t stream) {
  CUtensorMap mq, mk, mv;
  Params p;
  int32_t st = make_map(&mq, a.q, a.batch, a.heads, a.q_len, a.q_strides, BM, &p.q_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mk, a.k, a.batch, a.heads, a.kv_len, a.k_strides, BN, &p.k_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mv, a.v, a.batch, a.heads, a.kv_len, a.v_strides, BN, &p.v_heads_inner);
  if (st != B200_OK) return st;

  p.o = static_cast<__nv_bfloat16*>(a.o);
  p.lse = a.lse;
  p.heads = a.heads; p.q_len = a.q_len; p.kv_len = a.kv_len;
  p.os_b = a.o_strides[0]; p.os_h = a.o_strides[1]; p.os_t = a.o_strides[2];
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.causal = a.causal;
  p.q_tiles = (int)((a.q_len + BM - 1) / BM);
  p.bh = a.batch * a.heads;
  p.num_items = (int64_t)p.q_tiles * p.bh;
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
  const int64_t slots = 2 * (int64_t)sm_count();  // two resident CTAs per SM
  const unsigned grid = (unsigned)(p.num_items < slots ? p.num_items : slots);
  sdpa_tcgen05_kernel<<<grid, kThreads, SMEM_BYTES, stream>>>(mq, mk, mv, p);
  B200_CHECK_LAUNCH("sdpa(tcgen05)");
  return B200_OK;
}

}  // namespace b200
