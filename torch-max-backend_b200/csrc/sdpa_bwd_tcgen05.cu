// Attention backward on the 5th-generation tensor cores for head_dim 64, bf16.
//
// One work item is a 128-key tile (K_i, V_i) of one (batch, head); the CTA that owns it keeps dK_i and
// dV_i in tensor memory and walks the 128-row query tiles j that attend to it (all of them, or
// j >= i under a causal mask). Per (i, j), with the forward's LSE and delta = rowsum(dO * O):
//   S  = Q_j K_i^T            dP = dO_j V_i^T                       (two MMAs into tensor memory)
//   P  = exp2(S scale log2e - LSE log2e),  dS = scale P (dP - delta) (one thread per query row)
//   dV_i += P^T dO_j          dK_i += dS^T Q_j      dQ_j(i) = dS K_i (three MMAs)
// P and dS go to shared memory as bf16 in the [query row][key] layout with the 128-byte swizzle of
// the TMA tiles; that one layout is the K-major A operand of dS K and, read through the MN-major
// descriptor, the transposed A operand of P^T dO and dS^T Q. K, V, Q and dO tiles are [row][64]
// TMA tiles exactly as in the forward kernel, used K-major for S and dP and MN-major (as B) for the
// three products that contract over rows.
// dQ_j gets a contribution from every key tile; tile i writes its own to a partial buffer
// [batch*heads, key tile, query tile, 64 columns, 128 rows] (fp32, rows innermost so that a warp's
// stores are contiguous) and a second kernel adds the tiles up in tile order, so the gradient does
// not depend on which CTA ran first (no atomics).
// Steps overlap: Q_j / dO_j have a three-deep ring, the score MMAs of step n + 1 are issued as soon
// as the row threads have pulled S and dP of step n into registers -- BEFORE the three products of
// step n --, the row threads do the arithmetic of step n + 1 in registers while those products run
// and store P / dS only when they have completed, and they read dQ of step n after that.
//   warp 0      TMA producer: K_i, V_i per item (two stages: the next item's land while this one
//               computes); Q_j, dO_j into a three-deep ring.
//   warp 1      MMA issuer (converged warp, one elected lane).
//   warps 2-9   two threads per query row (warps w and w + 4 address the same 32 TMEM lanes): each
//               takes 64 of the tile's 128 keys for P and dS -- with the LSE given, no value
//               crosses between them --, 32 of the 64 columns of the dQ partial, and at the end
//               of the item one of dK, dV.
// Tensor memory: S 128 columns, dP 128, dV 64, dK 64, dQ 64. Items are ordered by key tile, so
// the tiles with the most query tiles (the first ones under a causal mask) start first.
// Every wait is bounded (ptx::mbar_wait); a CTA that gives up raises its abort flag, sets the
// device status bit and leaves through the normal teardown.
#include "ptx.cuh"
#include "sdpa_internal.cuh"
#include "tma.cuh"

namespace b200 {
namespace {

constexpr int BM = 128;  // query rows per tile
constexpr int BN = 128;  // keys per tile
constexpr int D = 64;
constexpr int kRowWarps = 8;
constexpr int kThreads = (2 + kRowWarps) * 32;
constexpr int TILE_BYTES = 128 * D * 2;  // 16 KiB: a [128][64] bf16 tile; also one 64-key half of P / dS
constexpr int kTmemCols = 512;
constexpr int TMEM_S = 0, TMEM_DP = 128, TMEM_DV = 256, TMEM_DK = 320, TMEM_DQ = 384;

constexpr int SMEM_K = 0;                           // two stages: the next item's K_i / V_i land during this one
constexpr int SMEM_V = SMEM_K + 2 * TILE_BYTES;
constexpr int kStages = 3;                          // Q_j / dO_j ring
constexpr int SMEM_Q = SMEM_V + 2 * TILE_BYTES;
constexpr int SMEM_DO = SMEM_Q + kStages * TILE_BYTES;
constexpr int SMEM_P = SMEM_DO + kStages * TILE_BYTES;  // [2 key halves][128 rows][64 keys]
constexpr int SMEM_DS = SMEM_P + 2 * TILE_BYTES;
constexpr int SMEM_BAR = SMEM_DS + 2 * TILE_BYTES;
constexpr int kNumBars = 18;
constexpr int SMEM_MISC = SMEM_BAR + kNumBars * 8;
constexpr int SMEM_BYTES = SMEM_MISC + 16 + 1024;
static_assert(SMEM_BYTES <= 227 * 1024, "shared memory of one SM exceeded");

struct Params {
  const float* lse;    // [bh, q_len] natural log
  const float* delta;  // [bh, q_len]
  float* dq_part;      // [bh, kv_tiles, q_tiles, 64, 128]
  __nv_bfloat16* dk;   // element strides (batch, head, position) below; 64 contiguous
  __nv_bfloat16* dv;
  int64_t dk_sb, dk_sh, dk_st, dv_sb, dv_sh, dv_st;
  uint32_t heads, bh;
  int32_t q_len, kv_len, q_tiles, kv_tiles;
  float scale, scale_log2;
  int causal;
  uint32_t num_items;  // kv_tiles * bh
  int q_heads_inner, k_heads_inner, v_heads_inner, do_heads_inner;
  unsigned int* status;
};

#ifdef B200_SDPA_PROBE
// Development build only: per-CTA cycle counters of the row threads, read back by b200_debug_sdpa_bwd_probe.
__device__ unsigned long long g_bwd_probe[160][16];
#define PROBE_DECL(n) long long n = 0
#define PROBE_T0(t) const long long t = clock64()
#define PROBE_ADD(n, t) n += clock64() - t
#else
#define PROBE_DECL(n)
#define PROBE_T0(t)
#define PROBE_ADD(n, t)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 16 bytes (eight bf16) of row r, 16-byte unit u of a [rows][64] tile with the 128-byte swizzle.
__device__ __forceinline__ uint32_t swz(uint32_t tile, int r, int u) {
  return tile + (uint32_t)r * 128u + (uint32_t)((u ^ (r & 7)) << 4);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1)
sdpa_bwd_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                        const __grid_constant__ CUtensorMap tmap_v, const __grid_constant__ CUtensorMap tmap_do,
                        Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t base = ptx::smem_u32(smem);
  const uint32_t k_smem = base + SMEM_K, v_smem = base + SMEM_V, q_smem = base + SMEM_Q, do_smem = base + SMEM_DO;
  const uint32_t p_smem = base + SMEM_P, ds_smem = base + SMEM_DS;
  const uint32_t bar = base + SMEM_BAR;
  // Each barrier is used once per item or once per (i, j) step by one producer and one consumer
  // side, in strict alternation, so use n is waited for with parity n & 1.
  auto kv_full = [&](int st) { return bar + 8u * st; };              // per item, two stages (bars 0-1)
  auto kv_empty = [&](int st) { return bar + 8u * (16 + st); };       // (bars 16-17)
  auto qd_full = [&](int s) { return bar + 8u * (2 + s); };         // per step, kStages stages (bars 2-4)
  auto qd_empty = [&](int s) { return bar + 8u * (13 + s); };       // (bars 13-15)
  const uint32_t sdp_full = bar + 8 * 6;    // S and dP are in tensor memory
  const uint32_t sdp_free = bar + 8 * 7;    // the row threads have read them (one arrival per warp)
  const uint32_t pds_full = bar + 8 * 8;    // P and dS are in shared memory (one arrival per warp)
  const uint32_t pds_free = bar + 8 * 9;    // the three MMAs that read them have completed
  const uint32_t dq_full = bar + 8 * 10;    // dQ_j(i) is in tensor memory
  const uint32_t dq_free = bar + 8 * 11;    // the row threads have read it
  const uint32_t acc_full = bar + 8 * 12;   // dK_i, dV_i complete (per item)
  const uint32_t acc_free = bar + 8 * 5;    // the row threads have read them
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + SMEM_MISC);
  volatile uint32_t* tmem_holder = misc;
  volatile uint32_t* abort_flag = misc + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int st = 0; st < 2; ++st) {
      ptx::mbar_init(kv_full(st), 1);
      ptx::mbar_init(kv_empty(st), 1);
    }
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(qd_full(s), 1);
      ptx::mbar_init(qd_empty(s), 1);
    }
    ptx::mbar_init(sdp_full, 1);
    ptx::mbar_init(sdp_free, kRowWarps);
    ptx::mbar_init(pds_full, kRowWarps);
    ptx::mbar_init(pds_free, 1);
    ptx::mbar_init(dq_full, 1);
    ptx::mbar_init(dq_free, kRowWarps);
    ptx::mbar_init(acc_full, 1);
    ptx::mbar_init(acc_free, kRowWarps);
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_q);
    ptx::prefetch_tensormap(&tmap_k);
    ptx::prefetch_tensormap(&tmap_v);
    ptx::prefetch_tensormap(&tmap_do);
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), kTmemCols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem = *tmem_holder;

  // item w -> (key tile i, batch*head index): key tiles outermost, so the longest items start first
  auto item_tile = [&](uint32_t w) { return (int)(w / p.bh); };
  auto item_bh = [&](uint32_t w) { return w - (w / p.bh) * p.bh; };
  auto first_q_tile = [&](int i) { return p.causal ? i : 0; };  // rows of tile j >= i see keys of tile i

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      uint32_t items = 0, steps = 0;
      bool ok = true;
      for (uint32_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++items) {
        const int i = item_tile(w);
        const uint32_t bh = item_bh(w);
        const int32_t b = (int32_t)(bh / p.heads), h = (int32_t)(bh - (uint32_t)b * p.heads);
        const int st = items & 1;
        if (!ptx::mbar_wait_relaxed(kv_empty(st), ((items >> 1) & 1) ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(kv_full(st), 2 * TILE_BYTES);
        if (p.k_heads_inner) ptx::tma_load_4d(k_smem + st * TILE_BYTES, &tmap_k, kv_full(st), 0, h, i * BN, b);
        else ptx::tma_load_4d(k_smem + st * TILE_BYTES, &tmap_k, kv_full(st), 0, i * BN, h, b);
        if (p.v_heads_inner) ptx::tma_load_4d(v_smem + st * TILE_BYTES, &tmap_v, kv_full(st), 0, h, i * BN, b);
        else ptx::tma_load_4d(v_smem + st * TILE_BYTES, &tmap_v, kv_full(st), 0, i * BN, h, b);
        for (int j = first_q_tile(i); j < p.q_tiles; ++j, ++steps) {
          const int s = steps % kStages;
          if (!ptx::mbar_wait_relaxed(qd_empty(s), ((steps / kStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(qd_full(s), 2 * TILE_BYTES);
          if (p.q_heads_inner) ptx::tma_load_4d(q_smem + s * TILE_BYTES, &tmap_q, qd_full(s), 0, h, j * BM, b);
          else ptx::tma_load_4d(q_smem + s * TILE_BYTES, &tmap_q, qd_full(s), 0, j * BM, h, b);
          if (p.do_heads_inner) ptx::tma_load_4d(do_smem + s * TILE_BYTES, &tmap_do, qd_full(s), 0, h, j * BM, b);
          else ptx::tma_load_4d(do_smem + s * TILE_BYTES, &tmap_do, qd_full(s), 0, j * BM, h, b);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    constexpr uint32_t idesc_s = ptx::idesc_bf16_f32(BM, BN, 0, 0);   // S, dP: both operands K-major
    constexpr uint32_t idesc_t = ptx::idesc_bf16_f32(BN, D, 1, 1);    // dV, dK: A read transposed, B = [row][d]
    constexpr uint32_t idesc_q = ptx::idesc_bf16_f32(BM, D, 0, 1);    // dQ: A = dS K-major, B = K_i [key][d]
    uint32_t items = 0, steps = 0, accs = 0;  // accs: items that had query tiles (the ones that use dK / dV)
    bool ok = true;
    for (uint32_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++items) {
      const int i = item_tile(w);
      const int j0 = first_q_tile(i);
      const int st = items & 1;  // K / V stage of this item
      const uint32_t kt = k_smem + st * TILE_BYTES, vt = v_smem + st * TILE_BYTES;
      if (j0 >= p.q_tiles) {
        // no query row attends to this key tile: nothing to accumulate; free its K/V stage
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(kv_full(st), (items >> 1) & 1, abort_flag))) break;
        if (ptx::elect_one()) ptx::tc_commit(kv_empty(st));
        __syncwarp();
        continue;
      }
      bool go = ptx::mbar_wait(kv_full(st), (items >> 1) & 1, abort_flag);
      // dK / dV restart with this item: the row threads must have read the previous item's
      if (accs > 0) go = go && ptx::mbar_wait(acc_free, (accs - 1) & 1, abort_flag);
      if (!__all_sync(0xffffffffu, go)) break;
      ++accs;
      // dV += P^T dO, dK += dS^T Q, dQ = dS K of step n (the j-th query tile), from P / dS buffer n & 1
      auto issue_products = [&](uint32_t n, int j, bool last) -> bool {
        const int sb = n % kStages;
        bool ready = ptx::mbar_wait(pds_full, n & 1, abort_flag);
        if (n > 0) ready = ready && ptx::mbar_wait(dq_free, (n - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, ready)) return false;
        ptx::tc_fence_after_sync();
        const uint32_t qs = q_smem + sb * TILE_BYTES, dos = do_smem + sb * TILE_BYTES;
        const uint32_t pb = p_smem, dsb = ds_smem;
        if (ptx::elect_one()) {
          const uint32_t acc = j > j0 ? 1u : 0u;
          // contraction over the 128 query rows: eight steps of 16 rows; A = P^T / dS^T through the
          // MN-major descriptor (two 64-key halves 16 KiB apart, 8-row groups 1 KiB apart)
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk) {
            ptx::mma_f16_ss(tmem + TMEM_DV, ptx::smem_desc_sw128(pb + kk * 2048, TILE_BYTES, 1024),
                            ptx::smem_desc_sw128(dos + kk * 2048, 0, 1024), idesc_t, (acc | (kk > 0)) ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < BM / 16; ++kk) {
            ptx::mma_f16_ss(tmem + TMEM_DK, ptx::smem_desc_sw128(dsb + kk * 2048, TILE_BYTES, 1024),
                            ptx::smem_desc_sw128(qs + kk * 2048, 0, 1024), idesc_t, (acc | (kk > 0)) ? 1u : 0u);
          }
          // contraction over the 128 keys: A = dS K-major (16 keys = 32 bytes inside a 64-key half)
#pragma unroll
          for (int kk = 0; kk < BN / 16; ++kk) {
            ptx::mma_f16_ss(tmem + TMEM_DQ,
                            ptx::smem_desc_sw128(dsb + (kk >> 2) * TILE_BYTES + (kk & 3) * 32, 0, 1024),
                            ptx::smem_desc_sw128(kt + kk * 2048, 0, 1024), idesc_q, kk > 0 ? 1u : 0u);
          }
          ptx::tc_commit(dq_full);
          ptx::tc_commit(pds_free);
          ptx::tc_commit(qd_empty(sb));
          if (last) {
            ptx::tc_commit(acc_full);
            ptx::tc_commit(kv_empty(st));
          }
        }
        __syncwarp();
        return true;
      };
      for (int j = j0; j < p.q_tiles; ++j, ++steps) {
        const int s = steps % kStages;
        go = ptx::mbar_wait(qd_full(s), (steps / kStages) & 1, abort_flag);
        if (steps > 0) go = go && ptx::mbar_wait(sdp_free, (steps - 1) & 1, abort_flag);
        if (!__all_sync(0xffffffffu, go)) { ok = false; break; }
        ptx::tc_fence_after_sync();
        const uint32_t qs = q_smem + s * TILE_BYTES, dos = do_smem + s * TILE_BYTES;
        if (ptx::elect_one()) {
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            ptx::mma_f16_ss(tmem + TMEM_S, ptx::smem_desc_sw128(qs + kk * 32, 0, 1024),
                            ptx::smem_desc_sw128(kt + kk * 32, 0, 1024), idesc_s, kk > 0 ? 1u : 0u);
          }
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            ptx::mma_f16_ss(tmem + TMEM_DP, ptx::smem_desc_sw128(dos + kk * 32, 0, 1024),
                            ptx::smem_desc_sw128(vt + kk * 32, 0, 1024), idesc_s, kk > 0 ? 1u : 0u);
          }
          ptx::tc_commit(sdp_full);
        }
        __syncwarp();
        // the products of the PREVIOUS step go behind this step's score MMAs: the row threads work
        // on this step while the tensor core is busy with them
        if (j > j0 && !issue_products(steps - 1, j - 1, false)) { ok = false; break; }
      }
      if (!ok) break;
      if (!issue_products(steps - 1, p.q_tiles - 1, true)) break;  // the item's last step
    }
  } else {
    // ---------------- row threads: warps 2-9 ----------------
    const int half = (warp - 2) >> 2;  // which 64 keys of P / dS, which 32 columns of dQ, which of dK / dV
    const int quad = warp & 3;       // TMEM lane quadrant this warp may access
    const int r = quad * 32 + lane;  // row of the tile == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    uint32_t items = 0, steps = 0, accs = 0;
    bool ok = true;
    PROBE_DECL(c_wait_sdp); PROBE_DECL(c_math); PROBE_DECL(c_wait_dq); PROBE_DECL(c_dq); PROBE_DECL(c_wait_acc); PROBE_DECL(c_acc);
    PROBE_T0(t_start);
    for (uint32_t w = blockIdx.x; w < p.num_items && ok; w += gridDim.x, ++items) {
      const int i = item_tile(w);
      const uint32_t bh = item_bh(w);
      const int j0 = first_q_tile(i);
      const int32_t kv0 = i * BN;
      const int32_t key = kv0 + r;  // the key this thread owns in the dK / dV epilogue
      const int64_t ob = bh / p.heads, oh = bh - (bh / p.heads) * p.heads;
      __nv_bfloat16* dk_row = p.dk + ob * p.dk_sb + oh * p.dk_sh + (int64_t)key * p.dk_st;
      __nv_bfloat16* dv_row = p.dv + ob * p.dv_sb + oh * p.dv_sh + (int64_t)key * p.dv_st;
      if (j0 >= p.q_tiles) {
        if (key < p.kv_len) {
#pragma unroll
          for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(half ? dv_row : dk_row)[c] = make_uint4(0, 0, 0, 0);
        }
        continue;
      }
      // this key tile's share of dQ of step n (query tile j): 32 of the 64 columns per thread
      auto dq_epilogue = [&](uint32_t n, int j) -> bool {
        PROBE_T0(t2);
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(dq_full, n & 1, abort_flag))) return false;
        ptx::tc_fence_after_sync();
        PROBE_ADD(c_wait_dq, t2);
        PROBE_T0(t3);
        float* part = p.dq_part + ((((int64_t)bh * p.kv_tiles + i) * p.q_tiles + j) * D + half * 32) * BM + r;
        uint32_t o[32];
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_DQ + half * 32 + lane_addr, o);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) part[c * BM] = __uint_as_float(o[c]);  // consecutive lanes, consecutive rows
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(dq_free);
        PROBE_ADD(c_dq, t3);
        return true;
      };
      // LSE and delta of this thread's row, fetched one step ahead of their use
      auto row_stats = [&](int j) {
        const int32_t row = j * BM + r;
        return row < p.q_len ? make_float2(p.lse[(int64_t)bh * p.q_len + row], p.delta[(int64_t)bh * p.q_len + row])
                             : make_float2(0.0f, 0.0f);
      };
      float2 stats = row_stats(j0);
      for (int j = j0; j < p.q_tiles; ++j, ++steps) {
        const int32_t row = j * BM + r;
        const bool live = row < p.q_len;
        const float lse2 = stats.x * 1.4426950408889634f;
        const float delta = stats.y;
        if (j + 1 < p.q_tiles) stats = row_stats(j + 1);
        PROBE_T0(t0);
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(sdp_full, steps & 1, abort_flag))) { ok = false; break; }
        ptx::tc_fence_after_sync();
        PROBE_ADD(c_wait_sdp, t0);
        PROBE_T0(t1);
        // keys [kv0, kv0 + visible) of the tile are visible to this row
        int32_t visible = p.kv_len - kv0;
        if (p.causal && row - kv0 + 1 < visible) visible = row - kv0 + 1;
        if (!live) visible = 0;
        // warp-uniform: does any row of this warp have a masked key among its 64? (diagonal and edge tiles only)
        const bool need_mask = __any_sync(0xffffffffu, visible < (half + 1) * 64);
        // this thread's 64 scores and 64 dP values: four loads in flight, one wait
        uint32_t sv[64], dpv[64];
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_S + half * 64 + lane_addr, reinterpret_cast<uint32_t(&)[32]>(sv[0]));
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_S + half * 64 + 32 + lane_addr, reinterpret_cast<uint32_t(&)[32]>(sv[32]));
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_DP + half * 64 + lane_addr, reinterpret_cast<uint32_t(&)[32]>(dpv[0]));
        ptx::tmem_ld_32x32b_x32(tmem + TMEM_DP + half * 64 + 32 + lane_addr, reinterpret_cast<uint32_t(&)[32]>(dpv[32]));
        ptx::tmem_ld_wait();
        // S and dP are in registers: the score MMAs of the next step may overwrite them right away
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(sdp_free);
        // packed two-wide arithmetic: P = exp2(S scale log2e - LSE log2e), dS = P (dP scale - delta scale)
        const float2 sl2 = make_float2(p.scale_log2, p.scale_log2), nlse2 = make_float2(-lse2, -lse2);
        const float2 sc2 = make_float2(p.scale, p.scale), nds2 = make_float2(-delta * p.scale, -delta * p.scale);
        const uint32_t half_p = p_smem + half * TILE_BYTES, half_d = ds_smem + half * TILE_BYTES;
        uint32_t pp[32], dd[32];  // the 64 probabilities and 64 dS values of this thread, as bf16 pairs
#pragma unroll
        for (int u = 0; u < 8; ++u) {  // eight 16-byte units of eight keys
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int c = 8 * u + 2 * e;
            const float2 arg = __ffma2_rn(make_float2(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), sl2, nlse2);
            float2 pr = make_float2(ex2(arg.x), ex2(arg.y));
            if (need_mask) {
              if (half * 64 + c >= visible) pr.x = 0.0f;
              if (half * 64 + c + 1 >= visible) pr.y = 0.0f;
            }
            const float2 t = __ffma2_rn(make_float2(__uint_as_float(dpv[c]), __uint_as_float(dpv[c + 1])), sc2, nds2);
            const float2 ds = __fmul2_rn(pr, t);
            pp[4 * u + e] = pack_bf16x2(pr.x, pr.y);
            dd[4 * u + e] = pack_bf16x2(ds.x, ds.y);
          }
        }
        // the products of the previous step read P / dS from shared memory: store only when they are done
        if (steps > 0 && !__all_sync(0xffffffffu, ptx::mbar_wait(pds_free, (steps - 1) & 1, abort_flag))) { ok = false; break; }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          st_shared_v4(swz(half_p, r, u), pp[4 * u], pp[4 * u + 1], pp[4 * u + 2], pp[4 * u + 3]);
          st_shared_v4(swz(half_d, r, u), dd[4 * u], dd[4 * u + 1], dd[4 * u + 2], dd[4 * u + 3]);
        }
        // P / dS are written: make them visible to the tensor core's proxy
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(pds_full);
        PROBE_ADD(c_math, t1);
        // dQ of the previous step, whose products ran on the tensor core during the arithmetic above
        if (j > j0 && !dq_epilogue(steps - 1, j - 1)) { ok = false; break; }
      }
      if (!ok) break;
      if (!dq_epilogue(steps - 1, p.q_tiles - 1)) { ok = false; break; }
      if (!ok) break;
      PROBE_T0(t4);
      // ---- end of the item: dK_i and dV_i, one key per thread
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(acc_full, accs & 1, abort_flag))) { ok = false; break; }
      ++accs;
      ptx::tc_fence_after_sync();
      PROBE_ADD(c_wait_acc, t4);
      PROBE_T0(t5);
      {
        __nv_bfloat16* out = half ? dv_row : dk_row;
#pragma unroll
        for (int hcol = 0; hcol < 2; ++hcol) {
          uint32_t o[32];
          ptx::tmem_ld_32x32b_x32(tmem + (half ? TMEM_DV : TMEM_DK) + hcol * 32 + lane_addr, o);
          ptx::tmem_ld_wait();
          if (key < p.kv_len) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
              uint4 t;
              t.x = pack_bf16x2(__uint_as_float(o[8 * c + 0]), __uint_as_float(o[8 * c + 1]));
              t.y = pack_bf16x2(__uint_as_float(o[8 * c + 2]), __uint_as_float(o[8 * c + 3]));
              t.z = pack_bf16x2(__uint_as_float(o[8 * c + 4]), __uint_as_float(o[8 * c + 5]));
              t.w = pack_bf16x2(__uint_as_float(o[8 * c + 6]), __uint_as_float(o[8 * c + 7]));
              reinterpret_cast<uint4*>(out)[hcol * 4 + c] = t;
            }
          }
        }
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_free);
      PROBE_ADD(c_acc, t5);
    }
#ifdef B200_SDPA_PROBE
    if (threadIdx.x == 64) {
      unsigned long long* o = g_bwd_probe[blockIdx.x];
      o[0] = clock64() - t_start; o[1] = steps; o[2] = items; o[3] = c_wait_sdp; o[4] = c_math; o[5] = c_wait_dq;
      o[6] = c_dq; o[7] = c_wait_acc; o[8] = c_acc;
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

// delta[bh, row] = sum_d dO * O: one thread per row, 16-byte loads.
__global__ void sdpa_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_out,
                                  float* __restrict__ delta, int64_t rows, int64_t heads, int64_t q_len,
                                  int64_t os_b, int64_t os_h, int64_t os_t, int64_t ds_b, int64_t ds_h,
                                  int64_t ds_t) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= rows) return;
  const int64_t t = idx % q_len, bh = idx / q_len;
  const int64_t b = bh / heads, h = bh - b * heads;
  const __nv_bfloat16* op = o + b * os_b + h * os_h + t * os_t;
  const __nv_bfloat16* dp = d_out + b * ds_b + h * ds_h + t * ds_t;
  float acc = 0.0f;
#pragma unroll
  for (int c = 0; c < D / 8; ++c) {
    float a[8], g[8];
    load16(op + 8 * c, a);
    load16(dp + 8 * c, g);
#pragma unroll
    for (int e = 0; e < 8; ++e) acc = fmaf(a[e], g[e], acc);
  }
  delta[idx] = acc;
}

// dq[bh, row, :] = sum over the key tiles that row attends to, in tile order. The partial tiles are
// [64 columns][128 rows]: consecutive threads take consecutive rows (contiguous reads), four columns each.
__global__ void sdpa_dq_reduce_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ dq, int64_t bh_count,
                                      int64_t heads, int64_t dq_sb, int64_t dq_sh, int64_t dq_st, int32_t q_len,
                                      int32_t q_tiles, int32_t kv_tiles, int causal) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;  // over bh * q_tiles * 16 * 128
  const int64_t total = bh_count * q_tiles * (D / 4) * BM;
  if (idx >= total) return;
  const int r = (int)(idx % BM);
  const int c4 = (int)((idx / BM) % (D / 4));
  const int j = (int)((idx / (BM * (D / 4))) % q_tiles);
  const int64_t bh = idx / ((int64_t)BM * (D / 4) * q_tiles);
  const int32_t row = j * BM + r;
  if (row >= q_len) return;
  int last = kv_tiles - 1;
  if (causal && j < last) last = j;
  float s[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  for (int i = 0; i <= last; ++i) {
    const float* t = part + ((((int64_t)bh * kv_tiles + i) * q_tiles + j) * D + 4 * c4) * BM + r;
#pragma unroll
    for (int c = 0; c < 4; ++c) s[c] += __ldcs(t + c * BM);
  }
  uint2 o;
  o.x = pack_bf16x2(s[0], s[1]);
  o.y = pack_bf16x2(s[2], s[3]);
  const int64_t b = bh / heads, h = bh - b * heads;
  reinterpret_cast<uint2*>(dq + b * dq_sb + h * dq_sh + (int64_t)row * dq_st)[c4] = o;
}

// Byte strides of the (position, head, batch) dims with legal stand-ins for size-1 dims.
void byte_strides(const int64_t* s, int64_t batch, int64_t heads, int64_t len, uint64_t* st, uint64_t* sh,
                  uint64_t* sb) {
  *st = (uint64_t)(len > 1 ? s[2] : D) * 2;
  *sh = heads > 1 ? (uint64_t)s[1] * 2 : *st * (uint64_t)(len > 0 ? len : 1);
  const uint64_t big = (*st * (uint64_t)len > *sh * (uint64_t)heads) ? *st * (uint64_t)len : *sh * (uint64_t)heads;
  *sb = batch > 1 ? (uint64_t)s[0] * 2 : big;
}

// Tensor map over [batch, heads, len, 64] with boxes of 128 positions; dims innermost first with
// ascending strides ((d, pos, head, batch) or (d, head, pos, batch)); *heads_inner says which.
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
  return sb >= st && sb >= sh;  // batch must be the outermost dim
}

size_t align256(size_t n) { return (n + 255) / 256 * 256; }

}  // namespace
}  // namespace b200

using namespace b200;

namespace {
const char* sdpa_bwd_ineligible(const b200_sdpa_bwd_args& a) {
  if (a.dtype != B200_BF16) return "tensors are not bf16";
  if (a.head_dim != D) return "head_dim is not 64";
  if (a.q_len <= 0 || a.kv_len <= 0) return "empty sequence";
  if (!(a.scale > 0.0f)) return "scale is not positive";
  if (!aligned_to(a.q, 16) || !aligned_to(a.k, 16) || !aligned_to(a.v, 16) || !aligned_to(a.o, 16) ||
      !aligned_to(a.d_out, 16) || !aligned_to(a.dq, 16) || !aligned_to(a.dk, 16) || !aligned_to(a.dv, 16))
    return "pointer not 16-byte aligned";
  if (!strides_ok(a.q_strides, a.batch, a.heads, a.q_len) || !strides_ok(a.k_strides, a.batch, a.heads, a.kv_len) ||
      !strides_ok(a.v_strides, a.batch, a.heads, a.kv_len) || !strides_ok(a.d_out_strides, a.batch, a.heads, a.q_len))
    return "stride not a multiple of 16 bytes";
  if (a.o_strides[0] % 8 != 0 || a.o_strides[1] % 8 != 0 || a.o_strides[2] % 8 != 0) return "output stride not a multiple of 16 bytes";
  for (int i = 0; i < 3; ++i)
    if (a.dq_strides[i] % 8 != 0 || a.dk_strides[i] % 8 != 0 || a.dv_strides[i] % 8 != 0 || a.dq_strides[i] < 0 ||
        a.dk_strides[i] < 0 || a.dv_strides[i] < 0)
      return "gradient stride not a non-negative multiple of 16 bytes";
  if (a.q_len > INT32_MAX - 512 || a.kv_len > INT32_MAX - 512) return "sequence too long";
  if (a.batch * a.heads > (1ll << 24) || (a.batch * a.heads) * ((a.kv_len + BN - 1) / BN) > (1ll << 30))
    return "too many (batch, head, key tile) work items";
  return nullptr;
}
}  // namespace

extern "C" B200_API size_t b200_sdpa_bwd_workspace_bytes(const b200_sdpa_bwd_args* a) {
  if (a == nullptr || a->batch <= 0 || a->heads <= 0 || a->q_len <= 0 || a->kv_len <= 0) return 0;
  const size_t bh = (size_t)a->batch * (size_t)a->heads;
  const size_t kv_tiles = (size_t)((a->kv_len + BN - 1) / BN), q_tiles = (size_t)((a->q_len + BM - 1) / BM);
  return align256(bh * (size_t)a->q_len * sizeof(float)) + bh * kv_tiles * q_tiles * BM * D * sizeof(float);
}

extern "C" B200_API int32_t b200_sdpa_bwd(const b200_sdpa_bwd_args* args, b200_stream_t stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  B200_REQUIRE(args != nullptr, B200_ERR_INVALID_ARG, "sdpa_bwd: null args");
  const b200_sdpa_bwd_args& a = *args;
  B200_REQUIRE(a.batch >= 0 && a.heads >= 0 && a.q_len >= 0 && a.kv_len >= 0, B200_ERR_INVALID_ARG,
               "sdpa_bwd: negative size");
  B200_REQUIRE(valid_dtype(a.dtype), B200_ERR_INVALID_ARG, "sdpa_bwd: bad dtype enum");
  if (a.batch == 0 || a.heads == 0) return B200_OK;
  B200_REQUIRE(a.q != nullptr && a.k != nullptr && a.v != nullptr && a.o != nullptr && a.d_out != nullptr &&
                   a.lse != nullptr && a.dq != nullptr && a.dk != nullptr && a.dv != nullptr,
               B200_ERR_INVALID_ARG, "sdpa_bwd: null pointer");
  const char* why = sdpa_bwd_ineligible(a);
  B200_REQUIRE(why == nullptr, B200_ERR_UNSUPPORTED, "sdpa_bwd: %s", why);
  const size_t need = b200_sdpa_bwd_workspace_bytes(args);
  B200_REQUIRE(a.workspace != nullptr && a.workspace_bytes >= need, B200_ERR_WORKSPACE,
               "sdpa_bwd: workspace of %zu bytes needed, %zu given", need, a.workspace_bytes);
  B200_REQUIRE(aligned_to(a.workspace, 256), B200_ERR_ALIGNMENT, "sdpa_bwd: workspace not 256-byte aligned");

  const int64_t bh = a.batch * a.heads;
  float* delta = static_cast<float*>(a.workspace);
  float* dq_part = reinterpret_cast<float*>(static_cast<unsigned char*>(a.workspace) +
                                            align256((size_t)bh * (size_t)a.q_len * sizeof(float)));
  {
    const int64_t rows = bh * a.q_len;
    sdpa_delta_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(a.o), static_cast<const __nv_bfloat16*>(a.d_out), delta, rows, a.heads,
        a.q_len, a.o_strides[0], a.o_strides[1], a.o_strides[2], a.d_out_strides[0], a.d_out_strides[1],
        a.d_out_strides[2]);
    B200_CHECK_LAUNCH("sdpa_bwd(delta)");
  }
  CUtensorMap mq, mk, mv, mdo;
  Params p;
  int32_t st = make_map(&mq, a.q, a.batch, a.heads, a.q_len, a.q_strides, &p.q_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mk, a.k, a.batch, a.heads, a.kv_len, a.k_strides, &p.k_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mv, a.v, a.batch, a.heads, a.kv_len, a.v_strides, &p.v_heads_inner);
  if (st != B200_OK) return st;
  st = make_map(&mdo, a.d_out, a.batch, a.heads, a.q_len, a.d_out_strides, &p.do_heads_inner);
  if (st != B200_OK) return st;
  p.lse = a.lse;
  p.delta = delta;
  p.dq_part = dq_part;
  p.dk = static_cast<__nv_bfloat16*>(a.dk);
  p.dv = static_cast<__nv_bfloat16*>(a.dv);
  p.dk_sb = a.dk_strides[0]; p.dk_sh = a.dk_strides[1]; p.dk_st = a.dk_strides[2];
  p.dv_sb = a.dv_strides[0]; p.dv_sh = a.dv_strides[1]; p.dv_st = a.dv_strides[2];
  p.heads = (uint32_t)a.heads;
  p.bh = (uint32_t)bh;
  p.q_len = (int32_t)a.q_len;
  p.kv_len = (int32_t)a.kv_len;
  p.q_tiles = (int32_t)((a.q_len + BM - 1) / BM);
  p.kv_tiles = (int32_t)((a.kv_len + BN - 1) / BN);
  p.scale = a.scale;
  p.scale_log2 = a.scale * 1.4426950408889634f;
  p.causal = a.causal;
  p.num_items = (uint32_t)p.kv_tiles * p.bh;
  p.status = device_status_ptr();
  B200_REQUIRE(p.status != nullptr, B200_ERR_CUDA, "sdpa_bwd: device status word unavailable");

  static thread_local bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(sdpa_bwd_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    if (e != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "sdpa_bwd: cannot opt in to %d bytes of shared memory: %s", SMEM_BYTES, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int64_t slots = sm_count();
  const int64_t grid = (int64_t)p.num_items < slots ? (int64_t)p.num_items : slots;
  sdpa_bwd_tcgen05_kernel<<<(unsigned)grid, kThreads, SMEM_BYTES, stream>>>(mq, mk, mv, mdo, p);
  B200_CHECK_LAUNCH("sdpa_bwd");
  {
    const int64_t total = bh * p.q_tiles * (D / 4) * BM;
    sdpa_dq_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        dq_part, static_cast<__nv_bfloat16*>(a.dq), bh, a.heads, a.dq_strides[0], a.dq_strides[1], a.dq_strides[2],
        p.q_len, p.q_tiles, p.kv_tiles, p.causal);
    B200_CHECK_LAUNCH("sdpa_bwd(dq)");
  }
  return B200_OK;
}

#ifdef B200_SDPA_PROBE
extern "C" B200_API int32_t b200_debug_sdpa_bwd_probe(unsigned long long* out) {
  return cudaMemcpyFromSymbol(out, g_bwd_probe, sizeof(g_bwd_probe)) == cudaSuccess ? 0 : -5;
}
#endif
