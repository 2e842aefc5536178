// bf16 GEMM on the 5th-generation tensor cores: TMA-fed shared-memory ring, tcgen05.mma with
// fp32 accumulators in TMEM, persistent CTAs, warp-specialised roles.
//
//   warp 0      TMA producer: one lane streams 128xBK A tiles and BNxBK B tiles into a
//               STAGES-deep ring (128-byte swizzle), signalling `full[s]` by transaction bytes.
//   warp 1      MMA issuer: the warp waits `full[s]` converged, one elected lane issues BK/16
//               tcgen05.mma (128 x BN x 16) per stage into one of two TMEM accumulators and
//               commits to `empty[s]`; after the last k-block it commits to `tmem_full[acc]`.
//   warps 2-9   epilogue: wait `tmem_full[acc]`; each warp owns 32 rows (its TMEM lane quadrant)
//               and half of the tile's columns. 32x32 chunks leave TMEM one row per lane, pass
//               through a per-warp swizzled shared-memory staging buffer and come back one
//               16-byte column group per lane, so that bias, residual and output accesses are
//               coalesced (8 lanes cover a 128-byte row segment); alpha/bias/activation/residual
//               are applied there, then the accumulator is released through `tmem_empty[acc]`.
//               Two accumulators let the epilogue of tile i overlap the main loop of tile i+1.
//
// Tiles are walked in bands of kBandM row-tiles (column-tile outer, row-tile inner inside a band):
// a band's slice of A is re-used from L2 across all its column tiles while the (smaller) B stays
// L2-resident.
// Large problems run the CTA-pair form (PAIR): clusters of two CTAs, each pair owning a 256 x BN
// tile through tcgen05.mma.cta_group::2. Each CTA stages its own 128 rows of A and its own half of
// the tile's B columns -- BN/2 rows of B^T for a K-major B, BN/2/64 boxes of 64 columns for an
// MN-major one (plain TMA loads whose completion bytes are counted on the even CTA's barrier), the even CTA's elected lane issues the 256 x BN x 16 MMAs for both and commits
// to the barriers of both, and each CTA's epilogue warps drain their own 128 accumulator rows and
// report to the even CTA's `tmem_empty`. A stage is a third smaller than the single-CTA stage of
// the same BN, so the ring is six stages deep instead of four.
// Every wait is bounded (ptx::mbar_wait); a CTA that gives up raises the device status word and
// leaves through the common teardown, which frees its TMEM.
#include "gemm_internal.cuh"
#include "ptx.cuh"
#include "tma.cuh"

#include <cstdlib>

namespace b200 {
namespace {

constexpr int BM = 128;
constexpr int BK = 64;                  // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kEpilogueWarps = 8;
constexpr int kEpilogueThreads = kEpilogueWarps * 32;
constexpr int kThreads = 64 + kEpilogueThreads;
constexpr int kStageChunkBytes = 32 * 32 * 4;  // one 32x32 fp32 chunk per epilogue warp
constexpr int kBandM = 16;                     // row-tiles per raster band
constexpr int A_STAGE_BYTES = BM * BK * 2;

// PAIR: two CTAs of a cluster share one 256 x BN tile (tcgen05 cta_group::2). Each CTA stages its
// own 128 rows of A and its own BN/2 rows of B^T, so a stage is a third smaller than the
// single-CTA stage of the same BN and the shared-memory fill traffic per flop drops with it.
template <int BN, bool PAIR = false>
struct Cfg {
  static constexpr int B_ROWS = PAIR ? BN / 2 : BN;  // rows of B^T this CTA stages
  static constexpr int B_STAGE_BYTES = B_ROWS * BK * 2;
  static constexpr int kStages = PAIR ? 6 : (BN == 128 ? 6 : 4);
  static constexpr int kTmemCols = BN == 128 ? 256 : 512;  // two accumulators, rounded up to a power of two
  static constexpr int kSmemA = 0;
  static constexpr int kSmemB = kStages * A_STAGE_BYTES;
  static constexpr int kSmemStaging = kSmemB + kStages * B_STAGE_BYTES;
  static constexpr int kSmemBar = kSmemStaging + kEpilogueWarps * kStageChunkBytes;
  static constexpr int kNumBars = 2 * kStages + 4;
  static constexpr int kSmemMisc = kSmemBar + kNumBars * 8;
  static constexpr int kSmemBytes = kSmemMisc + 16 + 1024;  // +1024: manual 1 KiB alignment
};

struct Params {
  int64_t M, N, K, batch;
  int64_t c_rs, c_bs;
  const void* bias;
  const void* residual;
  int64_t bias_rs, residual_rs;
  float alpha, beta;
  int32_t bias_dtype, residual_dtype, epilogue;
  int32_t tiles_m, tiles_n;
  int64_t num_tiles;
  unsigned int* status;
  int32_t fast_ok;  // pointers/pitches allow the branch-free vector epilogue on interior tiles
  // The K loop runs k_parts passes over K; pass i reads A at k offset a_part_off[i] and B at k offset
  // b_part_off[i] (elements). One pass with offsets 0 is a plain GEMM; three passes over operands
  // stored as [hi | lo] halves are the split-precision product a_hi b_lo + a_lo b_hi + a_hi b_hi.
  int32_t k_parts;
  int32_t a_part_off[3], b_part_off[3];
  // A is stored [K, M] with M contiguous (the transposed operand of a weight-gradient GEMM): its tile
  // arrives as two boxes of 64(m) x 64(k) and the MMA reads it through the MN-major descriptor.
  int32_t a_mn_major;
};

__device__ __forceinline__ float act(float v, int32_t epilogue) {
  if (epilogue == B200_EPILOGUE_GELU_TANH) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    // 0.5 v (1 + tanh u) == v / (1 + exp(-2u)) == v * rcp(1 + exp2(-2 log2(e) u)): two MUFU ops
    const float u = k0 * (v + k1 * v * v * v);
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-2.885390081777927f * u));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return v * r;
  }
  if (epilogue == B200_EPILOGUE_GELU_ERF) return gelu_erf_f32(v);
  return v;
}

// Tile index -> (batch, row-tile, column-tile): bands of kBandM row-tiles, column-tile outer,
// row-tile inner inside a band.
template <int BAND = kBandM>
__device__ __forceinline__ void tile_coords(int64_t t, const Params& p, int64_t& b, int32_t& mt, int32_t& nt) {
  const int64_t per_batch = (int64_t)p.tiles_m * p.tiles_n;
  b = t / per_batch;
  const int64_t r = t - b * per_batch;
  const int64_t band_tiles = (int64_t)BAND * p.tiles_n;
  const int32_t band = (int32_t)(r / band_tiles);
  const int32_t in_band = (int32_t)(r - (int64_t)band * band_tiles);
  const int32_t rows_in_band = min(BAND, p.tiles_m - band * BAND);
  nt = in_band / rows_in_band;
  mt = band * BAND + in_band % rows_in_band;
}

__device__ __forceinline__ void load4(const void* p, int64_t idx, int32_t dtype, int valid, float (&out)[4]) {
  if (dtype == B200_F32) {
    const float* q = static_cast<const float*>(p) + idx;
    if (valid == 4 && (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
      const float4 t = __ldg(reinterpret_cast<const float4*>(q));
      out[0] = t.x; out[1] = t.y; out[2] = t.z; out[3] = t.w;
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) out[j] = j < valid ? __ldg(q + j) : 0.0f;
    }
  } else {
    const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(p) + idx;
    if (valid == 4 && (reinterpret_cast<uintptr_t>(q) & 7) == 0) {
      const uint2 t = __ldg(reinterpret_cast<const uint2*>(q));
      out[0] = __uint_as_float(t.x << 16); out[1] = __uint_as_float(t.x & 0xffff0000u);
      out[2] = __uint_as_float(t.y << 16); out[3] = __uint_as_float(t.y & 0xffff0000u);
    } else {
#pragma unroll
      for (int j = 0; j < 4; ++j) out[j] = j < valid ? __bfloat162float(q[j]) : 0.0f;
    }
  }
}

__device__ __forceinline__ void store4_aligned(float* dst, const float (&v)[4]) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
}

__device__ __forceinline__ void store4_aligned(__nv_bfloat16* dst, const float (&v)[4]) {
  uint2 t;
  t.x = pack_bf16x2(v[0], v[1]);
  t.y = pack_bf16x2(v[2], v[3]);
  *reinterpret_cast<uint2*>(dst) = t;
}

__device__ __forceinline__ void store4(float* dst, const float (&v)[4], int valid) {
  if (valid == 4 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (j < valid) dst[j] = v[j];
  }
}

__device__ __forceinline__ void store4(__nv_bfloat16* dst, const float (&v)[4], int valid) {
  if (valid == 4 && (reinterpret_cast<uintptr_t>(dst) & 7) == 0) {
    uint2 t;
    t.x = pack_bf16x2(v[0], v[1]);
    t.y = pack_bf16x2(v[2], v[3]);
    *reinterpret_cast<uint2*>(dst) = t;
  } else {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (j < valid) dst[j] = __float2bfloat16_rn(v[j]);
  }
}

template <int BN, bool B_MN_MAJOR, typename Tout, bool PAIR = false>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a,
                    const __grid_constant__ CUtensorMap tmap_b, Tout* __restrict__ C, Params p) {
  static_assert(!(PAIR && B_MN_MAJOR) || (BN / 2) % 64 == 0,
                "MN-major B in the pair kernel: each CTA's half of the columns is a whole number of 64-column boxes");
  using C_ = Cfg<BN, PAIR>;
  constexpr int kStages = C_::kStages;
  constexpr int kTileM = PAIR ? 2 * BM : BM;        // rows of C per tile (per CTA pair when PAIR)
  constexpr int kBand = PAIR ? kBandM / 2 : kBandM;  // same rows per raster band either way
  // Rank inside the pair (0 = the CTA that issues the MMAs and owns the shared barriers).
  const uint32_t rank = PAIR ? ptx::cluster_ctarank() : 0u;
  const int64_t tile_first = PAIR ? (int64_t)(blockIdx.x >> 1) : (int64_t)blockIdx.x;
  const int64_t tile_step = PAIR ? (int64_t)(gridDim.x >> 1) : (int64_t)gridDim.x;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled operand tiles need a 1 KiB aligned base.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = ptx::smem_u32(smem);
  const uint32_t a_base = smem_base + C_::kSmemA;
  const uint32_t b_base = smem_base + C_::kSmemB;
  const uint32_t bar_base = smem_base + C_::kSmemBar;
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
  auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
  auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
  volatile uint32_t* misc = reinterpret_cast<volatile uint32_t*>(smem + C_::kSmemMisc);
  volatile uint32_t* tmem_holder = misc;      // TMEM base address written by tcgen05.alloc
  volatile uint32_t* abort_flag = misc + 1;   // set by any thread whose bounded wait ran out

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(full_bar(s), 1);
      ptx::mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      ptx::mbar_init(tmem_full_bar(a), 1);
      // one arrival per epilogue warp (of both CTAs when PAIR: the even CTA's barrier counts them)
      ptx::mbar_init(tmem_empty_bar(a), PAIR ? 2 * kEpilogueWarps : kEpilogueWarps);
    }
    *abort_flag = 0;
    ptx::fence_barrier_init();
    ptx::prefetch_tensormap(&tmap_a);
    ptx::prefetch_tensormap(&tmap_b);
  }
  if (warp == 1) {
    if (PAIR) {
      ptx::tmem_alloc_pair(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), C_::kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_holder)), C_::kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tc_fence_before_sync();
  if (PAIR) {
    __syncthreads();
    ptx::cluster_sync();  // the peer's barriers are initialised before anything signals them
  } else {
    __syncthreads();
  }
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_holder;

  const int64_t kb_per_part = (p.K + BK - 1) / BK;
  const int64_t num_kb = kb_per_part * p.k_parts;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int64_t t = tile_first; t < p.num_tiles && ok; t += tile_step) {
        int64_t b;
        int32_t mt, nt;
        tile_coords<kBand>(t, p, b, mt, nt);
        const int32_t m0 = mt * kTileM + (int32_t)rank * BM, n0 = nt * BN + (int32_t)rank * C_::B_ROWS * (PAIR ? 1 : 0);
        int32_t part = 0, k_in_part = 0;  // position of the k-block inside the (possibly multi-pass) K walk
        for (int64_t kb = 0; kb < num_kb; ++kb, k_in_part += BK) {
          if (!ptx::mbar_wait_relaxed(empty_bar(s), phase ^ 1, abort_flag)) { ok = false; break; }
          if (k_in_part >= (int32_t)(kb_per_part * BK)) { k_in_part = 0; ++part; }
          const int32_t k0 = k_in_part + p.a_part_off[part], k0b = k_in_part + p.b_part_off[part];
          if (PAIR) {
            // Both CTAs' copies are counted on the even CTA's barrier, which expects the bytes of
            // both. (The peer's bytes may land before the expectation is posted; the phase cannot
            // complete until the pending arrival below has happened.)
            const uint32_t bar = ptx::mapa(full_bar(s), 0);
            if (rank == 0) ptx::mbar_arrive_expect_tx(full_bar(s), 2 * (A_STAGE_BYTES + C_::B_STAGE_BYTES));
            if (!p.a_mn_major) {
              ptx::tma_load_3d_pair(a_base + s * A_STAGE_BYTES, &tmap_a, bar, k0, m0, (int32_t)b);
            } else {
#pragma unroll
              for (int j = 0; j < BM / 64; ++j)
                ptx::tma_load_3d_pair(a_base + s * A_STAGE_BYTES + j * (64 * BK * 2), &tmap_a, bar, m0 + j * 64, k0,
                                      (int32_t)b);
            }
            if (!B_MN_MAJOR) {
              ptx::tma_load_3d_pair(b_base + s * C_::B_STAGE_BYTES, &tmap_b, bar, k0b, n0, (int32_t)b);
            } else {
              // B stored [K, N]: this CTA's half of the tile's columns as boxes of 64(n) x 64(k)
#pragma unroll
              for (int j = 0; j < C_::B_ROWS / 64; ++j)
                ptx::tma_load_3d_pair(b_base + s * C_::B_STAGE_BYTES + j * (64 * BK * 2), &tmap_b, bar,
                                      n0 + j * 64, k0b, (int32_t)b);
            }
            if (++s == kStages) { s = 0; phase ^= 1; }
            continue;
          }
          ptx::mbar_arrive_expect_tx(full_bar(s), A_STAGE_BYTES + C_::B_STAGE_BYTES);
          if (!p.a_mn_major) {
            ptx::tma_load_3d(a_base + s * A_STAGE_BYTES, &tmap_a, full_bar(s), k0, m0, (int32_t)b);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)
              ptx::tma_load_3d(a_base + s * A_STAGE_BYTES + j * (64 * BK * 2), &tmap_a, full_bar(s), m0 + j * 64, k0,
                               (int32_t)b);
          }
          if (!B_MN_MAJOR) {
            ptx::tma_load_3d(b_base + s * C_::B_STAGE_BYTES, &tmap_b, full_bar(s), k0b, n0, (int32_t)b);
          } else {
            // B stored [K, N]: BN/64 boxes of 64(n) x 64(k), each one swizzle atom wide in n.
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              ptx::tma_load_3d(b_base + s * C_::B_STAGE_BYTES + j * (64 * BK * 2), &tmap_b,
                               full_bar(s), n0 + j * 64, k0b, (int32_t)b);
          }
          if (++s == kStages) { s = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    // The whole warp walks the loop converged (so that addresses and descriptors are warp-uniform
    // values) and one elected lane issues the MMAs and commits; tcgen05.commit tracks the MMAs of
    // the thread that executes it, and the election returns the same lane every time.
    if (rank == 0) {
      const uint32_t idesc = p.a_mn_major ? ptx::idesc_bf16_f32(kTileM, BN, 1, B_MN_MAJOR ? 1 : 0)
                                          : ptx::idesc_bf16_f32(kTileM, BN, 0, B_MN_MAJOR ? 1 : 0);
      const bool a_mn = p.a_mn_major != 0;
      int s = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int64_t t = tile_first; t < p.num_tiles && ok; t += tile_step) {
        if (!__all_sync(0xffffffffu, ptx::mbar_wait(tmem_empty_bar(acc), acc_phase ^ 1, abort_flag))) break;
        ptx::tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int64_t kb = 0; kb < num_kb; ++kb) {
          if (!__all_sync(0xffffffffu, ptx::mbar_wait(full_bar(s), phase, abort_flag))) { ok = false; break; }
          ptx::tc_fence_after_sync();
          const uint32_t a_addr = a_base + s * A_STAGE_BYTES;
          const uint32_t b_addr = b_base + s * C_::B_STAGE_BYTES;
          if (ptx::elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k) {
              const uint64_t a_desc = a_mn ? ptx::smem_desc_sw128(a_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                                           : ptx::smem_desc_sw128(a_addr + k * (UMMA_K * 2), 0, 1024);
              const uint64_t b_desc =
                  B_MN_MAJOR ? ptx::smem_desc_sw128(b_addr + k * (UMMA_K * 128), 64 * BK * 2, 1024)
                             : ptx::smem_desc_sw128(b_addr + k * (UMMA_K * 2), 0, 1024);
              if (PAIR) ptx::mma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
              else ptx::mma_f16_ss(d_tmem, a_desc, b_desc, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            }
            // frees the smem slot (in both CTAs when PAIR) when these MMAs have read it
            if (PAIR) {
              ptx::tc_commit_pair(ptx::mapa(empty_bar(s), 0));
              ptx::tc_commit_pair(ptx::mapa(empty_bar(s), 1));
            } else {
              ptx::tc_commit(empty_bar(s));
            }
            // after the last k-block: the accumulator is complete when these MMAs are
            if (kb == num_kb - 1) {
              if (PAIR) {
                ptx::tc_commit_pair(ptx::mapa(tmem_full_bar(acc), 0));
                ptx::tc_commit_pair(ptx::mapa(tmem_full_bar(acc), 1));
              } else {
                ptx::tc_commit(tmem_full_bar(acc));
              }
            }
          }
          __syncwarp();
          if (++s == kStages) { s = 0; phase ^= 1; }
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    const int q = warp & 3;              // TMEM lane quadrant this warp may access
    const int half = (warp - 2) >> 2;    // which half of the tile's columns
    constexpr int kChunks = BN / 64;     // 32-column chunks per warp
    float* stage = reinterpret_cast<float*>(smem + C_::kSmemStaging + (warp - 2) * kStageChunkBytes);
    const int rr = lane >> 3;            // row inside a group of 4 rows
    const int c4 = lane & 7;             // 16-byte column group inside the chunk
    int acc = 0;
    uint32_t acc_phase = 0;
    // where this warp reports a drained accumulator (the even CTA's barrier when PAIR)
    const uint32_t tmem_empty_remote0 = PAIR ? ptx::mapa(tmem_empty_bar(0), 0) : 0u;
    const uint32_t tmem_empty_remote1 = PAIR ? ptx::mapa(tmem_empty_bar(1), 0) : 0u;
    for (int64_t t = tile_first; t < p.num_tiles; t += tile_step) {
      int64_t b;
      int32_t mt, nt;
      tile_coords<kBand>(t, p, b, mt, nt);
      const int64_t m0 = (int64_t)mt * kTileM + (int64_t)rank * BM, n0 = (int64_t)nt * BN;
      Tout* cbase = C + b * p.c_bs;
      const int64_t row0 = m0 + q * 32;
      // Interior tiles with vector-friendly pointers take a branch-free path in which all loads
      // of a chunk are issued before they are needed.
      // (a column tile that ends on a 32-column boundary only has whole chunks inside or outside)
      const bool fast = p.fast_ok && m0 + BM <= p.M && (n0 + BN <= p.N || (p.N - n0) % 32 == 0);
      // beta * bias for the 4 columns this lane owns in chunk c (zeros without a row bias)
      auto bias_of_chunk = [&](int c, float (&out)[4]) {
#pragma unroll
        for (int j = 0; j < 4; ++j) out[j] = 0.0f;
        if (p.bias != nullptr && p.bias_rs == 0) {
          const int64_t col = n0 + half * (BN / 2) + c * 32 + c4 * 4;
          const int64_t rem = p.N - col;
          const int valid = rem >= 4 ? 4 : (rem > 0 ? (int)rem : 0);
          if (valid > 0) load4(p.bias, col, p.bias_dtype, valid, out);
#pragma unroll
          for (int j = 0; j < 4; ++j) out[j] *= p.beta;
        }
      };
      // The first chunk's bias is fetched before the accumulator is waited for.
      float bias_next[4];
      bias_of_chunk(0, bias_next);
      // Interior tiles also prefetch the fp32 residual one chunk ahead (8 rows x 16 bytes per
      // lane): under a saturated main loop a global load takes thousands of cycles, and exposing
      // that once per chunk was what made residual epilogues slower than their main loops.
      float4 res_next[8];
      auto residual_of_chunk = [&](int c, float4 (&out)[8]) {
        const int64_t col = n0 + half * (BN / 2) + c * 32 + c4 * 4;
        if (col < p.N) {
          const float* rbase = static_cast<const float*>(p.residual) + (row0 + rr) * p.residual_rs + col;
#pragma unroll
          for (int i = 0; i < 8; ++i) out[i] = __ldg(reinterpret_cast<const float4*>(rbase + (int64_t)i * 4 * p.residual_rs));
        }
      };
      if (fast && p.residual != nullptr) residual_of_chunk(0, res_next);
      // warp-uniform result: the TMEM loads below need the whole warp
      if (!__all_sync(0xffffffffu, ptx::mbar_wait(tmem_full_bar(acc), acc_phase, abort_flag))) break;
      ptx::tc_fence_after_sync();
      if (fast) {
        // (kept rolled: the unrolled form of both epilogue paths overflowed the instruction cache)
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
          const int col_in_tile = half * (BN / 2) + c * 32;
          if (n0 + col_in_tile >= p.N) break;  // uniform: chunk entirely past the last column
          const int64_t col = n0 + col_in_tile + c4 * 4;
          float bias_cur[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) bias_cur[j] = bias_next[j];
          if (c + 1 < kChunks) bias_of_chunk(c + 1, bias_next);  // in flight during this chunk
          float4 res[8];
          if (p.residual != nullptr) {
#pragma unroll
            for (int i = 0; i < 8; ++i) res[i] = res_next[i];
            if (c + 1 < kChunks) residual_of_chunk(c + 1, res_next);  // in flight during this chunk
          }
          uint32_t raw[32];
          ptx::tmem_ld_32x32b_x32(tmem_base + (uint32_t)(acc * BN + col_in_tile) + ((uint32_t)(q * 32) << 16), raw);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4)
            *reinterpret_cast<float4*>(stage + lane * 32 + ((g4 ^ (lane & 7)) << 2)) =
                make_float4(__uint_as_float(raw[4 * g4]), __uint_as_float(raw[4 * g4 + 1]),
                            __uint_as_float(raw[4 * g4 + 2]), __uint_as_float(raw[4 * g4 + 3]));
          __syncwarp();
          float4 a4[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int r = i * 4 + rr;
            a4[i] = *reinterpret_cast<const float4*>(stage + r * 32 + ((c4 ^ (r & 7)) << 2));
          }
          __syncwarp();  // staging buffer may be rewritten by the next chunk
          Tout* crow = cbase + (row0 + rr) * p.c_rs + col;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float v[4] = {fmaf(a4[i].x, p.alpha, bias_cur[0]), fmaf(a4[i].y, p.alpha, bias_cur[1]),
                          fmaf(a4[i].z, p.alpha, bias_cur[2]), fmaf(a4[i].w, p.alpha, bias_cur[3])};
            if (p.epilogue != B200_EPILOGUE_NONE) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] = act(v[j], p.epilogue);
            }
            if (p.residual != nullptr) {
              v[0] += res[i].x; v[1] += res[i].y; v[2] += res[i].z; v[3] += res[i].w;
            }
            store4_aligned(crow + (int64_t)i * 4 * p.c_rs, v);
          }
        }
        ptx::tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) {
          if (PAIR) ptx::mbar_arrive_cluster(acc ? tmem_empty_remote1 : tmem_empty_remote0);
          else ptx::mbar_arrive(tmem_empty_bar(acc));
        }
        if (++acc == 2) { acc = 0; acc_phase ^= 1; }
        continue;
      }
#pragma unroll 1
      for (int c = 0; c < kChunks; ++c) {
        const int col_in_tile = half * (BN / 2) + c * 32;
        const int64_t col0 = n0 + col_in_tile;
        if (col0 >= p.N || row0 >= p.M) break;  // uniform across the warp
        float bias_cur[4];
        if (c == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j) bias_cur[j] = bias_next[j];
        } else {
          bias_of_chunk(c, bias_cur);
        }
        uint32_t raw[32];
        ptx::tmem_ld_32x32b_x32(tmem_base + (uint32_t)(acc * BN + col_in_tile) + ((uint32_t)(q * 32) << 16), raw);
        ptx::tmem_ld_wait();
        // lane == row: row `lane`, 8 groups of 4 columns, group index XOR (row mod 8)
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4)
          *reinterpret_cast<float4*>(stage + lane * 32 + ((g4 ^ (lane & 7)) << 2)) =
              make_float4(__uint_as_float(raw[4 * g4]), __uint_as_float(raw[4 * g4 + 1]),
                          __uint_as_float(raw[4 * g4 + 2]), __uint_as_float(raw[4 * g4 + 3]));
        __syncwarp();
        // lane == (row group, column group): 8 lanes cover one 128-byte row segment
        const int64_t col = col0 + c4 * 4;
        const int64_t rem = p.N - col;
        const int valid = rem >= 4 ? 4 : (rem > 0 ? (int)rem : 0);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = i * 4 + rr;
          const int64_t row = row0 + r;
          const float4 a4 = *reinterpret_cast<const float4*>(stage + r * 32 + ((c4 ^ (r & 7)) << 2));
          if (row < p.M && valid > 0) {
            float v[4] = {a4.x * p.alpha, a4.y * p.alpha, a4.z * p.alpha, a4.w * p.alpha};
            if (p.bias != nullptr) {
              if (p.bias_rs == 0) {
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] += bias_cur[j];
              } else {
                float bb[4];
                load4(p.bias, row * p.bias_rs + col, p.bias_dtype, valid, bb);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = fmaf(p.beta, bb[j], v[j]);
              }
            }
            if (p.epilogue != B200_EPILOGUE_NONE) {
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] = act(v[j], p.epilogue);
            }
            if (p.residual != nullptr) {
              float res[4];
              load4(p.residual, row * p.residual_rs + col, p.residual_dtype, valid, res);
#pragma unroll
              for (int j = 0; j < 4; ++j) v[j] += res[j];
            }
            store4(cbase + row * p.c_rs + col, v, valid);
          }
        }
        __syncwarp();  // staging buffer is rewritten by the next chunk
      }
      ptx::tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (PAIR) ptx::mbar_arrive_cluster(acc ? tmem_empty_remote1 : tmem_empty_remote0);
        else ptx::mbar_arrive(tmem_empty_bar(acc));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------- teardown ----------------
  __syncthreads();
  if (*abort_flag != 0) {
    if (threadIdx.x == 0) atomicOr(p.status, STATUS_GEMM_TIMEOUT);
    // Let copies and MMAs that may still be in flight drain before TMEM and smem go away.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (PAIR) {
    // Neither CTA may free its tensor memory or leave (its shared memory is read by the pair's
    // MMAs and its barriers are signalled by the peer) before both are done.
    ptx::tc_fence_before_sync();
    ptx::cluster_sync();
  }
  if (warp == 1) {
    ptx::tc_fence_after_sync();
    if (PAIR) ptx::tmem_dealloc_pair(tmem_base, C_::kTmemCols);
    else ptx::tmem_dealloc(tmem_base, C_::kTmemCols);
  }
}

// ---- host side -----------------------------------------------------------------------------

bool b_is_k_major(const b200_gemm_args& g) { return g.b_row_stride == 1 && (g.b_col_stride != 1 || g.n == 1); }
bool b_is_n_major(const b200_gemm_args& g) { return g.b_col_stride == 1; }

// Kernel parameters common to both launchers; tile_m x tile_n is the tile one CTA (or pair) owns.
int32_t fill_params(const b200_gemm_args& g, Params& p, int tile_m, int tile_n, size_t out_elem_bytes) {
  p.M = g.m; p.N = g.n; p.K = g.k; p.batch = g.batch;
  p.c_rs = g.c_row_stride; p.c_bs = g.c_batch_stride;
  p.bias = g.bias; p.residual = g.residual;
  p.bias_rs = g.bias_row_stride; p.residual_rs = g.residual_row_stride;
  p.alpha = g.alpha; p.beta = g.beta;
  p.bias_dtype = g.bias_dtype; p.residual_dtype = g.residual_dtype; p.epilogue = g.epilogue;
  p.tiles_m = (int32_t)((g.m + tile_m - 1) / tile_m);
  p.tiles_n = (int32_t)((g.n + tile_n - 1) / tile_n);
  p.num_tiles = (int64_t)p.tiles_m * p.tiles_n * g.batch;
  p.k_parts = 1;
  for (int i = 0; i < 3; ++i) { p.a_part_off[i] = 0; p.b_part_off[i] = 0; }
  p.a_mn_major = 0;
  p.status = device_status_ptr();
  B200_REQUIRE(p.status != nullptr, B200_ERR_CUDA, "gemm(tcgen05): device status word unavailable");
  {
    const size_t out_vec = out_elem_bytes * 4;  // bytes of one 4-column group
    bool ok = aligned_to(g.c, out_vec) && g.c_row_stride % 4 == 0 && (g.batch == 1 || g.c_batch_stride % 4 == 0);
    if (g.bias != nullptr)
      ok = ok && g.bias_row_stride == 0 && aligned_to(g.bias, g.bias_dtype == B200_F32 ? 16 : 8);
    if (g.residual != nullptr)
      ok = ok && g.residual_dtype == B200_F32 && aligned_to(g.residual, 16) && g.residual_row_stride % 4 == 0;
    p.fast_ok = ok ? 1 : 0;
  }
  return B200_OK;
}

// Copies a multi-pass K schedule into the kernel parameters (after fill_params set the defaults).
void apply_k_parts(Params& p, const GemmKParts* kp) {
  if (kp == nullptr) return;
  p.k_parts = kp->parts;
  for (int i = 0; i < 3; ++i) { p.a_part_off[i] = kp->a_off[i]; p.b_part_off[i] = kp->b_off[i]; }
}

bool a_is_m_major(const b200_gemm_args& g) { return g.a_col_stride != 1 && g.a_row_stride == 1; }

// A as [m, k] with k contiguous (boxes of 64 k x 128 rows), or as [k, m] with m contiguous (boxes of
// 64 m x 64 k, two per tile).
int32_t encode_a_map(CUtensorMap* map, const b200_gemm_args& g, uint64_t k_extent) {
  if (!a_is_m_major(g)) {
    const uint64_t dims[3] = {k_extent, (uint64_t)g.m, (uint64_t)g.batch};
    const uint64_t strides[2] = {(uint64_t)g.a_row_stride * 2,
                                 (uint64_t)(g.batch > 1 ? g.a_batch_stride : g.a_row_stride * g.m) * 2};
    const uint32_t box[3] = {BK, BM, 1};
    return encode_tensor_map(map, B200_BF16, 3, g.a, dims, strides, box, true);
  }
  const uint64_t dims[3] = {(uint64_t)g.m, k_extent, (uint64_t)g.batch};
  const uint64_t strides[2] = {(uint64_t)g.a_col_stride * 2,
                               (uint64_t)(g.batch > 1 ? g.a_batch_stride : g.a_col_stride * (int64_t)k_extent) * 2};
  const uint32_t box[3] = {64, BK, 1};
  return encode_tensor_map(map, B200_BF16, 3, g.a, dims, strides, box, true);
}

template <int BN, bool B_MN_MAJOR, typename Tout>
int32_t launch_cfg(const b200_gemm_args& g, cudaStream_t stream, const GemmKParts* kp) {
  using C_ = Cfg<BN>;
  CUtensorMap tmap_a, tmap_b;
  const uint64_t k_extent = kp != nullptr ? (uint64_t)kp->k_storage : (uint64_t)g.k;  // K extent of the stored operands
  {
    int32_t st = encode_a_map(&tmap_a, g, k_extent);
    if (st != B200_OK) return st;
  }
  if (!B_MN_MAJOR) {
    // B^T is [n, k] with row pitch b_col_stride.
    const uint64_t dims[3] = {k_extent, (uint64_t)g.n, (uint64_t)g.batch};
    const uint64_t strides[2] = {(uint64_t)g.b_col_stride * 2,
                                 (uint64_t)(g.batch > 1 ? g.b_batch_stride : g.b_col_stride * g.n) * 2};
    const uint32_t box[3] = {BK, BN, 1};
    int32_t st = encode_tensor_map(&tmap_b, B200_BF16, 3, g.b, dims, strides, box, true);
    if (st != B200_OK) return st;
  } else {
    // B is [k, n] with row pitch b_row_stride.
    const uint64_t dims[3] = {(uint64_t)g.n, k_extent, (uint64_t)g.batch};
    const uint64_t strides[2] = {(uint64_t)g.b_row_stride * 2,
                                 (uint64_t)(g.batch > 1 ? g.b_batch_stride : g.b_row_stride * k_extent) * 2};
    const uint32_t box[3] = {64, BK, 1};
    int32_t st = encode_tensor_map(&tmap_b, B200_BF16, 3, g.b, dims, strides, box, true);
    if (st != B200_OK) return st;
  }
  Params p;
  {
    int32_t st = fill_params(g, p, BM, BN, sizeof(Tout));
    if (st != B200_OK) return st;
    apply_k_parts(p, kp);
    p.a_mn_major = a_is_m_major(g) ? 1 : 0;
  }

  auto kernel = gemm_tcgen05_kernel<BN, B_MN_MAJOR, Tout>;
  static thread_local bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::kSmemBytes);
    if (e != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "gemm(tcgen05): cannot opt in to %d bytes of shared memory: %s",
                C_::kSmemBytes, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int64_t grid = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  kernel<<<(unsigned)grid, kThreads, C_::kSmemBytes, stream>>>(tmap_a, tmap_b, static_cast<Tout*>(g.c), p);
  B200_CHECK_LAUNCH("gemm(tcgen05)");
  return B200_OK;
}

// The CTA-pair form: clusters of two CTAs, each pair walking 256 x BN tiles.
template <int BN, bool B_MN_MAJOR, typename Tout>
int32_t launch_pair_cfg(const b200_gemm_args& g, cudaStream_t stream, const GemmKParts* kp) {
  using C_ = Cfg<BN, true>;
  static_assert(C_::kSmemBytes <= 227 * 1024, "pair configuration exceeds the shared memory of an SM");
  CUtensorMap tmap_a, tmap_b;
  const uint64_t k_extent = kp != nullptr ? (uint64_t)kp->k_storage : (uint64_t)g.k;
  {
    int32_t st = encode_a_map(&tmap_a, g, k_extent);
    if (st != B200_OK) return st;
  }
  if (!B_MN_MAJOR) {
    const uint64_t dims[3] = {k_extent, (uint64_t)g.n, (uint64_t)g.batch};
    const uint64_t strides[2] = {(uint64_t)g.b_col_stride * 2,
                                 (uint64_t)(g.batch > 1 ? g.b_batch_stride : g.b_col_stride * g.n) * 2};
    const uint32_t box[3] = {BK, (uint32_t)C_::B_ROWS, 1};
    int32_t st = encode_tensor_map(&tmap_b, B200_BF16, 3, g.b, dims, strides, box, true);
    if (st != B200_OK) return st;
  } else {
    // B is [k, n] with row pitch b_row_stride.
    const uint64_t dims[3] = {(uint64_t)g.n, k_extent, (uint64_t)g.batch};
    const uint64_t strides[2] = {(uint64_t)g.b_row_stride * 2,
                                 (uint64_t)(g.batch > 1 ? g.b_batch_stride : g.b_row_stride * k_extent) * 2};
    const uint32_t box[3] = {64, BK, 1};
    int32_t st = encode_tensor_map(&tmap_b, B200_BF16, 3, g.b, dims, strides, box, true);
    if (st != B200_OK) return st;
  }
  Params p;
  int32_t st = fill_params(g, p, 2 * BM, BN, sizeof(Tout));
  if (st != B200_OK) return st;
  apply_k_parts(p, kp);
  p.a_mn_major = a_is_m_major(g) ? 1 : 0;

  auto kernel = gemm_tcgen05_kernel<BN, B_MN_MAJOR, Tout, true>;
  static thread_local bool attr_set[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C_::kSmemBytes);
    if (e != cudaSuccess)
      B200_FAIL(B200_ERR_CUDA, "gemm(tcgen05 pair): cannot opt in to %d bytes of shared memory: %s",
                C_::kSmemBytes, cudaGetErrorString(e));
    attr_set[dev] = true;
  }
  const int64_t pairs_avail = sm_count() / 2;
  const int64_t pairs = p.num_tiles < pairs_avail ? p.num_tiles : pairs_avail;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C_::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, tmap_a, tmap_b, static_cast<Tout*>(g.c), p);
  if (e != cudaSuccess)
    B200_FAIL(B200_ERR_CUDA, "gemm(tcgen05 pair): launch failed: %s", cudaGetErrorString(e));
  return B200_OK;
}

// Tuning switches, read from the environment on every call only while B200_GEMM_ENV_LIVE is set (the
// tests flip them between calls); otherwise once, at the first GEMM.
struct Tuning {
  int pair_mode;  // B200_GEMM_PAIR: -1 unset, 0 off, 1 forced wherever eligible
  int tile_n;     // B200_GEMM_TILE_N: 0 unset, else 128 | 192 | 256
};

Tuning read_tuning() {
  Tuning t = {-1, 0};
  if (const char* v = getenv("B200_GEMM_PAIR")) t.pair_mode = atoi(v);
  if (const char* v = getenv("B200_GEMM_TILE_N")) {
    const int n = atoi(v);
    if (n == 128 || n == 192 || n == 256) t.tile_n = n;
  }
  return t;
}

Tuning tuning() {
  static const bool live = getenv("B200_GEMM_ENV_LIVE") != nullptr;
  static const Tuning at_load = read_tuning();
  return live ? read_tuning() : at_load;
}

// Whether the CTA-pair kernel is used, and with which tile width (0 = not used).
// B200_GEMM_PAIR=0 turns it off, =1 forces it wherever it is eligible (tuning and tests).
int pick_pair_bn(const b200_gemm_args& g) {
  // MN-major B ([K, N] contiguous) comes in 64-column boxes, so a CTA's half of the tile must be a
  // multiple of 64 columns: tile widths 128 and 256 only.
  const bool mn_major = !b_is_k_major(g);
  const Tuning t = tuning();
  const int mode = t.pair_mode;
  if (mode == 0) return 0;
  // Small problems have too few 256-row tiles to fill 74 pairs; they keep the single-CTA kernel.
  if (mode != 1 && (g.m < 1024 || g.n < 512)) return 0;
  if (t.tile_n != 0) return (mn_major && t.tile_n == 192) ? 0 : t.tile_n;
  const int64_t pairs = sm_count() / 2;
  // Time of a tile ~ (BN + 270) columns' worth: the measured fixed share per tile (issue loop,
  // accumulator hand-off, epilogue) is about as large as the width-proportional part, so wide
  // tiles win unless they cost an extra wave.
  auto cost = [&](int bn) {
    const int64_t tiles = ((g.m + 2 * BM - 1) / (2 * BM)) * ((g.n + bn - 1) / bn) * g.batch;
    const int64_t waves = (tiles + pairs - 1) / pairs;
    return (double)waves * (bn + 270);
  };
  const double c256 = cost(256), c192 = mn_major ? 1e300 : cost(192), c128 = cost(128);
  if (c256 <= c192 && c256 <= c128) return 256;
  return c192 <= c128 ? 192 : 128;
}

// Wave-quantisation cost of a tile width: waves of CTAs times the per-tile cost (main loop
// proportional to BN plus a fixed epilogue/prologue share).
int pick_bn(const b200_gemm_args& g) {
  // B200_GEMM_TILE_N=128|192|256 pins the tile width (tuning and tests).
  if (tuning().tile_n != 0) return tuning().tile_n;
  if (g.n <= 128) return 128;
  const int sms = sm_count();
  // Per-tile cost: the main loop is proportional to BN, but narrower tiles need more operand
  // bytes per flop (1.33x at 128, 1.14x at 192 relative to 256), which is what bounds them; plus
  // a fixed share. The number of waves carries the quantisation loss of the last partial wave.
  auto cost = [&](int bn, double per_col) {
    const int64_t tiles = ((g.m + BM - 1) / BM) * ((g.n + bn - 1) / bn) * g.batch;
    const int64_t waves = (tiles + sms - 1) / sms;
    return (double)waves * (bn * per_col + 24);
  };
  const double c256 = cost(256, 1.0), c192 = cost(192, 1.08), c128 = cost(128, 1.25);
  if (c256 <= c192 && c256 <= c128) return 256;
  return c192 <= c128 ? 192 : 128;
}

}  // namespace

const char* gemm_tcgen05_ineligible(const b200_gemm_args& g) {
  if (g.in_dtype != B200_BF16) return "operands are not bf16";
  if (g.k <= 0) return "k is zero";
  if (g.a_col_stride != 1 && g.a_row_stride != 1) return "A has no unit stride";
  if (!b_is_k_major(g) && !b_is_n_major(g)) return "B has no unit stride";
  if (!aligned_to(g.a, 16) || !aligned_to(g.b, 16)) return "operand pointer not 16-byte aligned";
  if (a_is_m_major(g)) {
    if (g.a_col_stride % 8 != 0 || g.a_col_stride < g.m) return "A column pitch not a multiple of 16 bytes";
  } else if (g.a_row_stride % 8 != 0 || g.a_row_stride < g.k) {
    return "A row pitch not a multiple of 16 bytes";
  }
  if (g.batch > 1 && (g.a_batch_stride % 8 != 0 || g.b_batch_stride % 8 != 0))
    return "batch stride not a multiple of 16 bytes";
  if (b_is_n_major(g)) {
    if (g.b_row_stride % 8 != 0 || g.b_row_stride < g.n) return "B row pitch not a multiple of 16 bytes";
  } else {
    if (g.b_col_stride % 8 != 0 || g.b_col_stride < g.k) return "B column pitch not a multiple of 16 bytes";
  }
  if (g.m > INT32_MAX - 256 || g.n > INT32_MAX - 256 || g.k > INT32_MAX - 256 || g.batch > INT32_MAX)
    return "extent exceeds TMA coordinate range";
  if ((g.bias != nullptr && g.bias_row_stride != 0 && g.batch > 1) || (g.residual != nullptr && g.batch > 1))
    return "matrix bias/residual with batch > 1";
  return nullptr;
}

int32_t launch_gemm_tcgen05(const b200_gemm_args& g, cudaStream_t stream, const GemmKParts* kp) {
  const bool mn = !b_is_k_major(g);
  const bool f32 = g.out_dtype == B200_F32;
  if (const int pbn = pick_pair_bn(g)) {
#define PAIR_LAUNCH(BN_, MN_) \
  (f32 ? launch_pair_cfg<BN_, MN_, float>(g, stream, kp) : launch_pair_cfg<BN_, MN_, __nv_bfloat16>(g, stream, kp))
    if (pbn == 256) return mn ? PAIR_LAUNCH(256, true) : PAIR_LAUNCH(256, false);
    if (pbn == 192) return PAIR_LAUNCH(192, false);
    return mn ? PAIR_LAUNCH(128, true) : PAIR_LAUNCH(128, false);
#undef PAIR_LAUNCH
  }
  const int bn = pick_bn(g);
#define TC_LAUNCH(BN_, MN_)                                                   \
  (f32 ? launch_cfg<BN_, MN_, float>(g, stream, kp) : launch_cfg<BN_, MN_, __nv_bfloat16>(g, stream, kp))
  if (bn == 256) return mn ? TC_LAUNCH(256, true) : TC_LAUNCH(256, false);
  if (bn == 192) return mn ? TC_LAUNCH(192, true) : TC_LAUNCH(192, false);
  return mn ? TC_LAUNCH(128, true) : TC_LAUNCH(128, false);
#undef TC_LAUNCH
}

}  // namespace b200

