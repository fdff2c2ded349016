// Pair form of the tcgen05 3xTF32 GEMM: the two CTAs of a 2-CTA cluster (an SM pair) compute one
// 256 x 256 tile of C with tcgen05.mma.cta_group::2.  Each CTA stages its own 128 rows of A and its
// own 128 of the tile's 256 B rows; the MMA reads B from both CTAs' shared memory, so per SM the
// operand traffic into shared memory and out of it to the tensor pipe is 2/3 of the one-CTA kernel's
// (A 128 + B 128 rows per K-block instead of 128 + 256).  Each CTA keeps the accumulator of its own
// 128 rows in its own TMEM and drains it exactly as the one-CTA kernel does; full tiles are stored with TMA
// (32-row x 16-column bulk tensor stores from the drain warps' swizzled staging tiles, two in flight), ragged ones with plain stores.
//
// Operands, template parameter LO_PLANE:
//   false  the padded [hi | lo] planes of the pre-pass (both operands padded to 256 rows): one TMA box per operand
//          brings both planes
//   true   hi = the caller's tensor read in place (out-of-range parts of a box read as zero, so nothing is padded),
//          lo = a plane of the same layout (written by a one-pass pre-pass, by an earlier product's epilogue, or
//          handed in by the caller): two boxes per operand, same shared-memory layout
// The K-block is a template parameter: 32 (three stages of 64 KiB, K-major rows of 128 bytes in the 128-byte
// swizzle; the default, ~3 % faster) or 16 (six stages of 32 KiB, 64-byte rows; padded planes only).
//
// Roles per CTA (320 threads): warp 0 producer, warp 1 MMA issuer (only in the cluster's CTA 0),
// warps 2-9 drain + epilogue.  Signals:
//   full[s]        lives in CTA 0; CTA 0's producer arms it with the bytes of BOTH CTAs' boxes; every
//                  TMA load of either CTA completes on it (cp.async.bulk.tensor ... .cta_group::2)
//   empty[s]       one in each CTA; the issuer's tcgen05.commit arrives on both (CTA mask 0b11)
//   tmem_full[a]   one in each CTA; committed on both after each K-chunk
//   tmem_empty[a]  lives in CTA 0, 16 arrivals: the 8 drain warps of each CTA (CTA 1's arrive remotely)
// Every wait is bounded as in the one-CTA kernel; a CTA that gives up raises its own abort flag and
// reports; its peer then runs into its own limit.  TMEM is freed by both CTAs after a cluster barrier.
#include "tc_common.cuh"

namespace cleave {

constexpr int kRingBytesPair = 192 * 1024;
template <int BK>
struct PairCfg {
  static constexpr int kPlaneBytes = 128 * BK * 4;         // 128 rows x BK floats: one plane of A, or of half of B
  static constexpr int kStageBytes = 4 * kPlaneBytes;      // [A hi | A lo | B hi | B lo]
  static constexpr int kStages = kRingBytesPair / kStageBytes;   // 6 (BK 16) or 3 (BK 32)
};
constexpr int kPairSmemBytes = kRingBytesPair + kEpiWarps * 32 * 128 + 1024;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in the CTA of rank `rank` (shared::cluster window).
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA loads of a CTA pair: data into this CTA's shared memory, completion on CTA 0's mbarrier.
__device__ __forceinline__ void tma_pair_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0,
                                                 int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_pair_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar_cluster, int c0,
                                                 int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar_cluster), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
// Arrives on the mbarrier at this offset in both CTAs once all MMAs issued so far have retired.
__device__ __forceinline__ void tcgen05_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
      ::"r"(bar), "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ void umma_tf32_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                               uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// M = 256 over the pair, N = 256.
__host__ __device__ constexpr uint32_t instr_desc_pair(bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(256 >> 3) << 17) | ((uint32_t)(256 >> 4) << 24);
}

// Tile index -> (batch, 256-row tile-row, 256-column tile-column), tile-rows in groups of p.pair_group_m.
__device__ __forceinline__ void decode_pair_tile(int t, const TcParams& p, int& b, int& mb, int& nb) {
  const int per_batch = p.mblks * p.nblks;
  b = t / per_batch;
  int r = t - b * per_batch;
  const int group_span = p.pair_group_m * p.nblks;
  const int gid = r / group_span;
  const int first_m = gid * p.pair_group_m;
  const int rows_here = (p.mblks - first_m) < p.pair_group_m ? (p.mblks - first_m) : p.pair_group_m;
  r -= gid * group_span;
  mb = first_m + r % rows_here;
  nb = r / rows_here;
}

// ---- what a cluster works on ------------------------------------------------------------------------------------------
// Whole tiles first: t = cluster + i * clusters over the tiles below the cut region.  The cut region is the last,
// partly filled wave of a product whose tile count is not a multiple of the cluster count: each of its sk_tiles tiles
// is cut along K into sk_slices equal runs of K-blocks and cluster c < sk_tiles * sk_slices takes run c / sk_tiles of
// tile c % sk_tiles, leaving raw partial sums in slot c of p.sk_part; pair_streamk_fixup_kernel adds a tile's runs in
// ascending K order.  All clusters walk K at the same pace, as in a full wave, so operand panels are still shared
// through L2 (handing every cluster an equal share of one long K-block sequence instead -- stream-K proper -- was
// measured slower: clusters then sit at unrelated K offsets and the panels come from DRAM again and again).  Which
// cluster adds which K-blocks is a function of the shape alone, so the result is reproducible.
struct PairItem {
  int tile, kb0, kb1, slot;   // slot < 0: the whole K, result goes to C through the epilogue
};
__device__ __forceinline__ bool pair_item(const TcParams& p, int total_tiles, int cluster_id, int n_clusters, int idx,
                                          PairItem& w) {
  const int whole_tiles = total_tiles - p.sk_tiles;
  const int n_whole = whole_tiles > cluster_id ? (whole_tiles - cluster_id + n_clusters - 1) / n_clusters : 0;
  if (idx < n_whole) {
    w.tile = cluster_id + idx * n_clusters;
    w.kb0 = 0;
    w.kb1 = p.num_kb;
    w.slot = -1;
    return true;
  }
  if (idx > n_whole || cluster_id >= p.sk_tiles * p.sk_slices) return false;
  const int run = cluster_id / p.sk_tiles;
  w.tile = whole_tiles + cluster_id % p.sk_tiles;
  w.kb0 = (int)((long long)p.num_kb * run / p.sk_slices);
  w.kb1 = (int)((long long)p.num_kb * (run + 1) / p.sk_slices);
  w.slot = cluster_id;
  return true;
}

// A drain warp's 32 rows x 128 columns of raw partial sums -> slot `slot` of the partial-sum workspace (a 256 x 256
// tile; this CTA owns rows 128 * rank ..), through the warp's staging tile so that every store instruction writes
// whole 128-byte lines.
__device__ __forceinline__ void store_partial(const float (&sum)[BN / 2], float* ws, int slot, int rank, int q, int half,
                                              int lane, float4* stage) {
  float* block = ws + ((int64_t)slot * 256 + rank * 128 + q * 32) * 256 + half * 128;
#pragma unroll
  for (int pass = 0; pass < BN / 64; ++pass) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      stage[lane * 8 + (j ^ (lane & 7))] = make_float4(sum[32 * pass + 4 * j], sum[32 * pass + 4 * j + 1],
                                                       sum[32 * pass + 4 * j + 2], sum[32 * pass + 4 * j + 3]);
    __syncwarp();
#pragma unroll
    for (int it = 0; it < 8; ++it) {
      const int r = it * 4 + (lane >> 3), slot4 = lane & 7;
      __stcg(reinterpret_cast<float4*>(block + r * 256 + 32 * pass + 4 * slot4), stage[r * 8 + (slot4 ^ (r & 7))]);
    }
    __syncwarp();
  }
}

template <bool A_MN, bool B_MN, int BK, bool LO_PLANE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kGemmThreads, 1)
gemm_3xtf32_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                        const __grid_constant__ CUtensorMap map_c, const __grid_constant__ CUtensorMap map_a_lo,
                        const __grid_constant__ CUtensorMap map_b_lo, TcParams p) {
  constexpr int kPairStages = PairCfg<BK>::kStages;
  constexpr int kPairPlaneBytes = PairCfg<BK>::kPlaneBytes;
  constexpr int kPairStageBytes = PairCfg<BK>::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kPairStages];
  __shared__ __align__(8) uint64_t bar_empty[kPairStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[kAccStages];
  __shared__ __align__(8) uint64_t bar_tmem_empty[kAccStages];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0: issues the MMAs for the pair
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int total_tiles = p.batch * p.mblks * p.nblks;          // 256 x 256 tiles
  const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kPairStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), 2 * kEpiWarps);   // the drain warps of both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    // one warp of each CTA, together: the same columns in both CTAs' TMEM
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  // both CTAs' barriers are initialised and both TMEM allocations exist before anything crosses over
  cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      if constexpr (LO_PLANE) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a_lo) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b_lo) : "memory");
      }
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed[kPairStages];
#pragma unroll
      for (int s = 0; s < kPairStages; ++s) armed[s] = 0;
      bool ok = true;
      PairItem w;
      for (int idx = 0; ok && pair_item(p, total_tiles, cluster_id, n_clusters, idx, w); ++idx) {
        int b, mb, nb;
        decode_pair_tile(w.tile, p, b, mb, nb);
        const int a_row0 = mb * 256 + (int)rank * 128, b_row0 = nb * 256 + (int)rank * 128;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
            report(p.status, 1, 100 + stage, kb);
            ok = false;
            break;
          }
          const uint32_t full_own = smem_u32(&bar_full[stage]);
          const uint32_t full0 = map_to_cta(full_own, 0);
          if (rank == 0) mbar_arrive_expect_tx(full_own, 2 * kPairStageBytes);
          const uint32_t sa = ring + stage * kPairStageBytes, sb = sa + 2 * kPairPlaneBytes;
          if constexpr (LO_PLANE) {
            // hi from the caller's tensor, lo from the plane: same geometry, same coordinates, one plane each
            if (A_MN) {
              tma_pair_load_4d(sa, &map_a, full0, 0, kb * BK, a_row0 / 32, b);
              tma_pair_load_4d(sa + kPairPlaneBytes, &map_a_lo, full0, 0, kb * BK, a_row0 / 32, b);
            } else {
              tma_pair_load_3d(sa, &map_a, full0, kb * BK, a_row0, b);
              tma_pair_load_3d(sa + kPairPlaneBytes, &map_a_lo, full0, kb * BK, a_row0, b);
            }
            if (B_MN) {
              tma_pair_load_4d(sb, &map_b, full0, 0, kb * BK, b_row0 / 32, b);
              tma_pair_load_4d(sb + kPairPlaneBytes, &map_b_lo, full0, 0, kb * BK, b_row0 / 32, b);
            } else {
              tma_pair_load_3d(sb, &map_b, full0, kb * BK, b_row0, b);
              tma_pair_load_3d(sb + kPairPlaneBytes, &map_b_lo, full0, kb * BK, b_row0, b);
            }
          } else {
            if (A_MN) tma_pair_load_4d(sa, &map_a, full0, 0, kb * BK, a_row0 / 32, b * 2);
            else tma_pair_load_3d(sa, &map_a, full0, kb * BK, a_row0, b * 2);
            if (B_MN) tma_pair_load_4d(sb, &map_b, full0, 0, kb * BK, b_row0 / 32, b * 2);
            else tma_pair_load_3d(sb, &map_b, full0, kb * BK, b_row0, b * 2);
          }
#pragma unroll
          for (int s = 0; s < kPairStages; ++s)
            if (s == stage) armed[s]++;
          if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && rank == 0) {
        // Leaving early: give the copies in flight a bounded chance to land (CTA 0 sees their completion).
#pragma unroll
        for (int s = 0; s < kPairStages; ++s) {
          if (armed[s] == 0) continue;
          const uint32_t par = (armed[s] - 1u) & 1u;
          for (int spin = 0; spin < (1 << 20); ++spin)
            if (mbar_try_wait(smem_u32(&bar_full[s]), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (CTA 0 only)
    if (lane == 0 && rank == 0) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      constexpr uint32_t idesc = instr_desc_pair(A_MN, B_MN);
      PairItem w;
      for (int idx = 0; ok && pair_item(p, total_tiles, cluster_id, n_clusters, idx, w); ++idx) {
        for (int kb0 = w.kb0; ok && kb0 < w.kb1; kb0 += p.chunk_kb) {
          if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag)) {
            report(p.status, 2, 200 + acc, w.tile);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          const int kb_end = (kb0 + p.chunk_kb) < w.kb1 ? (kb0 + p.chunk_kb) : w.kb1;
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag)) {
              report(p.status, 3, 300 + stage, kb);
              ok = false;
              break;
            }
            tcgen05_fence_after();
            const uint32_t a_hi = ring + stage * kPairStageBytes;
            const uint32_t a_lo = a_hi + kPairPlaneBytes;
            const uint32_t b_hi = a_hi + 2 * kPairPlaneBytes;
            const uint32_t b_lo = b_hi + kPairPlaneBytes;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              const uint32_t off_a = A_MN ? kk * 1024 : kk * UMMA_K * 4;
              const uint32_t off_b = B_MN ? kk * 1024 : kk * UMMA_K * 4;
              // K-major rows are BK * 4 bytes: 64-byte swizzle (BK 16) or 128-byte swizzle (BK 32), 8-row groups
              constexpr uint32_t kmaj_sbo = 8 * BK * 4, kmaj_lay = BK == 32 ? 2u : 4u;
              constexpr uint32_t sbo_a = A_MN ? 512u : kmaj_sbo, lay_a = A_MN ? 1u : kmaj_lay;
              constexpr uint32_t sbo_b = B_MN ? 512u : kmaj_sbo, lay_b = B_MN ? 1u : kmaj_lay;
              constexpr uint32_t lbo_a = A_MN ? BK * 128u : 16u, lbo_b = B_MN ? BK * 128u : 16u;
              const uint64_t da_hi = make_smem_desc(a_hi + off_a, sbo_a, lay_a, lbo_a);
              const uint64_t da_lo = make_smem_desc(a_lo + off_a, sbo_a, lay_a, lbo_a);
              const uint64_t db_hi = make_smem_desc(b_hi + off_b, sbo_b, lay_b, lbo_b);
              const uint64_t db_lo = make_smem_desc(b_lo + off_b, sbo_b, lay_b, lbo_b);
              umma_tf32_pair(d_tmem, da_lo, db_hi, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
              umma_tf32_pair(d_tmem, da_hi, db_lo, idesc, 1u);
              umma_tf32_pair(d_tmem, da_hi, db_hi, idesc, 1u);
            }
            tcgen05_commit_pair(smem_u32(&bar_empty[stage]));   // both CTAs' stage s reusable once these retire
            if (++stage == kPairStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          tcgen05_commit_pair(smem_u32(&bar_tmem_full[acc]));   // chunk complete, in both CTAs' TMEM
          if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ drain + epilogue (warps 2..9, both CTAs)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = (p.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0);
    float4* stage_tile = reinterpret_cast<float4*>(smem_raw + (ring - smem_u32(smem_raw)) + kRingBytesPair) +
                         (warp - 2) * (32 * 8);
    bool ok = true;
    PairItem w;
    for (int idx = 0; ok && pair_item(p, total_tiles, cluster_id, n_clusters, idx, w); ++idx) {
      int b, mb, nb;
      decode_pair_tile(w.tile, p, b, mb, nb);
      float sum[BN / 2];
#pragma unroll
      for (int j = 0; j < BN / 2; ++j) sum[j] = 0.0f;
      for (int kb0 = w.kb0; kb0 < w.kb1; kb0 += p.chunk_kb) {
        ok = mbar_wait(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 4, 400 + acc, w.tile);
          break;
        }
        tcgen05_fence_after();
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(acc * BN + half * (BN / 2));
#pragma unroll
        for (int cb = 0; cb < BN / 64; ++cb) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + cb * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) sum[cb * 32 + j] = __fadd_rn(sum[cb * 32 + j], __uint_as_float(r[j]));
        }
        tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_tmem_empty[acc]), 0));
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) break;
      if (w.slot < 0)
        tile_epilogue(sum, p, b, mb * 256 + (int)rank * 128, nb, q, half, lane, vec_ok, stage_tile,
                      p.c_tma ? &map_c : nullptr);
      else
        store_partial(sum, p.sk_part, w.slot, (int)rank, q, half, lane, stage_tile);
    }
    // this warp's bulk stores have reached memory before the CTA may exit
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  // ------------------------------------------------------------------ teardown
  // Neither CTA may free its TMEM (or exit, taking its shared memory and barriers along) while its peer
  // can still issue an MMA into it or signal it.
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// Second pass of a product with a cut region: adds the K-runs of each cut tile in ascending K order and
// applies the epilogue exactly as tile_epilogue does (same expressions).  grid = (8 bands of 32 rows, sk_tiles).
__device__ __forceinline__ float sk_epilogue_value(float v, int act) {
  if (act == CLEAVE_ACT_TANH) return tanhf(v);
  if (act == CLEAVE_ACT_SIGMOID) return __fdividef(1.0f, 1.0f + __expf(-v));
  if (act == CLEAVE_ACT_RELU) return act_apply(v, CLEAVE_ACT_RELU);
  return v;
}
__global__ void __launch_bounds__(256) pair_streamk_fixup_kernel(TcParams p) {
  const int r = blockIdx.y;
  const int total_tiles = p.batch * p.mblks * p.nblks;
  int b, mb, nb;
  decode_pair_tile(total_tiles - p.sk_tiles + r, p, b, mb, nb);
  const bool vec = (p.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0) &&
                   (p.c_lo == nullptr || (reinterpret_cast<uintptr_t>(p.c_lo) & 15u) == 0);
#pragma unroll 2
  for (int j = 0; j < 8; ++j) {
    const int idx = threadIdx.x + 256 * j;          // 32 rows x 64 four-column groups
    const int row_t = blockIdx.x * 32 + (idx >> 6), c4 = idx & 63;
    const int grow = mb * 256 + row_t, gcol = nb * 256 + 4 * c4;
    if (grow >= p.m || gcol >= p.n) continue;
    const float4* part = reinterpret_cast<const float4*>(p.sk_part + ((int64_t)r * 256 + row_t) * 256) + c4;
    float4 acc = __ldcg(part);
    for (int run = 1; run < p.sk_slices; ++run) {
      const float4 v = __ldcg(part + (int64_t)run * p.sk_tiles * (256 * 256 / 4));
      acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    float o[4] = {acc.x, acc.y, acc.z, acc.w};
    const int64_t at = ((int64_t)b * p.m + grow) * (int64_t)p.n + gcol;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      if (gcol + e >= p.n) break;
      if (p.bias != nullptr) o[e] = __fadd_rn(o[e], __ldg(p.bias + gcol + e));
      o[e] = sk_epilogue_value(o[e], p.act);
      if (p.dact_y != nullptr) o[e] = dact_apply(__ldg(p.dact_y + at + e), o[e], p.dact);
    }
    if (vec && gcol + 4 <= p.n) {
      *reinterpret_cast<float4*>(p.c + at) = make_float4(o[0], o[1], o[2], o[3]);
      if (p.c_lo != nullptr)
        *reinterpret_cast<float4*>(p.c_lo + at) = make_float4(split_lo(o[0]), split_lo(o[1]), split_lo(o[2]), split_lo(o[3]));
    } else {
      for (int e = 0; e < 4 && gcol + e < p.n; ++e) {
        p.c[at + e] = o[e];
        if (p.c_lo != nullptr) p.c_lo[at + e] = split_lo(o[e]);
      }
    }
  }
}

// Cut region for this launch: *slices = K-runs per tile (0: none), returns the tiles of the region.  It pays when the
// last wave fills at most half of the SM pairs (so every tile gets at least two runs) and the K-blocks saved,
// num_kb * (1 - 1/slices), outweigh the second pass (measured: ~9 us, i.e. ~9 K-blocks of 32): at least 16, or what
// CLEAVE_CUDA_GEMM_CUT_MIN_KB says (4096 x 4096 x K1024, 34 tiles cut in two: 163 -> 156 us).
// CLEAVE_CUDA_GEMM_STREAMK=0 turns it off.
int gemm_cut_plan(int tiles, int num_kb, int sm_pairs, int* slices) {
  static const bool on = !(getenv("CLEAVE_CUDA_GEMM_STREAMK") && getenv("CLEAVE_CUDA_GEMM_STREAMK")[0] == '0');
  *slices = 0;
  if (!on || tiles <= 0 || num_kb <= 0 || sm_pairs <= 0) return 0;
  const int rem = tiles % sm_pairs;
  if (tiles < sm_pairs || rem == 0) return 0;
  int s = sm_pairs / rem;
  if (s > 8) s = 8;
  while (s > 2 && num_kb / s < 8) --s;   // runs of at least 8 K-blocks (one accumulation chunk)
  static const int min_saved = [] {
    const char* e = getenv("CLEAVE_CUDA_GEMM_CUT_MIN_KB");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 16;
  }();
  if (s < 2 || (int64_t)num_kb * (s - 1) < (int64_t)min_saved * s || num_kb / s < 8) return 0;
  *slices = s;
  return rem;
}

template <bool A_MN, bool B_MN, int BK, bool LO_PLANE>
static bool run_pair(const CUtensorMap* maps, const TcParams& p_in) {
  static bool attr_set = false;
  if (!attr_set) {
    if (!cuda_ok(cudaFuncSetAttribute(gemm_3xtf32_pair_kernel<A_MN, B_MN, BK, LO_PLANE>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemBytes),
                 "cudaFuncSetAttribute(pair gemm)"))
      return false;
    attr_set = true;
  }
  TcParams p = p_in;
  const int tiles = p.batch * p.mblks * p.nblks;
  const int sm_pairs = ctx().sm_count / 2;
  p.sk_tiles = gemm_cut_plan(tiles, p.num_kb, sm_pairs, &p.sk_slices);
  const int clusters = tiles < sm_pairs ? tiles : sm_pairs;
  if (p.sk_tiles) {
    p.sk_part = scratch_alloc((int64_t)p.sk_tiles * p.sk_slices * 256 * 256 * sizeof(float));
    if (!p.sk_part) return false;
  }
  profile_mark(true);
  gemm_3xtf32_pair_kernel<A_MN, B_MN, BK, LO_PLANE>
      <<<2 * clusters, kGemmThreads, kPairSmemBytes, ctx().stream>>>(maps[0], maps[1], maps[2], maps[3], maps[4], p);
  count_launch();
  bool ok = cuda_ok(cudaGetLastError(), "tcgen05 pair GEMM launch");
  if (ok && p.sk_tiles) {
    pair_streamk_fixup_kernel<<<dim3(8, p.sk_tiles), 256, 0, ctx().stream>>>(p);
    count_launch();
    ok = cuda_ok(cudaGetLastError(), "stream-K second pass launch");
  }
  profile_mark(false);
  if (p.sk_part) scratch_free(p.sk_part);
  return ok;
}

template <int BK, bool LO_PLANE>
static bool run_pair_bk(bool a_mn, bool b_mn, const CUtensorMap* maps, const TcParams& p) {
  return a_mn ? (b_mn ? run_pair<true, true, BK, LO_PLANE>(maps, p) : run_pair<true, false, BK, LO_PLANE>(maps, p))
              : (b_mn ? run_pair<false, true, BK, LO_PLANE>(maps, p) : run_pair<false, false, BK, LO_PLANE>(maps, p));
}

// maps = {A, B, C, A lo, B lo}; the last two are read in lo-plane mode only.
bool run_tc_pair(bool a_mn, bool b_mn, const CUtensorMap* maps, const TcParams& p, int bk, bool lo_plane) {
  if (lo_plane) return run_pair_bk<32, true>(a_mn, b_mn, maps, p);
  return bk == 32 ? run_pair_bk<32, false>(a_mn, b_mn, maps, p) : run_pair_bk<16, false>(a_mn, b_mn, maps, p);
}

// ---- short K ------------------------------------------------------------------------------------------------------
// With K <= 256 a tile is one accumulation chunk: 2 us of MMAs at K = 64, against ~3.3 us that the memory system
// needs for a CTA's 128 KiB of the tile when all SMs store at once, and in the kernel above the 8 drain warps
// cannot start on the next accumulator before their last store has left (measured at 16384 x 16384 x K64: 4.7 us per
// tile, tensor pipe 33 % busy, DRAM 41 %).  This variant has 16 drain warps in two groups of 8, one group per TMEM
// accumulator: while one group stores tile t the other drains and stores tile t + 1, so the stores of a CTA never
// pause.  No running sums (the single chunk goes from TMEM through a staging tile into a bulk store, 32 columns at a
// time, the next TMEM load in flight meanwhile), hence few registers.  Shared memory: a two-stage ring (128 KiB; a
// tile is at most 8 K-blocks and the MMAs of one tile overlap the loads of the next) + 64 KiB of staging tiles.
// Plain products only (no bias, activation, derivative or lo-plane output); padded [hi | lo] planes, K-block 32.
constexpr int kShortDrainWarps = 16;
constexpr int kShortThreads = 64 + 32 * kShortDrainWarps;        // producer, issuer, 16 drain warps
constexpr int kShortStages = 2;
constexpr int kShortRingBytes = kShortStages * PairCfg<32>::kStageBytes;                    // 128 KiB
constexpr int kShortSmemBytes = kShortRingBytes + kShortDrainWarps * 32 * 128 + 1024;

template <bool A_MN, bool B_MN>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kShortThreads, 1)
gemm_3xtf32_pair_shortk_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                               const __grid_constant__ CUtensorMap map_c, TcParams p) {
  constexpr int BK = 32;
  constexpr int kPlaneBytes = PairCfg<BK>::kPlaneBytes;
  constexpr int kStageBytes = PairCfg<BK>::kStageBytes;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[kShortStages];
  __shared__ __align__(8) uint64_t bar_empty[kShortStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[kAccStages];
  __shared__ __align__(8) uint64_t bar_tmem_empty[kAccStages];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int total_tiles = p.batch * p.mblks * p.nblks;
  const int n_clusters = gridDim.x >> 1, cluster_id = blockIdx.x >> 1;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < kShortStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), kShortDrainWarps);   // the 8 warps of its drain group, in both CTAs
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed[kShortStages] = {0, 0};
      bool ok = true;
      for (int t = cluster_id; ok && t < total_tiles; t += n_clusters) {
        int b, mb, nb;
        decode_pair_tile(t, p, b, mb, nb);
        const int a_row0 = mb * 256 + (int)rank * 128, b_row0 = nb * 256 + (int)rank * 128;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
            report(p.status, 1, 100 + stage, kb);
            ok = false;
            break;
          }
          const uint32_t full_own = smem_u32(&bar_full[stage]);
          const uint32_t full0 = map_to_cta(full_own, 0);
          if (rank == 0) mbar_arrive_expect_tx(full_own, 2 * kStageBytes);
          const uint32_t sa = ring + stage * kStageBytes, sb = sa + 2 * kPlaneBytes;
          if (A_MN) tma_pair_load_4d(sa, &map_a, full0, 0, kb * BK, a_row0 / 32, b * 2);
          else tma_pair_load_3d(sa, &map_a, full0, kb * BK, a_row0, b * 2);
          if (B_MN) tma_pair_load_4d(sb, &map_b, full0, 0, kb * BK, b_row0 / 32, b * 2);
          else tma_pair_load_3d(sb, &map_b, full0, kb * BK, b_row0, b * 2);
          armed[stage]++;
          if (++stage == kShortStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok && rank == 0) {
        for (int s = 0; s < kShortStages; ++s) {
          if (armed[s] == 0) continue;
          const uint32_t par = (armed[s] - 1u) & 1u;
          for (int spin = 0; spin < (1 << 20); ++spin)
            if (mbar_try_wait(smem_u32(&bar_full[s]), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (CTA 0 only): one chunk per tile
    if (lane == 0 && rank == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      constexpr uint32_t idesc = instr_desc_pair(A_MN, B_MN);
      for (int t = cluster_id; ok && t < total_tiles; t += n_clusters) {
        if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag)) {
          report(p.status, 2, 200 + acc, t);
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag)) {
            report(p.status, 3, 300 + stage, kb);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t a_hi = ring + stage * kStageBytes;
          const uint32_t a_lo = a_hi + kPlaneBytes;
          const uint32_t b_hi = a_hi + 2 * kPlaneBytes;
          const uint32_t b_lo = b_hi + kPlaneBytes;
#pragma unroll
          for (int kk = 0; kk < BK / UMMA_K; ++kk) {
            const uint32_t off_a = A_MN ? kk * 1024 : kk * UMMA_K * 4;
            const uint32_t off_b = B_MN ? kk * 1024 : kk * UMMA_K * 4;
            constexpr uint32_t kmaj_sbo = 8 * BK * 4, kmaj_lay = 2u;
            constexpr uint32_t sbo_a = A_MN ? 512u : kmaj_sbo, lay_a = A_MN ? 1u : kmaj_lay;
            constexpr uint32_t sbo_b = B_MN ? 512u : kmaj_sbo, lay_b = B_MN ? 1u : kmaj_lay;
            constexpr uint32_t lbo_a = A_MN ? BK * 128u : 16u, lbo_b = B_MN ? BK * 128u : 16u;
            const uint64_t da_hi = make_smem_desc(a_hi + off_a, sbo_a, lay_a, lbo_a);
            const uint64_t da_lo = make_smem_desc(a_lo + off_a, sbo_a, lay_a, lbo_a);
            const uint64_t db_hi = make_smem_desc(b_hi + off_b, sbo_b, lay_b, lbo_b);
            const uint64_t db_lo = make_smem_desc(b_lo + off_b, sbo_b, lay_b, lbo_b);
            umma_tf32_pair(d_tmem, da_lo, db_hi, idesc, (kb != 0 || kk != 0) ? 1u : 0u);
            umma_tf32_pair(d_tmem, da_hi, db_lo, idesc, 1u);
            umma_tf32_pair(d_tmem, da_hi, db_hi, idesc, 1u);
          }
          tcgen05_commit_pair(smem_u32(&bar_empty[stage]));
          if (++stage == kShortStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tcgen05_commit_pair(smem_u32(&bar_tmem_full[acc]));
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ drain + store: two groups of 8 warps
    // Group g (warps 2 + 8g .. 9 + 8g) owns accumulator g and with it every second tile of the cluster; a warp takes
    // 32 rows x 128 columns in four 32-column pieces, each from TMEM through its staging tile into a bulk store, and
    // hands the accumulator back after the last TMEM load.
    const int q = warp & 3;                       // TMEM lane quarter this warp may read
    const int grp = (warp - 2) >> 3;              // accumulator / tile parity
    const int half = ((warp - 2) >> 2) & 1;       // which 128 of the tile's 256 columns
    uint32_t acc_phase = 0;
    const bool vec_ok = (p.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0);
    float4* stage_tile = reinterpret_cast<float4*>(smem_raw + (ring - smem_u32(smem_raw)) + kShortRingBytes) +
                         (warp - 2) * (32 * 8);
    const uint32_t stage_addr = smem_u32(stage_tile);
    int i = 0;
    for (int t = cluster_id; t < total_tiles; t += n_clusters, ++i) {
      if ((i & 1) != grp) continue;
      int b, mb, nb;
      decode_pair_tile(t, p, b, mb, nb);
      bool ok = mbar_wait(smem_u32(&bar_tmem_full[grp]), acc_phase, &abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        if (lane == 0) report(p.status, 4, 400 + grp, t);
        break;
      }
      acc_phase ^= 1u;
      tcgen05_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(grp * BN + half * 128);
      const int tile_row0 = mb * 256 + (int)rank * 128;
      const int row = tile_row0 + q * 32 + lane;
      const int col0 = nb * 256 + half * 128;
      const bool full_tile = (tile_row0 + 128 <= p.m) && (nb * 256 + 256 <= p.n);
      const bool bulk = full_tile && p.c_tma;
      float* crow = p.c + ((int64_t)b * p.m + row) * (int64_t)p.n + col0;
      uint32_t r[2][32];
      tmem_ld_32x32(taddr, r[0]);
#pragma unroll
      for (int piece = 0; piece < 4; ++piece) {
        tmem_ld_wait_for(r[piece & 1]);                                   // piece `piece` has arrived
        if (piece < 3) {
          tmem_ld_32x32(taddr + (piece + 1) * 32, r[(piece + 1) & 1]);    // in flight while this piece is stored
        } else {
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&bar_tmem_empty[grp]), 0));
        }
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __fadd_rn(0.0f, __uint_as_float(r[piece & 1][j]));   // as the chunked kernels do
        if (bulk) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            stage_tile[lane * 8 + (j ^ (lane & 7))] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp();
          if (lane == 0) {
            asm volatile(
                "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                ::"l"(&map_c), "r"(stage_addr), "r"(col0 + 32 * piece), "r"(tile_row0 + q * 32), "r"(b)
                : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          }
          __syncwarp();
        } else if (row < p.m) {
          const int c0 = col0 + 32 * piece;
          if (vec_ok && c0 + 32 <= p.n) {
            float4* dst = reinterpret_cast<float4*>(crow + 32 * piece);
#pragma unroll
            for (int j = 0; j < 8; ++j) dst[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
              if (c0 + j < p.n) crow[32 * piece + j] = v[j];
          }
        }
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
  }

  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

template <bool A_MN, bool B_MN>
static bool run_pair_shortk(const CUtensorMap* maps, const TcParams& p) {
  static bool attr_set = false;
  if (!attr_set) {
    if (!cuda_ok(cudaFuncSetAttribute(gemm_3xtf32_pair_shortk_kernel<A_MN, B_MN>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, kShortSmemBytes),
                 "cudaFuncSetAttribute(short-K pair gemm)"))
      return false;
    attr_set = true;
  }
  const int tiles = p.batch * p.mblks * p.nblks;
  int clusters = ctx().sm_count / 2;
  if (tiles < clusters) clusters = tiles;
  profile_mark(true);
  gemm_3xtf32_pair_shortk_kernel<A_MN, B_MN>
      <<<2 * clusters, kShortThreads, kShortSmemBytes, ctx().stream>>>(maps[0], maps[1], maps[2], p);
  profile_mark(false);
  count_launch();
  return cuda_ok(cudaGetLastError(), "tcgen05 short-K pair GEMM launch");
}

// Padded planes (K-block 32), one accumulation chunk (K_padded <= 256), plain product.  maps = {A planes, B planes, C}.
bool run_tc_pair_shortk(bool a_mn, bool b_mn, const CUtensorMap* maps, const TcParams& p) {
  return a_mn ? (b_mn ? run_pair_shortk<true, true>(maps, p) : run_pair_shortk<true, false>(maps, p))
              : (b_mn ? run_pair_shortk<false, true>(maps, p) : run_pair_shortk<false, false>(maps, p));
}

}  // namespace cleave
