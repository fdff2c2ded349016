// Tensor-core f32 GEMM for sm_100a: tcgen05.mma (kind::tf32) with TMEM accumulators, operands
// staged by TMA into a multi-stage shared-memory ring guarded by mbarriers, and a 3xTF32
// split so that the f32 result stays within rounding distance of the reference's f32 loop.
//
// Split precision.  Every f32 operand value x is used as hi + lo and a*b is accumulated as
// a_lo*b_hi + a_hi*b_lo + a_hi*b_hi in the f32 TMEM accumulator.  Two ways to get the planes:
//   pre-pass path   hi = tf32(x) (round to nearest), lo = tf32(x - hi); dropped a_lo*b_lo and the
//                   rounding of lo are each <= 2^-22 |a b|
//   direct path     hi = x as the tensor pipe reads it: the pipe ignores the 13 low mantissa bits of an
//                   f32 operand (measured), i.e. truncates; lo = tf32(x - truncate(x)), exact
//                   subtraction, so the terms above are <= 2^-20 / 2^-21 |a b|
// Both stay an order of magnitude inside the 1e-5 tolerance (measured ~5e-7 componentwise).
//
// Data path, pre-pass.  split_copy_kernel writes both operands as two planes [hi | lo], padded
// (rows to the tile height, K to 32) and zero-filled so every TMA box is in bounds; an operand whose
// contraction index is strided keeps its [K][rows] order and is read as an MN-major operand.
// Data path, direct.  TMA reads the caller's tensors themselves (16-byte aligned, contiguous extent
// a multiple of 4; out-of-range parts of a box read as zero) into a deep ring of raw stages, and
// four "split" warps write the lo planes of each stage into a second, shallow ring just ahead of
// the MMAs.  No workspace and no extra HBM pass, but the split warps' shared-memory traffic competes
// with the MMAs' operand reads, so the kernel itself runs ~1.2x longer: the host picks this path
// for small and narrow problems, where the pre-pass would cost more than that.
//
// Kernel.  Persistent, one CTA per SM; 320 threads (pre-pass path) or 512 (direct path):
//   producer    one elected lane: per K-block one TMA box per operand -> shared memory, completion
//               on the stage's "full" mbarrier
//   MMA issuer  one elected lane: 3 x (BK/8) tcgen05.mma per K-block into one of two 128x256 f32
//               accumulators in TMEM; tcgen05.commit releases the stage ("empty") and, after each
//               K-chunk, publishes the accumulator ("tmem_full").  On the last tile column the
//               MMA's N shrinks to the live columns of C.
//   8 drain     after every K-chunk (256 values of k) tcgen05.ld the chunk's partial sums and add
//   warps       them, round-to-nearest, to 128 running sums per thread in registers; hand the
//               accumulator back ("tmem_empty"); after the last chunk apply bias + activation and
//               store C through a swizzled shared tile with full 128-byte lines
//   4 split     direct path only: raw stage -> lo stage, then fence.proxy.async and an arrival on
//   warps       the lo stage's "lo_full" mbarrier, which the issuer waits for
// On the direct path the warps form four warpgroups and registers move (setmaxnreg) from the
// producer/issuer and split groups to the drain groups.
// The two TMEM accumulators alternate per chunk, so draining chunk i overlaps the MMAs of
// chunk i+1 (and the stores of one tile overlap the first chunk of the next).
//
// Why chunks.  The tensor pipe adds into its f32 accumulator with truncation, not round to
// nearest (measured: at K = 8192 a single accumulation chain ends ~1e-3 too close to zero, a bias
// linear in K and 14x the error of the reference's f32 loop).  Restarting the chain every 256 k
// and summing the chunks in registers with round-to-nearest keeps each chain short and its
// partial sums small, which brings the error below that of the reference loop itself.
// Tiles are visited in groups of 16 tile-rows so that the ~148 tiles in flight share operand
// panels through L2.
//
// Every mbarrier wait is bounded (wall-clock limit on %globaltimer).  A wait that gives up sets a
// CTA-wide abort flag and a status word the host reads; the CTA then drains its own TMA copies
// (bounded), frees its TMEM and returns, so the context stays usable.
#include <cuda.h>

#include <cstdio>
#include <utility>
#include <vector>

#include "common.cuh"
#include "gemm.cuh"
#include "tc_common.cuh"

namespace cleave {

// PATH: where the hi / lo planes of a stage come from.
constexpr int kPathPlanes = 0;   // pre-pass wrote padded [hi | lo] planes; one TMA box per operand brings both
constexpr int kPathDirect = 1;   // TMA brings the caller's raw tile (= hi); split warps write lo in shared memory
constexpr int kPathLoPlane = 2;  // TMA brings the raw tile (= hi) from the caller's tensor and lo from a plane
                                 // that a one-pass pre-pass wrote in the same (unpadded) layout

template <int BK, bool A_MN, bool B_MN, int PATH>
__global__ void __launch_bounds__(PATH == kPathDirect ? kDirectThreads : kGemmThreads, 1)
gemm_3xtf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                   const __grid_constant__ CUtensorMap map_a_lo, const __grid_constant__ CUtensorMap map_b_lo,
                   TcParams p) {
  constexpr bool DIRECT = PATH == kPathDirect;
  using C = Cfg<BK, DIRECT>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];
  __shared__ __align__(8) uint64_t bar_lo_full[C::kLoStages];    // direct path: lo planes written
  __shared__ __align__(8) uint64_t bar_lo_empty[C::kLoStages];   // direct path: lo planes consumed
  __shared__ __align__(8) uint64_t bar_tmem_full[kAccStages];
  __shared__ __align__(8) uint64_t bar_tmem_empty[kAccStages];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  constexpr int kDrainFirst = DIRECT ? 4 : 2;                 // first of the kEpiWarps drain warps
  constexpr int kSplitFirst = kDrainFirst + kEpiWarps;        // direct path only
  // Operand ring, 1024-byte aligned (the swizzle pattern is a function of address bits 4-9).
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int total_tiles = p.batch * p.mblks * p.nblks;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
    }
    for (int s = 0; s < C::kLoStages; ++s) {
      mbar_init(smem_u32(&bar_lo_full[s]), 32 * kSplitWarps);   // every split thread arrives
      mbar_init(smem_u32(&bar_lo_empty[s]), 1);
    }
    for (int a = 0; a < kAccStages; ++a) {
      mbar_init(smem_u32(&bar_tmem_full[a]), 1);
      mbar_init(smem_u32(&bar_tmem_empty[a]), kEpiWarps);   // one arrival per drain warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)),
                 "r"((uint32_t)kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = tmem_slot;

  if (warp < kDrainFirst) {
  if constexpr (DIRECT) asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsLight));
  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
      if constexpr (PATH == kPathLoPlane) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a_lo) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b_lo) : "memory");
      }
      int stage = 0;
      uint32_t phase = 0;
      uint32_t armed[C::kStages];
#pragma unroll
      for (int s = 0; s < C::kStages; ++s) armed[s] = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        int b, mb, nb;
        decode_tile(t, p, b, mb, nb);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(smem_u32(&bar_empty[stage]), phase ^ 1u, &abort_flag)) {
            report(p.status, 1, 100 + stage, kb);
            ok = false;
            break;
          }
          const uint32_t full = smem_u32(&bar_full[stage]);
          const uint32_t sa = ring + stage * C::kStageBytes;
          if constexpr (DIRECT) {
            // Raw f32 tiles straight from the caller's tensors (out-of-range parts read as zero).
            // An MN-major tile is fetched as 32-wide blocks of BK rows x 128 bytes.
            const uint32_t sb = sa + C::kABytes;
            mbar_arrive_expect_tx(full, C::kABytes + p.b_box_rows * C::kRowBytes);
            if (A_MN) {
              if (p.a_blocked) {
                tma_load_4d(sa, &map_a, full, 0, kb * BK, mb * (BM / 32), b);
              } else {
#pragma unroll
                for (int j = 0; j < BM / 32; ++j)
                  tma_load_3d(sa + j * (BK * 128), &map_a, full, mb * BM + j * 32, kb * BK, b);
              }
            } else if (p.a_sliced) {
              tma_load_3d(sa, &map_a, full, kb * BK, b, mb * BM);   // K-sliced view: {k in slice, slice, row}
            } else {
              tma_load_3d(sa, &map_a, full, kb * BK, mb * BM, b);
            }
            if (B_MN) {
              if (p.b_blocked) {
                tma_load_4d(sb, &map_b, full, 0, kb * BK, nb * (BN / 32), b);
              } else {
#pragma unroll
                for (int j = 0; j < BN / 32; ++j)
                  if (j * 32 < p.b_box_rows) tma_load_3d(sb + j * (BK * 128), &map_b, full, nb * BN + j * 32, kb * BK, b);
              }
            } else if (p.b_sliced) {
              // K-sliced view of a row-major operand: the map's dimensions are {k in slice, slice, row}
              tma_load_3d(sb, &map_b, full, kb * BK, b, nb * BN);
            } else {
              tma_load_3d(sb, &map_b, full, kb * BK, nb * BN, b);
            }
          } else if constexpr (PATH == kPathLoPlane) {
            // hi from the caller's tensor, lo from the lo plane: same geometry, same coordinates
            // (an MN-major operand reaches this path only in its blocked, one-box form)
            mbar_arrive_expect_tx(full, C::kStageBytes);
            const uint32_t sb = sa + 2 * C::kABytes;
            if (A_MN) {
              tma_load_4d(sa, &map_a, full, 0, kb * BK, mb * (BM / 32), b);
              tma_load_4d(sa + C::kABytes, &map_a_lo, full, 0, kb * BK, mb * (BM / 32), b);
            } else {
              tma_load_3d(sa, &map_a, full, kb * BK, mb * BM, b);
              tma_load_3d(sa + C::kABytes, &map_a_lo, full, kb * BK, mb * BM, b);
            }
            if (B_MN) {
              tma_load_4d(sb, &map_b, full, 0, kb * BK, nb * (BN / 32), b);
              tma_load_4d(sb + C::kBBytes, &map_b_lo, full, 0, kb * BK, nb * (BN / 32), b);
            } else {
              tma_load_3d(sb, &map_b, full, kb * BK, nb * BN, b);
              tma_load_3d(sb + C::kBBytes, &map_b_lo, full, kb * BK, nb * BN, b);
            }
          } else {
            mbar_arrive_expect_tx(full, C::kStageBytes);
            if (A_MN) tma_load_4d(sa, &map_a, full, 0, kb * BK, mb * (BM / 32), b * 2);
            else tma_load_3d(sa, &map_a, full, kb * BK, mb * BM, b * 2);
            if (B_MN) tma_load_4d(sa + 2 * C::kABytes, &map_b, full, 0, kb * BK, nb * (BN / 32), b * 2);
            else tma_load_3d(sa + 2 * C::kABytes, &map_b, full, kb * BK, nb * BN, b * 2);
          }
#pragma unroll
          for (int s = 0; s < C::kStages; ++s)
            if (s == stage) armed[s]++;
          if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        }
      }
      if (!ok) {
        // Leaving early: give this CTA's copies in flight a bounded chance to land before the
        // shared memory they target is released.
#pragma unroll
        for (int s = 0; s < C::kStages; ++s) {
          if (armed[s] == 0) continue;
          const uint32_t par = (armed[s] - 1u) & 1u;
          for (int spin = 0; spin < (1 << 20); ++spin)
            if (mbar_try_wait(smem_u32(&bar_full[s]), par)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      int stage = 0, slot = 0;
      uint32_t phase = 0, lo_phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        // Columns past the edge of C need no arithmetic: the MMA's N shrinks to the live part of
        // the tile (a multiple of 16); the accumulator columns beyond it are never stored.
        int tb, tmb, tnb;
        decode_tile(t, p, tb, tmb, tnb);
        const int live_n = (p.n - tnb * BN) < BN ? (p.n - tnb * BN) : BN;
        const uint32_t idesc = instr_desc(A_MN, B_MN, (live_n + 15) & ~15);
        for (int kb0 = 0; ok && kb0 < p.num_kb; kb0 += p.chunk_kb) {
          if (!mbar_wait(smem_u32(&bar_tmem_empty[acc]), acc_phase ^ 1u, &abort_flag)) {
            report(p.status, 2, 200 + acc, t);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
          const int kb_end = (kb0 + p.chunk_kb) < p.num_kb ? (kb0 + p.chunk_kb) : p.num_kb;
          for (int kb = kb0; kb < kb_end; ++kb) {
            if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag) ||
                (DIRECT && !mbar_wait(smem_u32(&bar_lo_full[slot]), lo_phase, &abort_flag))) {
              report(p.status, 3, 300 + stage, kb);
              ok = false;
              break;
            }
            tcgen05_fence_after();
            const uint32_t a_hi = ring + stage * C::kStageBytes;
            const uint32_t a_lo = DIRECT ? ring + C::kLoRingOffset + slot * (C::kABytes + C::kBBytes) : a_hi + C::kABytes;
            const uint32_t b_hi = DIRECT ? a_hi + C::kABytes : a_hi + 2 * C::kABytes;
            const uint32_t b_lo = DIRECT ? a_lo + C::kABytes : b_hi + C::kBBytes;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // K-major: 32 bytes along K inside the swizzled row; MN-major: the next 8-row group
              const uint32_t off_a = A_MN ? kk * 1024 : kk * UMMA_K * 4;
              const uint32_t off_b = B_MN ? kk * 1024 : kk * UMMA_K * 4;
              constexpr uint32_t sbo_a = A_MN ? 512u : C::kSBO, lay_a = A_MN ? 1u : C::kLayoutType;
              constexpr uint32_t sbo_b = B_MN ? 512u : C::kSBO, lay_b = B_MN ? 1u : C::kLayoutType;
              constexpr uint32_t lbo_a = A_MN ? BK * 128u : 16u, lbo_b = B_MN ? BK * 128u : 16u;
              const uint64_t da_hi = make_smem_desc(a_hi + off_a, sbo_a, lay_a, lbo_a);
              const uint64_t da_lo = make_smem_desc(a_lo + off_a, sbo_a, lay_a, lbo_a);
              const uint64_t db_hi = make_smem_desc(b_hi + off_b, sbo_b, lay_b, lbo_b);
              const uint64_t db_lo = make_smem_desc(b_lo + off_b, sbo_b, lay_b, lbo_b);
              // the first MMA of a chunk overwrites the accumulator; small terms go first
              umma_tf32(d_tmem, da_lo, db_hi, idesc, (kb != kb0 || kk != 0) ? 1u : 0u);
              umma_tf32(d_tmem, da_hi, db_lo, idesc, 1u);
              umma_tf32(d_tmem, da_hi, db_hi, idesc, 1u);
            }
            tcgen05_commit(smem_u32(&bar_empty[stage]));   // stage reusable once these MMAs retire
            if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
            if constexpr (DIRECT) {
              tcgen05_commit(smem_u32(&bar_lo_empty[slot]));
              if (++slot == C::kLoStages) { slot = 0; lo_phase ^= 1u; }
            }
          }
          if (!ok) break;
          tcgen05_commit(smem_u32(&bar_tmem_full[acc]));   // chunk complete
          if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
  }
  } else if (DIRECT && warp >= kSplitFirst) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kRegsSplit));
    // ------------------------------------------------------------------ operand split (warps 12..15)
    // The tensor pipe reads an f32 operand as tf32 by dropping its 13 low mantissa bits, so the raw
    // tile itself serves as the hi plane.  These warps write the matching lo plane,
    // lo = tf32(x - truncate(x)), at the same (swizzled) offsets of the stage's lo buffers; the
    // subtraction is exact.  A non-finite x gives lo = NaN, as documented for this path.
    const int st = threadIdx.x - 32 * kSplitFirst;
    uint8_t* ring_ptr = smem_raw + (ring - smem_u32(smem_raw));
    int stage = 0, slot = 0;
    uint32_t phase = 0, lo_phase = 0;
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      for (int kb = 0; kb < p.num_kb; ++kb) {
        if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag) ||
            !mbar_wait(smem_u32(&bar_lo_empty[slot]), lo_phase ^ 1u, &abort_flag)) {
          if (lane == 0) report(p.status, 6, 600 + stage, kb);
          ok = false;
          break;
        }
        const float4* a_raw = reinterpret_cast<const float4*>(ring_ptr + stage * C::kStageBytes);
        const float4* b_raw = a_raw + C::kABytes / 16;
        float4* a_lo = reinterpret_cast<float4*>(ring_ptr + C::kLoRingOffset + slot * (C::kABytes + C::kBBytes));
        float4* b_lo = a_lo + C::kABytes / 16;
        constexpr int kA4 = C::kABytes / 16 / (32 * kSplitWarps), kB4 = C::kBBytes / 16 / (32 * kSplitWarps);
        float4 v[kA4 + kB4];
#pragma unroll
        for (int i = 0; i < kA4; ++i) v[i] = a_raw[st + i * 32 * kSplitWarps];
        const int b_f4 = p.b_box_rows * (C::kRowBytes / 16);   // 16-byte words of B present in the stage
#pragma unroll
        for (int i = 0; i < kB4; ++i)
          if (st + i * 32 * kSplitWarps < b_f4) v[kA4 + i] = b_raw[st + i * 32 * kSplitWarps];
#pragma unroll
        for (int i = 0; i < kA4 + kB4; ++i) {
          v[i].x = split_lo(v[i].x);
          v[i].y = split_lo(v[i].y);
          v[i].z = split_lo(v[i].z);
          v[i].w = split_lo(v[i].w);
        }
#pragma unroll
        for (int i = 0; i < kA4; ++i) a_lo[st + i * 32 * kSplitWarps] = v[i];
#pragma unroll
        for (int i = 0; i < kB4; ++i)
          if (st + i * 32 * kSplitWarps < b_f4) b_lo[st + i * 32 * kSplitWarps] = v[kA4 + i];
        // make these generic-proxy writes visible to the tensor pipe's (async-proxy) reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(smem_u32(&bar_lo_full[slot]));
        if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
        if (++slot == C::kLoStages) { slot = 0; lo_phase ^= 1u; }
      }
    }
  } else {
    // ------------------------------------------------------------------ drain + epilogue (kEpiWarps warps)
    if constexpr (DIRECT) asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kRegsDrain));
    const int q = warp & 3;             // TMEM lane quarter this warp may read: lanes 32q .. 32q+31
    const int half = (warp - kDrainFirst) >> 2;   // which 128 of the tile's 256 columns
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec_ok = (p.n % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.c) & 15u) == 0);
    bool ok = true;
    for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
      int b, mb, nb;
      decode_tile(t, p, b, mb, nb);
      float sum[BN / 2];
#pragma unroll
      for (int j = 0; j < BN / 2; ++j) sum[j] = 0.0f;
      for (int kb0 = 0; kb0 < p.num_kb; kb0 += p.chunk_kb) {
        ok = mbar_wait(smem_u32(&bar_tmem_full[acc]), acc_phase, &abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          if (lane == 0) report(p.status, 4, 400 + acc, t);
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
        if (lane == 0) mbar_arrive(smem_u32(&bar_tmem_empty[acc]));
        if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) break;
      float4* stage = reinterpret_cast<float4*>(smem_raw + (ring - smem_u32(smem_raw)) + C::kRingBytes) +
                      (warp - kDrainFirst) * (32 * 8);
      tile_epilogue(sum, p, b, mb * BM, nb, q, half, lane, vec_ok, stage);
    }
  }

  // ------------------------------------------------------------------ teardown
  __syncwarp();
  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                 : "memory");
  }
}

// ---- operand pre-pass: split into tf32 hi / lo planes, K-major, zero padded ----------------------
__device__ __forceinline__ float tf32_round(float x) {
  uint32_t u;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
  return __uint_as_float(u);
}
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  hi = tf32_round(x);
  // A finite x just below FLT_MAX must not round up to infinity: truncate instead.
  if (fabsf(hi) == INFINITY && fabsf(x) != INFINITY) hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  // Non-finite values carry no low part (inf - inf would inject a NaN of its own).
  lo = (fabsf(hi) == INFINITY || hi != hi) ? 0.0f : tf32_round(__fsub_rn(x, hi));
}

// Source already K-major: src[b][r][k] (r < rows, k < K).  dst planes [b][2][rows_p][Kp].
__global__ void __launch_bounds__(256, 4) split_copy_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                            int rows, int K, int rows_p, int Kp, int vec) {
  const int b = blockIdx.z;
  const float* s = src + (int64_t)b * rows * K;
  float* hi_p = dst + (int64_t)b * 2 * rows_p * Kp;
  float* lo_p = hi_p + (int64_t)rows_p * Kp;
  const int kq = Kp >> 2;   // Kp is a multiple of 16
  const int64_t total = (int64_t)rows_p * kq;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  constexpr int U = 4;      // 16-byte words in flight per thread
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += U * stride) {
    float4 x[U];
    int64_t o[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int64_t i = i0 + u * stride;
      x[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      o[u] = -1;
      if (i < total) {
        const int r = (int)(i / kq);
        const int k = (int)(i - (int64_t)r * kq) * 4;
        o[u] = (int64_t)r * Kp + k;
        if (r < rows) {
          const float* q = s + (int64_t)r * K + k;
          if (vec && k + 3 < K) {
            x[u] = __ldcs(reinterpret_cast<const float4*>(q));
          } else {
            if (k < K) x[u].x = q[0];
            if (k + 1 < K) x[u].y = q[1];
            if (k + 2 < K) x[u].z = q[2];
            if (k + 3 < K) x[u].w = q[3];
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      if (o[u] < 0) continue;
      float4 h, l;
      split_tf32(x[u].x, h.x, l.x);
      split_tf32(x[u].y, h.y, l.y);
      split_tf32(x[u].z, h.z, l.z);
      split_tf32(x[u].w, h.w, l.w);
      *reinterpret_cast<float4*>(hi_p + o[u]) = h;
      *reinterpret_cast<float4*>(lo_p + o[u]) = l;
    }
  }
}

// Source has the row index contiguous: src[b][k][r].  32x32 tiles through shared memory so both
// the read (along r) and the writes (along k) are coalesced.  grid = (Kp/32, rows_p/32, batch).
__global__ void __launch_bounds__(256) split_transpose_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                              int rows, int K, int rows_p, int Kp) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z;
  const float* s = src + (int64_t)b * rows * K;
  float* hi_p = dst + (int64_t)b * 2 * rows_p * Kp;
  float* lo_p = hi_p + (int64_t)rows_p * Kp;
  const int k0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 32 x 8
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int k = k0 + ty + j * 8, r = r0 + tx;
    tile[ty + j * 8][tx] = (k < K && r < rows) ? __ldcs(s + (int64_t)k * rows + r) : 0.0f;
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = r0 + ty + j * 8, k = k0 + tx;
    if (r < rows_p && k < Kp) {
      float h, l;
      split_tf32(tile[tx][ty + j * 8], h, l);
      hi_p[(int64_t)r * Kp + k] = h;
      lo_p[(int64_t)r * Kp + k] = l;
    }
  }
}

// Lo-plane pre-pass: dst[i] = lo part of src[i], same layout as the source (n4 16-byte words).
__global__ void __launch_bounds__(256, 4) split_lo_kernel(const float4* __restrict__ src, float4* __restrict__ dst,
                                                          int64_t n4) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      dst[i + j * stride] = make_float4(split_lo(v[j].x), split_lo(v[j].y), split_lo(v[j].z), split_lo(v[j].w));
  }
  for (; i < n4; i += stride) {
    const float4 v = __ldcs(src + i);
    dst[i] = make_float4(split_lo(v.x), split_lo(v.y), split_lo(v.z), split_lo(v.w));
  }
}

// The same for the two operands of one product in a single launch (blockIdx.y selects the operand): saves the
// second launch's ramp, which at 2048^3 is a quarter of the pre-pass.
__global__ void __launch_bounds__(256, 4) split_lo2_kernel(const float4* __restrict__ src0, float4* __restrict__ dst0,
                                                           int64_t n0, const float4* __restrict__ src1,
                                                           float4* __restrict__ dst1, int64_t n1) {
  const float4* src = blockIdx.y ? src1 : src0;
  float4* dst = blockIdx.y ? dst1 : dst0;
  const int64_t n4 = blockIdx.y ? n1 : n0;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + 3 * stride < n4; i += 4 * stride) {
    float4 v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = __ldcs(src + i + j * stride);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      dst[i + j * stride] = make_float4(split_lo(v[j].x), split_lo(v[j].y), split_lo(v[j].z), split_lo(v[j].w));
  }
  for (; i < n4; i += stride) {
    const float4 v = __ldcs(src + i);
    dst[i] = make_float4(split_lo(v.x), split_lo(v.y), split_lo(v.z), split_lo(v.w));
  }
}

__global__ void split_lo_scalar_kernel(const float* __restrict__ src, float* __restrict__ dst, int64_t n) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
    dst[i] = split_lo(src[i]);
}

// ---- host side ---------------------------------------------------------------------------------
bool split_lo_plane(const float* src, float* dst, int64_t n, cudaStream_t on_stream) {
  cudaStream_t s = on_stream ? on_stream : ctx().stream;
  if (aligned16(src) && aligned16(dst)) {
    const int64_t n4 = n / 4;
    if (n4 > 0) {
      split_lo_kernel<<<stream_grid(n4, 256, 4), 256, 0, s>>>(reinterpret_cast<const float4*>(src),
                                                              reinterpret_cast<float4*>(dst), n4);
      count_launch();
    }
    if (n % 4) {
      split_lo_scalar_kernel<<<1, 32, 0, s>>>(src + 4 * n4, dst + 4 * n4, n % 4);
      count_launch();
    }
  } else {
    split_lo_scalar_kernel<<<stream_grid(n, 256, 4), 256, 0, s>>>(src, dst, n);
    count_launch();
  }
  return cuda_ok(cudaGetLastError(), "lo-plane split launch");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
    else
      cudaGetLastError();
  }
  return fn;
}

// Tensor map over the split planes of one operand.
// K-major planes [2*batch][rows_p][Kp]: 3-D, dims {Kp, rows_p, 2*batch}, box {BK, tile_rows, 2}.
// MN-major planes [2*batch][Kp][rows_p]: 4-D with the row index cut into blocks of 32 so that one
// box lands as tile_rows/32 blocks of BK rows x 128 bytes: dims {32, Kp, rows_p/32, 2*batch},
// box {32, BK, tile_rows/32, 2}, 128-byte swizzle.
static bool make_operand_map(CUtensorMap* map, float* planes, int rows_p, int Kp, int batch, int bk, int box_rows,
                             bool mn_major) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  CUresult r;
  if (!mn_major) {
    cuuint64_t dims[3] = {(cuuint64_t)Kp, (cuuint64_t)rows_p, (cuuint64_t)(2 * batch)};
    cuuint64_t strides[2] = {(cuuint64_t)Kp * 4, (cuuint64_t)rows_p * Kp * 4};
    cuuint32_t box[3] = {(cuuint32_t)bk, (cuuint32_t)box_rows, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, planes, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[4] = {32, (cuuint64_t)Kp, (cuuint64_t)(rows_p / 32), (cuuint64_t)(2 * batch)};
    cuuint64_t strides[3] = {(cuuint64_t)rows_p * 4, 128, (cuuint64_t)rows_p * Kp * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)bk, (cuuint32_t)(box_rows / 32), 2};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, planes, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (rows %d, K %d, batch %d, %s-major)",
              (int)r, rows_p, Kp, batch, mn_major ? "MN" : "K");
    return false;
  }
  return true;
}

static int round_up(int x, int m) { return (x + m - 1) / m * m; }

// Batch entries processed per pass: as many as fit the operand workspace (4 GiB unless
// CLEAVE_CUDA_GEMM_WORKSPACE_MB says otherwise; read at every call so a test can lower it), at least one,
// and never more than a grid's z dimension can index (the pre-pass kernels put the batch there).
constexpr int kMaxGridZ = 65535;
int gemm_batch_chunk(int64_t bytes_per_entry, int batch) {
  int64_t limit = 4ll << 30;
  const char* e = getenv("CLEAVE_CUDA_GEMM_WORKSPACE_MB");
  if (e && atoll(e) > 0) limit = atoll(e) << 20;
  int64_t chunk = limit / (bytes_per_entry > 0 ? bytes_per_entry : 1);
  if (chunk < 1) chunk = 1;
  if (chunk > batch) chunk = batch;
  if (chunk > kMaxGridZ) chunk = kMaxGridZ;
  return (int)chunk;
}

// Switches for measurements (read once).  CLEAVE_CUDA_GEMM_DIRECT forces one operand path for every
// problem it can serve: 0 = padded [hi | lo] planes, 2 = split in the kernel, 3 = lo planes; otherwise
// the choice in launch_gemm_3xtf32.  CLEAVE_CUDA_GEMM_MN=0 makes the planes pre-pass transpose instead
// of writing MN-major planes.
static bool g_mn_major = true;
static int g_direct = 1;
static bool g_narrow = true;   // CLEAVE_CUDA_GEMM_NARROW=0: no transposed split-K route for narrow outputs
static bool g_splitk = true;   // CLEAVE_CUDA_GEMM_SPLITK=0: no split-K route for products with few tiles
static int g_pair = -1;   // CLEAVE_CUDA_GEMM_PAIR: 1 / 0 = always / never run the padded-planes path on CTA pairs
static void read_options() {
  static bool done = false;
  if (done) return;
  done = true;
  const char* mn = getenv("CLEAVE_CUDA_GEMM_MN");
  if (mn && mn[0] == '0') g_mn_major = false;
  const char* d = getenv("CLEAVE_CUDA_GEMM_DIRECT");
  if (d && (d[0] == '0' || d[0] == '2' || d[0] == '3')) g_direct = d[0] - '0';
  const char* nr = getenv("CLEAVE_CUDA_GEMM_NARROW");
  if (nr && nr[0] == '0') g_narrow = false;
  const char* sk = getenv("CLEAVE_CUDA_GEMM_SPLITK");
  if (sk && sk[0] == '0') g_splitk = false;
  const char* pr = getenv("CLEAVE_CUDA_GEMM_PAIR");
  if (pr && (pr[0] == '0' || pr[0] == '1')) g_pair = pr[0] - '0';
}

bool gemm_3xtf32_supported(const GemmArgs& g) {
  // Problem dimensions must fit the 32-bit coordinates of the tensor map and the tile counters.
  return g.m > 0 && g.n > 0 && g.k > 0 && g.batch > 0 && (int64_t)g.m * g.n < (1ll << 40) &&
         (int64_t)g.batch * ceil_div(g.m, BM) * ceil_div(g.n, BN) < (1ll << 30);
}

// Writes the hi / lo planes of one operand.  `k_contiguous`: the source has the contraction index
// contiguous ([rows][K]); otherwise it is stored [K][rows].  `mn_major`: the planes keep the
// [K][rows] order (no transpose; the kernel reads them as an MN-major operand) -- only
// meaningful for a source that is not k-contiguous.
static bool split_operand(const float* src, float* dst, int batch, int rows, int K, int rows_p, int Kp,
                          bool k_contiguous, bool mn_major) {
  cudaStream_t s = ctx().stream;
  if (k_contiguous || mn_major) {
    // a padded 2-D split copy: R x C source -> Rp x Cp planes
    const int R = k_contiguous ? rows : K, Cc = k_contiguous ? K : rows;
    const int Rp = k_contiguous ? rows_p : Kp, Cp = k_contiguous ? Kp : rows_p;
    int vec = (aligned16(src) && Cc % 4 == 0) ? 1 : 0;
    int64_t items = (int64_t)Rp * (Cp / 4);
    int grid = stream_grid((items + 3) / 4, 256, 4);
    split_copy_kernel<<<dim3(grid, 1, batch), 256, 0, s>>>(src, dst, R, Cc, Rp, Cp, vec);
  } else {
    split_transpose_kernel<<<dim3(ceil_div(Kp, 32), ceil_div(rows_p, 32), batch), 256, 0, s>>>(src, dst, rows, K,
                                                                                               rows_p, Kp);
  }
  count_launch();
  return cuda_ok(cudaGetLastError(), "operand split launch");
}

template <int BK, bool A_MN, bool B_MN, int PATH>
static bool run_tc(const CUtensorMap* maps, const TcParams& p) {
  using C = Cfg<BK, PATH == kPathDirect>;
  static bool attr_set = false;
  if (!attr_set) {
    if (!cuda_ok(cudaFuncSetAttribute(gemm_3xtf32_kernel<BK, A_MN, B_MN, PATH>,
                                      cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes),
                 "cudaFuncSetAttribute(gemm)"))
      return false;
    attr_set = true;
  }
  const int tiles = p.batch * p.mblks * p.nblks;
  const int grid = tiles < ctx().sm_count ? tiles : ctx().sm_count;
  profile_mark(true);
  gemm_3xtf32_kernel<BK, A_MN, B_MN, PATH>
      <<<grid, PATH == kPathDirect ? kDirectThreads : kGemmThreads, C::kSmemBytes, ctx().stream>>>(
          maps[0], maps[1], maps[2], maps[3], p);
  profile_mark(false);
  count_launch();
  return cuda_ok(cudaGetLastError(), "tcgen05 GEMM launch");
}

// maps: {A, B, A lo, B lo}; the last two are read on the lo-plane path only.
template <int PATH>
static bool run_tc_layout(bool a_mn, bool b_mn, const CUtensorMap* maps, const TcParams& p) {
  return a_mn ? (b_mn ? run_tc<16, true, true, PATH>(maps, p) : run_tc<16, true, false, PATH>(maps, p))
              : (b_mn ? run_tc<16, false, true, PATH>(maps, p) : run_tc<16, false, false, PATH>(maps, p));
}

// Tensor map straight over a caller's operand ([batch] matrices, row-major, unpadded).
// `k_contiguous` ([rows][K]): dims {K, rows, batch}, box {BK, tile_rows, 1}, 64-byte swizzle.
// Otherwise ([K][rows], read MN-major), 128-byte swizzle with 32-byte atoms, either
//   blocked (rows a multiple of 32): dims {32, K, rows/32, batch}, box {32, BK, tile_rows/32, 1} -- one box
//   per stage lands as tile_rows/32 blocks of BK rows x 128 bytes; or
//   plain: dims {rows, K, batch}, box {32, BK, 1}; the kernel issues tile_rows/32 such boxes per stage.
// Needs a 16-byte aligned base and a contiguous extent that is a multiple of 4 elements.
static bool make_direct_map(CUtensorMap* map, const float* base, int rows, int K, int batch, bool k_contiguous,
                            int tile_rows, bool blocked, int bk = 16) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  const cuuint64_t inner = k_contiguous ? K : rows, outer = k_contiguous ? rows : K;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r;
  if (blocked) {
    cuuint64_t dims[4] = {32, (cuuint64_t)K, (cuuint64_t)(rows / 32), (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)rows * 4, 128, (cuuint64_t)rows * K * 4};
    cuuint32_t box[4] = {32, (cuuint32_t)bk, (cuuint32_t)(tile_rows / 32), 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  } else {
    cuuint64_t dims[3] = {inner, outer, (cuuint64_t)batch};
    cuuint64_t strides[2] = {inner * 4, inner * outer * 4};
    // K-major rows are bk * 4 bytes: 64-byte swizzle for bk 16, 128-byte swizzle for bk 32
    cuuint32_t box[3] = {k_contiguous ? (cuuint32_t)bk : 32u, k_contiguous ? (cuuint32_t)tile_rows : (cuuint32_t)bk, 1};
    r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE,
            k_contiguous ? (bk == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)
                         : CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  }
  if (r != CUDA_SUCCESS) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (operand %d x %d, batch %d)", (int)r,
              rows, K, batch);
    return false;
  }
  return true;
}

// TMA can read the caller's tensors themselves when they are 16-byte aligned and their contiguous
// extent is a multiple of 4 elements.
static bool addressable(const GemmArgs& g) {
  const int a_inner = g.trans_a ? g.m : g.k, b_inner = g.trans_b ? g.k : g.n;
  return aligned16(g.a) && aligned16(g.b) && a_inner % 4 == 0 && b_inner % 4 == 0;
}

// Splitting in the kernel costs shared-memory bandwidth that the MMAs also need (measured: the kernel
// runs ~1.2x longer); a pre-pass costs an HBM round trip over both operands.  The pre-pass is the
// cheaper of the two once 1/M + 1/N drops below ~1/1000 (large, square-ish outputs; CLEAVE_CUDA_GEMM_DIRECT_BELOW
// moves the threshold for measurements).  At 2048^3 the lo-plane route wins (80 us against 88), at 4096 x 1024 x K4096
// the two are level (161 / 162 us).
static bool prefer_direct(const GemmArgs& g) {
  static const int64_t threshold = [] {
    const char* e = getenv("CLEAVE_CUDA_GEMM_DIRECT_BELOW");
    const long v = e ? atol(e) : 0;
    return (int64_t)(v > 0 ? v : 1000);
  }();
  return (int64_t)g.m * g.n < threshold * ((int64_t)g.m + g.n);
}

// The lo-plane path fetches an MN-major operand as one blocked box, which needs whole 32-wide blocks.
static bool lo_plane_eligible(const GemmArgs& g) {
  return addressable(g) && (!g.trans_a || g.m % 32 == 0) && (g.trans_b || g.n % 32 == 0);
}

static bool launch_direct(const GemmArgs& g) {
  const bool a_mn = g.trans_a != 0, b_mn = g.trans_b == 0;
  const bool a_blocked = a_mn && g.m % 32 == 0, b_blocked = b_mn && g.n % 32 == 0;
  // A narrow C needs only the first round_up(n, 32) rows of each B tile.
  const int b_box_rows = g.n < BN ? round_up(g.n, 32) : BN;
  CUtensorMap maps[4];
  if (!make_direct_map(&maps[0], g.a, g.m, g.k, g.batch, !a_mn, BM, a_blocked) ||
      !make_direct_map(&maps[1], g.b, g.n, g.k, g.batch, !b_mn, b_box_rows, b_blocked))
    return false;
  maps[2] = maps[0];
  maps[3] = maps[1];
  TcParams p;
  p.a_blocked = a_blocked;
  p.b_blocked = b_blocked;
  p.c_tma = 0;
  p.b_sliced = 0;
  p.b_box_rows = b_box_rows;
  p.c = g.c;
  p.c_lo = g.c_lo;
  p.bias = g.bias;
  p.dact_y = g.dact_y;
  p.dact = g.dact;
  p.m = g.m;
  p.n = g.n;
  p.num_kb = ceil_div(g.k, 16);
  p.chunk_kb = kChunkK / 16;
  p.batch = g.batch;
  p.mblks = ceil_div(g.m, BM);
  p.nblks = ceil_div(g.n, BN);
  p.act = g.act;
  p.status = ctx().status_dev;
  return run_tc_layout<kPathDirect>(a_mn, b_mn, maps, p);
}

// ---- narrow C (n <= 128): transposed, split-K ---------------------------------------------------------------
// A tcgen05.mma with M = 128 takes about as long at N = 64 as at N = 256 (measured), so with C's narrow
// dimension on N the kernel is bound by its MMA count.  Here C^T = B^T A^T is computed instead: the narrow
// dimension lies on M (one tile row, padded to 128) and the long one runs along N in full 256-wide
// tiles -- half as many MMAs or fewer.  That leaves only m/256 tiles, so K is cut into S slices that run as the S
// entries of a batch (B is [k, n]: a K-slice of it is a dense block; A is [m, k]: a K-slice is a strided
// view, which a tensor map expresses), and a last pass adds the S partial results in slice order and
// transposes them into C.
__global__ void __launch_bounds__(256) sum_transpose_kernel(const float* __restrict__ part, float* __restrict__ c,
                                                            int slices, int n, int m) {
  // part: [slices][n][m]; c: [m][n].  32 x 32 tiles through shared memory, both sides coalesced.
  __shared__ float tile[32][33];
  const int i0 = blockIdx.x * 32, j0 = blockIdx.y * 32;      // i along m, j along n
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;    // 32 x 8
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = j0 + ty + 8 * r, i = i0 + tx;
    float acc = 0.0f;
    if (j < n && i < m)
      for (int sl = 0; sl < slices; ++sl) acc = __fadd_rn(acc, part[((int64_t)sl * n + j) * m + i]);
    tile[ty + 8 * r][tx] = acc;
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int i = i0 + ty + 8 * r, j = j0 + tx;
    if (i < m && j < n) c[(int64_t)i * n + j] = tile[tx][ty + 8 * r];
  }
}

// Number of K slices for the transposed route, 0 if it does not apply.
static int narrow_slices(const GemmArgs& g) {
  if (g.batch != 1 || g.trans_a || g.trans_b || g.bias || g.dact_y || g.act != CLEAVE_ACT_IDENTITY) return 0;
  if (g.n > BM || g.n % 4 != 0 || g.m < 2048 || g.k < 2048 || g.k % 16 != 0) return 0;
  if (!aligned16(g.a) || !aligned16(g.b) || !aligned16(g.c)) return 0;
  const int tiles = ceil_div(g.m, BN);
  int s = ctx().sm_count / tiles;
  if (s < 1) s = 1;
  if (s > 16) s = 16;
  while (s > 1 && (g.k % s != 0 || (g.k / s) % 16 != 0 || g.k / s < 512)) --s;
  return s;
}

static bool launch_narrow_transposed(const GemmArgs& g, int slices) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  const int ks = g.k / slices;
  float* part = scratch_alloc((int64_t)slices * g.n * g.m * 4);
  if (!part) return false;
  CUtensorMap maps[4];
  // operand "A" of the transposed product is B: stored [k, n], read MN-major; its K slices are the batch
  const bool a_blocked = g.n % 32 == 0;
  bool ok = make_direct_map(&maps[0], g.b, g.n, ks, slices, false, BM, a_blocked);
  if (ok) {
    // operand "B" is A: stored [m, k], K-major; slice sl is the view A[:, sl*ks : (sl+1)*ks]
    // (dimensions ordered by stride: k within the slice, slice, row)
    cuuint64_t dims[3] = {(cuuint64_t)ks, (cuuint64_t)slices, (cuuint64_t)g.m};
    cuuint64_t strides[2] = {(cuuint64_t)ks * 4, (cuuint64_t)g.k * 4};
    cuuint32_t box[3] = {16, 1, (cuuint32_t)BN};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = enc(&maps[1], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(g.a), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
      set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (K-sliced operand %d x %d / %d)", (int)r,
                g.m, g.k, slices);
      ok = false;
    }
  }
  if (ok) {
    maps[2] = maps[0];
    maps[3] = maps[1];
    TcParams p;
    p.a_blocked = a_blocked;
    p.b_blocked = 0;
    p.b_sliced = 1;
    p.c_tma = 0;
    p.b_box_rows = BN;
    p.c = part;
    p.bias = nullptr;
    p.dact_y = nullptr;
    p.dact = CLEAVE_ACT_IDENTITY;
    p.m = g.n;                 // the transposed product is [n, m]
    p.n = g.m;
    p.num_kb = ceil_div(ks, 16);
    p.chunk_kb = kChunkK / 16;
    p.batch = slices;
    p.mblks = ceil_div(g.n, BM);
    p.nblks = ceil_div(g.m, BN);
    p.act = CLEAVE_ACT_IDENTITY;
    p.status = ctx().status_dev;
    ok = run_tc_layout<kPathDirect>(true, false, maps, p);
  }
  if (ok) {
    sum_transpose_kernel<<<dim3(ceil_div(g.m, 32), ceil_div(g.n, 32)), 256, 0, ctx().stream>>>(part, g.c, slices, g.n,
                                                                                              g.m);
    count_launch();
    ok = cuda_ok(cudaGetLastError(), "sum-transpose launch");
  }
  scratch_free(part);
  return ok;
}

// ---- few tiles: split K ------------------------------------------------------------------------------------
// A product with fewer tiles than half the SMs leaves most of the machine idle for the whole of K.  Here K is cut
// into S slices that run as the S entries of a batch on the in-kernel-split kernel (a K-slice of a K-major operand
// is a strided view, which a tensor map expresses; a K-slice of an MN-major operand is a contiguous block), so
// tiles * S CTAs are busy, and one pass adds the S partial results in slice order -- a fixed order, so the result
// is reproducible -- and applies bias / activation / derivative exactly as the GEMM epilogue would.
__global__ void __launch_bounds__(256) sum_slices_kernel(const float4* __restrict__ part, float4* __restrict__ c,
                                                         float4* __restrict__ c_lo, int slices, int64_t n4, int n,
                                                         const float* __restrict__ bias, int act,
                                                         const float* __restrict__ dact_y, int dact) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 acc = __ldcg(part + i);
    for (int sl = 1; sl < slices; ++sl) {
      const float4 v = __ldcg(part + (int64_t)sl * n4 + i);
      acc.x = __fadd_rn(acc.x, v.x); acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z); acc.w = __fadd_rn(acc.w, v.w);
    }
    if (bias != nullptr) {
      const float4 bv = __ldg(reinterpret_cast<const float4*>(bias + (int)((4 * i) % n)));   // n is a multiple of 4
      acc.x = __fadd_rn(acc.x, bv.x); acc.y = __fadd_rn(acc.y, bv.y);
      acc.z = __fadd_rn(acc.z, bv.z); acc.w = __fadd_rn(acc.w, bv.w);
    }
    if (act != CLEAVE_ACT_IDENTITY) {
      acc.x = act_apply(acc.x, act); acc.y = act_apply(acc.y, act);
      acc.z = act_apply(acc.z, act); acc.w = act_apply(acc.w, act);
    }
    if (dact_y != nullptr) {
      const float4 y = __ldg(reinterpret_cast<const float4*>(dact_y) + i);
      acc.x = dact_apply(y.x, acc.x, dact); acc.y = dact_apply(y.y, acc.y, dact);
      acc.z = dact_apply(y.z, acc.z, dact); acc.w = dact_apply(y.w, acc.w, dact);
    }
    c[i] = acc;
    if (c_lo != nullptr) c_lo[i] = make_float4(split_lo(acc.x), split_lo(acc.y), split_lo(acc.z), split_lo(acc.w));
  }
}

// Number of K slices for the split-K route, 0 if it does not apply.
static int splitk_slices(const GemmArgs& g) {
  if (g.batch != 1 || !addressable(g) || g.n % 4 != 0 || !aligned16(g.c) || g.k < 1024) return 0;
  if ((g.bias && !aligned16(g.bias)) || (g.dact_y && !aligned16(g.dact_y)) || (g.c_lo && !aligned16(g.c_lo))) return 0;
  const int tiles = ceil_div(g.m, BM) * ceil_div(g.n, BN);
  const int sms = ctx().sm_count;
  if (tiles * 2 > sms) return 0;
  int s = sms / tiles;
  if (s > 16) s = 16;
  while (s > 1 && (g.k % s != 0 || (g.k / s) % 16 != 0 || g.k / s < 256)) --s;
  return s > 1 ? s : 0;
}

// Tensor map over the K slices of a K-major operand ([rows][K], K contiguous): dimensions ordered by stride
// {k within the slice, slice, row}, box {16, 1, tile_rows}.
static bool make_sliced_map(CUtensorMap* map, const float* base, int rows, int K, int slices, int tile_rows) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    return false;
  }
  const int ks = K / slices;
  cuuint64_t dims[3] = {(cuuint64_t)ks, (cuuint64_t)slices, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)ks * 4, (cuuint64_t)K * 4};
  cuuint32_t box[3] = {16, 1, (cuuint32_t)tile_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    set_error(CLEAVE_CUDA_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d (K-sliced operand %d x %d / %d)", (int)r,
              rows, K, slices);
    return false;
  }
  return true;
}

static bool launch_split_k(const GemmArgs& g, int slices) {
  const int ks = g.k / slices;
  const bool a_mn = g.trans_a != 0, b_mn = g.trans_b == 0;
  const bool a_blocked = a_mn && g.m % 32 == 0, b_blocked = b_mn && g.n % 32 == 0;
  const int b_box_rows = g.n < BN ? round_up(g.n, 32) : BN;
  const int64_t out = (int64_t)g.m * g.n;
  float* part = scratch_alloc((int64_t)slices * out * 4);
  if (!part) return false;
  CUtensorMap maps[4];
  // an MN-major operand is stored [K][rows]: its K slices are consecutive blocks, i.e. a batch of [ks][rows] matrices
  bool ok = (a_mn ? make_direct_map(&maps[0], g.a, g.m, ks, slices, false, BM, a_blocked)
                  : make_sliced_map(&maps[0], g.a, g.m, g.k, slices, BM)) &&
            (b_mn ? make_direct_map(&maps[1], g.b, g.n, ks, slices, false, b_box_rows, b_blocked)
                  : make_sliced_map(&maps[1], g.b, g.n, g.k, slices, b_box_rows));
  if (ok) {
    maps[2] = maps[0];
    maps[3] = maps[1];
    TcParams p;
    p.a_blocked = a_blocked;
    p.b_blocked = b_blocked;
    p.a_sliced = a_mn ? 0 : 1;
    p.b_sliced = b_mn ? 0 : 1;
    p.c_tma = 0;
    p.b_box_rows = b_box_rows;
    p.c = part;
    p.bias = nullptr;
    p.dact_y = nullptr;
    p.dact = CLEAVE_ACT_IDENTITY;
    p.m = g.m;
    p.n = g.n;
    p.num_kb = ceil_div(ks, 16);
    p.chunk_kb = kChunkK / 16;
    p.batch = slices;
    p.mblks = ceil_div(g.m, BM);
    p.nblks = ceil_div(g.n, BN);
    p.act = CLEAVE_ACT_IDENTITY;
    p.status = ctx().status_dev;
    ok = run_tc_layout<kPathDirect>(a_mn, b_mn, maps, p);
  }
  if (ok) {
    const int64_t n4 = out / 4;
    sum_slices_kernel<<<stream_grid(n4, 256, 4), 256, 0, ctx().stream>>>(
        reinterpret_cast<const float4*>(part), reinterpret_cast<float4*>(g.c), reinterpret_cast<float4*>(g.c_lo), slices,
        n4, g.n, g.bias, g.act, g.dact_y, g.dact);
    count_launch();
    ok = cuda_ok(cudaGetLastError(), "slice-sum launch");
  }
  scratch_free(part);
  return ok;
}

static bool make_c_map(CUtensorMap* map, float* c, int m, int n, int batch, int mode);

// hi planes are the caller's tensors, lo planes come from one streaming pass per operand.
static bool launch_lo_plane(const GemmArgs& g) {
  const bool a_mn = g.trans_a != 0, b_mn = g.trans_b == 0;
  const int64_t a_elems = (int64_t)g.m * g.k, b_elems = (int64_t)g.n * g.k;
  // planes the caller holds are used as they are; a missing one is written here, in chunks of the batch
  const int64_t scratch_per_entry = ((g.a_lo ? 0 : a_elems) + (g.b_lo ? 0 : b_elems)) * 4;
  const int chunk = scratch_per_entry ? gemm_batch_chunk(scratch_per_entry, g.batch) : (g.batch < 65535 ? g.batch : 65535);
  // Larger outputs run their 256 x 256 tiles on CTA pairs (measured at 4096 x 4096 x K1024: 132 us against 144 us on
  // single CTAs; level at 2048^3), unless padding to 256 would waste more than ~7 % of the tile area.
  // CLEAVE_CUDA_GEMM_LO_PAIR = 0 / 1 forces the choice.
  static const int lo_pair = [] {
    const char* e = getenv("CLEAVE_CUDA_GEMM_LO_PAIR");
    return (e && (e[0] == '0' || e[0] == '1')) ? e[0] - '0' : -1;
  }();
  const int64_t padded = (int64_t)round_up(g.m, 256) * round_up(g.n, 256);
  const bool pair = lo_pair >= 0 ? lo_pair == 1
                                 : ((int64_t)g.m * g.n >= (1ll << 22) && padded * 100 <= (int64_t)g.m * g.n * 107);
  float* wa = nullptr;
  float* wb = nullptr;
  if (!g.a_lo) {
    wa = scratch_alloc(chunk * a_elems * 4);
    if (!wa) return false;
  }
  if (!g.b_lo) {
    wb = scratch_alloc(chunk * b_elems * 4);
    if (!wb) { scratch_free(wa); return false; }
  }
  bool ok = true;
  for (int b0 = 0; ok && b0 < g.batch; b0 += chunk) {
    const int nb = (g.batch - b0) < chunk ? (g.batch - b0) : chunk;
    const float* a = g.a + b0 * a_elems;
    const float* b = g.b + b0 * b_elems;
    const float* a_lo = g.a_lo ? g.a_lo + b0 * a_elems : wa;
    const float* b_lo = g.b_lo ? g.b_lo + b0 * b_elems : wb;
    if (!g.a_lo && !g.b_lo) {
      // both planes in one launch (the operands of this route are 16-byte aligned, their sizes multiples of 4)
      const int64_t a4 = nb * a_elems / 4, b4 = nb * b_elems / 4;
      const int64_t per_operand = (a4 > b4 ? a4 : b4);
      int grid = stream_grid((per_operand + 3) / 4, 256, 2);
      split_lo2_kernel<<<dim3(grid, 2), 256, 0, ctx().stream>>>(reinterpret_cast<const float4*>(a),
                                                                 reinterpret_cast<float4*>(wa), a4,
                                                                 reinterpret_cast<const float4*>(b),
                                                                 reinterpret_cast<float4*>(wb), b4);
      count_launch();
      ok = cuda_ok(cudaGetLastError(), "lo-plane split launch");
    } else {
      if (!g.a_lo) ok = split_lo_plane(a, wa, nb * a_elems);
      if (ok && !g.b_lo) ok = split_lo_plane(b, wb, nb * b_elems);
    }
    if (!ok) break;
    if (pair) {
      // 256 x 256 tiles on CTA pairs: each CTA loads 128 rows of A and 128 of the tile's 256 rows of B, K-block 32
      CUtensorMap pm[5];
      ok = make_direct_map(&pm[0], a, g.m, g.k, nb, !a_mn, 128, a_mn, 32) &&
           make_direct_map(&pm[1], b, g.n, g.k, nb, !b_mn, 128, b_mn, 32) &&
           make_direct_map(&pm[3], a_lo, g.m, g.k, nb, !a_mn, 128, a_mn, 32) &&
           make_direct_map(&pm[4], b_lo, g.n, g.k, nb, !b_mn, 128, b_mn, 32);
      if (!ok) break;
      TcParams p;
      p.a_blocked = a_mn;
      p.b_blocked = b_mn;
      p.b_sliced = 0;
      p.b_box_rows = BN;
      p.c = g.c + (int64_t)b0 * g.m * g.n;
      p.c_lo = g.c_lo ? g.c_lo + (int64_t)b0 * g.m * g.n : nullptr;
      p.bias = g.bias;
      p.dact_y = g.dact_y ? g.dact_y + (int64_t)b0 * g.m * g.n : nullptr;
      p.dact = g.dact;
      p.m = g.m;
      p.n = g.n;
      p.num_kb = ceil_div(g.k, 32);
      p.chunk_kb = kChunkK / 32;
      p.batch = nb;
      p.mblks = ceil_div(g.m, 256);
      p.nblks = ceil_div(g.n, 256);
      p.act = g.act;
      p.status = ctx().status_dev;
      p.c_tma = (aligned16(p.c) && g.n % 4 == 0 && make_c_map(&pm[2], p.c, g.m, g.n, nb, 1)) ? 1 : 0;
      if (!p.c_tma) pm[2] = pm[0];
      ok = run_tc_pair(a_mn, b_mn, pm, p, 32, true);
      continue;
    }
    CUtensorMap maps[4];
    ok = make_direct_map(&maps[0], a, g.m, g.k, nb, !a_mn, BM, a_mn) &&
         make_direct_map(&maps[1], b, g.n, g.k, nb, !b_mn, BN, b_mn) &&
         make_direct_map(&maps[2], a_lo, g.m, g.k, nb, !a_mn, BM, a_mn) &&
         make_direct_map(&maps[3], b_lo, g.n, g.k, nb, !b_mn, BN, b_mn);
    if (!ok) break;
    TcParams p;
    p.a_blocked = a_mn;
    p.b_blocked = b_mn;
    p.c_tma = 0;
    p.b_sliced = 0;
    p.b_box_rows = BN;
    p.c = g.c + (int64_t)b0 * g.m * g.n;
    p.c_lo = g.c_lo ? g.c_lo + (int64_t)b0 * g.m * g.n : nullptr;
    p.bias = g.bias;
    p.dact_y = g.dact_y ? g.dact_y + (int64_t)b0 * g.m * g.n : nullptr;
    p.dact = g.dact;
    p.m = g.m;
    p.n = g.n;
    p.num_kb = ceil_div(g.k, 16);
    p.chunk_kb = kChunkK / 16;
    p.batch = nb;
    p.mblks = ceil_div(g.m, BM);
    p.nblks = ceil_div(g.n, BN);
    p.act = g.act;
    p.status = ctx().status_dev;
    ok = run_tc_layout<kPathLoPlane>(a_mn, b_mn, maps, p);
  }
  scratch_free(wa);
  scratch_free(wb);
  return ok;
}

// Tensor map over the output for TMA stores: dims {n, m, batch}; box 32 x 32 floats with the 128-byte swizzle
// (mode 1: the layout of a drain warp's shared staging tile) or 16 columns x 32 rows with the 64-byte swizzle
// (mode 2: the layout of its halves).  Needs a 16-byte aligned C and n a multiple of 4.
static bool make_c_map(CUtensorMap* map, float* c, int m, int n, int batch, int mode) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {(cuuint64_t)n, (cuuint64_t)m, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)n * 4, (cuuint64_t)m * n * 4};
  cuuint32_t box[3] = {mode == 2 ? 16u : 32u, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, c, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             mode == 2 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
         CUDA_SUCCESS;
}

bool launch_gemm_3xtf32(const GemmArgs& g) {
  if (!gemm_3xtf32_supported(g)) {
    set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "3xTF32 GEMM: problem %d x %d x %d (batch %d) is out of range", g.m, g.n,
              g.k, g.batch);
    return false;
  }
  read_options();
  // Routes chosen by shape alone come first, so that a call gives the same bits whether or not the caller also
  // hands in lo planes.  (1) A narrow output with long m and k: the transposed split-K route; it adds its partial
  // results in a pass of its own that cannot write C's lo plane.  (2) Few tiles: split K.
  if (g_direct == 1) {
    if (g_narrow && g.c_lo == nullptr) {
      const int slices = narrow_slices(g);
      if (slices > 0) return launch_narrow_transposed(g, slices);
    }
    if (g_splitk) {
      const int slices = splitk_slices(g);
      if (slices > 0) return launch_split_k(g, slices);
    }
    // (3) Lo planes handed in by the caller (an earlier GEMM's epilogue wrote them, or they are reused across
    // calls): the lo-plane route then needs no pre-pass at all, which beats every other route where it applies.
    if ((g.a_lo || g.b_lo) && lo_plane_eligible(g) && aligned16(g.a_lo) && aligned16(g.b_lo)) return launch_lo_plane(g);
  }
  // Measured choice.  Small / narrow problems: split in the kernel.  Up to 4096^2 outputs: lo planes (the
  // pre-pass moves 2/3 of the bytes of the padded one: 183 vs 300 us at 8192^3, 50 vs 80 us at 4096^3).
  // Beyond that the padded [hi | lo] planes win although their pre-pass is longer: the kernel runs
  // 3-5 % slower when its hi operand is the raw tensor (low mantissa bits that the tensor pipe ignores
  // still travel through shared memory; the kernel runs under the power cap).
  if (g_direct == 2 || (g_direct == 1 && prefer_direct(g))) {
    if (addressable(g)) return launch_direct(g);
  } else if (g_direct == 3 || (g_direct == 1 && (int64_t)g.m * g.n <= (1ll << 24))) {
    if (lo_plane_eligible(g)) return launch_lo_plane(g);
  }
  // K-block of the pair kernel: 32 (three 64 KiB stages, 128-byte rows) unless CLEAVE_CUDA_GEMM_PAIR_BK=16 asks for
  // six 32 KiB stages; measured on one box at 8192^3: 3.85-3.90 ms against 3.97-4.04 ms
  static const int pair_bk =
      (getenv("CLEAVE_CUDA_GEMM_PAIR_BK") && atoi(getenv("CLEAVE_CUDA_GEMM_PAIR_BK")) == 16) ? 16 : 32;
  // 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2) for the large problems this path serves:
  // measured 1-2 % faster at 4096^3 and 8192^3 (3.71-3.79 vs 3.74-3.84 ms); small ragged problems
  // keep 128-row tiles, which pad less.
  const bool pair = g_pair >= 0 ? g_pair == 1 : (int64_t)g.m * g.n > (1ll << 24);
  const int bk = pair ? pair_bk : 16;
  const int Kp = round_up(g.k, 32);
  const int Mp = round_up(g.m, pair ? 256 : BM);
  const int Np = round_up(g.n, BN);
  // Bound the split workspace: process the batch in chunks of at most ~4 GiB of planes.
  const int64_t per_batch_bytes = 2ll * ((int64_t)Mp + Np) * Kp * 4;
  const int chunk = gemm_batch_chunk(per_batch_bytes, g.batch);

  float* wa = scratch_alloc((int64_t)chunk * 2 * Mp * Kp * 4);
  if (!wa) return false;
  float* wb = scratch_alloc((int64_t)chunk * 2 * Np * Kp * 4);
  if (!wb) { scratch_free(wa); return false; }

  bool ok = true;
  for (int b0 = 0; ok && b0 < g.batch; b0 += chunk) {
    const int nb = (g.batch - b0) < chunk ? (g.batch - b0) : chunk;
    const float* a = g.a + (int64_t)b0 * g.m * g.k;
    const float* b = g.b + (int64_t)b0 * g.k * g.n;
    // A is K-contiguous when stored [m,k]; B is K-contiguous when stored [n,k].  An operand stored
    // the other way round is left in that order and read as an MN-major operand (no transpose).
    const bool a_mn = g.trans_a != 0 && g_mn_major, b_mn = g.trans_b == 0 && g_mn_major;
    ok = split_operand(a, wa, nb, g.m, g.k, Mp, Kp, g.trans_a == 0, a_mn) &&
         split_operand(b, wb, nb, g.n, g.k, Np, Kp, g.trans_b != 0, b_mn);
    if (!ok) break;
    CUtensorMap maps[5];
    ok = make_operand_map(&maps[0], wa, Mp, Kp, nb, bk, BM, a_mn) &&
         make_operand_map(&maps[1], wb, Np, Kp, nb, bk, pair ? 128 : BN, b_mn);
    if (!ok) break;
    maps[2] = maps[0];
    maps[3] = maps[1];
    maps[4] = maps[1];
    TcParams p;
    p.c = g.c + (int64_t)b0 * g.m * g.n;
    p.c_lo = g.c_lo ? g.c_lo + (int64_t)b0 * g.m * g.n : nullptr;
    p.bias = g.bias;
    p.dact_y = g.dact_y ? g.dact_y + (int64_t)b0 * g.m * g.n : nullptr;
    p.dact = g.dact;
    p.m = g.m;
    p.n = g.n;
    p.num_kb = Kp / bk;
    p.chunk_kb = kChunkK / bk;
    p.batch = nb;
    p.mblks = Mp / BM;
    p.nblks = Np / BN;
    p.act = g.act;
    p.a_blocked = p.b_blocked = 0;
    p.c_tma = 0;
    p.b_sliced = 0;
    p.b_box_rows = BN;
    p.status = ctx().status_dev;
    if (pair) {
      p.mblks = Mp / 256;
      // tile-rows per rasterisation group (CLEAVE_CUDA_GEMM_GROUP_M, 1 .. 64): the ~74 tiles in flight span
      // group x (74 / group) panels of A and B; 8 x 9 is the squarest split
      static const int group_m = [] {
        const char* e = getenv("CLEAVE_CUDA_GEMM_GROUP_M");
        const int v = e ? atoi(e) : 0;
        return (v >= 1 && v <= 64) ? v : 8;
      }();
      p.pair_group_m = group_m;
      // full tiles leave through TMA stores when a tensor map can describe C
      // CLEAVE_CUDA_GEMM_TMA_STORE: 0 = the warps' own stores, 1 = 32 x 32 bulk stores one at a time, 2 = 32 x 16
      // bulk stores, two in flight
      static const int tma_store = [] {
        const char* e = getenv("CLEAVE_CUDA_GEMM_TMA_STORE");
        return (e && e[0] >= '0' && e[0] <= '2') ? e[0] - '0' : 1;
      }();
      p.c_tma = (tma_store && aligned16(p.c) && g.n % 4 == 0 && make_c_map(&maps[2], p.c, g.m, g.n, nb, tma_store))
                    ? tma_store : 0;
      // one accumulation chunk and nothing but the product: the variant with twice the drain warps
      // (CLEAVE_CUDA_GEMM_SHORTK=0 turns it off)
      static const bool shortk_on = !(getenv("CLEAVE_CUDA_GEMM_SHORTK") && getenv("CLEAVE_CUDA_GEMM_SHORTK")[0] == '0');
      if (shortk_on && bk == 32 && Kp <= kChunkK && !g.bias && g.act == CLEAVE_ACT_IDENTITY && !g.dact_y && !g.c_lo) {
        if (p.c_tma == 2) p.c_tma = make_c_map(&maps[2], p.c, g.m, g.n, nb, 1) ? 1 : 0;   // this variant stores 32 x 32 blocks
        ok = run_tc_pair_shortk(a_mn, b_mn, maps, p);
      } else {
        ok = run_tc_pair(a_mn, b_mn, maps, p, bk);   // maps[3] (a copy of maps[1]) and maps[4] are not read in this mode
      }
    } else {
      ok = run_tc_layout<kPathPlanes>(a_mn, b_mn, maps, p);
    }
  }
  scratch_free(wa);
  scratch_free(wb);
  return ok;
}

}  // namespace cleave
