// Tensor-core f32 GEMM for sm_100a: tcgen05.mma (kind::tf32) with TMEM accumulators, operands
// staged by TMA into a multi-stage shared-memory ring guarded by mbarriers, and a 3xTF32
// split so that the f32 result stays within rounding distance of the reference's f32 loop.
//
// Split precision.  Every f32 operand value x is written as hi + lo with
//   hi = tf32(x)  (round to nearest, 10 explicit mantissa bits),  lo = tf32(x - hi),
// and a*b is accumulated as  a_lo*b_hi + a_hi*b_lo + a_hi*b_hi  in the f32 TMEM accumulator.
// The dropped a_lo*b_lo term and the rounding of lo are each <= 2^-22 |a b|.
//
// Data path.  A pre-pass writes both operands K-major (the contraction index contiguous) as two
// planes [hi | lo] of shape [rows_padded, K_padded], transposing where the caller's layout has
// the other index contiguous; this makes NN / NT / TN one kernel.  Padding (rows to the tile
// height, K to the K-block) is zero-filled so every TMA box is fully in bounds.
//
// Kernel.  Persistent, one CTA per SM, 192 threads:
//   warp 0      TMA producer (one elected lane): per K-block one 3-D box per operand
//               {BK, rows, 2 planes} -> shared memory, completion on the stage's "full" mbarrier
//   warp 1      MMA issuer (one elected lane): 3 x (BK/8) tcgen05.mma per K-block into one of two
//               128x256 f32 accumulators in TMEM; tcgen05.commit releases the stage ("empty")
//               and, after each K-chunk, publishes the accumulator ("tmem_full")
//   warps 2-9   drain + epilogue: after every K-chunk (256 values of k) tcgen05.ld the chunk's
//               partial sums and add them, round-to-nearest, to 128 running sums per thread in
//               registers; hand the accumulator back ("tmem_empty"); after the last chunk apply
//               bias + activation and store C with 128-bit stores
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

namespace cleave {

constexpr int BM = 128;          // tile rows  (UMMA M)
constexpr int BN = 256;          // tile cols  (UMMA N)
constexpr int UMMA_K = 8;        // tf32 MMA K (32 bytes)
constexpr int kEpiWarps = 8;     // two per TMEM lane quarter, 128 columns each
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr int kChunkK = 256;     // k values accumulated in TMEM before a drain into registers
constexpr int kAccStages = 2;
constexpr int kTmemCols = kAccStages * BN;   // 512: all of TMEM
constexpr int kGroupM = 16;      // tile-rows per rasterisation group
constexpr unsigned long long kWaitLimitNs = 4000000000ull;   // 4 s per wait

template <int BK>
struct Cfg {
  static_assert(BK == 16 || BK == 32, "BK must give a 64- or 128-byte row");
  static constexpr int kRowBytes = BK * 4;
  static constexpr int kStages = BK == 32 ? 2 : 4;
  static constexpr int kABytes = BM * kRowBytes;          // one plane of A
  static constexpr int kBBytes = BN * kRowBytes;          // one plane of B
  static constexpr int kStageBytes = 2 * kABytes + 2 * kBBytes;
  static constexpr int kStoreStageBytes = kEpiWarps * 32 * 128;      // per drain warp: 32 rows x 32 floats
  static constexpr int kSmemBytes = kStages * kStageBytes + kStoreStageBytes + 1024;   // + alignment slack
  static constexpr uint32_t kLayoutType = BK == 32 ? 2u : 4u;       // SWIZZLE_128B : SWIZZLE_64B
  static constexpr uint32_t kSBO = 8 * kRowBytes;                   // bytes between 8-row groups
};

// ---- PTX wrappers ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

// Bounded wait.  Returns false if the CTA is aborting or the wall-clock limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 0xFFu) == 0) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > kWaitLimitNs) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2,
                                            int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

__device__ __forceinline__ void tcgen05_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tcgen05_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tcgen05_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc], tf32 inputs, f32 accumulate.
__device__ __forceinline__ void umma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Shared-memory matrix descriptor.
// K-major operand (contraction index contiguous), swizzled rows of `kRowBytes`: start + k-step * 32 B,
// stride byte offset = pitch of 8-row groups, leading byte offset unused.
// MN-major operand (row / column index contiguous), 128-byte swizzle: the tile is a sequence of
// 32-wide blocks along M or N, each block BK rows of 128 bytes; a k-step (8 rows) is 1024 bytes,
// stride byte offset = 1024 (pitch of 8-row groups), leading byte offset = BK * 128 (pitch of blocks).
//   bits  0-13 start address >> 4     bits 16-29 leading byte offset >> 4 (1: unused when swizzled)
//   bits 32-45 stride byte offset >> 4 (8-row group pitch)   bits 46-47 descriptor version (1)
//   bits 61-63 swizzle mode (2 = 128 B, 4 = 64 B)
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr, uint32_t sbo_bytes, uint32_t layout_type,
                                                   uint32_t lbo_bytes = 16) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(sbo_bytes >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)layout_type << 61;
  return d;
}

// Instruction descriptor: f32 accumulator (bits 4-5 = 1), A and B tf32 (bits 7-9, 10-12 = 2),
// bit 15 / 16 = 1 for an MN-major A / B operand, N >> 3 in bits 17-22, M >> 4 in bits 24-28.
__host__ __device__ constexpr uint32_t instr_desc(bool a_mn, bool b_mn) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ float act_apply(float v, int act) {
  switch (act) {
    case CLEAVE_ACT_RELU: return v != v ? v : (v > 0.0f ? v : 0.0f);
    case CLEAVE_ACT_SIGMOID: return __frcp_rn(__fadd_rn(1.0f, expf(-v)));
    case CLEAVE_ACT_TANH: return tanhf(v);
    default: return v;
  }
}

struct TcParams {
  float* c;             // [batch][m][n]
  const float* bias;    // [n] or null
  int m, n;
  int num_kb;           // K_padded / BK
  int chunk_kb;         // K-blocks per accumulation chunk (kChunkK / BK)
  int batch, mblks, nblks;
  int act;
  DeviceStatus* status;
};

// Tile index -> (batch, tile-row, tile-col); tile-rows are walked in groups of kGroupM with the
// row index fastest inside a group, so consecutive tiles share a B panel and nearby A panels.
__device__ __forceinline__ void decode_tile(int t, const TcParams& p, int& b, int& mb, int& nb) {
  const int per_batch = p.mblks * p.nblks;
  b = t / per_batch;
  int r = t - b * per_batch;
  const int group_span = kGroupM * p.nblks;
  const int gid = r / group_span;
  const int first_m = gid * kGroupM;
  const int rows_here = (p.mblks - first_m) < kGroupM ? (p.mblks - first_m) : kGroupM;
  r -= gid * group_span;
  mb = first_m + r % rows_here;
  nb = r / rows_here;
}

__device__ __forceinline__ void report(DeviceStatus* st, int code, int where, int detail) {
  // Plain stores to mapped host memory (several CTAs may report; any one record will do).
  volatile DeviceStatus* v = st;
  v->where = where;
  v->block = blockIdx.x;
  v->detail = detail;
  v->code = code;
  __threadfence_system();
}

template <int BK, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_3xtf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, TcParams p) {
  using C = Cfg<BK>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t bar_full[C::kStages];
  __shared__ __align__(8) uint64_t bar_empty[C::kStages];
  __shared__ __align__(8) uint64_t bar_tmem_full[kAccStages];
  __shared__ __align__(8) uint64_t bar_tmem_empty[kAccStages];
  __shared__ uint32_t tmem_slot;
  __shared__ volatile int abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Operand ring, 1024-byte aligned (the swizzle pattern is a function of address bits 4-9).
  const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const int total_tiles = p.batch * p.mblks * p.nblks;

  if (threadIdx.x == 0) {
    abort_flag = 0;
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(smem_u32(&bar_full[s]), 1);
      mbar_init(smem_u32(&bar_empty[s]), 1);
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

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
      asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
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
          mbar_arrive_expect_tx(full, C::kStageBytes);
          if (A_MN) tma_load_4d(sa, &map_a, full, 0, kb * BK, mb * (BM / 32), b * 2);
          else tma_load_3d(sa, &map_a, full, kb * BK, mb * BM, b * 2);
          if (B_MN) tma_load_4d(sa + 2 * C::kABytes, &map_b, full, 0, kb * BK, nb * (BN / 32), b * 2);
          else tma_load_3d(sa + 2 * C::kABytes, &map_b, full, kb * BK, nb * BN, b * 2);
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
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
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
            if (!mbar_wait(smem_u32(&bar_full[stage]), phase, &abort_flag)) {
              report(p.status, 3, 300 + stage, kb);
              ok = false;
              break;
            }
            tcgen05_fence_after();
            const uint32_t a_hi = ring + stage * C::kStageBytes;
            const uint32_t a_lo = a_hi + C::kABytes;
            const uint32_t b_hi = a_hi + 2 * C::kABytes;
            const uint32_t b_lo = b_hi + C::kBBytes;
#pragma unroll
            for (int kk = 0; kk < BK / UMMA_K; ++kk) {
              // K-major: 32 bytes along K inside the swizzled row; MN-major: the next 8-row group
              const uint32_t off_a = A_MN ? kk * 1024 : kk * UMMA_K * 4;
              const uint32_t off_b = B_MN ? kk * 1024 : kk * UMMA_K * 4;
              constexpr uint32_t sbo_a = A_MN ? 512u : C::kSBO, lay_a = A_MN ? 1u : C::kLayoutType;
              constexpr uint32_t sbo_b = B_MN ? 512u : C::kSBO, lay_b = B_MN ? 1u : C::kLayoutType;
              constexpr uint32_t lbo_a = A_MN ? BK * 128u : 16u, lbo_b = B_MN ? BK * 128u : 16u;
              constexpr uint32_t kInstrDesc = instr_desc(A_MN, B_MN);
              const uint64_t da_hi = make_smem_desc(a_hi + off_a, sbo_a, lay_a, lbo_a);
              const uint64_t da_lo = make_smem_desc(a_lo + off_a, sbo_a, lay_a, lbo_a);
              const uint64_t db_hi = make_smem_desc(b_hi + off_b, sbo_b, lay_b, lbo_b);
              const uint64_t db_lo = make_smem_desc(b_lo + off_b, sbo_b, lay_b, lbo_b);
              // the first MMA of a chunk overwrites the accumulator; small terms go first
              umma_tf32(d_tmem, da_lo, db_hi, kInstrDesc, (kb != kb0 || kk != 0) ? 1u : 0u);
              umma_tf32(d_tmem, da_hi, db_lo, kInstrDesc, 1u);
              umma_tf32(d_tmem, da_hi, db_hi, kInstrDesc, 1u);
            }
            tcgen05_commit(smem_u32(&bar_empty[stage]));   // stage reusable once these MMAs retire
            if (++stage == C::kStages) { stage = 0; phase ^= 1u; }
          }
          if (!ok) break;
          tcgen05_commit(smem_u32(&bar_tmem_full[acc]));   // chunk complete
          if (++acc == kAccStages) { acc = 0; acc_phase ^= 1u; }
        }
      }
    }
  } else {
    // ------------------------------------------------------------------ drain + epilogue (warps 2..9)
    const int q = warp & 3;             // TMEM lane quarter this warp may read: lanes 32q .. 32q+31
    const int half = (warp - 2) >> 2;   // which 128 of the tile's 256 columns
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
      const int row = mb * BM + q * 32 + lane;
      const int col0 = nb * BN + half * (BN / 2);
      const bool full_tile = (mb * BM + BM <= p.m) && (nb * BN + BN <= p.n);   // uniform over the CTA
      if (row < p.m) {
        float* crow = p.c + ((int64_t)b * p.m + row) * (int64_t)p.n + col0;
        if (p.bias != nullptr) {
          if (vec_ok && col0 + BN / 2 <= p.n && (reinterpret_cast<uintptr_t>(p.bias) & 15u) == 0) {
            const float4* b4 = reinterpret_cast<const float4*>(p.bias + col0);
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) {
              const float4 bv = __ldg(b4 + j);
              sum[4 * j] = __fadd_rn(sum[4 * j], bv.x);
              sum[4 * j + 1] = __fadd_rn(sum[4 * j + 1], bv.y);
              sum[4 * j + 2] = __fadd_rn(sum[4 * j + 2], bv.z);
              sum[4 * j + 3] = __fadd_rn(sum[4 * j + 3], bv.w);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 2; ++j)
              if (col0 + j < p.n) sum[j] = __fadd_rn(sum[j], __ldg(p.bias + col0 + j));
          }
        }
        // One loop per activation (the choice is uniform for the launch), so each is a straight
        // unrolled sequence over independent elements.
        if (p.act == CLEAVE_ACT_TANH) {
#pragma unroll
          for (int j = 0; j < BN / 2; ++j) sum[j] = tanhf(sum[j]);
        } else if (p.act == CLEAVE_ACT_SIGMOID) {
#pragma unroll
          for (int j = 0; j < BN / 2; ++j) sum[j] = __frcp_rn(__fadd_rn(1.0f, expf(-sum[j])));
        } else if (p.act == CLEAVE_ACT_RELU) {
#pragma unroll
          for (int j = 0; j < BN / 2; ++j) sum[j] = act_apply(sum[j], CLEAVE_ACT_RELU);
        }
        if (!(full_tile && vec_ok)) {
          if (vec_ok && col0 + BN / 2 <= p.n) {
            float4* dst = reinterpret_cast<float4*>(crow);
#pragma unroll
            for (int j = 0; j < BN / 8; ++j) dst[j] = make_float4(sum[4 * j], sum[4 * j + 1], sum[4 * j + 2], sum[4 * j + 3]);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 2; ++j)
              if (col0 + j < p.n) crow[j] = sum[j];
          }
        }
      }
      if (full_tile && vec_ok) {
        // Coalesced store of the warp's 32 x 128 block.  A thread owns one ROW (what tcgen05.ld
        // hands out), but a store instruction is efficient when the warp covers whole 128-byte
        // lines.  So, 32 columns at a time, every thread parks its 8 16-byte words in a
        // warp-private shared tile (word j of row r at slot j ^ (r & 7): conflict free both ways)
        // and the warp then writes 4 rows x 128 bytes per instruction.
        float4* stage = reinterpret_cast<float4*>(smem_raw + (ring - smem_u32(smem_raw)) +
                                                  C::kStages * C::kStageBytes) + (warp - 2) * (32 * 8);
        float* cblock = p.c + ((int64_t)b * p.m + mb * BM + q * 32) * (int64_t)p.n + col0;
#pragma unroll
        for (int pass = 0; pass < BN / 64; ++pass) {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            stage[lane * 8 + (j ^ (lane & 7))] = make_float4(sum[32 * pass + 4 * j], sum[32 * pass + 4 * j + 1],
                                                             sum[32 * pass + 4 * j + 2], sum[32 * pass + 4 * j + 3]);
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int r = it * 4 + (lane >> 3), slot = lane & 7;
            const float4 v = stage[r * 8 + (slot ^ (r & 7))];
            *reinterpret_cast<float4*>(cblock + (int64_t)r * p.n + 32 * pass + 4 * slot) = v;
          }
          __syncwarp();
        }
      }
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
// Experiment switch (CLEAVE_CUDA_SPLIT_MODE): 0 = hi rounded to tf32 (product default);
// 1 = hi left as the raw f32 value, lo = x - truncate_to_tf32(x); 2 = raw hi, lo = x - round_to_tf32(x).
// Modes 1 and 2 probe what the tensor pipe does with the 13 low mantissa bits of an f32 operand.
__constant__ int c_split_mode = 0;

__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  if (c_split_mode != 0) {
    const float t = c_split_mode == 1 ? __uint_as_float(__float_as_uint(x) & 0xFFFFE000u) : tf32_round(x);
    hi = x;
    lo = tf32_round(__fsub_rn(x, t));
    return;
  }
  hi = tf32_round(x);
  // A finite x just below FLT_MAX must not round up to infinity: truncate instead.
  if (fabsf(hi) == INFINITY && fabsf(x) != INFINITY) hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  // Non-finite values carry no low part (inf - inf would inject a NaN of its own).
  lo = (fabsf(hi) == INFINITY || hi != hi) ? 0.0f : tf32_round(__fsub_rn(x, hi));
}

// Source already K-major: src[b][r][k] (r < rows, k < K).  dst planes [b][2][rows_p][Kp].
__global__ void __launch_bounds__(256) split_copy_kernel(const float* __restrict__ src, float* __restrict__ dst,
                                                         int rows, int K, int rows_p, int Kp, int vec) {
  const int b = blockIdx.z;
  const float* s = src + (int64_t)b * rows * K;
  float* hi_p = dst + (int64_t)b * 2 * rows_p * Kp;
  float* lo_p = hi_p + (int64_t)rows_p * Kp;
  const int kq = Kp >> 2;   // Kp is a multiple of 16
  const int64_t total = (int64_t)rows_p * kq;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / kq);
    const int k = (int)(i - (int64_t)r * kq) * 4;
    float x[4] = {0.f, 0.f, 0.f, 0.f};
    if (r < rows) {
      if (vec && k + 3 < K) {
        const float4 v = __ldcs(reinterpret_cast<const float4*>(s + (int64_t)r * K + k));
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (k + j < K) x[j] = s[(int64_t)r * K + k + j];
      }
    }
    float h[4], l[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) split_tf32(x[j], h[j], l[j]);
    const int64_t o = (int64_t)r * Kp + k;
    *reinterpret_cast<float4*>(hi_p + o) = make_float4(h[0], h[1], h[2], h[3]);
    *reinterpret_cast<float4*>(lo_p + o) = make_float4(l[0], l[1], l[2], l[3]);
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

// ---- host side ---------------------------------------------------------------------------------
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

static bool g_mn_major = true;   // CLEAVE_CUDA_GEMM_MN=0: transpose such operands in the pre-pass instead
static int g_bk = 0;   // K-block: 16 (64-byte rows, 4 stages) or 32 (128-byte rows, 2 stages)
static int choose_bk() {
  if (g_bk == 0) {
    const char* e = getenv("CLEAVE_CUDA_GEMM_BK");
    g_bk = (e && atoi(e) == 32) ? 32 : 16;
    const char* mn = getenv("CLEAVE_CUDA_GEMM_MN");
    if (mn && mn[0] == '0') g_mn_major = false;
    const char* sm = getenv("CLEAVE_CUDA_SPLIT_MODE");
    if (sm && sm[0] >= '1' && sm[0] <= '2') {
      const int mode = sm[0] - '0';
      cudaMemcpyToSymbol(c_split_mode, &mode, sizeof(int));
    }
  }
  return g_bk;
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
    int grid = stream_grid(items, 256, 8);
    split_copy_kernel<<<dim3(grid, 1, batch), 256, 0, s>>>(src, dst, R, Cc, Rp, Cp, vec);
  } else {
    split_transpose_kernel<<<dim3(ceil_div(Kp, 32), ceil_div(rows_p, 32), batch), 256, 0, s>>>(src, dst, rows, K,
                                                                                               rows_p, Kp);
  }
  count_launch();
  return cuda_ok(cudaGetLastError(), "operand split launch");
}

template <int BK, bool A_MN, bool B_MN>
static bool run_tc(const CUtensorMap& ma, const CUtensorMap& mb, const TcParams& p) {
  using C = Cfg<BK>;
  static bool attr_set = false;
  if (!attr_set) {
    if (!cuda_ok(cudaFuncSetAttribute(gemm_3xtf32_kernel<BK, A_MN, B_MN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                      C::kSmemBytes),
                 "cudaFuncSetAttribute(gemm)"))
      return false;
    attr_set = true;
  }
  const int tiles = p.batch * p.mblks * p.nblks;
  const int grid = tiles < ctx().sm_count ? tiles : ctx().sm_count;
  profile_mark(true);
  gemm_3xtf32_kernel<BK, A_MN, B_MN><<<grid, kGemmThreads, C::kSmemBytes, ctx().stream>>>(ma, mb, p);
  profile_mark(false);
  count_launch();
  return cuda_ok(cudaGetLastError(), "tcgen05 GEMM launch");
}

bool launch_gemm_3xtf32(const GemmArgs& g) {
  if (!gemm_3xtf32_supported(g)) {
    set_error(CLEAVE_CUDA_ERR_UNSUPPORTED, "3xTF32 GEMM: problem %d x %d x %d (batch %d) is out of range", g.m, g.n,
              g.k, g.batch);
    return false;
  }
  const int bk = choose_bk();
  const int Kp = round_up(g.k, 32);        // multiple of both K-block sizes
  const int Mp = round_up(g.m, BM);
  const int Np = round_up(g.n, BN);
  // Bound the split workspace: process the batch in chunks of at most ~4 GiB of planes.
  const int64_t per_batch_bytes = 2ll * ((int64_t)Mp + Np) * Kp * 4;
  int chunk = (int)((4ll << 30) / per_batch_bytes);
  if (chunk < 1) chunk = 1;
  if (chunk > g.batch) chunk = g.batch;

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
    CUtensorMap ma, mb;
    ok = make_operand_map(&ma, wa, Mp, Kp, nb, bk, BM, a_mn) && make_operand_map(&mb, wb, Np, Kp, nb, bk, BN, b_mn);
    if (!ok) break;
    TcParams p;
    p.c = g.c + (int64_t)b0 * g.m * g.n;
    p.bias = g.bias;
    p.m = g.m;
    p.n = g.n;
    p.num_kb = Kp / bk;
    p.chunk_kb = kChunkK / bk;
    p.batch = nb;
    p.mblks = Mp / BM;
    p.nblks = Np / BN;
    p.act = g.act;
    p.status = ctx().status_dev;
    if (bk == 32) {
      ok = a_mn ? (b_mn ? run_tc<32, true, true>(ma, mb, p) : run_tc<32, true, false>(ma, mb, p))
                : (b_mn ? run_tc<32, false, true>(ma, mb, p) : run_tc<32, false, false>(ma, mb, p));
    } else {
      ok = a_mn ? (b_mn ? run_tc<16, true, true>(ma, mb, p) : run_tc<16, true, false>(ma, mb, p))
                : (b_mn ? run_tc<16, false, true>(ma, mb, p) : run_tc<16, false, false>(ma, mb, p));
    }
  }
  scratch_free(wa);
  scratch_free(wb);
  return ok;
}

}  // namespace cleave
