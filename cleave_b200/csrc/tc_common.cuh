// Shared pieces of the tcgen05 GEMM kernels: tile constants, the shared-memory plan, PTX wrappers
// (mbarrier, TMA, tcgen05), shared-memory / instruction descriptors, kernel parameters.
#pragma once
#include <cuda.h>

#include <cstdint>

#include "common.cuh"
#include "gemm.cuh"

namespace cleave {

constexpr int BM = 128;          // tile rows  (UMMA M)
constexpr int BN = 256;          // tile cols  (UMMA N)
constexpr int UMMA_K = 8;        // tf32 MMA K (32 bytes)
constexpr int kEpiWarps = 8;     // two per TMEM lane quarter, 128 columns each
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;     // producer, issuer, drain warps
// Direct path (the kernel splits raw operands itself): four warpgroups.  0: producer, issuer and
// two idle warps; 1-2: drain warps; 3: split warps.  Registers move from groups 0 and 3 to the
// drain groups (setmaxnreg), whose 128 running sums per thread do not fit the 128 registers that
// 512 threads would get each.
constexpr int kSplitWarps = 4;
constexpr int kDirectThreads = 512;
constexpr int kRegsLight = 64, kRegsSplit = 72, kRegsDrain = 184;   // 128*64 + 128*72 + 256*184 <= 65536
constexpr int kChunkK = 256;     // k values accumulated in TMEM before a drain into registers
constexpr int kAccStages = 2;
constexpr int kTmemCols = kAccStages * BN;   // 512: all of TMEM
constexpr int kGroupM = 16;      // tile-rows per rasterisation group
constexpr unsigned long long kWaitLimitNs = 4000000000ull;   // 4 s per wait

#ifndef CLEAVE_RAW_STAGES
#define CLEAVE_RAW_STAGES 6
#endif
// Shared-memory plan.  Pre-pass path: kStages stages of [A hi | A lo | B hi | B lo], all written by
// TMA.  Direct path: a deep ring of raw stages [A | B] written by TMA plus a shallow ring of lo
// stages [A lo | B lo] written by the split warps just ahead of the MMAs, so the depth that hides
// the TMA latency costs 24 KiB per stage instead of 48.
template <int BK, bool DIRECT>
struct Cfg {
  static_assert(BK == 16, "one K-block size is built: 64-byte rows (K-major) / 16 rows of 128 bytes (MN-major)");
  static constexpr int kRowBytes = BK * 4;
  static constexpr int kABytes = BM * kRowBytes;          // one plane of A
  static constexpr int kBBytes = BN * kRowBytes;          // one plane of B
  static constexpr int kStages = DIRECT ? CLEAVE_RAW_STAGES : 4;        // ring that TMA fills
  static constexpr int kLoStages = DIRECT ? 8 - CLEAVE_RAW_STAGES : 1;  // direct path: ring of lo planes
  static constexpr int kStageBytes = DIRECT ? kABytes + kBBytes : 2 * (kABytes + kBBytes);
  static constexpr int kLoRingOffset = kStages * kStageBytes;
  static constexpr int kRingBytes = kLoRingOffset + (DIRECT ? kLoStages * (kABytes + kBBytes) : 0);
  static constexpr int kStoreStageBytes = kEpiWarps * 32 * 128;      // per drain warp: 32 rows x 32 floats
  static constexpr int kSmemBytes = kRingBytes + kStoreStageBytes + 1024;   // + alignment slack
  static constexpr uint32_t kLayoutType = 4u;                       // K-major planes: SWIZZLE_64B
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
// MN-major operand (row / column index contiguous): for 4-byte elements the only layout the tensor
// pipe takes is the 128-byte swizzle with 32-byte atoms (TMA: CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B).
// The tile is a sequence of 32-wide blocks along M or N, each block BK rows of 128 bytes; the
// swizzle pattern spans 4 rows (512 bytes), a k-step (8 rows) is 1024 bytes, stride byte offset =
// 512 (pitch of 4-row groups), leading byte offset = BK * 128 (pitch of blocks).
//   bits  0-13 start address >> 4     bits 16-29 leading byte offset >> 4 (1: unused when swizzled)
//   bits 32-45 stride byte offset >> 4 (8-row group pitch)   bits 46-47 descriptor version (1)
//   bits 61-63 swizzle mode (1 = 128 B with 32-byte atoms, 2 = 128 B, 4 = 64 B)
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
__host__ __device__ constexpr uint32_t instr_desc(bool a_mn, bool b_mn, int n) {
  return (1u << 4) | (2u << 7) | (2u << 10) | ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) |
         ((uint32_t)(n >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
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
// The same wait for a load that was issued further back with other work in between: the registers pass through the
// statement as in/out operands, so that no use of them can be scheduled above it.
__device__ __forceinline__ void tmem_ld_wait_for(uint32_t (&r)[32]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
                 "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
                 "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
               :
               : "memory");
}

__device__ __forceinline__ float act_apply(float v, int act) {
  switch (act) {
    case CLEAVE_ACT_RELU: return v != v ? v : (v > 0.0f ? v : 0.0f);
    case CLEAVE_ACT_SIGMOID: return __frcp_rn(__fadd_rn(1.0f, expf(-v)));
    case CLEAVE_ACT_TANH: return tanhf(v);
    default: return v;
  }
}

// Low part of the in-kernel split: d = x minus x with its 13 low mantissa bits cleared (exact), then
// half a tf32 unit is added to d's magnitude so that the tensor pipe's own truncation of the 13 low
// bits rounds d to the nearest tf32 value.  Integer / full-rate instructions only: a cvt per
// element would make the split warps slower than the MMAs they feed.
__device__ __forceinline__ float split_lo(float x) {
  const float d = __fsub_rn(x, __uint_as_float(__float_as_uint(x) & 0xFFFFE000u));
  return __uint_as_float(__float_as_uint(d) + 0x1000u);
}

struct TcParams {
  float* c;             // [batch][m][n]
  float* c_lo = nullptr;   // [batch][m][n] or null: also store the low split part of every result (see split_lo),
                           // i.e. the lo plane a following GEMM needs when C is one of its operands
  const float* bias;    // [n] or null
  const float* dact_y;  // [batch][m][n] or null: multiply the product by dact'(y) (backward form)
  int dact;
  int m, n;
  int num_kb;           // K_padded / BK
  int chunk_kb;         // K-blocks per accumulation chunk (kChunkK / BK)
  int batch, mblks, nblks;
  int act;
  int a_blocked, b_blocked;   // direct path, MN-major operand: one 4-D box per stage instead of 32-wide boxes
  int b_box_rows;             // direct path: rows of B fetched and split per stage (BN, less when n is small)
  int b_sliced;               // direct path: B is a K-sliced view, map dimensions {k, slice, row}
  int a_sliced = 0;           // direct path: the same for a K-major A
  int pair_group_m = 8;       // pair kernel: 256-row tile-rows per rasterisation group
  int sk_tiles = 0;           // pair kernel: the last sk_tiles tiles (a partly filled wave) are each cut along K into
  int sk_slices = 0;          // sk_slices runs that different clusters add up; their partial sums go to sk_part and a
                              // second kernel adds them in K order; 0 = off
  float* sk_part = nullptr;   // [sk_slices][sk_tiles][256][256]: slot = run * sk_tiles + tile of the region
  int c_tma;                  // pair kernel: a tensor map over C exists (16-byte aligned, n a multiple of 4): TMA stores
                              // of 32 x 32 blocks (1) or of 32 x 16 blocks, two in flight (2)
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

// Stores one drain warp's 32 x 128 block (one row per lane in `sum`) into the matrix `cmat` ([batch][m][n]).
// Ragged tiles: every lane writes its own row.  Full tiles: a thread owns one ROW (what tcgen05.ld hands
// out), but a store instruction is efficient when the warp covers whole 128-byte lines, so, 32 columns at a
// time, every thread parks its 8 16-byte words in the warp-private shared tile `stage` (word j of row r at
// slot j ^ (r & 7): conflict free both ways) and the warp then writes 4 rows x 128 bytes per instruction --
// or, with `map_c` (tensor map over cmat {n, m, batch}), one lane hands blocks to TMA as bulk tensor stores:
// p.c_tma == 1: 32 x 32 blocks (box 32 x 32, 128-byte swizzle), one at a time; p.c_tma == 2: 32-row x 16-column
// blocks (box 16 x 32, 64-byte swizzle), two in flight.
__device__ __forceinline__ void store_block(const float (&sum)[BN / 2], float* cmat, const TcParams& p, int b,
                                            int tile_row0, int nb, int q, int half, int lane, bool vec_ok, float4* stage,
                                            const CUtensorMap* map_c) {
  const int row = tile_row0 + q * 32 + lane;
  const int col0 = nb * BN + half * (BN / 2);
  const bool full_tile = (tile_row0 + BM <= p.m) && (nb * BN + BN <= p.n);   // uniform over the warps of a tile
  if (!(full_tile && vec_ok)) {
    if (row < p.m) {
      float* crow = cmat + ((int64_t)b * p.m + row) * (int64_t)p.n + col0;
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
    return;
  }
  if (map_c != nullptr && p.c_tma == 1) {
    // One 32 x 32 block per bulk store: the shared tile (word j of row r at slot j ^ (r & 7), rows of 128 bytes) is
    // exactly TMA's 128-byte swizzle.  The warp waits for the copy engine to have read the tile before repacking it.
    const uint32_t stage_addr = smem_u32(stage);
#pragma unroll
    for (int pass = 0; pass < BN / 64; ++pass) {
#pragma unroll
      for (int j = 0; j < 8; ++j)
        stage[lane * 8 + (j ^ (lane & 7))] = make_float4(sum[32 * pass + 4 * j], sum[32 * pass + 4 * j + 1],
                                                         sum[32 * pass + 4 * j + 2], sum[32 * pass + 4 * j + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the copy engine
      __syncwarp();
      if (lane == 0) {
        asm volatile(
            "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
            ::"l"(map_c), "r"(stage_addr), "r"(col0 + 32 * pass), "r"(tile_row0 + q * 32), "r"(b)
            : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the tile may be overwritten
      }
      __syncwarp();
    }
    return;
  }
  if (map_c != nullptr) {
    // p.c_tma == 2: two 2 KiB halves of the warp's staging tile alternate, each a 32-row x 16-column block (rows of
    // 64 bytes in TMA's 64-byte swizzle: 16-byte word j of row r at slot j ^ ((r >> 1) & 3), conflict free for the
    // row-per-lane writes).  While the copy engine reads one half the warp already packs the other, so the latency
    // of a bulk store is hidden behind the next one.
    const uint32_t stage_addr = smem_u32(stage);
    constexpr int kPasses = BN / 2 / 16;
#pragma unroll
    for (int pass = 0; pass < kPasses; ++pass) {
      const int half_buf = pass & 1;
      if (pass >= 2) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");   // this half has been read
        __syncwarp();
      }
      float4* buf = stage + half_buf * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j)
        buf[lane * 4 + (j ^ ((lane >> 1) & 3))] = make_float4(sum[16 * pass + 4 * j], sum[16 * pass + 4 * j + 1],
                                                              sum[16 * pass + 4 * j + 2], sum[16 * pass + 4 * j + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // generic writes -> visible to the copy engine
      __syncwarp();
      if (lane == 0) {
        asm volatile(
            "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
            ::"l"(map_c), "r"(stage_addr + half_buf * 2048), "r"(col0 + 16 * pass), "r"(tile_row0 + q * 32), "r"(b)
            : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
      }
    }
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // the staging tile may be reused
    __syncwarp();
    return;
  }
  float* cblock = cmat + ((int64_t)b * p.m + tile_row0 + q * 32) * (int64_t)p.n + col0;
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

// Epilogue of one drain warp: its 32 rows x 128 columns of a tile (rows tile_row0 + 32q .., columns
// nb*BN + 128*half ..), one row per lane in `sum`: + bias[col], activation or activation derivative, store to C
// (and, when p.c_lo is set, the low split part of the same values to that plane).
// `stage`: this warp's 4 KiB of shared memory for the coalesced store; `map_c`: see store_block.
__device__ __forceinline__ void tile_epilogue(float (&sum)[BN / 2], const TcParams& p, int b, int tile_row0, int nb,
                                              int q, int half, int lane, bool vec_ok, float4* stage,
                                              const CUtensorMap* map_c = nullptr) {
  const int row = tile_row0 + q * 32 + lane;
  const int col0 = nb * BN + half * (BN / 2);
  if (row < p.m) {
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
      // 1 / (1 + e^-z) with the hardware exponential and reciprocal: within a few ulp (~3e-7 relative) of the
      // IEEE sequence the elementwise kernel runs, at a third of its instructions -- the epilogue of a product
      // with one tile per CTA is fully exposed (measured: 12 us of a 146 us product with the IEEE sequence)
#pragma unroll
      for (int j = 0; j < BN / 2; ++j) sum[j] = __fdividef(1.0f, 1.0f + __expf(-sum[j]));
    } else if (p.act == CLEAVE_ACT_RELU) {
#pragma unroll
      for (int j = 0; j < BN / 2; ++j) sum[j] = act_apply(sum[j], CLEAVE_ACT_RELU);
    }
  }
  if (p.dact_y != nullptr) {
    // backward form: times the activation derivative taken from the forward output y at the same place; one
    // straight loop per activation (the choice is uniform for the launch)
    const bool full_tile = (tile_row0 + BM <= p.m) && (nb * BN + BN <= p.n);   // uniform over the warps of a tile
    const bool y_aligned = vec_ok && (reinterpret_cast<uintptr_t>(p.dact_y) & 15u) == 0;
    if (full_tile && y_aligned) {
      // y is read the way C is stored: the warp fetches a 32 x 32 block with whole 128-byte lines (4 rows per
      // instruction), parks it in its swizzled staging tile, and every lane then picks up its own row.  A lane
      // reading its row straight from global memory touches 32 different lines per instruction.
      const float* yblock = p.dact_y + ((int64_t)b * p.m + tile_row0 + q * 32) * (int64_t)p.n + col0;
#define CLEAVE_DACT_STAGED(ACT)                                                                                   \
  _Pragma("unroll") for (int pass = 0; pass < BN / 64; ++pass) {                                                  \
    _Pragma("unroll") for (int it = 0; it < 8; ++it) {                                                            \
      const int r = it * 4 + (lane >> 3), slot = lane & 7;                                                        \
      stage[r * 8 + (slot ^ (r & 7))] =                                                                           \
          __ldg(reinterpret_cast<const float4*>(yblock + (int64_t)r * p.n + 32 * pass + 4 * slot));               \
    }                                                                                                             \
    __syncwarp();                                                                                                 \
    _Pragma("unroll") for (int j = 0; j < 8; ++j) {                                                               \
      const float4 y = stage[lane * 8 + (j ^ (lane & 7))];                                                        \
      sum[32 * pass + 4 * j] = dact_apply(y.x, sum[32 * pass + 4 * j], ACT);                                      \
      sum[32 * pass + 4 * j + 1] = dact_apply(y.y, sum[32 * pass + 4 * j + 1], ACT);                              \
      sum[32 * pass + 4 * j + 2] = dact_apply(y.z, sum[32 * pass + 4 * j + 2], ACT);                              \
      sum[32 * pass + 4 * j + 3] = dact_apply(y.w, sum[32 * pass + 4 * j + 3], ACT);                              \
    }                                                                                                             \
    __syncwarp();                                                                                                 \
  }
      if (p.dact == CLEAVE_ACT_TANH) {
        CLEAVE_DACT_STAGED(CLEAVE_ACT_TANH)
      } else if (p.dact == CLEAVE_ACT_SIGMOID) {
        CLEAVE_DACT_STAGED(CLEAVE_ACT_SIGMOID)
      } else if (p.dact == CLEAVE_ACT_RELU) {
        CLEAVE_DACT_STAGED(CLEAVE_ACT_RELU)
      }
#undef CLEAVE_DACT_STAGED
    } else if (row < p.m) {
      const float* yrow = p.dact_y + ((int64_t)b * p.m + row) * (int64_t)p.n + col0;
      const bool yvec = y_aligned && col0 + BN / 2 <= p.n;
#define CLEAVE_DACT_LOOP(ACT)                                                                   \
  if (yvec) {                                                                                   \
    _Pragma("unroll") for (int j = 0; j < BN / 8; ++j) {                                        \
      const float4 y = __ldg(reinterpret_cast<const float4*>(yrow) + j);                        \
      sum[4 * j] = dact_apply(y.x, sum[4 * j], ACT);                                            \
      sum[4 * j + 1] = dact_apply(y.y, sum[4 * j + 1], ACT);                                    \
      sum[4 * j + 2] = dact_apply(y.z, sum[4 * j + 2], ACT);                                    \
      sum[4 * j + 3] = dact_apply(y.w, sum[4 * j + 3], ACT);                                    \
    }                                                                                           \
  } else {                                                                                      \
    _Pragma("unroll") for (int j = 0; j < BN / 2; ++j)                                          \
      if (col0 + j < p.n) sum[j] = dact_apply(__ldg(yrow + j), sum[j], ACT);                    \
  }
      if (p.dact == CLEAVE_ACT_TANH) {
        CLEAVE_DACT_LOOP(CLEAVE_ACT_TANH)
      } else if (p.dact == CLEAVE_ACT_SIGMOID) {
        CLEAVE_DACT_LOOP(CLEAVE_ACT_SIGMOID)
      } else if (p.dact == CLEAVE_ACT_RELU) {
        CLEAVE_DACT_LOOP(CLEAVE_ACT_RELU)
      }
#undef CLEAVE_DACT_LOOP
    }
  }
  store_block(sum, p.c, p, b, tile_row0, nb, q, half, lane, vec_ok, stage, map_c);
  if (p.c_lo != nullptr) {
    // the same block once more, as the low part of the split-precision representation of what was just stored
#pragma unroll
    for (int j = 0; j < BN / 2; ++j) sum[j] = split_lo(sum[j]);
    store_block(sum, p.c_lo, p, b, tile_row0, nb, q, half, lane, vec_ok && ((reinterpret_cast<uintptr_t>(p.c_lo) & 15u) == 0),
                stage, nullptr);
  }
}

// Pair kernel (gemm_tc_pair.cu): two CTAs of a cluster share one 256 x 256 tile (tcgen05 cta_group::2).
// `maps` = {A planes, B planes, C}; the planes must be padded to 256 rows for both operands; the map over C
// ({n, m, batch}; box and swizzle as p.c_tma says, see store_block) is read only when p.c_tma is set.
// In lo-plane mode `maps` = {A, B, C, A lo, B lo} over the caller's tensors and their lo planes (K-block 32).
bool run_tc_pair(bool a_mn, bool b_mn, const CUtensorMap* maps, const TcParams& p, int bk, bool lo_plane = false);
// Short-K variant (K_padded <= 256, plain product, padded planes with K-block 32): 16 drain warps per CTA.
bool run_tc_pair_shortk(bool a_mn, bool b_mn, const CUtensorMap* maps, const TcParams& p);

}  // namespace cleave
