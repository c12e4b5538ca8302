// uint8 weight x fixed-point activation GEMM for sm_100a: the many-rows path (prompt ingestion with
// T tokens per stream, decode with B streams) of the same arithmetic contract as stream_gemv.cuh.
//
//   out[r][n] = epilogue( contract(matrix, x[r])[n] )      r = 0..R-1 activation rows
//
// Arithmetic is identical to the one-row kernel: every activation row is turned into 24-bit fixed
// point X = rint(xs * QMAX / max|xs|), split into three signed base-256 digits, and the dot products
// with the uint8 weights are exact integer sums recombined in int64.  Here the digit rows are the
// B operand of 5th-generation tensor-core MMAs (tcgen05.mma kind::i8, u8 x s8 -> s32):
//
//   A  = mt weight rows    x 128 bytes of K   (one TMA box of qt[N][K], 128-byte swizzle, K-major; mt = 128 or 256)
//   B  = 3*Rt digit rows   x 128 bytes of K   (three TMA boxes, [digit][Rt activation rows], Rt = 16..80)
//   D  = 128 lanes x 3*Rt int32 columns per 128 weight rows in tensor memory (TMEM),
//        column = digit*Rt + row.  A 256-row tile keeps its second accumulator at column 256 (two
//        weight sub-tiles share one digit tile); with 128-row tiles columns 0 and 256 are two
//        buffers, so the epilogue of one tile runs under the MMAs of the next.
//
// Persistent kernel, one CTA per SM looping over tiles; a CTA walks K in 128-byte steps through a
// ring of shared-memory stages that runs on across tiles: warp 0 issues the TMA copies, warp 1
// issues the MMAs (one elected thread; completion is signalled to the ring by tcgen05.commit on the
// stage's mbarrier), warps 4-19 read the accumulators with tcgen05.ld and apply the affine terms
// and the fused element-wise op.  The kernel is bound by operand traffic from L2 to shared memory
// (int8 MMAs need ~250 MACs per byte to saturate, the 256 x 240 tile gives M*N/(M+N) = 124) until
// the tensor pipe saturates (81 % active on the largest shapes).  Tiles that share a weight tile
// are adjacent in issue order so it is read from HBM once and from L2 afterwards.  The host picks
// mt, Rt and, for launches with too few tiles, a split of K over several CTAs (see GemmParams).
//
// Every wait is bounded (common.cuh): on expiry the CTA raises its abort flag, sets a status bit,
// skips its remaining work, and still frees its tensor memory before it retires.
#pragma once

#include "stream_gemv.cuh"

namespace b200 {

constexpr int kGemmM = 256;                              // weight rows per tile = two MMA M=128 sub-tiles
constexpr int kGemmRowsMax = 80;                         // activation rows per tile (multiple of 16)
constexpr int kDigits = 3;
constexpr int kGemmStages = 3;
constexpr int kGemmABytes = kGemmM * 128;                // 32 KB
constexpr int kGemmStageBytes = kGemmABytes + kDigits * kGemmRowsMax * 128;   // 62 KB
constexpr int kGemmTmemCols = 512;                       // both accumulators; one CTA per SM (shared memory)
constexpr int kGemmAcc1Col = 256;                        // first column of the second accumulator
constexpr int kGemmEpiWarps = 16;                        // four per TMEM lane quadrant
constexpr int kGemmThreads = 128 + kGemmEpiWarps * 32;   // warp 0 TMA, 1 MMA, 2 TMEM allocation, 4.. epilogue
constexpr int kGemmChunk = 8;                            // activation rows an epilogue warp handles per TMEM read
// 8-row chunks of both 128-row sub-tiles that one epilogue warp takes at most (every fourth of its lane quadrant's)
constexpr int kGemmItemsPerWarp = (2 * (kGemmRowsMax / kGemmChunk) + kGemmEpiWarps / 4 - 1) / (kGemmEpiWarps / 4);
constexpr int kSplitMaxTiles = 320;                      // tiles a split-K launch may have
constexpr int kSplitMaxRt = 32;                          // and its tile height
constexpr size_t kSplitAccBytes = size_t(kSplitMaxTiles) * kDigits * kSplitMaxRt * 128 * 4;   // 15.7 MB
constexpr int kGemmOffScal = 1024;                       // SegScalars[80]
constexpr int kGemmOffRing = 4096;
constexpr int kGemmSmem = kGemmOffRing + kGemmStages * kGemmStageBytes;

// The digit rows of a launch are laid out [matrix][digit][Rpad][K] with Rpad = R rounded up to 16,
// whatever tile height the GEMM then picks: a tile that reaches past row R reads the next digit
// plane (or TMA's zero fill past the end) into accumulator columns that are never stored.
inline int gemm_padded_rows(int R) { return (R + 15) / 16 * 16; }

struct GemmSeg {
  CUtensorMap wmap;    // u8 qt as [K/128][N][128 B], box [1][mt][128], 128-byte swizzle
  CUtensorMap xmap;    // s8 digits as [K/128][3*Rpad][128 B], box [1][Rt][128], 128-byte swizzle
  const float* rx;     // [N] or null
  const float* mx;     // [N] or null
  const SegScalars* scal;  // [R] per activation row: sd, zp, sumxs, sumx
  float* out;          // [R][ldo]
  const float* res;    // [R][ldres] added to the output, or null
  const float* gate;   // [R][ldgate] multiplies act(y), or null
  long long ldo, ldres, ldgate;
  float half;
  int N;
  int act;
};

struct GemmParams {
  GemmSeg seg[kMaxSeg];
  int nseg, K, R, Rpad;
  int Rt;              // activation rows per tile (multiple of 16, <= 80)
  int mt;              // weight rows per tile: 256 (two accumulators) or 128 (small grids: more CTAs)
  int row_tiles;       // ceil(R / Rt)
  int block_tiles;     // row tiles per row block (tile order below); row_tiles when all digit rows fit L2 at once
  int tiles_seg[kMaxSeg];  // tiles per matrix = row_tiles * ceil(N / mt)
  int ntiles;          // all tiles of the launch; the grid is min(ntiles * ksplit, SMs), CTAs loop over work items
  // Split-K for launches with few tiles (few activation rows): work item = (tile, K slice); every
  // slice adds its int32 digit sums into sk_acc with integer atomics (exact, order-free), takes a
  // ticket, and the CTA that draws the last ticket of a tile reads the totals, runs the epilogue and
  // leaves sk_acc / sk_count zero again.  Nobody waits for anybody.
  int ksplit;          // 1, 2, 4 or 8 slices (divides K/128; only with 128-row tiles and Rt <= 32)
  int* sk_acc;         // [kSplitMaxTiles][3*Rt][128] int32, zero between launches
  unsigned* sk_count;  // [kSplitMaxTiles] tickets, zero between launches
  int* status;
};

// ---- tcgen05 wrappers ------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor: K-major tile of 128-byte rows, 128-byte swizzle; groups of 8
// rows are 1024 bytes apart.  `addr` is the shared-memory byte address of the tile (1024-aligned)
// plus the byte offset of the K slice inside the 128-byte row.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr) {
  uint64_t d = 0;
  d |= uint64_t((addr & 0x3FFFFu) >> 4);   // start address, 16-byte units
  d |= uint64_t(1024 >> 4) << 32;          // stride between 8-row groups
  d |= uint64_t(1) << 46;                  // descriptor version of this architecture
  d |= uint64_t(2) << 61;                  // 128-byte swizzle
  return d;
}

// Instruction descriptor: D s32, A u8, B s8, both K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc_u8s8(int M, int N) {
  return (2u << 4) | (0u << 7) | (1u << 10) | (uint32_t(N >> 3) << 17) | (uint32_t(M >> 4) << 24);
}

__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The mbarrier receives one arrival when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// 16 consecutive int32 columns of this warp's 32 lanes.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, int (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
        "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// 8 consecutive int32 columns of this warp's 32 lanes.
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, int (&v)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
               : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tile t of a launch -> (segment, first weight row, first activation row).  Within a matrix the order is
// row block, weight tile, row tile of the block: the CTAs working side by side share a weight tile, and
// all weight tiles sweep over one block of digit rows (sized by the launcher to stay in L2) before the
// next block is touched, so the digit rows come from DRAM once instead of once per few weight tiles.
struct GemmTile { int seg, n0, row0; };
__device__ __forceinline__ GemmTile gemm_tile(const GemmParams& P, int t) {
  int s = 0;
  while (s < P.nseg - 1 && t >= P.tiles_seg[s]) { t -= P.tiles_seg[s]; ++s; }
  const int wtiles = P.tiles_seg[s] / P.row_tiles;
  const int per_block = P.block_tiles * wtiles;
  const int blk = t / per_block, first = blk * P.block_tiles;
  const int nb = min(P.block_tiles, P.row_tiles - first);     // row tiles of this (maybe last, shorter) block
  const int idx = t - blk * per_block;
  const int wt = idx / nb;
  return {s, wt * P.mt, (first + idx - wt * nb) * P.Rt};
}

// Row tiles per block: three digit planes of a block's rows take at most kGemmDigitBlockBytes.
constexpr long long kGemmDigitBlockBytes = 16ll << 20;   // measured best of 8 / 16 / 24 / 32 / 48 MB on the 126 MB L2
inline int gemm_block_tiles(int row_tiles, int Rt, int K) {
  const long long per_tile = (long long)kDigits * Rt * K;
  const long long fit = per_tile > 0 ? kGemmDigitBlockBytes / per_tile : row_tiles;
  return int(fit < 1 ? 1 : fit > row_tiles ? row_tiles : fit);
}

__global__ void __launch_bounds__(kGemmThreads, 1) tile_gemm_kernel(const __grid_constant__ GemmParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Rt = P.Rt;
  const int S = P.ksplit;
  const int nk = P.K / 128 / S;          // K steps of one work item
  const int nitems_all = P.ntiles * S;
  const uint32_t a_bytes = uint32_t(P.mt) * 128u;
  const uint32_t b_bytes = uint32_t(kDigits * Rt * 128);

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 8);
  const uint32_t acc_full0 = smem_u32(bars + 16), acc_empty0 = smem_u32(bars + 18);   // two of each (8 bytes apart)
  // With 128-row tiles one accumulator needs 3*Rt <= 240 columns, so two fit in TMEM: tile i+1 is
  // accumulated at column 256 while the epilogue still reads tile i at column 0.  With 256-row tiles
  // the second accumulator of the SAME tile lives at column 256 and tiles alternate on one buffer.
  const bool dbuf = P.mt != kGemmM;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 256);
  volatile int* issued_ptr = reinterpret_cast<volatile int*>(smem + 260);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 264);
  SegScalars* scal = reinterpret_cast<SegScalars*>(smem + kGemmOffScal);
  unsigned char* ring = smem + kGemmOffRing;

  if (tid == 0) {
    for (int i = 0; i < kGemmStages; ++i) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
    for (int i = 0; i < 2; ++i) { mbar_init(acc_full0 + 8 * i, 1); mbar_init(acc_empty0 + 8 * i, kGemmEpiWarps); }
    *abort_flag = 0;
    *issued_ptr = 0;
    fence_mbar_init();
  }
  if (warp == 2) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kGemmTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  griddep_launch_dependents();

  // Persistent: CTA c handles tiles c, c + grid, c + 2*grid, ...  The operand ring runs on across
  // tiles (the producer is already fetching the next tile while the epilogue of this one runs).
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      griddep_wait();   // the digit rows come from the preparation kernel in front of this launch
      int issued = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < nitems_all && ok; it += gridDim.x) {
        const GemmTile T = gemm_tile(P, it / S);
        const GemmSeg& Sg = P.seg[T.seg];
        const int kbase = (it % S) * nk;
        for (int kc = 0; kc < nk; ++kc, ++issued) {
          const int slot = issued % kGemmStages;
          const uint32_t phase = uint32_t(issued / kGemmStages) & 1u;
          if (!mbar_wait_bounded(empty0 + 8 * slot, phase ^ 1u, abort_flag)) {
            if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
            ok = false;
            break;
          }
          const uint32_t bar = full0 + 8 * slot;
          const uint32_t dst = smem_u32(ring + size_t(slot) * kGemmStageBytes);
          mbar_arrive_expect_tx(bar, a_bytes + b_bytes);
          tma_load_3d(dst, &Sg.wmap, 0, T.n0, kbase + kc, bar);   // rows past N are zero-filled
#pragma unroll
          for (int d = 0; d < kDigits; ++d)
            tma_load_3d(dst + kGemmABytes + uint32_t(d * Rt * 128), &Sg.xmap, 0, d * P.Rpad + T.row0, kbase + kc, bar);
        }
      }
      *issued_ptr = issued;
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_u8s8(128, kDigits * Rt);
      bool ok = true;
      int step = 0, iter = 0;
      for (int it = blockIdx.x; it < nitems_all && ok; it += gridDim.x, ++iter) {
        const GemmTile T = gemm_tile(P, it / S);
        const bool two = P.mt == kGemmM && T.n0 + 128 < P.seg[T.seg].N;   // second 128-row sub-tile holds real rows
        // the epilogue must have read this buffer's previous tile out of TMEM
        const int buf = dbuf ? (iter & 1) : 0, use = dbuf ? (iter >> 1) : iter;
        const uint32_t tacc = tmem + uint32_t(buf * kGemmAcc1Col);
        if (!mbar_wait_bounded(acc_empty0 + 8 * buf, uint32_t(use & 1) ^ 1u, abort_flag)) {
          if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kc = 0; kc < nk; ++kc, ++step) {
          const int slot = step % kGemmStages;
          const uint32_t phase = uint32_t(step / kGemmStages) & 1u;
          if (!mbar_wait_bounded(full0 + 8 * slot, phase, abort_flag)) {
            if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_u32(ring + size_t(slot) * kGemmStageBytes);
          const uint64_t ad0 = umma_desc(a), ad1 = umma_desc(a + 128 * 128), bd = umma_desc(a + kGemmABytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {   // 32 bytes of K per instruction: +2 in the descriptors' 16-byte address units
            const uint32_t acc = (kc | k) != 0 ? 1u : 0u;
            umma_i8(tacc, ad0 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
            if (two) umma_i8(tmem + kGemmAcc1Col, ad1 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
          }
          umma_commit(empty0 + 8 * slot);   // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);   // accumulators of this tile complete
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- epilogue: 16 warps.  A warp can
    // read TMEM lanes 32*(warp%4)..+31 only, so four warps share each lane quadrant and take every
    // fourth 8-row chunk of the accumulators (many warps with short chains: the epilogue is bound by
    // instruction latency, not by issue slots).
    const int q = warp & 3, eg = (warp - 4) >> 2;
    constexpr int EG = kGemmEpiWarps / 4, CH = kGemmChunk;
    const int et = tid - 128;
    griddep_wait();
    bool ok = true;
    int iter = 0;
    volatile int* last_flag = reinterpret_cast<volatile int*>(smem + 272);   // split-K: this CTA drew a tile's last ticket
    for (int it = blockIdx.x; it < nitems_all && ok; it += gridDim.x, ++iter) {
      const int tile = it / S;
      const GemmTile T = gemm_tile(P, tile);
      const GemmSeg& Sg = P.seg[T.seg];
      const int n0 = T.n0, row0 = T.row0;
      const bool two = P.mt == kGemmM && n0 + 128 < Sg.N;
      named_bar_sync(1, kGemmEpiWarps * 32);   // every epilogue warp is done with the previous tile's scalars
      for (int i = et; i < Rt * 8; i += kGemmEpiWarps * 32) {
        const int r = row0 + (i >> 3);
        reinterpret_cast<float*>(scal)[i] = r < P.R ? __ldcg(reinterpret_cast<const float*>(Sg.scal + r) + (i & 7)) : 0.f;
      }
      named_bar_sync(1, kGemmEpiWarps * 32);
      const int buf = dbuf ? (iter & 1) : 0, use = dbuf ? (iter >> 1) : iter;
      const uint32_t acc_empty = acc_empty0 + 8 * buf;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(acc_full0 + 8 * buf, uint32_t(use & 1), abort_flag));
      if (!ok) {
        if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
        break;
      }
      tc_fence_after();
      const int nchunks = Rt / CH, nitems = (two ? 2 : 1) * nchunks;
      // this warp's last item that really reads TMEM: after it the accumulators may be overwritten
      int last_item = -1;
      for (int item = eg; item < nitems; item += EG)
        if (row0 + (item % nchunks) * CH < P.R) last_item = item;
      if (last_item < 0) {
        tc_fence_before();
        if (lane == 0) mbar_arrive(acc_empty);
      }
      // exact dot products of 8 rows of one output column from their three digit sums, as fp32
      auto recombine = [&](const int (&da)[CH], const int (&db)[CH], const int (&dc)[CH], float (&yf)[CH]) {
#pragma unroll
        for (int j = 0; j < CH; ++j)
          yf[j] = __ll2float_rn((long long)da[j] * 65536 + (long long)db[j] * 256 + (long long)dc[j]);
      };
      // affine terms + fused element-wise op for 8 rows of one output column
      auto finish = [&](const float (&yf)[CH], int h, int j0) {
        const int n = n0 + h * 128 + q * 32 + lane;
        const bool nvalid = n < Sg.N;
        const int nc = nvalid ? n : Sg.N - 1;   // clamped: loads stay in bounds, the store is predicated
        const float rx = Sg.rx ? Sg.rx[nc] : 1.f, mx = Sg.mx ? Sg.mx[nc] : 0.f;
        // branch-free over the rows so that their dependency chains interleave
        float yv[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const float4 sc = *reinterpret_cast<const float4*>(&scal[j0 + j]);   // sd, zp, sumxs, sumx
          float y = __fmul_rn(yf[j], sc.x) + Sg.half * sc.z;
          y *= rx;               // rx = 1, mx = 0 when the matrix has no per-output terms: exact no-ops
          y += sc.y;
          y += mx * sc.w;
          yv[j] = y;
        }
        if (Sg.act == ACT_RELUSQ) {
#pragma unroll
          for (int j = 0; j < CH; ++j) { const float t = fmaxf(yv[j], 0.f); yv[j] = t * t; }
        } else if (Sg.act == ACT_SIGMOID) {
#pragma unroll
          for (int j = 0; j < CH; ++j) yv[j] = sigmoidf_(yv[j]);
        }
        const int rlast = P.R - 1;
        if (Sg.gate) {
          float gv[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) { const int r = min(row0 + j0 + j, rlast); gv[j] = __ldcg(Sg.gate + size_t(r) * Sg.ldgate + nc); }
#pragma unroll
          for (int j = 0; j < CH; ++j) yv[j] *= gv[j];
        }
        if (Sg.res) {
          float rv[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) { const int r = min(row0 + j0 + j, rlast); rv[j] = __ldcg(Sg.res + size_t(r) * Sg.ldres + nc); }
#pragma unroll
          for (int j = 0; j < CH; ++j) yv[j] += rv[j];
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int r = row0 + j0 + j;
          if (r <= rlast && nvalid) Sg.out[size_t(r) * Sg.ldo + n] = yv[j];
        }
      };
      // split-K scratch of this tile: [column = digit*Rt + row][128 weight rows] (mt = 128 only)
      int* sk = S > 1 ? P.sk_acc + size_t(tile) * (kDigits * Rt) * 128 + q * 32 + lane : nullptr;
      if (S == 1) {
        // Two passes, so that the accumulators are free again as early as possible (a 256-row tile has no
        // second buffer: the next tile's MMAs wait for this): first every item of this warp leaves TMEM and
        // is recombined to one fp32 per output (40 registers at most), then the affine terms, the gate and
        // residual loads and the stores run from registers under the next tile's MMAs.
        float yf[kGemmItemsPerWarp][CH];
#pragma unroll
        for (int u = 0; u < kGemmItemsPerWarp; ++u) {
          const int item = eg + u * EG;
          if (item < nitems) {
            const int h = item / nchunks, j0 = (item - h * nchunks) * CH;
            if (row0 + j0 < P.R) {   // warp-uniform
              const uint32_t tbase = tmem + (uint32_t(q * 32) << 16) + uint32_t((h + buf) * kGemmAcc1Col + j0);
              int da[CH], db[CH], dc[CH];
              tmem_ld8(tbase, da);
              tmem_ld8(tbase + uint32_t(Rt), db);
              tmem_ld8(tbase + uint32_t(2 * Rt), dc);
              tmem_ld_wait();
              if (item == last_item) {
                tc_fence_before();
                if (lane == 0) mbar_arrive(acc_empty);
              }
              recombine(da, db, dc, yf[u]);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kGemmItemsPerWarp; ++u) {
          const int item = eg + u * EG;
          if (item < nitems) {
            const int h = item / nchunks, j0 = (item - h * nchunks) * CH;
            if (row0 + j0 < P.R) finish(yf[u], h, j0);
          }
        }
      } else {
#pragma unroll 1
        for (int item = eg; item < nitems; item += EG) {
          const int h = item / nchunks, j0 = (item - h * nchunks) * CH;
          if (row0 + j0 >= P.R) continue;   // warp-uniform
          const uint32_t tbase = tmem + (uint32_t(q * 32) << 16) + uint32_t((h + buf) * kGemmAcc1Col + j0);
          int da[CH], db[CH], dc[CH];
          tmem_ld8(tbase, da);
          tmem_ld8(tbase + uint32_t(Rt), db);
          tmem_ld8(tbase + uint32_t(2 * Rt), dc);
          tmem_ld_wait();
          if (item == last_item) {   // the rest works from registers: let the next tile's MMAs start
            tc_fence_before();
            if (lane == 0) mbar_arrive(acc_empty);
          }
#pragma unroll
          for (int j = 0; j < CH; ++j) {   // 32 lanes = 32 consecutive ints per atomic instruction
            atomicAdd(sk + size_t(j0 + j) * 128, da[j]);
            atomicAdd(sk + size_t(Rt + j0 + j) * 128, db[j]);
            atomicAdd(sk + size_t(2 * Rt + j0 + j) * 128, dc[j]);
          }
        }
      }
      if (S > 1) {
        __threadfence();                                   // this thread's additions are visible before the ticket
        named_bar_sync(1, kGemmEpiWarps * 32);
        if (et == 0) {
          const unsigned ticket = atomicAdd(P.sk_count + tile, 1u);
          __threadfence();                                 // and the other slices' additions before the reads below
          *last_flag = ticket == unsigned(S - 1) ? 1 : 0;
        }
        named_bar_sync(1, kGemmEpiWarps * 32);
        if (*last_flag) {
#pragma unroll 1
          for (int item = eg; item < nchunks; item += EG) {
            const int j0 = item * CH;
            if (row0 + j0 >= P.R) continue;
            int da[CH], db[CH], dc[CH];
#pragma unroll
            for (int j = 0; j < CH; ++j) {
              da[j] = __ldcg(sk + size_t(j0 + j) * 128);
              db[j] = __ldcg(sk + size_t(Rt + j0 + j) * 128);
              dc[j] = __ldcg(sk + size_t(2 * Rt + j0 + j) * 128);
            }
#pragma unroll
            for (int j = 0; j < CH; ++j) {   // leave the scratch zero for the next launch
              sk[size_t(j0 + j) * 128] = 0; sk[size_t(Rt + j0 + j) * 128] = 0; sk[size_t(2 * Rt + j0 + j) * 128] = 0;
            }
            float yf[CH];
            recombine(da, db, dc, yf);
            finish(yf, 0, j0);
          }
          if (et == 0) P.sk_count[tile] = 0u;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  // After an aborted wait copies may still be in flight into this CTA's shared memory: give each
  // issued copy a bounded chance to land before the CTA retires.
  if (tid == 0 && *abort_flag) {
    const int issued = *issued_ptr;
    const unsigned long long t0 = globaltimer_ns();
    for (int i = issued > kGemmStages ? issued - kGemmStages : 0; i < issued; ++i) {
      const uint32_t bar = full0 + 8 * (i % kGemmStages), parity = uint32_t(i / kGemmStages) & 1u;
      while (!mbar_try_wait(bar, parity) && globaltimer_ns() - t0 < kWaitLimitNs / 10) {
      }
    }
  }
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGemmTmemCols) : "memory");
  }
}

// ======================================================================================================
// Row-wise activation preparation: CTA (s, r) turns activation row r into the digit rows and scalars
// of matrix s.  Same arithmetic per row as vector_prep.cuh; the statistics are block reductions
// (nothing is published between launches on this path).
//   ROWS_PLAIN  v = xin_s[r]
//   ROWS_LN     v = mix_s * LN(ln_x[r]) + (1 - mix_s) * carry, where the carry of a stream's first row
//               is its state row and that of every later row is LN(ln_x[r-1]) (modules/block.py:58-67)
// Row r belongs to stream r / T at position r % T.
enum RowsMode : int { ROWS_PLAIN = 0, ROWS_LN = 1 };

struct RowsPrepParams {
  PrepSeg seg[kMaxSeg];
  int nseg, K, R, T, Rpad;
  int mode, need_sums;
  long long ldx;              // floats between consecutive rows of xin / ln_x
  const float* ln_x;
  const float* ln_w;
  const float* ln_b;
  const float* shift;         // carry of stream b at shift + b * shift_stride, or null (zeros)
  long long shift_stride;
  float* shift_out;           // [R/T][K]: LN of every stream's last row = its next carry (or null)
  signed char* digits;        // [nseg][3][Rpad][K]
  SegScalars* scal;           // [nseg][R]
  // Deferred commit of a token-shift carry that an EARLIER preparation launch parked (it could not
  // write the state row its sibling CTAs were reading): stream b's commit_n floats go from
  // commit_src + b*commit_n to commit_dst + b*commit_stride.  Done by the CTA of matrix 0 and the
  // stream's last row.
  const float* commit_src;
  float* commit_dst;
  long long commit_stride;
  int commit_n;
  // Grouping of the work, filled in by the launcher: a CTA takes one matrix (blockIdx.x) or all of them,
  // and rows_per_cta consecutive rows from blockIdx.y * rows_per_cta.
  int segs_per_cta, rows_per_cta;
};

// Sums of four per-thread values over a CTA of NT threads; every thread gets the totals.
template <int NT>
__device__ __forceinline__ void block_sum4(float (&v)[4], float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
#pragma unroll
  for (int i = 0; i < 4; ++i) v[i] = warp_sum(v[i]);
  __syncthreads();   // red may still be read from an earlier use
  if (lane == 0) reinterpret_cast<float4*>(red)[warp] = make_float4(v[0], v[1], v[2], v[3]);
  __syncthreads();
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int w = 0; w < NT / 32; ++w) {
    const float4 t = reinterpret_cast<const float4*>(red)[w];
    s.x += t.x; s.y += t.y; s.z += t.z; s.w += t.w;
  }
  v[0] = s.x; v[1] = s.y; v[2] = s.z; v[3] = s.w;
}

// max of v[0] and sums of v[1..3] over a CTA of NT threads (statistics of one row: max|xs|, sum v*my,
// sum xs, sum v); every thread gets the totals.
template <int NT>
__device__ __forceinline__ void block_stats(float (&v)[4], float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  v[0] = warp_max(v[0]); v[1] = warp_sum(v[1]); v[2] = warp_sum(v[2]); v[3] = warp_sum(v[3]);
  __syncthreads();
  if (lane == 0) reinterpret_cast<float4*>(red)[warp] = make_float4(v[0], v[1], v[2], v[3]);
  __syncthreads();
  float4 s = reinterpret_cast<const float4*>(red)[0];
  for (int w = 1; w < NT / 32; ++w) {
    const float4 t = reinterpret_cast<const float4*>(red)[w];
    s.x = fmaxf(s.x, t.x); s.y += t.y; s.z += t.z; s.w += t.w;
  }
  v[0] = s.x; v[1] = s.y; v[2] = s.z; v[3] = s.w;
}

// Digit words of four inputs (same digit arithmetic as store_digits in vector_prep.cuh).
__device__ __forceinline__ void rows_store_digits(uint32_t* da, uint32_t* db, uint32_t* dc, int g, float4 xs, float inv) {
  const float v[4] = {xs.x, xs.y, xs.z, xs.w};
  uint32_t y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // round to nearest even of the fp32 product, sign included (|v * inv| <= kQMax < 2^23): one conversion
    // instead of the five instructions of the magnitude-and-sign form, same integer
    const int X = __float2int_rn(__fmul_rn(v[i], inv));
    y[i] = uint32_t(X + 0x8080) ^ 0x8080u;   // bytes: (c, b, a, sign extension)
  }
  const uint32_t c01 = __byte_perm(y[0], y[1], 0x0040), c23 = __byte_perm(y[2], y[3], 0x0040);
  const uint32_t b01 = __byte_perm(y[0], y[1], 0x0051), b23 = __byte_perm(y[2], y[3], 0x0051);
  const uint32_t a01 = __byte_perm(y[0], y[1], 0x0062), a23 = __byte_perm(y[2], y[3], 0x0062);
  da[g] = __byte_perm(a01, a23, 0x5410);
  db[g] = __byte_perm(b01, b23, 0x5410);
  dc[g] = __byte_perm(c01, c23, 0x5410);
}

__device__ __forceinline__ float4 ln_apply(float4 x, float mean, float rstd, float4 w, float4 b) {
  return make_float4(w.x * ((x.x - mean) * rstd) + b.x, w.y * ((x.y - mean) * rstd) + b.y,
                     w.z * ((x.z - mean) * rstd) + b.z, w.w * ((x.w - mean) * rstd) + b.w);
}

// Totals of NV per-thread values over a CTA of NT threads, in every thread: sums, except that v[0] is a
// maximum when MAX0.  Warp butterflies, one float4 slot per warp in shared memory, one barrier: the
// slots alternate between two buffers (phase), so the next reduction cannot overwrite partials that
// a slower warp is still reading.
template <int NT, int NV, bool MAX0>
__device__ __forceinline__ void span_reduce(float (&v)[NV], float* red, int& phase) {
  constexpr int NW = NT / 32;
  static_assert(NV <= 4 && (NW == 8 || NW == 16), "one float4 slot per warp, 8 or 16 warps");
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int k = 0; k < NV; ++k) v[k] = (MAX0 && k == 0) ? warp_max(v[k]) : warp_sum(v[k]);
  float* slots = red + phase * (NW * 4);
  phase ^= 1;
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < NV; ++k) slots[warp * 4 + k] = v[k];
  }
  __syncthreads();
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    float t = slots[(lane & (NW - 1)) * 4 + k];   // every aligned group of NW lanes holds all partials
#pragma unroll
    for (int o = NW / 2; o > 0; o >>= 1) {
      const float u = __shfl_xor_sync(0xffffffffu, t, o);
      t = (MAX0 && k == 0) ? fmaxf(t, u) : t + u;
    }
    v[k] = t;
  }
}

// A CTA prepares rows [blockIdx.y * rows_per_cta, ...) for the matrices of its range (one matrix per
// blockIdx.x, or all of them), each row held in registers (up to G groups of four inputs per thread).
// With thousands of rows a CTA walks several consecutive rows: the layer norm of a row is computed
// once for all matrices, its result stays in registers as the token-shift carry of the next row, and
// the parameter vectors come from L1.  The kernel is bound by instruction issue, so groups beyond the
// row's end are skipped by a CTA-uniform test and the reductions carry only the values in use.
// The arithmetic of a row (which thread holds which input, the order of every reduction) does not
// depend on how rows and matrices are grouped, so a row's digits and scalars are the same bits in
// every grouping.
template <int NT, int G, bool LN>
__device__ __forceinline__ void rows_prep_span(const RowsPrepParams& P, float* red) {
  const int tid = threadIdx.x;
  const int K = P.K, NG = K / 4;
  const int s0 = P.segs_per_cta == 1 ? int(blockIdx.x) : 0, s1 = P.segs_per_cta == 1 ? s0 + 1 : P.nseg;
  const int r0 = int(blockIdx.y) * P.rows_per_cta, r1 = min(r0 + P.rows_per_cta, P.R);
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  const float invk = 1.0f / float(K);
  const bool sums = P.need_sums != 0;
  int phase = 0;
  bool any_mix = false;
  if (LN)
    for (int s = s0; s < s1; ++s) any_mix = any_mix || P.seg[s].mix != nullptr;

  float4 xv[G];               // the row: raw, then its layer norm (LN) or the matrix input (plain)
  float4 pv[LN ? G : 1];      // token-shift partner: LN of the previous row, or the stream's state row
  bool have_prev = false;     // pv holds LN(row r-1) from the previous turn of the loop

  for (int r = r0; r < r1; ++r) {
    const int b = r / P.T, t = r - b * P.T;
    if (P.commit_n > 0 && s0 == 0 && t == P.T - 1) {
      const float4* src = reinterpret_cast<const float4*>(P.commit_src + size_t(b) * P.commit_n);
      float4* dst = reinterpret_cast<float4*>(P.commit_dst + size_t(b) * P.commit_stride);
      for (int g = tid; g < P.commit_n / 4; g += NT) dst[g] = __ldcg(src + g);
    }
    if (LN) {
      const float4* xr = reinterpret_cast<const float4*>(P.ln_x + size_t(r) * P.ldx);
      const bool fetch_prev = any_mix && t > 0 && !have_prev;   // first row of this CTA inside a stream
      const float4* xp = fetch_prev ? reinterpret_cast<const float4*>(P.ln_x + size_t(r - 1) * P.ldx) : nullptr;
#pragma unroll
      for (int i = 0; i < G; ++i)
        if (i * NT < NG) {
          const int g = tid + i * NT;
          xv[i] = g < NG ? __ldcg(xr + g) : zero4;
          if (fetch_prev) pv[i] = g < NG ? __ldcg(xp + g) : zero4;
        }
      // mean of the row (and of the previous one when it has to be rebuilt), then the sums of squared
      // deviations: two passes over registers and two reductions, the centred form of
      // modules/layernorm.py:11-20 (a single pass with E[x^2] - mean^2 cancels in fp32 when |mean| is
      // large against the spread)
      float s[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < G; ++i)
        if (i * NT < NG) {
          s[0] += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w);     // groups past the end hold zeros
          if (fetch_prev) s[1] += (pv[i].x + pv[i].y) + (pv[i].z + pv[i].w);
        }
      if (fetch_prev) span_reduce<NT, 2, false>(s, red, phase);
      else { float s1v[1] = {s[0]}; span_reduce<NT, 1, false>(s1v, red, phase); s[0] = s1v[0]; }
      const float mean = s[0] * invk, meanp = s[1] * invk;
      float q[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < G; ++i)
        if (tid + i * NT < NG) {
          const float a0 = xv[i].x - mean, a1 = xv[i].y - mean, a2 = xv[i].z - mean, a3 = xv[i].w - mean;
          q[0] += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
          if (fetch_prev) {
            const float b0 = pv[i].x - meanp, b1 = pv[i].y - meanp, b2 = pv[i].z - meanp, b3 = pv[i].w - meanp;
            q[1] += (b0 * b0 + b1 * b1) + (b2 * b2 + b3 * b3);
          }
        }
      if (fetch_prev) span_reduce<NT, 2, false>(q, red, phase);
      else { float q1v[1] = {q[0]}; span_reduce<NT, 1, false>(q1v, red, phase); q[0] = q1v[0]; }
      const float rstd = 1.0f / sqrtf(q[0] * invk + 1e-5f), rstdp = 1.0f / sqrtf(q[1] * invk + 1e-5f);
      const bool park_carry = s0 == 0 && P.shift_out && t == P.T - 1;
      const float4* carry = (any_mix && t == 0 && P.shift) ? reinterpret_cast<const float4*>(P.shift + size_t(b) * P.shift_stride) : nullptr;
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int g = tid + i * NT;
        if (g < NG) {
          const float4 w = __ldg(reinterpret_cast<const float4*>(P.ln_w) + g), bb = __ldg(reinterpret_cast<const float4*>(P.ln_b) + g);
          xv[i] = ln_apply(xv[i], mean, rstd, w, bb);
          if (park_carry) reinterpret_cast<float4*>(P.shift_out + size_t(b) * K)[g] = xv[i];
          if (fetch_prev) pv[i] = ln_apply(pv[i], meanp, rstdp, w, bb);
          else if (any_mix && t == 0) pv[i] = carry ? __ldcg(carry + g) : zero4;
        }
      }
    }

    for (int sidx = s0; sidx < s1; ++sidx) {
      const PrepSeg& S = P.seg[sidx];
      const bool mixing = LN && S.mix != nullptr;
      float4 xs_ln[LN ? G : 1];
      float4* xs = LN ? xs_ln : xv;   // scaled values: beside the layer-normed row, or in place of the plain input
      if (!LN) {
        const float4* xr = reinterpret_cast<const float4*>(S.xin + size_t(r) * P.ldx);
#pragma unroll
        for (int i = 0; i < G; ++i) {
          const int g = tid + i * NT;
          if (g < NG) xv[i] = __ldcg(xr + g);
        }
      }
      float st[4] = {0.f, 0.f, 0.f, 0.f};   // max |xs|, sum v*my, sum xs, sum v
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int g = tid + i * NT;
        if (g < NG) {
          float4 v = xv[i];
          if (mixing) {
            const float4 xy = xv[i], tc = pv[LN ? i : 0];
            const float4 mu = __ldg(reinterpret_cast<const float4*>(S.mix) + g);
            v.x = xy.x * mu.x + tc.x * (1.f - mu.x);
            v.y = xy.y * mu.y + tc.y * (1.f - mu.y);
            v.z = xy.z * mu.z + tc.z * (1.f - mu.z);
            v.w = xy.w * mu.w + tc.w * (1.f - mu.w);
          }
          const float4 ry = __ldg(reinterpret_cast<const float4*>(S.ry) + g), my = __ldg(reinterpret_cast<const float4*>(S.my) + g);
          const float4 y = make_float4(v.x * ry.x, v.y * ry.y, v.z * ry.z, v.w * ry.w);
          st[0] = fmaxf(st[0], fmaxf(fmaxf(fabsf(y.x), fabsf(y.y)), fmaxf(fabsf(y.z), fabsf(y.w))));
          st[1] += (v.x * my.x + v.y * my.y) + (v.z * my.z + v.w * my.w);
          if (sums) {
            st[2] += (y.x + y.y) + (y.z + y.w);
            st[3] += (v.x + v.y) + (v.z + v.w);
          }
          xs[i] = y;
        }
      }
      if (sums) span_reduce<NT, 4, true>(st, red, phase);
      else { float st2[2] = {st[0], st[1]}; span_reduce<NT, 2, true>(st2, red, phase); st[0] = st2[0]; st[1] = st2[1]; }
      const float amax = st[0];
      const float inv = amax > 0.f ? kQMax / amax : 0.f;
      if (tid == 0) {
        SegScalars sc;
        sc.sd = amax > 0.f ? __fdiv_rn(1.0f, inv) : 0.f;   // IEEE fp32 division, no fp64 on this path
        sc.zp = st[1]; sc.sumxs = st[2]; sc.sumx = st[3];
        sc.pad[0] = sc.pad[1] = sc.pad[2] = sc.pad[3] = 0.f;
        P.scal[size_t(sidx) * P.R + r] = sc;
      }
      // digit d of row r of matrix s: digits[((s*3 + d) * Rpad + r) * K ...], four inputs per word
      uint32_t* da = reinterpret_cast<uint32_t*>(P.digits + (size_t(sidx * kDigits + 0) * P.Rpad + r) * K);
      uint32_t* db = reinterpret_cast<uint32_t*>(P.digits + (size_t(sidx * kDigits + 1) * P.Rpad + r) * K);
      uint32_t* dc = reinterpret_cast<uint32_t*>(P.digits + (size_t(sidx * kDigits + 2) * P.Rpad + r) * K);
#pragma unroll
      for (int i = 0; i < G; ++i) {
        const int g = tid + i * NT;
        if (g < NG) rows_store_digits(da, db, dc, g, xs[i], inv);
      }
    }
    if (LN && any_mix) {
#pragma unroll
      for (int i = 0; i < G; ++i) pv[LN ? i : 0] = xv[i];
      have_prev = true;
    }
  }
}

// Rows too long for the registers of a CTA: one row and one matrix per CTA, the row is re-read for
// every pass and its scaled values are parked in shared memory between the statistics and the digits.
template <int NT>
__device__ __forceinline__ void rows_prep_long(const RowsPrepParams& P, float* red, float4* park) {
  const int tid = threadIdx.x;
  const int K = P.K, NG = K / 4;
  const int sidx = blockIdx.x, r = blockIdx.y;
  const int b = r / P.T, t = r - b * P.T;
  const PrepSeg& S = P.seg[sidx];
  const bool ln = P.mode == ROWS_LN;
  const bool mixing = ln && S.mix != nullptr;
  const float4* xr = reinterpret_cast<const float4*>((ln ? P.ln_x : S.xin) + size_t(r) * P.ldx);
  const float4* xp = nullptr;     // previous row (t > 0)
  const float4* carry = nullptr;  // state row (t == 0)
  if (mixing) {
    if (t > 0) xp = reinterpret_cast<const float4*>(P.ln_x + size_t(r - 1) * P.ldx);
    else if (P.shift) carry = reinterpret_cast<const float4*>(P.shift + size_t(b) * P.shift_stride);
  }
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  if (P.commit_n > 0 && sidx == 0 && t == P.T - 1) {
    const float4* src = reinterpret_cast<const float4*>(P.commit_src + size_t(b) * P.commit_n);
    float4* dst = reinterpret_cast<float4*>(P.commit_dst + size_t(b) * P.commit_stride);
    for (int g = tid; g < P.commit_n / 4; g += NT) dst[g] = __ldcg(src + g);
  }
  auto p_at = [&](int g) -> float4 { return xp ? __ldcg(xp + g) : (carry ? __ldcg(carry + g) : zero4); };

  float mean = 0.f, rstd = 1.f, meanp = 0.f, rstdp = 1.f;
  if (ln) {
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    for (int g = tid; g < NG; g += NT) {
      const float4 x = __ldcg(xr + g);
      s[0] += (x.x + x.y) + (x.z + x.w);
      if (xp) {
        const float4 y = __ldcg(xp + g);
        s[2] += (y.x + y.y) + (y.z + y.w);
      }
    }
    block_sum4<NT>(s, red);
    const float invk = 1.0f / float(K);
    mean = s[0] * invk; meanp = s[2] * invk;
    float q[4] = {0.f, 0.f, 0.f, 0.f};
    for (int g = tid; g < NG; g += NT) {
      const float4 x = __ldcg(xr + g);
      const float a0 = x.x - mean, a1 = x.y - mean, a2 = x.z - mean, a3 = x.w - mean;
      q[0] += (a0 * a0 + a1 * a1) + (a2 * a2 + a3 * a3);
      if (xp) {
        const float4 y = __ldcg(xp + g);
        const float b0 = y.x - meanp, b1 = y.y - meanp, b2 = y.z - meanp, b3 = y.w - meanp;
        q[2] += (b0 * b0 + b1 * b1) + (b2 * b2 + b3 * b3);
      }
    }
    block_sum4<NT>(q, red);
    rstd = 1.0f / sqrtf(q[0] * invk + 1e-5f);
    rstdp = 1.0f / sqrtf(q[2] * invk + 1e-5f);
  }

  float amax = 0.f, szp = 0.f, sxs = 0.f, sx = 0.f;
  const bool last_of_stream = ln && sidx == 0 && P.shift_out && t == P.T - 1;
  for (int g = tid; g < NG; g += NT) {
    float4 v = __ldcg(xr + g);
    if (ln) {
      const float4 w = __ldg(reinterpret_cast<const float4*>(P.ln_w) + g), bb = __ldg(reinterpret_cast<const float4*>(P.ln_b) + g);
      const float4 xy = ln_apply(v, mean, rstd, w, bb);
      if (last_of_stream) reinterpret_cast<float4*>(P.shift_out + size_t(b) * K)[g] = xy;
      v = xy;
      if (mixing) {
        float4 tc = p_at(g);
        if (xp) tc = ln_apply(tc, meanp, rstdp, w, bb);
        const float4 mu = __ldg(reinterpret_cast<const float4*>(S.mix) + g);
        v.x = xy.x * mu.x + tc.x * (1.f - mu.x);
        v.y = xy.y * mu.y + tc.y * (1.f - mu.y);
        v.z = xy.z * mu.z + tc.z * (1.f - mu.z);
        v.w = xy.w * mu.w + tc.w * (1.f - mu.w);
      }
    }
    const float4 ry = __ldg(reinterpret_cast<const float4*>(S.ry) + g), my = __ldg(reinterpret_cast<const float4*>(S.my) + g);
    const float4 xs = make_float4(v.x * ry.x, v.y * ry.y, v.z * ry.z, v.w * ry.w);
    amax = fmaxf(amax, fmaxf(fmaxf(fabsf(xs.x), fabsf(xs.y)), fmaxf(fabsf(xs.z), fabsf(xs.w))));
    szp += (v.x * my.x + v.y * my.y) + (v.z * my.z + v.w * my.w);
    if (P.need_sums) {
      sxs += (xs.x + xs.y) + (xs.z + xs.w);
      sx += (v.x + v.y) + (v.z + v.w);
    }
    park[g] = xs;
  }
  {
    float st[4] = {amax, szp, sxs, sx};
    block_stats<NT>(st, red);
    amax = st[0]; szp = st[1]; sxs = st[2]; sx = st[3];
  }
  const float inv = amax > 0.f ? kQMax / amax : 0.f;
  if (tid == 0) {
    SegScalars sc;
    sc.sd = amax > 0.f ? __fdiv_rn(1.0f, inv) : 0.f;
    sc.zp = szp; sc.sumxs = sxs; sc.sumx = sx;
    sc.pad[0] = sc.pad[1] = sc.pad[2] = sc.pad[3] = 0.f;
    P.scal[size_t(sidx) * P.R + r] = sc;
  }
  uint32_t* da = reinterpret_cast<uint32_t*>(P.digits + (size_t(sidx * kDigits + 0) * P.Rpad + r) * K);
  uint32_t* db = reinterpret_cast<uint32_t*>(P.digits + (size_t(sidx * kDigits + 1) * P.Rpad + r) * K);
  uint32_t* dc = reinterpret_cast<uint32_t*>(P.digits + (size_t(sidx * kDigits + 2) * P.Rpad + r) * K);
  for (int g = tid; g < NG; g += NT) rows_store_digits(da, db, dc, g, park[g], inv);
}

// Register-resident rows: up to 4 groups of four inputs per thread with the layer norm (row, carry and
// scaled values live at once), 8 without; the kernel is instantiated for the exact number of groups a
// row needs (fewer registers, more resident CTAs).  256 threads while a row fits, else 512.
constexpr int kRowsPrepGroupsLn = 4, kRowsPrepGroupsPlain = 8;
constexpr int rows_prep_min_ctas(int NT, int mode, int G) {
  return mode == ROWS_LN ? (NT == 256 ? (G <= 2 ? 5 : G == 3 ? 4 : 3) : (G <= 3 ? 2 : 1))
                         : (NT == 256 ? (G <= 4 ? 5 : 4) : 2);
}

template <int NT, int MODE, int G>
__global__ void __launch_bounds__(NT, rows_prep_min_ctas(NT, MODE, G)) rows_prep_kernel(const __grid_constant__ RowsPrepParams P) {
  extern __shared__ __align__(128) unsigned char prep_smem[];
  griddep_launch_dependents();
  griddep_wait();
  rows_prep_span<NT, G, MODE == ROWS_LN>(P, reinterpret_cast<float*>(prep_smem));
}

// Rows beyond the registers: one CTA of 512 threads per (matrix, row).
__global__ void __launch_bounds__(512, 2) rows_prep_long_kernel(const __grid_constant__ RowsPrepParams P) {
  extern __shared__ __align__(128) unsigned char prep_smem[];
  griddep_launch_dependents();
  griddep_wait();
  rows_prep_long<512>(P, reinterpret_cast<float*>(prep_smem), reinterpret_cast<float4*>(prep_smem + kPrepRedBytes));
}

inline bool rows_prep_in_regs(int K, int mode, int threads) {
  return K / 4 <= (mode == ROWS_LN ? kRowsPrepGroupsLn : kRowsPrepGroupsPlain) * threads;
}
inline int rows_prep_threads(int K, int mode) { return rows_prep_in_regs(K, mode, 256) ? 256 : 512; }
inline int rows_prep_groups(int K, int threads) { return (K / 4 + threads - 1) / threads; }

// Shared memory: the reduction scratch, plus 4*K bytes of parked xs when the row does not fit the registers.
inline size_t rows_prep_smem(int K, int mode) {
  return size_t(kPrepRedBytes) + (rows_prep_in_regs(K, mode, rows_prep_threads(K, mode)) ? 0 : size_t(4) * K);
}

// How a launch groups its work: while one CTA per (matrix, row) does not fill the GPU twice over, keep
// that (shortest chain per CTA); beyond, one CTA takes all matrices of ceil(R / resident CTAs) consecutive
// rows, so that the whole launch is one wave.
inline void rows_prep_grouping(int nseg, int K, int mode, int R, int sms, int* segs_per_cta, int* rows_per_cta) {
  *segs_per_cta = 1; *rows_per_cta = 1;
  const int threads = rows_prep_threads(K, mode);
  if (!rows_prep_in_regs(K, mode, threads)) return;
  const long long slots = (long long)sms * rows_prep_min_ctas(threads, mode, rows_prep_groups(K, threads));
  if ((long long)nseg * R <= 2 * slots) return;
  *segs_per_cta = nseg;
  *rows_per_cta = int((R + slots - 1) / slots);
}
}  // namespace b200
