// Many activation rows through UNQUANTISED bf16 / fp16 matrices on the 5th-generation tensor cores:
// the reference's TORCH-mode matvec for T > 1 rows (agnostic/backends/torch.py:162-164,
// `x.to(W.dtype).matmul(W).to(x.dtype)`; AgnosticRWKV applies every matrix to all rows of a sequence
// at once, agnosticRwkv.py:123-169).
//
//   out[r][n] = epilogue( round_T( sum_k x_T[r][k] * W[n][k] ) )        fp32 accumulation
//
//   A = mt weight rows     x 128 bytes of K (64 elements; one TMA box of W[N][K], 128-byte swizzle; mt = 128 or 256)
//   B = Rt activation rows x 128 bytes of K (one TMA box of the rows already rounded to T; Rt = 16..240)
//   D = 128 lanes x Rt fp32 columns per 128 weight rows in tensor memory; a 256-row tile keeps its
//       second accumulator at column 256, with 128-row tiles columns 0 and 256 are two buffers.
//
// Same skeleton as tile_gemm.cuh (persistent CTAs, a three-stage operand ring that runs on across
// tiles, warp 0 = TMA producer, warp 1 = MMA issuer with tcgen05.mma kind::f16, warps 4..19 =
// epilogue through tcgen05.ld); no digit planes, no per-row scalars.  With few rows and therefore few
// tiles K is cut into slices (work item = tile x slice): a slice parks its fp32 partial sums in a scratch
// buffer and draws a ticket; the CTA that draws a tile's last ticket adds the slices IN SLICE ORDER (so
// the result does not depend on which CTA finished when) and runs the epilogue.  Nobody waits for anybody.
// Every wait is bounded; on expiry the CTA sets a status bit, drains its copies and still frees its
// tensor memory.
#pragma once

#include "dense_step.cuh"
#include "tile_gemm.cuh"

namespace b200 {

constexpr int kDgRowsMax = 240;                                  // activation rows per tile: 30 KB of a stage
constexpr int kDgStageBytes = kGemmABytes + kDgRowsMax * 128;    // 62 KB
constexpr int kDgRingBytes = kGemmStages * kDgStageBytes;          // 186 KB: three stages of the largest tile, up to eight of a small one
constexpr int kDgMaxStages = 8;                                  // barriers: full 0..7, empty 8..15
constexpr int kDgSmem = kGemmOffRing + kDgRingBytes;
constexpr int kDgSplitMaxItems = 640;                            // tiles x slices of a split launch (its tickets)
constexpr int kDgSplitMaxRows = 1024;                            // calls of up to this many rows may split K
constexpr long long kDgSplitMaxCells = 640ll * 64;               // tiles x slices x tile height that the scratch holds
constexpr size_t kDgSplitBytes = size_t(kDgSplitMaxCells) * 128 * 4;   // 21 MB of partial sums

struct DGemmSeg {
  CUtensorMap wmap;     // W as bytes [K*2/128][N][128 B], box [1][mt][128], 128-byte swizzle
  CUtensorMap xmap;     // rows as bytes [K*2/128][Rpad][128 B], box [1][Rt][128], 128-byte swizzle
  void* out;            // [R][ldo] of float, or of T when out_t is set
  const float* res;     // [R][ldres] added last, or null
  const float* gate;    // [R][ldgate] multiplies the product first, or null
  long long ldo, ldres, ldgate;
  int N, act, out_t;
};

struct DGemmParams {
  DGemmSeg seg[kMaxSeg];
  int nseg, ksteps, R;  // ksteps = K * 2 / 128
  int Rt, mt, row_tiles;
  int tiles_seg[kMaxSeg];
  int ntiles;
  int is_bf16;
  int stages;           // ring depth: as many stages of stage_bytes as fit the ring, at most 8
  int stage_bytes;      // mt * 128 (weights) + Rt * 128 (rows), a multiple of 1024
  int ksplit;           // K slices per tile (1: none; > 1 only with 128-row tiles; divides ksteps)
  float* sk_part;       // [ntiles][ksplit][Rt][128] partial sums of the slices
  unsigned* sk_count;   // [ntiles] tickets, zero between launches
  int* status;
};

// Instruction descriptor of kind::f16: D fp32, A and B of the same 16-bit type, both K-major, M x N.
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N, int is_bf16) {
  return (1u << 4) | (uint32_t(is_bf16 ? 1 : 0) << 7) | (uint32_t(is_bf16 ? 1 : 0) << 10) | (uint32_t(N >> 3) << 17) |
         (uint32_t(M >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float round16(float v, int is_bf16) {
  return is_bf16 ? __bfloat162float(__float2bfloat16_rn(v)) : __half2float(__float2half_rn(v));
}
__device__ __forceinline__ unsigned short bits16(float v, int is_bf16) {
  return is_bf16 ? __bfloat16_as_ushort(__float2bfloat16_rn(v)) : __half_as_ushort(__float2half_rn(v));
}

struct DGemmTile { int seg, n0, row0; };
__device__ __forceinline__ DGemmTile dgemm_tile(const DGemmParams& P, int t) {
  int s = 0;
  while (s < P.nseg - 1 && t >= P.tiles_seg[s]) { t -= P.tiles_seg[s]; ++s; }
  const int wt = t / P.row_tiles;                       // tiles that share a weight tile are consecutive
  return {s, wt * P.mt, (t - wt * P.row_tiles) * P.Rt};
}

__global__ void __launch_bounds__(kGemmThreads, 1) dense_tile_gemm_kernel(const __grid_constant__ DGemmParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int Rt = P.Rt, S = P.ksplit;
  const int nk = P.ksteps / S;            // K steps of one work item
  const int nitems_all = P.ntiles * S;
  const int NS = P.stages;
  const uint32_t a_bytes = uint32_t(P.mt) * 128u, b_bytes = uint32_t(Rt) * 128u;

  uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + 8);
  const uint32_t acc_full0 = smem_u32(bars + 16), acc_empty0 = smem_u32(bars + 18);
  const bool dbuf = P.mt != kGemmM;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 256);
  volatile int* issued_ptr = reinterpret_cast<volatile int*>(smem + 260);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 264);
  unsigned char* ring = smem + kGemmOffRing;

  if (tid == 0) {
    for (int i = 0; i < kDgMaxStages; ++i) { mbar_init(full0 + 8 * i, 1); mbar_init(empty0 + 8 * i, 1); }
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

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      griddep_wait();   // the activation rows come from the kernel in front of this launch
      int issued = 0;
      bool ok = true;
      for (int it = blockIdx.x; it < nitems_all && ok; it += gridDim.x) {
        const DGemmTile T = dgemm_tile(P, it / S);
        const DGemmSeg& Sg = P.seg[T.seg];
        const int kbase = (it % S) * nk;
        for (int kc = 0; kc < nk; ++kc, ++issued) {
          const int slot = issued % NS;
          const uint32_t phase = uint32_t(issued / NS) & 1u;
          if (!mbar_wait_bounded(empty0 + 8 * slot, phase ^ 1u, abort_flag)) {
            if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
            ok = false;
            break;
          }
          const uint32_t bar = full0 + 8 * slot;
          const uint32_t dst = smem_u32(ring + size_t(slot) * P.stage_bytes);
          mbar_arrive_expect_tx(bar, a_bytes + b_bytes);
          tma_load_3d(dst, &Sg.wmap, 0, T.n0, kbase + kc, bar);                    // rows past N are zero-filled
          tma_load_3d(dst + a_bytes, &Sg.xmap, 0, T.row0, kbase + kc, bar);    // rows past the buffer too
        }
      }
      *issued_ptr = issued;
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(128, Rt, P.is_bf16);
      bool ok = true;
      int step = 0, iter = 0;
      for (int it = blockIdx.x; it < nitems_all && ok; it += gridDim.x, ++iter) {
        const DGemmTile T = dgemm_tile(P, it / S);
        const bool two = P.mt == kGemmM && T.n0 + 128 < P.seg[T.seg].N;
        const int buf = dbuf ? (iter & 1) : 0, use = dbuf ? (iter >> 1) : iter;
        const uint32_t tacc = tmem + uint32_t(buf * kGemmAcc1Col);
        if (!mbar_wait_bounded(acc_empty0 + 8 * buf, uint32_t(use & 1) ^ 1u, abort_flag)) {
          if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
          ok = false;
          break;
        }
        tc_fence_after();
        for (int kc = 0; kc < nk; ++kc, ++step) {
          const int slot = step % NS;
          const uint32_t phase = uint32_t(step / NS) & 1u;
          if (!mbar_wait_bounded(full0 + 8 * slot, phase, abort_flag)) {
            if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a = smem_u32(ring + size_t(slot) * P.stage_bytes);
          const uint64_t ad0 = umma_desc(a), ad1 = umma_desc(a + 128 * 128), bd = umma_desc(a + a_bytes);
#pragma unroll
          for (int k = 0; k < 4; ++k) {   // 16 elements = 32 bytes of K per instruction: +2 in the descriptors' 16-byte units
            const uint32_t acc = (kc | k) != 0 ? 1u : 0u;
            umma_f16(tacc, ad0 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
            if (two) umma_f16(tmem + kGemmAcc1Col, ad1 + uint64_t(2 * k), bd + uint64_t(2 * k), idesc, acc);
          }
          umma_commit(empty0 + 8 * slot);
        }
        if (ok) umma_commit(acc_full0 + 8 * buf);
      }
    }
  } else if (warp >= 4) {
    // ---------------------------------------------------------------- epilogue: four warps per TMEM lane quadrant
    const int q = warp & 3, eg = (warp - 4) >> 2;
    constexpr int EG = kGemmEpiWarps / 4, CH = kGemmChunk;
    const int et = tid - 128;
    volatile int* last_flag = reinterpret_cast<volatile int*>(smem + 272);   // K split: this CTA drew a tile's last ticket
    griddep_wait();
    bool ok = true;
    int iter = 0;
    for (int it = blockIdx.x; it < nitems_all && ok; it += gridDim.x, ++iter) {
      const int tile = it / S, slice = it - tile * S;
      const DGemmTile T = dgemm_tile(P, tile);
      const DGemmSeg& Sg = P.seg[T.seg];
      const int n0 = T.n0, row0 = T.row0;
      const bool two = P.mt == kGemmM && n0 + 128 < Sg.N;
      const int buf = dbuf ? (iter & 1) : 0, use = dbuf ? (iter >> 1) : iter;
      const uint32_t acc_empty = acc_empty0 + 8 * buf;
      ok = __all_sync(0xffffffffu, mbar_wait_bounded(acc_full0 + 8 * buf, uint32_t(use & 1), abort_flag));
      if (!ok) {
        if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
        break;
      }
      tc_fence_after();
      const int nchunks = Rt / CH, nitems = (two ? 2 : 1) * nchunks;
      int last_item = -1;     // this warp's last item that really reads TMEM
      for (int item = eg; item < nitems; item += EG)
        if (row0 + (item % nchunks) * CH < P.R) last_item = item;
      if (last_item < 0) {
        tc_fence_before();
        if (lane == 0) mbar_arrive(acc_empty);
      }
      const int rlast = P.R - 1;
      // rounding to the matrices' type, activation, gate, residual and store for 8 rows of one output column
      auto finish = [&](const float (&acc)[CH], int h, int j0) {
        const int n = n0 + h * 128 + q * 32 + lane;
        const bool nvalid = n < Sg.N;
        const int nc = nvalid ? n : Sg.N - 1;
        float yv[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) yv[j] = round16(acc[j], P.is_bf16);
        if (Sg.act == ACT_RELUSQ) {
#pragma unroll
          for (int j = 0; j < CH; ++j) { const float t = fmaxf(yv[j], 0.f); yv[j] = __fmul_rn(t, t); }
        } else if (Sg.act == ACT_SIGMOID) {
#pragma unroll
          for (int j = 0; j < CH; ++j) yv[j] = sigmoidf_(yv[j]);
        }
        if (Sg.gate) {
          float gv[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) { const int r = min(row0 + j0 + j, rlast); gv[j] = __ldcg(Sg.gate + size_t(r) * Sg.ldgate + nc); }
#pragma unroll
          for (int j = 0; j < CH; ++j) yv[j] = __fmul_rn(yv[j], gv[j]);
        }
        if (Sg.res) {
          float rv[CH];
#pragma unroll
          for (int j = 0; j < CH; ++j) { const int r = min(row0 + j0 + j, rlast); rv[j] = __ldcg(Sg.res + size_t(r) * Sg.ldres + nc); }
#pragma unroll
          for (int j = 0; j < CH; ++j) yv[j] = __fadd_rn(rv[j], yv[j]);
        }
#pragma unroll
        for (int j = 0; j < CH; ++j) {
          const int r = row0 + j0 + j;
          if (r <= rlast && nvalid) {
            if (Sg.out_t) static_cast<unsigned short*>(Sg.out)[size_t(r) * Sg.ldo + n] = bits16(yv[j], P.is_bf16);
            else static_cast<float*>(Sg.out)[size_t(r) * Sg.ldo + n] = yv[j];
          }
        }
      };
      // K split: this slice's partial sums go to [tile][slice][row][128 weight rows] (mt = 128 only)
      float* sk = S > 1 ? P.sk_part + (size_t(tile) * S + slice) * Rt * 128 + q * 32 + lane : nullptr;
#pragma unroll 1
      for (int item = eg; item < nitems; item += EG) {
        const int h = item / nchunks, j0 = (item - h * nchunks) * CH;
        if (row0 + j0 >= P.R) continue;   // warp-uniform
        const uint32_t tbase = tmem + (uint32_t(q * 32) << 16) + uint32_t((h + buf) * kGemmAcc1Col + j0);
        int d[CH];
        tmem_ld8(tbase, d);
        tmem_ld_wait();
        if (item == last_item) {
          tc_fence_before();
          if (lane == 0) mbar_arrive(acc_empty);
        }
        float acc[CH];
#pragma unroll
        for (int j = 0; j < CH; ++j) acc[j] = __int_as_float(d[j]);
        if (S == 1) {
          finish(acc, h, j0);
        } else {
#pragma unroll
          for (int j = 0; j < CH; ++j) sk[size_t(j0 + j) * 128] = acc[j];   // 32 lanes = 128 consecutive bytes per store
        }
      }
      if (S > 1) {
        __threadfence();                                   // this thread's partial sums are visible before the ticket
        named_bar_sync(1, kGemmEpiWarps * 32);
        if (et == 0) {
          const unsigned ticket = atomicAdd(P.sk_count + tile, 1u);
          __threadfence();                                 // and the other slices' sums before the reads below
          *last_flag = ticket == unsigned(S - 1) ? 1 : 0;
        }
        named_bar_sync(1, kGemmEpiWarps * 32);
        if (*last_flag) {
          const float* all = P.sk_part + size_t(tile) * S * Rt * 128 + q * 32 + lane;
#pragma unroll 1
          for (int item = eg; item < nchunks; item += EG) {
            const int j0 = item * CH;
            if (row0 + j0 >= P.R) continue;
            float acc[CH];
#pragma unroll
            for (int j = 0; j < CH; ++j) acc[j] = 0.f;
            for (int sl = 0; sl < S; ++sl) {               // slice order: the sum does not depend on who came last
#pragma unroll
              for (int j = 0; j < CH; ++j) acc[j] += __ldcg(all + (size_t(sl) * Rt + j0 + j) * 128);
            }
            finish(acc, 0, j0);
          }
          if (et == 0) P.sk_count[tile] = 0u;              // leave the tickets zero for the next launch
        }
        named_bar_sync(1, kGemmEpiWarps * 32);             // last_flag is rewritten by the next work item
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (tid == 0 && *abort_flag) {      // copies that may still be in flight into this CTA's shared memory
    const int issued = *issued_ptr;
    const unsigned long long t0 = globaltimer_ns();
    for (int i = issued > NS ? issued - NS : 0; i < issued; ++i) {
      const uint32_t bar = full0 + 8 * (i % NS), parity = uint32_t(i / NS) & 1u;
      while (!mbar_try_wait(bar, parity) && globaltimer_ns() - t0 < kWaitLimitNs / 10) {
      }
    }
  }
  if (warp == 2) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kGemmTmemCols) : "memory");
  }
}

// ---- rows in front of the GEMMs ---------------------------------------------------------------------
// A CTA takes rows_per_cta consecutive activation rows (row r: stream r / Tn, position r % Tn): layer
// norm of x[r]; the token-shift carry is the stream's state row for its first row and the layer norm of
// x[r - 1] otherwise (agnosticRwkv.py:125-127: roll + push); out[m][r] = T(lerp(carry, ln, mix[m])).
// Walking consecutive rows, the CTA already holds the layer norm of x[r - 1] from its previous turn (the
// two shared-memory rows swap roles) and only rebuilds it for the first row it takes; a row's arithmetic
// is the same either way.  The layer norm of
// every stream's last row is the stream's next carry: with one row per stream the CTA that read the
// state row writes it back itself; with more rows it is parked in a scratch row that the caller copies
// to the state once this launch is over (sibling CTAs still read the old row).
// With `last_only` the CTA of stream b normalises x[(b+1)*Tn - 1] and writes out[0][b] = T(ln): the
// rows the head is applied to (agnosticRwkv.py:184).
struct DRowsPrepParams {
  const float* x;            // [R][D]
  const float *ln_w, *ln_b;
  const float* carry;        // state row of stream 0; stream b at carry + b * carry_stride
  long long carry_stride;
  float* carry_out;          // stream b's new carry goes to carry_out + b * carry_out_stride
  long long carry_out_stride;
  const float* mix[3];
  void* out[3];              // T [Rpad][D]
  int nmix, D, Tn, last_only, is_bf16, is_f32;
  int R, rows_per_cta;       // rows of the call (streams with last_only); consecutive rows per CTA
};

__global__ void __launch_bounds__(256)
dense_rows_prep_kernel(const DRowsPrepParams P) {
  extern __shared__ __align__(16) float rp_smem[];      // [2][D]
  __shared__ float red[8];
  griddep_launch_dependents();
  griddep_wait();
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, D = P.D, D4 = P.D >> 2;
  auto block_sum = [&](float v) -> float {
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    return t;
  };
  // thread t owns the float4 groups t, t + 256, ... of a row in every pass
  auto layer_norm = [&](const float* src, float* dst) {      // torch.py:102-110
    const float4* s4 = reinterpret_cast<const float4*>(src);
    float4* d4 = reinterpret_cast<float4*>(dst);
    float s = 0.f;
    for (int i = tid; i < D4; i += 256) { const float4 v = __ldcg(s4 + i); d4[i] = v; s += (v.x + v.y) + (v.z + v.w); }
    const float mean = block_sum(s) / float(D);
    float q = 0.f;
    for (int i = tid; i < D4; i += 256) {
      const float4 v = d4[i];
      const float a = v.x - mean, b = v.y - mean, c = v.z - mean, d = v.w - mean;
      q = fmaf(a, a, q); q = fmaf(b, b, q); q = fmaf(c, c, q); q = fmaf(d, d, q);
    }
    const float sd = sqrtf(block_sum(q) / float(D) + 1e-5f);
    for (int i = tid; i < D4; i += 256) {
      const float4 v = d4[i], w = __ldg(reinterpret_cast<const float4*>(P.ln_w) + i), b = __ldg(reinterpret_cast<const float4*>(P.ln_b) + i);
      d4[i] = make_float4(w.x * ((v.x - mean) / sd) + b.x, w.y * ((v.y - mean) / sd) + b.y, w.z * ((v.z - mean) / sd) + b.z,
                          w.w * ((v.w - mean) / sd) + b.w);
    }
  };
  float* cur = rp_smem;
  float* prev = rp_smem + D;
  const bool shift = !P.last_only && P.nmix > 0;
  const int first = blockIdx.x * P.rows_per_cta, end = min(first + P.rows_per_cta, P.R);
  for (int idx = first; idx < end; ++idx) {
    const int r = P.last_only ? (idx + 1) * P.Tn - 1 : idx;
    const int pos = r % P.Tn, stream = r / P.Tn;
    if (idx > first) { float* t = cur; cur = prev; prev = t; }     // prev now holds the layer norm of row r - 1
    layer_norm(P.x + size_t(r) * D, cur);
    if (shift) {
      if (pos == 0) {
        const float4* c4 = reinterpret_cast<const float4*>(P.carry + size_t(stream) * P.carry_stride);
        for (int i = tid; i < D4; i += 256) reinterpret_cast<float4*>(prev)[i] = __ldcg(c4 + i);
      } else if (idx == first) {
        layer_norm(P.x + size_t(r - 1) * D, prev);
      }
      if (pos == P.Tn - 1 && P.carry_out)
        for (int i = tid; i < D4; i += 256) reinterpret_cast<float4*>(P.carry_out + size_t(stream) * P.carry_out_stride)[i] = reinterpret_cast<const float4*>(cur)[i];
    }
    const size_t orow = size_t(idx) * D;
    auto store4 = [&](void* out, int i, float a, float b, float c, float d) {
      if (P.is_f32) {
        reinterpret_cast<float4*>(static_cast<float*>(out) + orow)[i] = make_float4(a, b, c, d);
      } else {
        ushort4 o;
        o.x = bits16(a, P.is_bf16); o.y = bits16(b, P.is_bf16); o.z = bits16(c, P.is_bf16); o.w = bits16(d, P.is_bf16);
        reinterpret_cast<ushort4*>(static_cast<unsigned short*>(out) + orow)[i] = o;
      }
    };
    if (!shift) {
      for (int i = tid; i < D4; i += 256) { const float4 v = reinterpret_cast<const float4*>(cur)[i]; store4(P.out[0], i, v.x, v.y, v.z, v.w); }
    } else {
      for (int i = tid; i < D4; i += 256) {
        const float4 c = reinterpret_cast<const float4*>(cur)[i], p = reinterpret_cast<const float4*>(prev)[i];
#pragma unroll
        for (int m = 0; m < 3; ++m) {
          if (m < P.nmix) {
            const float4 w = __ldg(reinterpret_cast<const float4*>(P.mix[m]) + i);
            store4(P.out[m], i, lerp_like_torch(p.x, c.x, w.x), lerp_like_torch(p.y, c.y, w.y), lerp_like_torch(p.z, c.z, w.z),
                   lerp_like_torch(p.w, c.w, w.w));
          }
        }
      }
    }
  }
}

// fp32 rows -> rows of the matrices' 16-bit type (the cast in front of torch.py:162-164's matmul).
__global__ void __launch_bounds__(256)
dense_rows_cast_kernel(const float* __restrict__ in, unsigned short* __restrict__ out, long long n4, int is_bf16) {
  griddep_launch_dependents();
  griddep_wait();
  for (long long i = blockIdx.x * 256ll + threadIdx.x; i < n4; i += (long long)gridDim.x * 256) {
    const float4 v = __ldcg(reinterpret_cast<const float4*>(in) + i);
    ushort4 o;
    o.x = bits16(v.x, is_bf16); o.y = bits16(v.y, is_bf16); o.z = bits16(v.z, is_bf16); o.w = bits16(v.w, is_bf16);
    reinterpret_cast<ushort4*>(out)[i] = o;
  }
}

}  // namespace b200
