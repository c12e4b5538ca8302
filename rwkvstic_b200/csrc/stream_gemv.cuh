// Streaming uint8 GEMV for sm_100a: the decode-time (one token) matrix-vector kernel.
//
// Data layout in HBM: every matrix is output-major bytes qt[N][K] (K contiguous).  One launch
// covers up to three matrices ("segments") with the same K.
//
// Work split: CTA c owns rows [N*c/G, N*(c+1)/G) of every segment and reads each of its bytes
// exactly once.  A producer lane streams them through a ring of shared-memory stages with TMA
// tensor copies (cp.async.bulk.tensor.3d + mbarrier complete_tx): the matrix is described to TMA
// as [K/128][N][128 bytes], a stage is one box of 16 rows x one K-chunk (<= 2048 bytes per row) and
// lands as [K-chunk/128][16 rows][128 B] with the 128-byte swizzle, so one instruction moves 32 KB
// and ldmatrix reads it bank-conflict free.  16 consumer warps split the K-chunk of every stage.  The grid
// leaves three SMs free: that is where the activation-preparation kernel (vector_prep.cuh, one CTA
// per matrix) of the NEXT launch runs while this one streams.
//
// Arithmetic: the activations arrive as 24-bit fixed point X[k] = rint(xs[k]*inv) in three signed
// base-256 digit planes (X = a*65536 + b*256 + c), prepared once per launch by vector_prep_kernel.
// The dot products with the uint8 weights are integer tensor-core MMAs (m16n8k32, u8 x s8 -> s32):
// a 16-row weight tile against the three digit planes in three of the eight B columns.  The digit
// columns are reduced across warps with 32-bit shared-memory integer atomics and recombined
// exactly in int64, so the result is order-independent and bit-reproducible for any partitioning; y = I/inv carries
// only the input rounding (2^-24 of the largest |xs|).
//
// Fusion: the epilogue applies the affine correction terms and the activation / gate / residual /
// WKV-state update that follows the matrix in the reference's modules/block.py:72-100.
#pragma once

#include <cuda.h>

#include <cstdlib>

#include "vector_prep.cuh"

namespace b200 {

constexpr int kConsumers = 512;                 // consumer threads (16 warps)
constexpr int kConsumerWarps = kConsumers / 32;
constexpr int kGemvThreads = kConsumers + 32;   // + one producer warp
constexpr int kMaxStages = 16;
constexpr int kTileRows = 16;                   // rows per stage = MMA M
constexpr int kChunkMax = 2048;                 // bytes of one row per stage
constexpr int kInFlight = 1;                    // stages in flight while the ring is first filled (pacing; 2: -2 %, 3+: -4 %)
constexpr int kSmemLimit = 227 * 1024;          // dynamic shared memory per CTA on sm_100

enum Act : int { ACT_NONE = 0, ACT_RELUSQ = 1, ACT_SIGMOID = 2 };
enum Epilogue : int { EPI_GENERIC = 0, EPI_WKV = 1 };

struct GemvSeg {
  const uint8_t* qt;   // [N][K]
  const float* rx;     // [N] or null
  const float* mx;     // [N] or null
  float* out;          // EPI_GENERIC: destination [N]
  const float* res;    // EPI_GENERIC: residual added to the output, or null
  const float* gate;   // EPI_GENERIC: multiplies act(y), or null
  // When the next launch's input is an element-wise function of this segment's outputs, the
  // epilogue writes it already scaled, xs_out[n] = out_value * xs_ry[n], and publishes max|xs| and
  // the sums of xs, value and value * xs_my[n] (EPI_WKV uses segment 0's fields for sigmoid(r)*wkv).
  float* xs_out;
  const float* xs_ry;
  const float* xs_my;
  PubSlot* pub_xs;
  float half;
  int N;
  int act;
};

struct GemvParams {
  CUtensorMap tmap[kMaxSeg];  // per segment: u8 [K/128][N][128], box [kc/128][16][128], 128-byte swizzle
  GemvSeg seg[kMaxSeg];
  int nseg, K;
  // geometry (derived from K on the host, see plan_gemv)
  int kc;           // bytes of one row per stage (multiple of 128); the last chunk may be shorter
  int nchunks;      // stages per 16-row tile
  int stages;       // ring depth
  int stage_bytes;  // ring slot size = 16 * kc
  int rpc16;        // max rows per CTA per segment, rounded up to 16
  // prepared activations (output of vector_prep_kernel)
  const unsigned char* planes;  // nseg * 4*K bytes
  const SegScalars* scal;       // nseg entries
  // epilogue
  int epi;
  int accumulate;          // EPI_GENERIC: out += result instead of out = result
  const float* wkv_w;      // EPI_WKV: decay w = -exp(time_decay) [N]
  const float* wkv_u;      // time_first [N]
  float* aa;               // state rows, updated in place [N]
  float* bb;
  float* pp;
  float* wkv_out;          // sigmoid(r) * wkv [N], or null when only seg[0].xs_out is wanted
  PubSlot* pub_ln;         // EPI_GENERIC: publish sum and sum of squares of segment 0's outputs, or null
  int* status;             // device status word or null
  unsigned long long* trace;  // diagnostics: 8 globaltimer stamps per CTA, or null
  // The launch that follows on the stream (same grid): once this CTA's own copies are all issued,
  // its producer asks L2 to fetch the first next_prefetch bytes of the rows the same CTA index will
  // stream next, so HBM stays busy while the next launch waits for its activations.
  const uint8_t* next_qt[kMaxSeg];
  int next_n[kMaxSeg];
  int next_nseg, next_k;
  int next_prefetch;       // bytes per CTA, 0 = none
  // deferred state commit done by CTA 0 once the dependency has resolved: dst[0..n) = src[0..n)
  // (the token-shift carry the preparation kernel computed but could not write in place)
  const float* commit_src;
  float* commit_dst;
  int commit_n;
};

// Shared-memory map (byte offsets)
constexpr int kOffFull = 0;        // 16 x u64
constexpr int kOffEmpty = 128;     // 16 x u64
constexpr int kOffAbort = 256;     // int abort flag, int stages issued
constexpr int kOffPlaneBar = 264;  // u64 mbarrier: digit planes have landed
constexpr int kOffScale = 384;     // SegScalars[3]
constexpr int kOffEpi = 512;       // epilogue reduction scratch: long long [16 warps][6] + float [16]
constexpr int kOffRows = 1536;     // int32 rowsum[nseg*rpc16][4], then digit planes, then ring

struct GemvPlan {
  int kc, nchunks, stages, stage_bytes, rpc16, grid;
  size_t smem;
};

// Choose the stage geometry for a reduction length K.  Returns false when K is unsupported.
inline bool plan_gemv(int K, int nseg, int max_n, int num_sms, GemvPlan* p) {
  if (K <= 0 || (K % 128) != 0 || K > 65536 || nseg < 1 || nseg > kMaxSeg || max_n <= 0) return false;
  p->nchunks = (K + kChunkMax - 1) / kChunkMax;
  p->kc = ((K + p->nchunks - 1) / p->nchunks + 127) / 128 * 128;
  p->stage_bytes = kTileRows * p->kc;
  p->grid = num_sms - kMaxSeg < max_n ? num_sms - kMaxSeg : max_n;  // three SMs stay free for vector_prep_kernel
  if (p->grid < 1) p->grid = 1;
  const int rpc = (max_n + p->grid - 1) / p->grid;
  p->rpc16 = (rpc + 15) / 16 * 16;
  size_t fixed = kOffRows + (size_t(nseg) * p->rpc16 * 16 + 127) / 128 * 128 + size_t(nseg) * 4 * K;
  fixed = (fixed + 1023) / 1024 * 1024;  // swizzled TMA tiles want 1024-byte aligned stages
  if (fixed + 2 * size_t(p->stage_bytes) > size_t(kSmemLimit)) return false;
  int stages = int((size_t(kSmemLimit) - fixed) / p->stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p->stages = stages;
  p->smem = fixed + size_t(stages) * p->stage_bytes;
  return true;
}

// One TMA tensor copy global -> shared of the box at coordinates (c0, c1, c2); completion in bytes on `bar`.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, uint32_t bar) {
  asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst),
               "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar)
               : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& a0, uint32_t& a1, uint32_t& a2, uint32_t& a3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a0), "=r"(a1), "=r"(a2), "=r"(a3)
               : "r"(addr));
}

// D(16x8, s32) += A(16x32, u8, row) * B(32x8, s8, col)
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Phase stamps written when P.trace is set (index: 0 entry, 1 dependency resolved, 4 digit planes
// in shared memory, 5 rows done, 6 epilogue done, 7 producer done; 2 and 3 unused).
#define B200_TRACE(i)                                                              \
  do {                                                                             \
    if (P.trace) P.trace[size_t(blockIdx.x) * 8 + (i)] = globaltimer_ns();         \
  } while (0)

__global__ void __launch_bounds__(kGemvThreads, 1) stream_gemv_kernel(const __grid_constant__ GemvParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int K = P.K;

  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffAbort);
  volatile int* issued_ptr = reinterpret_cast<volatile int*>(smem + kOffAbort + 4);  // stages the producer issued
  volatile int* go_flag = reinterpret_cast<volatile int*>(smem + kOffAbort + 16);    // digit planes have landed: stop pacing
  SegScalars* scal = reinterpret_cast<SegScalars*>(smem + kOffScale);
  int* rowsum = reinterpret_cast<int*>(smem + kOffRows);  // [segment][row][4]: sums of the digit columns
  const size_t rows_bytes = (size_t(P.nseg) * P.rpc16 * 16 + 127) / 128 * 128;
  unsigned char* planes = smem + kOffRows + rows_bytes;  // per segment 4*K bytes
  const uint32_t plane_bytes = uint32_t(P.nseg) * 4u * uint32_t(K);
  const size_t ring_off = (kOffRows + rows_bytes + plane_bytes + 1023) / 1024 * 1024;
  unsigned char* ring = smem + ring_off;
  const uint32_t full0 = smem_u32(smem + kOffFull), empty0 = smem_u32(smem + kOffEmpty);
  const uint32_t plane_bar = smem_u32(smem + kOffPlaneBar);

  int r0[kMaxSeg], nr[kMaxSeg];
#pragma unroll
  for (int s = 0; s < kMaxSeg; ++s) {
    if (s < P.nseg) {
      r0[s] = int((long long)P.seg[s].N * cta / G);
      nr[s] = int((long long)P.seg[s].N * (cta + 1) / G) - r0[s];
    } else {
      r0[s] = 0; nr[s] = 0;
    }
  }

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, kConsumerWarps);
    }
    mbar_init(plane_bar, 1);
    *abort_flag = 0;
    *issued_ptr = 0;
    *go_flag = 0;
    fence_mbar_init();
    B200_TRACE(0);
  }
  __syncthreads();
  griddep_launch_dependents();

  if (warp == kConsumerWarps) {
    // ------------------------------------------------------------------ producer: weights only,
    // which no earlier kernel writes, so it does not wait on the launch dependency.  One lane, one
    // tensor copy per stage; rows past the CTA's range belong to the next CTA (or are zero-filled
    // past the matrix) and are ignored by the consumers.
    bool ok = true;
    if (lane == 0) {
      int slot = 0, issued = 0;
      uint32_t phase = 0;
      for (int s = 0; s < P.nseg && ok; ++s) {
        for (int row = 0; row < nr[s] && ok; row += kTileRows) {
          for (int ch = 0; ch < P.nchunks; ++ch) {
            if (!mbar_wait_bounded(empty0 + 8 * slot, phase ^ 1u, abort_flag)) {
              if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
              ok = false;
              break;
            }
            // Pacing of the first ring fill: at most kInFlight stage requested but not yet landed.
            // All CTAs start their stream at the moment the preparation kernel of this very launch
            // does its one latency-critical round trip; without pacing that load would sit behind
            // ~24 MB of queued weight requests (3+ us).  Once the ring has been filled, requests
            // follow consumption and the full ring depth may be in flight; likewise as soon as the
            // digit planes have landed (go_flag), whatever is left of the first fill goes out at once.
            if (issued >= kInFlight && issued < P.stages && !*go_flag) {
              const int j = issued - kInFlight;
              if (!mbar_wait_bounded(full0 + 8 * (j % P.stages), uint32_t(j / P.stages) & 1u, abort_flag)) {
                if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
                ok = false;
                break;
              }
            }
            mbar_arrive_expect_tx(full0 + 8 * slot, uint32_t(P.stage_bytes));
            tma_load_3d(smem_u32(ring + size_t(slot) * P.stage_bytes), &P.tmap[s], 0, r0[s] + row, ch * (P.kc / 128),
                        full0 + 8 * slot);
            ++issued;
            if (++slot == P.stages) { slot = 0; phase ^= 1u; }
          }
        }
      }
      *issued_ptr = issued;
      B200_TRACE(7);
    }
    ok = __shfl_sync(0xffffffffu, ok, 0);
    if (ok && P.next_prefetch > 0) {
      long long left = P.next_prefetch;
      for (int s = 0; s < P.next_nseg && left > 0; ++s) {
        const long long b0 = (long long)P.next_n[s] * cta / G * P.next_k;
        const long long b1 = (long long)P.next_n[s] * (cta + 1) / G * P.next_k;
        const long long take = b1 - b0 < left ? b1 - b0 : left;   // a multiple of 32 bytes
        for (long long o = (long long)lane * 16384; o < take; o += 32ll * 16384) {
          const uint32_t n = uint32_t(take - o < 16384 ? take - o : 16384);
          asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(P.next_qt[s] + b0 + o), "r"(n) : "memory");
        }
        left -= take;
      }
    }
  } else {
    // ------------------------------------------------------------------ consumers
    for (int i = tid; i < P.nseg * P.rpc16 * 4; i += kConsumers) rowsum[i] = 0;

    griddep_wait();  // the prepared activations (and everything the epilogue reads) are now visible
    if (tid == 0) {
      B200_TRACE(1);
      mbar_arrive_expect_tx(plane_bar, plane_bytes);
      bulk_g2s(smem_u32(planes), P.planes, plane_bytes, plane_bar);
    }
    if (tid < P.nseg * 8) reinterpret_cast<float*>(scal)[tid] = __ldcg(reinterpret_cast<const float*>(P.scal) + tid);
    if (cta == 0 && P.commit_n > 0) {
      for (int i = tid; i < P.commit_n / 4; i += kConsumers)
        reinterpret_cast<float4*>(P.commit_dst)[i] = ld_act_v4(reinterpret_cast<const float4*>(P.commit_src) + i);
    }
    bool dead = !__all_sync(0xffffffffu, mbar_wait_bounded(plane_bar, 0, abort_flag));
    named_bar_sync(1, kConsumers);  // scalars and zeroed row sums visible to every consumer warp
    if (tid == 0) { *go_flag = 1; B200_TRACE(4); }   // the chain's critical loads are over: the producer may run ahead

    // ---- operands of the epilogue for this thread's first row of every segment: requested now,
    // used after the main loop, so their latency hides behind the weight stream
    float e_res[kMaxSeg], e_gate[kMaxSeg], e_ry[kMaxSeg], e_my[kMaxSeg], e_rx[kMaxSeg], e_mx[kMaxSeg];
    float e_aa = 0.f, e_bb = 0.f, e_pp = 0.f, e_w = 0.f, e_u = 0.f;
#pragma unroll
    for (int s = 0; s < kMaxSeg; ++s) {
      e_res[s] = 0.f; e_gate[s] = 1.f; e_ry[s] = 0.f; e_my[s] = 0.f; e_rx[s] = 1.f; e_mx[s] = 0.f;
      if (s < P.nseg && tid < nr[s]) {
        const int n = r0[s] + tid;
        if (P.seg[s].res) e_res[s] = ld_act_f32(P.seg[s].res + n);
        if (P.seg[s].gate) e_gate[s] = ld_act_f32(P.seg[s].gate + n);
        if (P.seg[s].rx) e_rx[s] = ld_param_f32(P.seg[s].rx + n);
        if (P.seg[s].mx) e_mx[s] = ld_param_f32(P.seg[s].mx + n);
        if (P.seg[s].pub_xs) { e_ry[s] = ld_param_f32(P.seg[s].xs_ry + n); e_my[s] = ld_param_f32(P.seg[s].xs_my + n); }
      }
    }
    if (P.epi == EPI_WKV && tid < nr[0]) {
      const int n = r0[0] + tid;
      e_aa = ld_act_f32(P.aa + n); e_bb = ld_act_f32(P.bb + n); e_pp = ld_act_f32(P.pp + n);
      e_w = ld_param_f32(P.wkv_w + n); e_u = ld_param_f32(P.wkv_u + n);
    }

    // ---- main loop: integer tensor-core dot products over the streamed 16-row tiles
    {
      const int gq = lane >> 2, tq = lane & 3;  // MMA group id / thread in group
      // ldmatrix row address inside a swizzled stage: row r of 128-byte chunk c sits at c*2048 + r*128,
      // its 16-byte unit j at ((j ^ (r & 7)) << 4)
      const uint32_t lm_row = uint32_t(((lane & 7) + 8 * ((lane >> 3) & 1)) * 128);
      const uint32_t lm_half = uint32_t(lane >> 4), lm_x = uint32_t(lane & 7);
      const int kbpc = P.kc / 32;  // 32-input blocks per full chunk
      int slot = 0;
      uint32_t phase = 0;
      for (int s = 0; s < P.nseg && !dead; ++s) {
        const int nrows = nr[s];
        const uint32_t* pw = reinterpret_cast<const uint32_t*>(planes + size_t(s) * 4 * K) + gq * 8 + tq;
        for (int tile = 0; tile * kTileRows < nrows && !dead; ++tile) {
          int c[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};  // two accumulator chains
          for (int ch = 0; ch < P.nchunks; ++ch) {
            const int k0 = ch * P.kc;
            const int kbn = (K - k0 < P.kc ? K - k0 : P.kc) / 32;
            const bool ok = mbar_wait_bounded(full0 + 8 * slot, phase, abort_flag);
            if (!__all_sync(0xffffffffu, ok)) {
              dead = true;
              if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
              break;
            }
            const uint32_t sbase = smem_u32(ring + size_t(slot) * P.stage_bytes) + lm_row;
            for (int kb0 = warp; kb0 < kbn; kb0 += 4 * kConsumerWarps) {
              uint32_t a[4][4], b[4][2];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const int kbi = kb0 + j * kConsumerWarps;
                b[j][0] = 0u; b[j][1] = 0u;
                if (kbi < kbn) {
                  ldmatrix_x4(sbase + uint32_t(kbi >> 2) * 2048u + (((2u * uint32_t(kbi & 3) + lm_half) ^ lm_x) << 4),
                              a[j][0], a[j][1], a[j][2], a[j][3]);
                  if (gq < 3) {
                    const uint32_t* bp = pw + size_t(ch * kbpc + kbi) * 32;
                    b[j][0] = bp[0];
                    b[j][1] = bp[4];
                  }
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j)
                if (kb0 + j * kConsumerWarps < kbn) mma_u8s8(c[j & 1], a[j][0], a[j][1], a[j][2], a[j][3], b[j][0], b[j][1]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            if (++slot == P.stages) { slot = 0; phase ^= 1u; }
          }
          if (dead) break;
          // Columns 0,1 (digits a,b) live in lanes with tq == 0, column 2 (digit c) in tq == 1.  Each
          // digit column is summed across the 16 warps with native 32-bit shared-memory atomics
          // (|sum| <= K*255*128 fits int32 for K <= 65536) and recombined in the epilogue.
          const int d0 = c[0][0] + c[1][0], d1 = c[0][1] + c[1][1], d2 = c[0][2] + c[1][2], d3 = c[0][3] + c[1][3];
          if (tq < 2) {
            const int row_lo = tile * kTileRows + gq, row_hi = row_lo + 8;
            int* lo = rowsum + (size_t(s) * P.rpc16 + row_lo) * 4 + 2 * tq;
            int* hi = rowsum + (size_t(s) * P.rpc16 + row_hi) * 4 + 2 * tq;
            if (row_lo < nrows) { atomicAdd(lo, d0); if (tq == 0) atomicAdd(lo + 1, d1); }
            if (row_hi < nrows) { atomicAdd(hi, d2); if (tq == 0) atomicAdd(hi + 1, d3); }
          }
        }
      }
    }
    named_bar_sync(1, kConsumers);
    if (tid == 0) B200_TRACE(5);

    // ---- epilogue: affine terms + the element-wise op that follows this matrix in the block.
    // `first` = this is the thread's first row of the segment, whose operands were preloaded.
    auto value = [&](int s, int row, int n, bool first) -> float {
      const int* rs = rowsum + (size_t(s) * P.rpc16 + row) * 4;
      const long long I = (long long)rs[0] * 65536 + (long long)rs[1] * 256 + (long long)rs[2];
      float y = __fmul_rn(__ll2float_rn(I), scal[s].sd) + P.seg[s].half * scal[s].sumxs;
      if (P.seg[s].rx) y *= first ? e_rx[s] : P.seg[s].rx[n];
      y += scal[s].zp;
      if (P.seg[s].mx) y += (first ? e_mx[s] : P.seg[s].mx[n]) * scal[s].sumx;
      return y;
    };
    // per-thread partials of what this launch publishes for the next one
    long long p_sum = 0, p_sq = 0, p_sqlo = 0, p_zp = 0, p_sxs = 0, p_sx = 0;
    float p_amax = 0.f;
    PubSlot* pub_xs = nullptr;
    auto publish_xs = [&](const GemvSeg& sg, int n, float v, float ry, float my) {
      const float xs = v * ry;
      sg.xs_out[n] = xs;
      p_amax = fmaxf(p_amax, fabsf(xs));
      p_zp += __float2ll_rn(v * my * kPubSumScale);   // scaling by a power of two is exact
      p_sxs += __float2ll_rn(xs * kPubXsScale);
      p_sx += __float2ll_rn(v * kPubSumScale);
    };
    if (P.epi == EPI_WKV) {
      pub_xs = P.seg[0].pub_xs;
      for (int row = tid; row < nr[0]; row += kConsumers) {
        const int n = r0[0] + row;
        const bool first = row == tid;
        const float k = value(0, row, n, first), v = value(1, row, n, first), r = sigmoidf_(value(2, row, n, first));
        float aa = first ? e_aa : P.aa[n], bb = first ? e_bb : P.bb[n], pp = first ? e_pp : P.pp[n];
        const float y = wkv_step(k, v, first ? e_w : P.wkv_w[n], first ? e_u : P.wkv_u[n], aa, bb, pp);
        P.aa[n] = aa; P.bb[n] = bb; P.pp[n] = pp;
        if (P.wkv_out) P.wkv_out[n] = r * y;
        if (pub_xs) publish_xs(P.seg[0], n, r * y, first ? e_ry[0] : P.seg[0].xs_ry[n], first ? e_my[0] : P.seg[0].xs_my[n]);
      }
    } else {
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) {
        if (s < P.nseg) {
          if (P.seg[s].pub_xs) pub_xs = P.seg[s].pub_xs;
          for (int row = tid; row < nr[s]; row += kConsumers) {
            const int n = r0[s] + row;
            const bool first = row == tid;
            float y = value(s, row, n, first);
            if (P.seg[s].act == ACT_RELUSQ) { y = fmaxf(y, 0.f); y *= y; }
            else if (P.seg[s].act == ACT_SIGMOID) y = sigmoidf_(y);
            if (P.seg[s].gate) y *= first ? e_gate[s] : P.seg[s].gate[n];
            if (P.seg[s].res) y += first ? e_res[s] : P.seg[s].res[n];
            if (P.accumulate) y += P.seg[s].out[n];
            if (P.seg[s].out) P.seg[s].out[n] = y;
            if (P.seg[s].pub_xs)
              publish_xs(P.seg[s], n, y, first ? e_ry[s] : P.seg[s].xs_ry[n], first ? e_my[s] : P.seg[s].xs_my[n]);
            if (s == 0 && P.pub_ln) {
              p_sum += __float2ll_rn(y * kPubSumScale);
              square_limbs(y, p_sq, p_sqlo);
            }
          }
        }
      }
    }
    if (pub_xs || P.pub_ln) {
      // exact block totals (integers; the max is order-independent too), one atomic per quantity and CTA
      long long* esum = reinterpret_cast<long long*>(smem + kOffEpi);
      float* emax = reinterpret_cast<float*>(smem + kOffEpi + kConsumerWarps * 6 * 8);
      long long v6[6] = {p_sum, p_sq, p_sqlo, p_zp, p_sxs, p_sx};
#pragma unroll
      for (int i = 0; i < 6; ++i)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v6[i] += __shfl_xor_sync(0xffffffffu, v6[i], o);
      p_amax = warp_max(p_amax);
      if (lane == 0) {
#pragma unroll
        for (int i = 0; i < 6; ++i) esum[warp * 6 + i] = v6[i];
        emax[warp] = p_amax;
      }
      named_bar_sync(1, kConsumers);
      if (tid < 6) {
        long long a = 0;
        for (int w = 0; w < kConsumerWarps; ++w) a += esum[w * 6 + tid];
        if (tid < 3) {
          if (P.pub_ln) atomicAdd(reinterpret_cast<unsigned long long*>(tid == 0 ? &P.pub_ln->sum : (tid == 1 ? &P.pub_ln->sq : &P.pub_ln->sq_lo)),
                                  (unsigned long long)a);
        } else if (pub_xs) {
          long long* dst = tid == 3 ? &pub_xs->zp : (tid == 4 ? &pub_xs->sumxs : &pub_xs->sumx);
          atomicAdd(reinterpret_cast<unsigned long long*>(dst), (unsigned long long)a);
        }
      } else if (tid == 6 && pub_xs) {
        float m = 0.f;
        for (int w = 0; w < kConsumerWarps; ++w) m = fmaxf(m, emax[w]);
        atomicMax(&pub_xs->amax_bits, __float_as_uint(m));   // non-negative floats order like their bits
      }
    }
  }

  __syncthreads();
  if (tid == 0) B200_TRACE(6);
  // After an aborted wait some bulk copies may still be in flight into this CTA's shared memory:
  // give every copy that was issued a bounded chance to land before the CTA retires.
  if (tid == 0 && *abort_flag) {
    const int issued = *issued_ptr;
    const unsigned long long t0 = globaltimer_ns();
    while (!mbar_try_wait(plane_bar, 0) && globaltimer_ns() - t0 < kWaitLimitNs / 10) {
    }
    for (int i = issued > P.stages ? issued - P.stages : 0; i < issued; ++i) {
      const uint32_t bar = full0 + 8 * (i % P.stages), parity = uint32_t(i / P.stages) & 1u;
      while (!mbar_try_wait(bar, parity) && globaltimer_ns() - t0 < kWaitLimitNs / 10) {
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------------------
cudaError_t launch_stream_gemv(GemvParams& P, int max_n, bool pdl, cudaStream_t stream, const char** why);
cudaError_t launch_vector_prep(const PrepParams& P, bool pdl, cudaStream_t stream, const char** why);

}  // namespace b200
