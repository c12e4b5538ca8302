// One decode step (one token, one stream) of the whole network as ONE persistent kernel.
//
// Why: a decode step is a chain of 4*L+1 matrix-vector products, each of which needs the complete
// output of the one before.  Launching them one by one leaves HBM idle at every link of the chain:
// a CTA's shared-memory ring - the only place weight bytes can wait - is torn down and rebuilt at
// each kernel boundary.  Here every SM runs one CTA for the whole step.  Its producer lane streams
// the CTA's rows of ALL matrices, one after the other, through one ring that never drains (weights
// are constants, so the stream does not depend on any activation) and asks L2 for the bytes that
// follow the ring; the 16 consumer warps meet the other CTAs only where the mathematics needs
// every output of a matrix: at a grid barrier (one release-increment and one acquire-poll of a
// counter in L2 per CTA).
//
// What crosses CTAs, and how.  CTA c owns rows [N*c/G, N*(c+1)/G) of every matrix.  For the D-wide
// vectors (residual stream, receptance gates, WKV state, token-shift carries) that is the same
// slice in every block, so they never leave their CTA: the residual lives in shared memory for the
// whole step.  Only three things are exchanged through global memory (L2):
//   * the input of the next matrix, already multiplied by its per-input scale (xs = v * ry), one
//     slice per CTA, with max|xs| (integer atomicMax on the float bits) and the fixed-point sums the
//     affine terms need (int64 atomics): exact and order-free, so a step is bit-reproducible;
//   * for a layer norm, the sum and sum of squares of the residual (int64 fixed point; the squares
//     in two limbs so that neither large nor tiny activations lose bits), finished in fp64 with the
//     centred form var = E[x^2] - mean^2 evaluated where it cannot cancel;
//   * the barrier counter.
// After the barrier every CTA reads the whole xs vector (4 bytes per input, L2 hits), turns it into
// the three signed base-256 digit planes in its own shared memory and runs the same integer
// tensor-core main loop as stream_gemv_kernel.  A layer norm needs two hops (statistics, then the
// normalised and mixed slices), an element-wise hand-off (attention output, ffn value) one.
//
// Every wait (mbarrier, grid barrier) is bounded by wait_limit_ns; on expiry the CTA raises a
// status bit and an abort word that the other CTAs see at their next poll, drains its own copies
// in flight and returns.
#pragma once

#include "stream_gemv.cuh"

namespace b200 {

#ifndef B200_STEP_CONSUMER_WARPS
#define B200_STEP_CONSUMER_WARPS 8
#endif
constexpr int kStepConsumerWarps = B200_STEP_CONSUMER_WARPS;   // a multiple of 4; 8 + the producer = 9 warps
constexpr int kStepConsumers = kStepConsumerWarps * 32;
constexpr int kStepThreads = kStepConsumers + 32;   // + one producer warp
constexpr int kStepLineBase = 5;                // publication lines 0 barrier, 1 abort, 2..4 first block's k/v/r
constexpr int kStepLinesPerLayer = 9;
constexpr int kStepTraceSlots = 8;              // u64 stamps per (phase, CTA)
constexpr int kStepPrefetchPiece = 16384;       // bytes per L2 prefetch request
constexpr int kStepPrefetchDefault = 256 * 1024; // bytes per CTA requested from L2 beyond the ring

// Shared-memory map of the step kernel (byte offsets; the rest is laid out by the host, see StepParams)
constexpr int kSOffDecision = 272;   // int: uniform abort decision of the last grid barrier
constexpr int kSOffRed = 512;        // reduction scratch: long long [16 warps][12], then float [16][4], then 16 floats
constexpr int kSOffRedF = kSOffRed + 16 * 12 * 8;
constexpr int kSOffBc = kSOffRedF + 16 * 4 * 4;
constexpr int kSOffDyn = 2560;       // first byte the host lays out

// Fixed-point units of the published quantities
constexpr float kSqHiScale = 256.0f;                 // 2^8: high limb of a square
constexpr float kSqLoScale = 1099511627776.0f;       // 2^40 on top of the 2^8: low limb in 2^-48 units

// One matrix as the step kernel sees it: a 256-byte entry of a table in global memory.
struct __align__(128) StepMat {
  CUtensorMap tmap;     // u8 [K/128][N][128], box [kc/128][16][128], 128-byte swizzle
  const uint8_t* qt;
  const float* ry;
  const float* my;
  const float* rx;      // or null
  const float* mx;      // or null
  float half;
  int N, K, kc, nchunks, need_sums;
  int pad[16];
};
static_assert(sizeof(StepMat) == 256, "StepMat is 256 bytes");

// The vector parameters of one block (all f32 [D]).
struct __align__(128) StepVec {
  const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
  const float *mix_k, *mix_v, *mix_r, *fmix_k, *fmix_r;
  const float *decay, *first;
  const float* pad[5];
};
static_assert(sizeof(StepVec) == 128, "StepVec is 128 bytes");

#ifdef B200_STEP_TMAP_CONST
__constant__ CUtensorMap c_step_tmaps[449];
#endif

struct StepParams {
  const StepMat* mats;    // [7*L + 1]: per block key, value, receptance, output, ffn key, ffn receptance, ffn value; then the head
  const StepVec* vecs;    // [L]
  int L, D, F, V;
  const float* emb;
  const float *ln0_w, *ln0_b, *lnout_w, *lnout_b;
  const long long* token;
  float* state;           // [L][5][D]
  float* logits;          // [V] or null (no head)
  float* xs_att;          // [D]   exchange buffers
  float* xs_ffn;          // [F]
  float* xs_ln;           // [3][D]
  unsigned char* pub;     // publication lines of 128 bytes, zero at kernel entry
  int* status;
  unsigned long long* trace;   // optional: [4L+1 phases][G][kStepTraceSlots]
  // shared-memory geometry (host: plan_step)
  int slot_bytes, stages, off_own, own_rows, off_park, park_stride, off_rows, off_planes, off_ring;
  // tuning
  int window;             // weight stages a CTA may have in flight (>= stages: no limit)
  int window_handoff;     // the same while the consumers are between two matrices
  int pf_bytes;           // bytes per CTA requested from L2 ahead of the ring
  unsigned long long wait_limit_ns;
  double inv_d;           // 1 / D
};

// ---- scoped memory operations ----------------------------------------------------------------------
__device__ __forceinline__ void red_release_add_u32(unsigned* p, unsigned v) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ long long ld_act_s64(const long long* p) {
  long long v;
  asm volatile("ld.global.cg.s64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned ld_act_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__device__ __forceinline__ bool mbar_wait_limited(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                  unsigned long long limit_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (globaltimer_ns() - t0 > limit_ns) {
      *abort_flag = 1;
      return false;
    }
  }
}

// Digits of four inputs -> one word per plane in the compact shared-memory layout: 96 bytes per
// 32 inputs, [a:32][b:32][c:32] (the global layout of vector_prep.cuh without its zero block).
__device__ __forceinline__ void store_digits_compact(unsigned char* planes, int g, float4 xs, float inv) {
  const float v[4] = {xs.x, xs.y, xs.z, xs.w};
  uint32_t y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int mag = rint_nonneg(__fmul_rn(fabsf(v[i]), inv));
    const int X = v[i] < 0.f ? -mag : mag;
    y[i] = uint32_t(X + 0x8080) ^ 0x8080u;
  }
  const uint32_t c01 = __byte_perm(y[0], y[1], 0x0040), c23 = __byte_perm(y[2], y[3], 0x0040);
  const uint32_t b01 = __byte_perm(y[0], y[1], 0x0051), b23 = __byte_perm(y[2], y[3], 0x0051);
  const uint32_t a01 = __byte_perm(y[0], y[1], 0x0062), a23 = __byte_perm(y[2], y[3], 0x0062);
  uint32_t* blk = reinterpret_cast<uint32_t*>(planes + size_t(g >> 3) * 96);
  const int j = g & 7;
  blk[j] = __byte_perm(a01, a23, 0x5410);
  blk[8 + j] = __byte_perm(b01, b23, 0x5410);
  blk[16 + j] = __byte_perm(c01, c23, 0x5410);
}

// y^2 as two integers: hi = rint(y^2 * 2^8), lo = (y^2 * 2^8 - hi) * 2^40.  Both products are exact
// (power-of-two scaling; the remainder of a float against its own rounding to an integer is a float),
// so the pair carries y^2 exactly for 2^-60 <= y^2 < 2^55 and sums of either limb are order-free.
__device__ __forceinline__ void square_limbs(float y, long long& hi, long long& lo) {
  const float s = __fmul_rn(__fmul_rn(y, y), kSqHiScale);
  const float sh = rintf(s);
  hi += __float2ll_rn(sh);
  lo += __float2ll_rn(__fmul_rn(__fsub_rn(s, sh), kSqLoScale));
}


// Sums of NV int64 quantities and maxima of NM floats over the consumer threads.  Afterwards
// thread i < NV holds total i in v[0] and thread 32 + j holds maximum j in m[0].  One named barrier
// inside; the scratch is free again after the caller's next named barrier.
template <int NV, int NM>
__device__ __forceinline__ void cta_reduce(long long (&v)[NV], float (&m)[NM > 0 ? NM : 1], long long* red_ll, float* red_f) {
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int i = 0; i < NV; ++i)
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v[i] += __shfl_xor_sync(0xffffffffu, v[i], o);
#pragma unroll
  for (int i = 0; i < NM; ++i) m[i] = warp_max(m[i]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) red_ll[warp * 12 + i] = v[i];
#pragma unroll
    for (int i = 0; i < NM; ++i) red_f[warp * 4 + i] = m[i];
  }
  named_bar_sync(1, kStepConsumers);
  if (tid < NV) {
    long long a = 0;
    for (int w = 0; w < kStepConsumerWarps; ++w) a += red_ll[w * 12 + tid];
    v[0] = a;
  } else if (tid >= 32 && tid < 32 + NM) {
    float a = 0.f;
    for (int w = 0; w < kStepConsumerWarps; ++w) a = fmaxf(a, red_f[w * 4 + tid - 32]);
    m[0] = a;
  }
}

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

// A warp's share of one landed stage: NJ blocks of 32 inputs x 16 rows, block j at a_addr + j * (W/4)
// * 2048 (weights, swizzled stage) and b_addr + j * W * 96 (digit planes).  Four accumulator chains.
template <int NJ>
__device__ __forceinline__ void consume_blocks(int (&c)[4][4], uint32_t a_addr, uint32_t b_addr, bool bvalid) {
  constexpr uint32_t kAStep = uint32_t(kStepConsumerWarps / 4) * 2048u, kBStep = uint32_t(kStepConsumerWarps) * 96u;
  uint32_t a[NJ][4], b[NJ][2];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    ldmatrix_x4(a_addr + uint32_t(j) * kAStep, a[j][0], a[j][1], a[j][2], a[j][3]);
    b[j][0] = 0u; b[j][1] = 0u;
    if (bvalid) {
      b[j][0] = lds_u32(b_addr + uint32_t(j) * kBStep);
      b[j][1] = lds_u32(b_addr + uint32_t(j) * kBStep + 16u);
    }
  }
#pragma unroll
  for (int j = 0; j < NJ; ++j) mma_u8s8(c[j & 3], a[j][0], a[j][1], a[j][2], a[j][3], b[j][0], b[j][1]);
}

// kbn blocks of 32 inputs in the stage (a multiple of 4); the unrolled forms cover every count that
// divides evenly among the warps, the loop the rest.
__device__ __forceinline__ void consume_stage(int (&c)[4][4], uint32_t a_addr, uint32_t b_addr, bool bvalid, int kbn, int warp) {
  static_assert(kStepConsumerWarps % 4 == 0, "a warp's blocks must share their position in the swizzle atom");
  constexpr int W = kStepConsumerWarps;
  if (kbn == 8 * W) consume_blocks<8>(c, a_addr, b_addr, bvalid);
  else if (kbn == 4 * W) consume_blocks<4>(c, a_addr, b_addr, bvalid);
  else if (kbn == 5 * W) consume_blocks<5>(c, a_addr, b_addr, bvalid);
  else if (kbn == 7 * W) consume_blocks<7>(c, a_addr, b_addr, bvalid);
  else if (kbn == 6 * W) consume_blocks<6>(c, a_addr, b_addr, bvalid);
  else if (kbn == 3 * W) consume_blocks<3>(c, a_addr, b_addr, bvalid);
  else if (kbn == 2 * W) consume_blocks<2>(c, a_addr, b_addr, bvalid);
  else {
    constexpr uint32_t kAStep = uint32_t(W / 4) * 2048u, kBStep = uint32_t(W) * 96u;
    for (int j0 = 0; warp + j0 * W < kbn; j0 += 4) {
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int j = j0 + jj;
        if (warp + j * W < kbn) {
          uint32_t a0, a1, a2, a3, b0 = 0u, b1 = 0u;
          ldmatrix_x4(a_addr + uint32_t(j) * kAStep, a0, a1, a2, a3);
          if (bvalid) { b0 = lds_u32(b_addr + uint32_t(j) * kBStep); b1 = lds_u32(b_addr + uint32_t(j) * kBStep + 16u); }
          mma_u8s8(c[jj], a0, a1, a2, a3, b0, b1);
        }
      }
    }
  }
}

// Digit planes of a launch's nseg segments from the exchanged xs vectors (segment s at
// xs + s * xs_stride, K inputs each) and their publication lines line0 + s; also the segments'
// scalars.  Called by all consumer threads.  The loads of all segments go out together: one L2
// round trip.
__device__ __forceinline__ void build_digit_planes(unsigned char* planes, SegScalars* scal, const unsigned char* pub,
                                                   const float* xs, size_t xs_stride, int line0, int nseg, int K, int tid) {
  constexpr int GB = (4096 + kStepConsumers - 1) / kStepConsumers;   // 16384 inputs in one batch
  const int NG = K / 4, TG = nseg * NG;
  float4 v[GB];
#pragma unroll
  for (int i = 0; i < GB; ++i) {
    const int f = tid + i * kStepConsumers;
    if (f < TG) {
      const int s = f >= 2 * NG ? 2 : (f >= NG ? 1 : 0), g = f - s * NG;
      v[i] = ld_act_v4(reinterpret_cast<const float4*>(xs + size_t(s) * xs_stride) + g);
    }
  }
  float inv[kMaxSeg];
#pragma unroll
  for (int s = 0; s < kMaxSeg; ++s) {
    inv[s] = 0.f;
    if (s < nseg) inv[s] = __uint_as_float(ld_act_u32(reinterpret_cast<const unsigned*>(pub + size_t(line0 + s) * 128)));   // max |xs|
  }
  if (tid < nseg) {
    const unsigned char* line = pub + size_t(line0 + tid) * 128;
    const long long zp = ld_act_s64(reinterpret_cast<const long long*>(line + 32));
    const long long sxs = ld_act_s64(reinterpret_cast<const long long*>(line + 64));
    const long long sx = ld_act_s64(reinterpret_cast<const long long*>(line + 96));
    const float amax = __uint_as_float(ld_act_u32(reinterpret_cast<const unsigned*>(line)));
    SegScalars sc;
    sc.sd = amax > 0.f ? __fdiv_rn(1.0f, kQMax / amax) : 0.f;
    sc.zp = __ll2float_rn(zp) * (1.0f / kPubSumScale);
    sc.sumxs = __ll2float_rn(sxs) * (1.0f / kPubXsScale);
    sc.sumx = __ll2float_rn(sx) * (1.0f / kPubSumScale);
    sc.pad[0] = sc.pad[1] = sc.pad[2] = sc.pad[3] = 0.f;
    scal[tid] = sc;
  }
#pragma unroll
  for (int s = 0; s < kMaxSeg; ++s) inv[s] = inv[s] > 0.f ? kQMax / inv[s] : 0.f;
#pragma unroll
  for (int i = 0; i < GB; ++i) {
    const int f = tid + i * kStepConsumers;
    if (f < TG) {
      const int s = f >= 2 * NG ? 2 : (f >= NG ? 1 : 0), g = f - s * NG;
      store_digits_compact(planes + size_t(s) * 3 * K, g, v[i], s == 0 ? inv[0] : (s == 1 ? inv[1] : inv[2]));
    }
  }
  for (int f = tid + GB * kStepConsumers; f < TG; f += kStepConsumers) {
    const int s = f >= 2 * NG ? 2 : (f >= NG ? 1 : 0), g = f - s * NG;
    store_digits_compact(planes + size_t(s) * 3 * K, g, ld_act_v4(reinterpret_cast<const float4*>(xs + size_t(s) * xs_stride) + g),
                         s == 0 ? inv[0] : (s == 1 ? inv[1] : inv[2]));
  }
}

#define STEP_TRACE(ph, i)                                                                               \
  do {                                                                                                  \
    if (P.trace && tid == 0)                                                                            \
      P.trace[(size_t(ph) * gridDim.x + blockIdx.x) * kStepTraceSlots + (i)] = globaltimer_ns();        \
  } while (0)

__global__ void __launch_bounds__(kStepThreads, 1) decode_step_kernel(const __grid_constant__ StepParams P) {
  extern __shared__ __align__(1024) unsigned char smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int D = P.D, L = P.L;

  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffAbort);
  volatile int* issued_ptr = reinterpret_cast<volatile int*>(smem + kOffAbort + 4);
  volatile int* handoff = reinterpret_cast<volatile int*>(smem + kOffAbort + 8);
  volatile int* decision = reinterpret_cast<volatile int*>(smem + kSOffDecision);
  SegScalars* scal = reinterpret_cast<SegScalars*>(smem + kOffScale);
  long long* red_ll = reinterpret_cast<long long*>(smem + kSOffRed);
  float* red_f = reinterpret_cast<float*>(smem + kSOffRedF);
  float* bc = reinterpret_cast<float*>(smem + kSOffBc);
  float* x_own = reinterpret_cast<float*>(smem + P.off_own);   // this CTA's slice of the residual stream
  float* rf_own = x_own + P.own_rows;                          // ... of sigmoid(ffn receptance)
  int* rowsum = reinterpret_cast<int*>(smem + P.off_rows);
  unsigned char* planes = smem + P.off_planes;
  unsigned char* ring = smem + P.off_ring;
  const uint32_t full0 = smem_u32(smem + kOffFull), empty0 = smem_u32(smem + kOffEmpty);
  unsigned* bar_counter = reinterpret_cast<unsigned*>(P.pub);
  unsigned* abort_word = reinterpret_cast<unsigned*>(P.pub + 128);
  const unsigned long long limit = P.wait_limit_ns;

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, kStepConsumerWarps);
    }
    *abort_flag = 0;
    *issued_ptr = 0;
    *handoff = 1;
    *decision = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const int nmat = 7 * L + (P.logits ? 1 : 0);

  if (warp == kStepConsumerWarps) {
    // ================================================================== producer: weights only.
    // The stream is the CTA's rows of matrix 0, 1, 2, ... in the order the consumers use them; it
    // depends on no activation, so it runs ahead of them by the ring and, in L2, by pf_bytes more.
    if (lane == 0) {
      struct Cur { int m, row, N, K, r0, nr; const uint8_t* qt; };
      auto load_mat = [&](Cur& c) __attribute__((always_inline)) {
        if (c.m < nmat) {
          const StepMat* M = P.mats + c.m;
          c.N = __ldg(&M->N); c.K = __ldg(&M->K);
          c.qt = reinterpret_cast<const uint8_t*>(__ldg(reinterpret_cast<const unsigned long long*>(&M->qt)));
          c.r0 = int((long long)c.N * cta / G);
          c.nr = int((long long)c.N * (cta + 1) / G) - c.r0;
        }
        c.row = 0;
      };
      auto skip_empty = [&](Cur& c) __attribute__((always_inline)) {
        while (c.m < nmat && c.row >= c.nr) { ++c.m; load_mat(c); }
      };
      auto tile_bytes = [&](const Cur& c) __attribute__((always_inline)) -> long long {
        const int rows = c.nr - c.row < kTileRows ? c.nr - c.row : kTileRows;
        return (long long)rows * c.K;
      };
      Cur ic, pc;
      ic.m = 0; load_mat(ic); skip_empty(ic);
      pc = ic;
      if (pc.m < nmat) { pc.row += kTileRows; skip_empty(pc); }   // the prefetch cursor stays ahead of the issue cursor
      long long ic_ord = 0, pc_ord = 1, pf_ahead = 0;
      int slot = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      while (ic.m < nmat && ok) {
        const StepMat* M = P.mats + ic.m;
        const int kc = __ldg(&M->kc), nchunks = __ldg(&M->nchunks);
        const uint32_t stage_bytes = uint32_t(kTileRows) * uint32_t(kc);
        for (int ch = 0; ch < nchunks; ++ch) {
          if (!mbar_wait_limited(empty0 + 8 * slot, phase ^ 1u, abort_flag, limit)) {
            if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
            ok = false;
            break;
          }
          // in-flight window: stage (issued - w) must have landed before another one is requested
          const int w = *handoff ? P.window_handoff : P.window;
          if (w < P.stages && issued >= w) {
            const int j = issued - w;
            if (!mbar_wait_limited(full0 + 8 * (j % P.stages), uint32_t(j / P.stages) & 1u, abort_flag, limit)) {
              if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
              ok = false;
              break;
            }
          }
          mbar_arrive_expect_tx(full0 + 8 * slot, stage_bytes);
#ifdef B200_STEP_TMAP_CONST
          tma_load_3d(smem_u32(ring + size_t(slot) * P.slot_bytes), &c_step_tmaps[ic.m], 0, ic.r0 + ic.row, ch * (kc / 128),
#else
          tma_load_3d(smem_u32(ring + size_t(slot) * P.slot_bytes), &M->tmap, 0, ic.r0 + ic.row, ch * (kc / 128),
#endif
                      full0 + 8 * slot);
          ++issued;
          if (++slot == P.stages) { slot = 0; phase ^= 1u; }
        }
        if (!ok) break;
        *issued_ptr = issued;
        // next tile; the prefetch cursor is topped up to pf_bytes beyond it
        ic.row += kTileRows; skip_empty(ic); ++ic_ord;
        if (pc_ord <= ic_ord) {            // the ring caught up with the prefetch cursor
          pc = ic; pc_ord = ic_ord; pf_ahead = 0;
          if (pc.m < nmat) { pc.row += kTileRows; skip_empty(pc); ++pc_ord; }
        } else if (ic.m < nmat) {
          pf_ahead -= tile_bytes(ic);
        }
        while (pc.m < nmat && pf_ahead < P.pf_bytes) {
          const long long nb = tile_bytes(pc);
          const uint8_t* src = pc.qt + (long long)(pc.r0 + pc.row) * pc.K;   // a multiple of 128 bytes from a 16-byte aligned base
          for (long long o = 0; o < nb; o += kStepPrefetchPiece) {
            const uint32_t n = uint32_t(nb - o < kStepPrefetchPiece ? nb - o : kStepPrefetchPiece);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src + o), "r"(n) : "memory");
          }
          pf_ahead += nb;
          pc.row += kTileRows; skip_empty(pc); ++pc_ord;
        }
      }
      *issued_ptr = issued;
    }
  } else {
    // ================================================================== consumers
    const int gq = lane >> 2, tq = lane & 3;
    const uint32_t lm_row = uint32_t(((lane & 7) + 8 * ((lane >> 3) & 1)) * 128);
    const uint32_t lm_half = uint32_t(lane >> 4), lm_x = uint32_t(lane & 7);
    int slot = 0;
    uint32_t ring_phase = 0;
    unsigned bar_target = 0;
    const int r0D = int((long long)D * cta / G), nrD = int((long long)D * (cta + 1) / G) - r0D;

    // ---- grid barrier over the consumer warps of all CTAs, in two halves so that work which does not
    // depend on the other CTAs (table look-ups, operand requests) runs between them.  bar_wait returns
    // true (for every thread alike) when the step is to be abandoned.
    auto bar_arrive = [&]() __attribute__((always_inline)) {
      named_bar_sync(1, kStepConsumers);            // every thread's stores and atomics are issued
      bar_target += unsigned(G);
      if (tid == 0) red_release_add_u32(bar_counter, 1u);
    };
    auto bar_wait = [&]() __attribute__((always_inline)) -> bool {
      if (tid == 0) {
        bool ok = true;
        if (ld_acquire_u32(bar_counter) < bar_target) {
          const unsigned long long t0 = globaltimer_ns();
          unsigned it = 0;
          for (;;) {
            if (ld_acquire_u32(bar_counter) >= bar_target) break;
            if ((++it & 15u) == 0u) {
              if (*abort_flag || ld_relaxed_u32(abort_word) != 0u) { ok = false; break; }
              if (globaltimer_ns() - t0 > limit) {
                if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_PEER);
                atomicExch(abort_word, 1u);
                ok = false;
                break;
              }
            }
          }
        }
        if (!ok) *abort_flag = 1;
        *decision = *abort_flag;
      }
      named_bar_sync(1, kStepConsumers);
      return *decision != 0;
    };

    // ---- headers of the matrices of the current launch
    int sr0[kMaxSeg], snr[kMaxSeg];
    int pK = 0, pkc = 0, pnchunks = 0, prpc16 = 16, pnseg = 0, pm0 = 0;
    int paffine = 0;   // bit s: segment s has per-output terms (rx / mx / half), read from the table when needed
    auto load_phase = [&](int m0, int nseg) __attribute__((always_inline)) {
      pnseg = nseg; pm0 = m0; paffine = 0;
      int rpc = 0;
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) {
        sr0[s] = 0; snr[s] = 0;
        if (s < nseg) {
          const StepMat* M = P.mats + m0 + s;
          const int N = __ldg(&M->N);
          sr0[s] = int((long long)N * cta / G);
          snr[s] = int((long long)N * (cta + 1) / G) - sr0[s];
          if (__ldg(&M->need_sums)) paffine |= 1 << s;
          const int r = (N + G - 1) / G;
          rpc = r > rpc ? r : rpc;
        }
      }
      const StepMat* M0 = P.mats + m0;
      pK = __ldg(&M0->K); pkc = __ldg(&M0->kc); pnchunks = __ldg(&M0->nchunks);
      prpc16 = (rpc + 15) / 16 * 16;
      for (int i = tid; i < nseg * prpc16 * 4; i += kStepConsumers) rowsum[i] = 0;
    };

    // ---- main loop: the rows of the current launch's matrices against the digit planes.  Warp w takes
    // the 32-input blocks w, w + W, w + 2W, ... of every stage (W = consumer warps, a multiple of 4, so
    // that a warp's blocks share their position inside the 128-byte swizzle atom and every address of
    // the unrolled loop is a per-thread constant plus an immediate).
    const uint32_t ring_s32 = smem_u32(ring), planes_s32 = smem_u32(planes);
    const uint32_t a_lane = lm_row + uint32_t(warp >> 2) * 2048u + (((2u * uint32_t(warp & 3) + lm_half) ^ lm_x) << 4);
    const uint32_t b_lane = uint32_t(warp) * 96u + uint32_t(gq * 8 + tq) * 4u;
    auto stream_rows = [&]() __attribute__((always_inline)) {
      const int K = pK, kc = pkc, nchunks = pnchunks;
      const int kbpc = kc / 32;
      bool dead = false;
      for (int s = 0; s < pnseg && !dead; ++s) {
        const int nrows = s == 0 ? snr[0] : (s == 1 ? snr[1] : snr[2]);
        const uint32_t b_seg = planes_s32 + uint32_t(s) * 3u * uint32_t(K) + b_lane;
        for (int tile = 0; tile * kTileRows < nrows && !dead; ++tile) {
          int c[4][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}};
          for (int ch = 0; ch < nchunks; ++ch) {
            const int k0 = ch * kc;
            const int kbn = (K - k0 < kc ? K - k0 : kc) / 32;
            const bool ok = mbar_wait_limited(full0 + 8 * slot, ring_phase, abort_flag, limit);
            if (!__all_sync(0xffffffffu, ok)) {
              dead = true;
              if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
              break;
            }
            const uint32_t a_addr = ring_s32 + uint32_t(slot) * uint32_t(P.slot_bytes) + a_lane;
            const uint32_t b_addr = b_seg + uint32_t(ch * kbpc) * 96u;
#ifndef B200_STEP_NO_MATH
            consume_stage(c, a_addr, b_addr, gq < 3, kbn, warp);
#endif
            __syncwarp();
            if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            if (++slot == P.stages) { slot = 0; ring_phase ^= 1u; }
          }
          if (dead) break;
          const int d0 = (c[0][0] + c[1][0]) + (c[2][0] + c[3][0]), d1 = (c[0][1] + c[1][1]) + (c[2][1] + c[3][1]);
          const int d2 = (c[0][2] + c[1][2]) + (c[2][2] + c[3][2]), d3 = (c[0][3] + c[1][3]) + (c[2][3] + c[3][3]);
          if (tq < 2) {
            const int row_lo = tile * kTileRows + gq, row_hi = row_lo + 8;
            int* lo = rowsum + (size_t(s) * prpc16 + row_lo) * 4 + 2 * tq;
            int* hi = rowsum + (size_t(s) * prpc16 + row_hi) * 4 + 2 * tq;
            if (row_lo < nrows) { atomicAdd(lo, d0); if (tq == 0) atomicAdd(lo + 1, d1); }
            if (row_hi < nrows) { atomicAdd(hi, d2); if (tq == 0) atomicAdd(hi + 1, d3); }
          }
        }
      }
    };

    // ---- value of output `row` of segment s (affine terms of the quantisation contract); s is a
    // compile-time constant at every call site
    auto value = [&](int s, int row) __attribute__((always_inline)) -> float {
      const int* rs = rowsum + (size_t(s) * prpc16 + row) * 4;
      const long long I = (long long)rs[0] * 65536 + (long long)rs[1] * 256 + (long long)rs[2];
      float y = __fmul_rn(__ll2float_rn(I), scal[s].sd);
      if (paffine & (1 << s)) {
        const StepMat* M = P.mats + pm0 + s;
        const float* rx = reinterpret_cast<const float*>(__ldg(reinterpret_cast<const unsigned long long*>(&M->rx)));
        const float* mx = reinterpret_cast<const float*>(__ldg(reinterpret_cast<const unsigned long long*>(&M->mx)));
        const int n = sr0[s] + row;
        y += __ldg(&M->half) * scal[s].sumxs;
        if (rx) y *= __ldg(rx + n);
        y += scal[s].zp;
        if (mx) y += __ldg(mx + n) * scal[s].sumx;
      } else {
        y += scal[s].zp;
      }
      return y;
    };

    auto pub_add = [&](unsigned char* line, int off, long long v) __attribute__((always_inline)) {
      atomicAdd(reinterpret_cast<unsigned long long*>(line + off), (unsigned long long)v);
    };
    auto pub_max = [&](unsigned char* line, float m) __attribute__((always_inline)) {
      atomicMax(reinterpret_cast<unsigned*>(line), __float_as_uint(m));   // non-negative floats order like their bits
    };
    auto line_of = [&](int i) -> unsigned char* { return P.pub + size_t(i) * 128; };

    // ---- one element-wise producer of a next-matrix input: xs = v * ry, partial max and sums
    struct XsAcc { long long zp, sxs, sx; float amax; };
    auto xs_emit = [&](XsAcc& a, float* dst, int n, float v, float ry, float my) __attribute__((always_inline)) {
      const float xs = v * ry;
      dst[n] = xs;
      a.amax = fmaxf(a.amax, fabsf(xs));
      a.zp += __float2ll_rn(v * my * kPubSumScale);
      a.sxs += __float2ll_rn(xs * kPubXsScale);
      a.sx += __float2ll_rn(v * kPubSumScale);
    };

    // ---- operands a thread needs after a matrix has streamed (constants, or state only this thread
    // touches) are requested before the grid barrier in front of that matrix and parked in a
    // thread-private shared-memory slot, so their latency is off the chain and they hold no register
    // while the weights stream.  Slot j of thread t: park[j * park_stride + t], 13 slots.
    float* park = reinterpret_cast<float*>(smem + P.off_park);
    const int pstride = P.park_stride;
    auto ptr_of = [&](const float* const* field) __attribute__((always_inline)) -> const float* {
      return reinterpret_cast<const float*>(__ldg(reinterpret_cast<const unsigned long long*>(field)));
    };
    // operands of a layer-norm hop for this thread's element of the residual: w, b, carry, then per
    // following matrix mu, ry, my
    auto hop_issue = [&](float (&pre)[13], const float* ln_w, const float* ln_b, const float* mix0, const float* mix1, const float* mix2,
                         const float* carry_row, int mfirst, int nseg) __attribute__((always_inline)) {
      if (tid < nrD) {
        const int n = r0D + tid;
        pre[0] = ld_param_f32(ln_w + n);
        pre[1] = ld_param_f32(ln_b + n);
        if (carry_row) pre[2] = ld_act_f32(carry_row + n);
#pragma unroll
        for (int s = 0; s < kMaxSeg; ++s) {
          if (s < nseg) {
            const StepMat* M = P.mats + mfirst + s;
            const float* mix = s == 0 ? mix0 : (s == 1 ? mix1 : mix2);
            if (mix) pre[3 + 3 * s] = ld_param_f32(mix + n);
            pre[4 + 3 * s] = ld_param_f32(ptr_of(&M->ry) + n);
            pre[5 + 3 * s] = ld_param_f32(ptr_of(&M->my) + n);
          }
        }
      }
    };
    auto park_all = [&](const float (&pre)[13], int rows) __attribute__((always_inline)) {
      if (tid < rows) {
#pragma unroll
        for (int j = 0; j < 13; ++j) park[j * pstride + tid] = pre[j];
      }
    };
    // layer norm + token-shift mix of this CTA's slice of the residual for the nseg matrices that
    // follow (modules/layernorm.py:11-20, modules/block.py:58-67, :82-91): writes their xs slices,
    // the new carry, and publishes max / sums per matrix on lines line0..
    auto ln_hop = [&](float mean, float rstd, float* carry_row, int nseg, int line0) __attribute__((always_inline)) {
      XsAcc acc[kMaxSeg];
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) { acc[s].zp = 0; acc[s].sxs = 0; acc[s].sx = 0; acc[s].amax = 0.f; }
      if (tid < nrD) {
        const int n = r0D + tid;
        const float x = x_own[tid];
        const float xy = park[tid] * ((x - mean) * rstd) + park[pstride + tid];
        const float carry = park[2 * pstride + tid];
        if (carry_row) carry_row[n] = xy;     // the state row: this thread is its only reader and writer
#pragma unroll
        for (int s = 0; s < kMaxSeg; ++s) {
          if (s < nseg) {
            const float mu = park[(3 + 3 * s) * pstride + tid];
            const float v = carry_row ? xy * mu + carry * (1.f - mu) : xy;
            xs_emit(acc[s], P.xs_ln + size_t(s) * D, n, v, park[(4 + 3 * s) * pstride + tid], park[(5 + 3 * s) * pstride + tid]);
          }
        }
      }
      long long v[9];
      float m[3];
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) { v[3 * s] = acc[s].zp; v[3 * s + 1] = acc[s].sxs; v[3 * s + 2] = acc[s].sx; m[s] = acc[s].amax; }
      cta_reduce<9, 3>(v, m, red_ll, red_f);
      if (tid < 3 * nseg) pub_add(line_of(line0 + tid / 3), 32 + 32 * (tid % 3), v[0]);
      else if (tid >= 32 && tid < 32 + nseg) pub_max(line_of(line0 + tid - 32), m[0]);
    };
    // statistics of the residual from sum and squares (two limbs) in fixed point, fp64 finish:
    // var = E[x^2] - mean^2 on exact sums does not cancel (modules/layernorm.py:11-20 centres first)
    auto stats_finish = [&](long long sum, long long sqhi, long long sqlo, float& mean, float& rstd) __attribute__((always_inline)) {
      // multiplications and one subtraction in fp64 (no fp64 division or square root: those are subroutines)
      const double mu = double(sum) * (P.inv_d * (1.0 / 4294967296.0));
      const double q = double(sqhi) * (1.0 / 256.0) + double(sqlo) * (1.0 / 281474976710656.0);
      const double var = q * P.inv_d - mu * mu;
      mean = float(mu);
      rstd = 1.0f / sqrtf(fmaxf(float(var), 0.f) + 1e-5f);
    };
    // publish the statistics of the residual slice this CTA just wrote into x_own
    auto publish_stats = [&](int line) __attribute__((always_inline)) {
      long long v[3] = {0, 0, 0};
      float m[1] = {0.f};
      if (tid < nrD) {
        const float y = x_own[tid];
        v[0] = __float2ll_rn(y * kPubSumScale);
        square_limbs(y, v[1], v[2]);
      }
      cta_reduce<3, 0>(v, m, red_ll, red_f);
      if (tid < 3) pub_add(line_of(line), 32 * tid, v[0]);
    };

    // ================================================================== the step
    float mean = 0.f, rstd = 1.f;
    {   // operands of the first block's ln1 hop
      const StepVec* V0 = P.vecs;
      float pre[13] = {0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 1.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f};
      hop_issue(pre, ptr_of(&V0->ln1_w), ptr_of(&V0->ln1_b), ptr_of(&V0->mix_k), ptr_of(&V0->mix_v), ptr_of(&V0->mix_r), P.state, 0, 3);
      park_all(pre, nrD);
    }
    // ---- embedding row + ln0 (emb.py:8-9, opt.py:63-64).  Every CTA evaluates the whole vector: it
    // needs the statistics of ln0's output for the first block's layer norm and keeps its own slice.
    {
      long long tok = *P.token;
      tok = tok < 0 ? 0 : (tok >= P.V ? P.V - 1 : tok);
      const float* row = P.emb + size_t(tok) * D;
      auto block_sum = [&](float v) __attribute__((always_inline)) -> float {
        v = warp_sum(v);
        if (lane == 0) red_f[warp] = v;
        named_bar_sync(1, kStepConsumers);
        if (tid == 0) {
          float a = 0.f;
          for (int i = 0; i < kStepConsumerWarps; ++i) a += red_f[i];
          bc[0] = a;
        }
        named_bar_sync(1, kStepConsumers);
        const float r = bc[0];
        named_bar_sync(1, kStepConsumers);
        return r;
      };
      float s = 0.f;
      for (int i = tid; i < D; i += kStepConsumers) s += row[i];
      const float mean0 = block_sum(s) / float(D);
      s = 0.f;
      for (int i = tid; i < D; i += kStepConsumers) { const float c = row[i] - mean0; s += c * c; }
      const float sdev = sqrtf(block_sum(s) / float(D) + 1e-5f);
      long long v[3] = {0, 0, 0};
      float m[1] = {0.f};
      for (int i = tid; i < D; i += kStepConsumers) {
        const float y = P.ln0_w[i] * ((row[i] - mean0) / sdev) + P.ln0_b[i];
        if (i >= r0D && i < r0D + nrD) x_own[i - r0D] = y;
        v[0] += __float2ll_rn(y * kPubSumScale);
        square_limbs(y, v[1], v[2]);
      }
      cta_reduce<3, 0>(v, m, red_ll, red_f);
      if (tid < 3) red_ll[16 * 12 - 3 + tid] = v[0];   // last three slots of the scratch: totals for everyone
      named_bar_sync(1, kStepConsumers);
      if (warp * 32 < nrD) stats_finish(red_ll[16 * 12 - 3], red_ll[16 * 12 - 2], red_ll[16 * 12 - 1], mean, rstd);
      named_bar_sync(1, kStepConsumers);
    }

    // ---- the launches: per block 0 key/value/receptance + WKV, 1 attention output, 2 ffn key +
    // receptance, 3 ffn value; then 4 = the head.  One copy of every stage of a launch; what differs
    // between the launch types is selected by `type`.
    const int nph = 4 * L + (P.logits ? 1 : 0);
    for (int ph = 0; ph < nph; ++ph) {
      const int type = ph < 4 * L ? (ph & 3) : 4;
      const int l = ph < 4 * L ? (ph >> 2) : L - 1;
      const int lines = kStepLineBase + kStepLinesPerLayer * l;
      const int kvr_line = l == 0 ? 2 : lines - kStepLinesPerLayer + 6;
      const bool more = l + 1 < L;
      float* st = P.state + size_t(l) * 5 * D;
      const int mfirst = 7 * l + (type == 0 ? 0 : type == 1 ? 3 : type == 2 ? 4 : type == 3 ? 6 : 7);
      const int nseg = type == 0 ? 3 : (type == 2 ? 2 : 1);
      const int line0 = type == 0 ? kvr_line : type == 1 ? lines : type == 2 ? lines + 2 : type == 3 ? lines + 4 : lines + 6;

      // ---- A. a layer norm in front of the matrices: normalise and mix this CTA's slice
      if (type == 0 || type == 2 || type == 4) {
        ln_hop(mean, rstd, type == 0 ? st : (type == 2 ? st + size_t(D) : nullptr), nseg, line0);
        STEP_TRACE(ph, 5);
      }
      bar_arrive();
      load_phase(mfirst, nseg);
#ifdef B200_STEP_STREAM_ONLY
      named_bar_sync(1, kStepConsumers);
      STEP_TRACE(ph, 1);
      stream_rows();
      named_bar_sync(1, kStepConsumers);
      STEP_TRACE(ph, 2);
      continue;
#endif

      // ---- B. operands for after the stream, grid barrier, digit planes
      {
        float pre[13] = {0.f, 0.f, 0.f, 1.f, 0.f, 0.f, 1.f, 0.f, 0.f, 1.f, 0.f, 0.f, 0.f};
        int prows = 0;
        const StepVec* Vv = P.vecs + l;
        if (type == 0) {          // WKV state and parameters; ry, my of the output projection
          prows = nrD;
          if (tid < nrD) {
            const int n = r0D + tid;
            const StepMat* Mo = P.mats + mfirst + 3;
            pre[0] = ld_act_f32(st + 2 * size_t(D) + n); pre[1] = ld_act_f32(st + 3 * size_t(D) + n); pre[2] = ld_act_f32(st + 4 * size_t(D) + n);
            pre[3] = ld_param_f32(ptr_of(&Vv->decay) + n);
            pre[4] = ld_param_f32(ptr_of(&Vv->first) + n);
            pre[5] = ld_param_f32(ptr_of(&Mo->ry) + n);
            pre[6] = ld_param_f32(ptr_of(&Mo->my) + n);
          }
        } else if (type == 1) {   // the ln2 hop that follows this matrix
          prows = nrD;
          hop_issue(pre, ptr_of(&Vv->ln2_w), ptr_of(&Vv->ln2_b), ptr_of(&Vv->fmix_k), ptr_of(&Vv->fmix_r), nullptr, st + size_t(D), mfirst + 1, 2);
        } else if (type == 2) {   // ry, my of the value projection at this thread's first ffn-key row
          prows = snr[0];
          if (tid < snr[0]) {
            const StepMat* Mv = P.mats + mfirst + 2;
            pre[0] = ld_param_f32(ptr_of(&Mv->ry) + sr0[0] + tid);
            pre[1] = ld_param_f32(ptr_of(&Mv->my) + sr0[0] + tid);
          }
        } else if (type == 3) {   // the next block's ln1 hop, or ln_out
          if (more) {
            prows = nrD;
            const StepVec* Vn = Vv + 1;
            hop_issue(pre, ptr_of(&Vn->ln1_w), ptr_of(&Vn->ln1_b), ptr_of(&Vn->mix_k), ptr_of(&Vn->mix_v), ptr_of(&Vn->mix_r),
                      st + size_t(5) * D, mfirst + 1, 3);
          } else if (P.logits) {
            prows = nrD;
            hop_issue(pre, P.lnout_w, P.lnout_b, nullptr, nullptr, nullptr, nullptr, mfirst + 1, 1);
          }
        }
        if (bar_wait()) break;
        STEP_TRACE(ph, 0);
        park_all(pre, prows);
      }
      build_digit_planes(planes, scal, P.pub, type == 1 ? P.xs_att : (type == 3 ? P.xs_ffn : P.xs_ln), type == 0 || type == 2 ? size_t(D) : 0,
                         line0, nseg, pK, tid);
      named_bar_sync(1, kStepConsumers);      // planes, scalars, zeroed row sums, parked operands
      if (tid == 0) *handoff = 0;
      STEP_TRACE(ph, 1);
      stream_rows();
      named_bar_sync(1, kStepConsumers);
      if (tid == 0) *handoff = 1;
      STEP_TRACE(ph, 2);

      // ---- C. what follows the matrices in the block (modules/block.py:72-100)
      if (type == 0) {            // WKV update, sigmoid(r) * wkv -> input of the output projection
        XsAcc acc; acc.zp = 0; acc.sxs = 0; acc.sx = 0; acc.amax = 0.f;
        if (tid < nrD) {
          const int n = r0D + tid;
          const float k = value(0, tid), v = value(1, tid), r = sigmoidf_(value(2, tid));
          float aa = park[tid], bb = park[pstride + tid], pp = park[2 * pstride + tid];
          const float y = wkv_step(k, v, park[3 * pstride + tid], park[4 * pstride + tid], aa, bb, pp);
          st[2 * size_t(D) + n] = aa; st[3 * size_t(D) + n] = bb; st[4 * size_t(D) + n] = pp;
          xs_emit(acc, P.xs_att, n, r * y, park[5 * pstride + tid], park[6 * pstride + tid]);
        }
        long long v3[3] = {acc.zp, acc.sxs, acc.sx};
        float m1[1] = {acc.amax};
        cta_reduce<3, 1>(v3, m1, red_ll, red_f);
        if (tid < 3) pub_add(line_of(lines + 0), 32 + 32 * tid, v3[0]);
        else if (tid == 32) pub_max(line_of(lines + 0), m1[0]);
      } else if (type == 2) {     // relu(key)^2 -> input of the value projection; sigmoid(receptance) stays here
        XsAcc acc; acc.zp = 0; acc.sxs = 0; acc.sx = 0; acc.amax = 0.f;
        const StepMat* Mv = P.mats + mfirst + 2;
        const float* vry = ptr_of(&Mv->ry);
        const float* vmy = ptr_of(&Mv->my);
        for (int row = tid; row < snr[0]; row += kStepConsumers) {
          const int n = sr0[0] + row;
          float y = fmaxf(value(0, row), 0.f);
          y *= y;
          const bool parked = row < kStepConsumers;    // row == tid then: this thread parked them
          xs_emit(acc, P.xs_ffn, n, y, parked ? park[row] : __ldg(vry + n), parked ? park[pstride + row] : __ldg(vmy + n));
        }
        if (tid < nrD) rf_own[tid] = sigmoidf_(value(1, tid));
        long long v3[3] = {acc.zp, acc.sxs, acc.sx};
        float m1[1] = {acc.amax};
        cta_reduce<3, 1>(v3, m1, red_ll, red_f);
        if (tid < 3) pub_add(line_of(lines + 4), 32 + 32 * tid, v3[0]);
        else if (tid == 32) pub_max(line_of(lines + 4), m1[0]);
      } else if (type == 4) {     // logits
        for (int row = tid; row < snr[0]; row += kStepConsumers) P.logits[sr0[0] + row] = value(0, row);
      } else {                    // residual update; a layer norm follows unless the step ends here
        if (tid < nrD) x_own[tid] = type == 1 ? value(0, tid) + x_own[tid] : value(0, tid) * rf_own[tid] + x_own[tid];
        if (type == 1 || more || P.logits) {
          const int sline = type == 1 ? lines + 1 : lines + 5;
          publish_stats(sline);
          STEP_TRACE(ph, 3);
          bar_arrive();
          if (bar_wait()) break;
          STEP_TRACE(ph + 1, 4);
          if (warp * 32 < nrD) {
            const unsigned char* line = line_of(sline);
            const long long a = ld_act_s64(reinterpret_cast<const long long*>(line));
            const long long b = ld_act_s64(reinterpret_cast<const long long*>(line + 32));
            const long long c = ld_act_s64(reinterpret_cast<const long long*>(line + 64));
            stats_finish(a, b, c, mean, rstd);
          }
          continue;
        }
      }
      STEP_TRACE(ph, 3);
    }
  }

  __syncthreads();
  // After an abandoned step some weight copies may still be in flight into this CTA's shared memory:
  // give every copy that was issued a bounded chance to land before the CTA retires.
  if (tid == 0 && *abort_flag) {
    const int issued = *issued_ptr;
    const unsigned long long t0 = globaltimer_ns();
    for (int i = issued > P.stages ? issued - P.stages : 0; i < issued; ++i) {
      const uint32_t bar = full0 + 8 * (i % P.stages), parity = uint32_t(i / P.stages) & 1u;
      while (!mbar_try_wait(bar, parity) && globaltimer_ns() - t0 < limit / 10 + 1000000ull) {
      }
    }
  }
}

// ---- host side: shared-memory layout -------------------------------------------------------------
struct StepPlan {
  int grid, slot_bytes, stages, off_own, own_rows, off_park, park_stride, off_rows, off_planes, off_ring;
  size_t smem;
};

inline void step_mat_geometry(int K, int* kc, int* nchunks) {
  *nchunks = (K + kChunkMax - 1) / kChunkMax;
  *kc = ((K + *nchunks - 1) / *nchunks + 127) / 128 * 128;
}

// Geometry for a model with n_embd D, n_ffn F, n_vocab V on a GPU with num_sms SMs.  False when the
// shape is unsupported (D, F multiples of 128 up to 65536; at least two ring stages must fit).
inline bool plan_step(int D, int F, int V, bool head, int num_sms, StepPlan* p) {
  if (D <= 0 || F <= 0 || (D % 128) != 0 || (F % 128) != 0 || D > 65536 || F > 65536 || num_sms < 1) return false;
  if (head && V <= 0) return false;
  p->grid = num_sms < D ? num_sms : D;
  const int G = p->grid;
  auto rpc16 = [&](int N) { return ((N + G - 1) / G + 15) / 16 * 16; };
  const int rD = rpc16(D), rF = rpc16(F), rV = head ? rpc16(V) : 16;
  if ((D + G - 1) / G > kStepConsumers) return false;      // the layer-norm hop handles one row per consumer thread
  int kcD, kcF, n;
  step_mat_geometry(D, &kcD, &n);
  step_mat_geometry(F, &kcF, &n);
  p->slot_bytes = kTileRows * (kcD > kcF ? kcD : kcF);
  // row sums: [segment][rows per CTA, rounded to 16][4] ints of the launch with the most rows
  size_t rows_bytes = size_t(3) * rD * 16;                                   // key, value, receptance
  if (size_t(2) * rF * 16 > rows_bytes) rows_bytes = size_t(2) * rF * 16;    // ffn key + receptance share the larger count
  if (size_t(rV) * 16 > rows_bytes) rows_bytes = size_t(rV) * 16;
  const size_t plane_bytes = size_t(3) * (3 * D > F ? 3 * D : F);            // 3 bytes per input and matrix
  p->own_rows = rD;
  p->off_own = kSOffDyn;
  p->off_park = (p->off_own + 2 * rD * 4 + 127) / 128 * 128;
  p->park_stride = rD > rF ? rD : rF;                                        // 13 thread-private slots per row a CTA can own
  p->off_rows = (p->off_park + 13 * p->park_stride * 4 + 127) / 128 * 128;
  p->off_planes = int((p->off_rows + rows_bytes + 127) / 128 * 128);
  const size_t ring = (p->off_planes + plane_bytes + 1023) / 1024 * 1024;
  if (ring + 2 * size_t(p->slot_bytes) > size_t(kSmemLimit)) return false;
  p->off_ring = int(ring);
  int stages = int((size_t(kSmemLimit) - ring) / p->slot_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p->stages = stages;
  p->smem = ring + size_t(stages) * p->slot_bytes;
  return true;
}

}  // namespace b200
