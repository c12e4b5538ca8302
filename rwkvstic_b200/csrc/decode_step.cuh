// One decode step (one token, one stream) of the whole network as ONE persistent kernel.
//
// Why: a decode step is a chain of 4*L+1 matrix-vector products, each of which needs the complete
// output of the one before.  Launching them one by one leaves HBM idle at every link of the chain:
// a CTA's shared-memory ring - the only place weight bytes can wait - is torn down and rebuilt at
// each kernel boundary.  Here every SM runs one CTA for the whole step.  Its producer lane streams
// the CTA's rows of ALL matrices, one after the other, through one ring that never drains (weights
// are constants, so the stream does not depend on any activation); the consumer warps meet the
// other CTAs only where the mathematics needs every output of a matrix.
//
// What crosses CTAs, and how.  CTA c owns rows [N*c/G, N*(c+1)/G) of every matrix.  For the D-wide
// vectors (residual stream, receptance gates, WKV state, token-shift carries) that is the same
// slice in every block, so they never leave their CTA: the residual lives in shared memory for the
// whole step.  Two kinds of data are exchanged through global memory (L2):
//   * the input of the next matrix, already multiplied by its per-input scale (xs = v * ry), one
//     slice per CTA, plus one 16-byte record per CTA with the slice's max|xs| and the sums the affine
//     terms need;
//   * for a layer norm, one record per CTA with the mean and the centred sum of squares of its
//     slice of the residual; every CTA combines the G records (Chan's parallel variance, fp64) in
//     the same order, so all CTAs get the same statistics bit for bit.
// There is no barrier, no atomic and no fence in the exchange: every 32-bit word that crosses carries
// the parity of its buffer's use count in its lowest mantissa bit (a relative change of 2^-23 at
// most, below the 24-bit fixed point the value is about to be rounded to).  A reader simply loads
// the words it needs and repeats the load of those whose bit is still the old one; the poll IS the
// read.  A buffer is rewritten completely at every use and a CTA cannot get a whole block ahead of
// another (every exchange needs everyone's data), so a word with the right parity is the right
// word.  A hand-off costs one store transit plus one load round trip.
// After the exchange every CTA turns the xs vector into the three signed base-256 digit planes in
// its own shared memory and runs the integer tensor-core main loop of stream_gemv_kernel.  A layer
// norm needs two exchanges (statistics, then the normalised and mixed slices), an element-wise
// hand-off (attention output, ffn value) one.
//
// Every wait (mbarrier, exchange poll) is bounded by wait_limit_ns; on expiry the CTA raises a
// status bit and an abort word that the other CTAs see at their next poll, drains its own copies
// in flight and returns.  After an abandoned step the plan (use counts) has to be initialised again.
#pragma once

#include "stream_gemv.cuh"

namespace b200 {

#ifndef B200_STEP_CONSUMER_WARPS
#define B200_STEP_CONSUMER_WARPS 16
#endif
constexpr int kStepConsumerWarps = B200_STEP_CONSUMER_WARPS;   // a multiple of 4; 16 + the producer = 17 warps: 96 registers per thread
constexpr int kStepConsumers = kStepConsumerWarps * 32;
constexpr int kStepThreads = kStepConsumers + 32;   // + one producer warp
constexpr int kStepTraceSlots = 8;              // u64 stamps per (launch, CTA)
constexpr int kStepPrefetchPiece = 16384;       // bytes per L2 prefetch request
constexpr int kStepPrefetchDefault = 0;         // bytes per CTA requested from L2 beyond the ring (measured: no gain)
constexpr int kStepPartPerLane = 5;             // warps of 32 per-CTA records: up to 160 CTAs
constexpr int kRecStride = 8;                   // float4s between two CTAs' records: one 128-byte line each, so that pollers spread over L2
constexpr int kStepGather = (4096 + kStepConsumers - 1) / kStepConsumers;   // float4 per thread in one exchange read: 16384 inputs

// Shared-memory map of the step kernel (byte offsets; the rest is laid out by the host, see StepParams)
constexpr int kSOffConsAbort = 272;  // int: set by consumer threads only, read after named barriers (uniform decisions)
constexpr int kSOffInv = 288;        // float[3]: fixed-point scale of each segment's digit planes
constexpr int kSOffRed = 512;        // reduction scratch: float [warps <= 16][16]
constexpr int kSOffBc = kSOffRed + 16 * 16 * 4;   // 16 floats
constexpr int kSOffStat = kSOffBc + 64;            // 2 * kStepPartPerLane doubles
constexpr int kSOffDyn = 2560;       // first byte the host lays out

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

// The vector parameters are copied into the plan at fixed offsets so that the kernel computes their
// addresses instead of chasing pointers.  Per block kStepVecs vectors of D floats, in this order:
enum StepVecId : int { VEC_LN1_W = 0, VEC_LN1_B, VEC_LN2_W, VEC_LN2_B, VEC_MIX_K, VEC_MIX_V, VEC_MIX_R, VEC_FMIX_K, VEC_FMIX_R,
                       VEC_DECAY, VEC_FIRST, kStepVecs };
// ... and the per-input scale / offset (ry, my) of every matrix: per block [6 matrices with D inputs:
// key, value, receptance, output, ffn key, ffn receptance][ry, my][D], then [ffn value][ry, my][F];
// after the last block [head][ry, my][D].

struct StepParams {
  const StepMat* mats;    // [7*L + 1]: per block key, value, receptance, output, ffn key, ffn receptance, ffn value; then the head
  const float* vpack;     // [L][kStepVecs][D]
  const float* rympack;   // [L][12*D + 2*F], then [2][D] for the head
  int L, D, F, V;
  const float* emb;
  const float *ln0_w, *ln0_b, *lnout_w, *lnout_b;
  const long long* token;
  float* state;           // [L][5][D]
  float* logits;          // [V] or null (no head)
  // exchange buffers: tagged words (see the header comment)
  // (each buffer is written completely at every one of its uses, which is what makes the tag sufficient)
  float* xs_kvr;          // [3][D]  inputs of key / value / receptance
  float* xs_att;          // [D]     input of the attention output projection
  float* xs_fkr;          // [2][D]  inputs of ffn key / receptance
  float* xs_ffn;          // [F]     input of the ffn value projection
  float* xs_head;         // [D]     input of the head
  float4* part_kvr;       // [3][G]  per CTA: max|xs|, sum v*my, sum xs, sum v of its slice
  float4* part_att;       // [G]
  float4* part_fkr;       // [2][G]
  float4* part_ffn;       // [G]
  float4* part_head;      // [G]
  float4* part_st;        // [G]     per CTA: mean and centred sum of squares of its slice of the residual
  unsigned* uses;         // [6]: how often the kvr, att, fkr, ffn, head buffers and part_st have been written so far
  unsigned* abort_word;
  int* status;
  unsigned long long* trace;   // optional: [4L+1 launches][G][kStepTraceSlots]
  // shared-memory geometry (host: plan_step)
  int slot_bytes, stages, off_own, own_rows, off_park, park_stride, off_rows, off_planes, off_ring;
  // tuning
  int window;             // weight stages a CTA may have in flight (>= stages: no limit)
  int window_handoff;     // the same while the consumers are between two matrices
  int pf_bytes;           // bytes per CTA requested from L2 ahead of the ring
  unsigned long long wait_limit_ns;
  double inv_d;           // 1 / D
};

// ---- memory operations -------------------------------------------------------------------------------
__device__ __forceinline__ unsigned ld_relaxed_u32(const unsigned* p) {
  unsigned v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Exchange words are read and written with strong (relaxed, gpu-scope) accesses: a weak load, even
// one that bypasses L1, may be served from a stale copy for microseconds.
__device__ __forceinline__ float4 ld_xchg_v4(const float4* p) {
  float4 v;
  asm volatile("ld.relaxed.gpu.global.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_xchg_f32(float* p, float v) {
  asm volatile("st.relaxed.gpu.global.f32 [%0], %1;" ::"l"(p), "f"(v) : "memory");
}
__device__ __forceinline__ void st_xchg_v4(float4* p, float4 v) {
  asm volatile("st.relaxed.gpu.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__device__ __forceinline__ void cp_async_f32(float* smem_dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// ---- tagged words ------------------------------------------------------------------------------------
__device__ __forceinline__ float tag_f32(float v, unsigned tag) { return __uint_as_float((__float_as_uint(v) & ~1u) | tag); }
__device__ __forceinline__ bool tagged(float v, unsigned tag) { return (__float_as_uint(v) & 1u) == tag; }
__device__ __forceinline__ bool tagged4(float4 v, unsigned tag) {
  return ((__float_as_uint(v.x) & __float_as_uint(v.y) & __float_as_uint(v.z) & __float_as_uint(v.w)) & 1u) == tag &&
         ((__float_as_uint(v.x) | __float_as_uint(v.y) | __float_as_uint(v.z) | __float_as_uint(v.w)) & 1u) == tag;
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

// Sums of NV floats and maxima of NM floats over the consumer threads, in a fixed order (the same
// inputs give the same bits).  Afterwards thread i < NV holds total i in v[0] and thread 32 + j holds
// maximum j in m[0].  One named barrier inside; the scratch is free again after the caller's next one.
template <int NV, int NM>
__device__ __forceinline__ void cta_reduce(float (&v)[NV], float (&m)[NM > 0 ? NM : 1], float* red) {
  static_assert(NV + NM <= 16, "scratch row holds 16 floats");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = warp_sum(v[i]);
#pragma unroll
  for (int i = 0; i < NM; ++i) m[i] = warp_max(m[i]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) red[warp * 16 + i] = v[i];
#pragma unroll
    for (int i = 0; i < NM; ++i) red[warp * 16 + NV + i] = m[i];
  }
  named_bar_sync(1, kStepConsumers);
  if (tid < NV) {
    float a = 0.f;
    for (int w = 0; w < kStepConsumerWarps; ++w) a += red[w * 16 + tid];
    v[0] = a;
  } else if (tid >= 32 && tid < 32 + NM) {
    float a = 0.f;
    for (int w = 0; w < kStepConsumerWarps; ++w) a = fmaxf(a, red[w * 16 + NV + tid - 32]);
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


// What a thread needs to give up a poll: the flags, the limit, where to report.
struct StepWaitCtx {
  volatile int* abort_flag;     // shared: anyone may raise it; waits return early when it is set
  volatile int* cons_abort;     // shared: raised by consumer threads only
  const unsigned* abort_word;   // global: another CTA gave up
  int* status;
  unsigned long long limit;
};

// true: go on polling.  Called every few iterations of a poll loop.
__device__ __forceinline__ bool poll_check(const StepWaitCtx& w, unsigned long long t0) {
  if (*w.abort_flag || ld_relaxed_u32(w.abort_word) != 0u) {
    *w.abort_flag = 1; *w.cons_abort = 1;
    return false;
  }
  if (globaltimer_ns() - t0 > w.limit) {
    if (w.status) atomicOr(w.status, B200RWKV_STATUS_WAIT_PEER);
    atomicExch(const_cast<unsigned*>(w.abort_word), 1u);
    *w.abort_flag = 1; *w.cons_abort = 1;
    return false;
  }
  return true;
}

// The read side of an xs exchange, called by all consumer threads: gathers the nseg vectors of K
// inputs (segment s at xs + s * xs_stride) and the G per-CTA records of each (segment s at
// part + s * G), repeating the loads of words that still carry the old tag, then writes the digit
// planes and the segments' scalars to shared memory.  Thread t reads record t % 160 of segment
// t / 160 beside its share of the vectors.  Two named barriers inside; the planes are complete after
// the caller's next one.
__device__ __forceinline__ void gather_digit_planes(unsigned char* planes, SegScalars* scal, float* inv_s, float* red, const float* xs,
                                                    size_t xs_stride, const float4* part, int G, int nseg, int K, unsigned tag,
                                                    const StepWaitCtx& w) {
  constexpr int kRecSpan = 32 * kStepPartPerLane;   // threads (and five warps) per segment's records
  static_assert(kStepConsumers >= kMaxSeg * kRecSpan, "one consumer thread per record of three segments");
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NG = K / 4, TG = nseg * NG;
  const int rs = tid / kRecSpan, rc = tid - rs * kRecSpan;
  const bool has_rec = rs < nseg && rc < G;
  float4 v[kStepGather], p = make_float4(0.f, 0.f, 0.f, 0.f);
  const unsigned long long t0 = globaltimer_ns();
  // 1. the records: small, one line per CTA, so polling them is cheap; they are written after the
  //    slice they describe
  if (has_rec) {
    const float4* rec = part + (size_t(rs) * G + rc) * kRecStride;
    p = ld_xchg_v4(rec);
    for (unsigned it = 1; !tagged4(p, tag); ++it) {
      if ((it & 15u) == 0u && !poll_check(w, t0)) break;
      __nanosleep(64);
      p = ld_xchg_v4(rec);
    }
  }
  named_bar_sync(2, kStepConsumers);      // every record has arrived: the slices are (almost always) visible too
  // 2. the vectors: one read; words that still carry the old tag are read again
  unsigned need = 0u;        // bit i: v[i] not yet valid
#pragma unroll
  for (int i = 0; i < kStepGather; ++i) if (tid + i * kStepConsumers < TG) need |= 1u << i;
  for (unsigned it = 1; need != 0u; ++it) {
#pragma unroll
    for (int i = 0; i < kStepGather; ++i) {
      if (need & (1u << i)) {
        const int f = tid + i * kStepConsumers;
        const int s = f >= 2 * NG ? 2 : (f >= NG ? 1 : 0), g = f - s * NG;
        v[i] = ld_xchg_v4(reinterpret_cast<const float4*>(xs + size_t(s) * xs_stride) + g);
      }
    }
#pragma unroll
    for (int i = 0; i < kStepGather; ++i)
      if ((need & (1u << i)) && tagged4(v[i], tag)) need &= ~(1u << i);
    if (need != 0u && (it & 15u) == 0u && !poll_check(w, t0)) break;
  }
  // the records: maximum and sums over the CTAs, in the same order in every CTA (warp, then the
  // five warps of a segment in sequence)
  {
    float amax = has_rec ? p.x : 0.f, zp = has_rec ? p.y : 0.f, sxs = has_rec ? p.z : 0.f, sx = has_rec ? p.w : 0.f;
    amax = warp_max(amax); zp = warp_sum(zp); sxs = warp_sum(sxs); sx = warp_sum(sx);
    if (lane == 0) { red[warp * 4] = amax; red[warp * 4 + 1] = zp; red[warp * 4 + 2] = sxs; red[warp * 4 + 3] = sx; }
  }
  named_bar_sync(1, kStepConsumers);
  if (tid < nseg) {
    float amax = 0.f, zp = 0.f, sxs = 0.f, sx = 0.f;
#pragma unroll
    for (int j = 0; j < kStepPartPerLane; ++j) {
      const float* r = red + (tid * kStepPartPerLane + j) * 4;
      amax = fmaxf(amax, r[0]); zp += r[1]; sxs += r[2]; sx += r[3];
    }
    const float inv = amax > 0.f ? kQMax / amax : 0.f;
    SegScalars sc;
    sc.sd = amax > 0.f ? __fdiv_rn(1.0f, inv) : 0.f;
    sc.zp = zp; sc.sumxs = sxs; sc.sumx = sx;
    sc.pad[0] = sc.pad[1] = sc.pad[2] = sc.pad[3] = 0.f;
    scal[tid] = sc;
    inv_s[tid] = inv;
  }
  named_bar_sync(1, kStepConsumers);
  const float inv0 = inv_s[0], inv1 = inv_s[1], inv2 = inv_s[2];
#pragma unroll
  for (int i = 0; i < kStepGather; ++i) {
    const int f = tid + i * kStepConsumers;
    if (f < TG) {
      const int s = f >= 2 * NG ? 2 : (f >= NG ? 1 : 0), g = f - s * NG;
      store_digits_compact(planes + size_t(s) * 3 * K, g, v[i], s == 0 ? inv0 : (s == 1 ? inv1 : inv2));
    }
  }
  // inputs beyond what one pass holds in registers (nseg * K > 16384): one more poll per piece
  for (int f = tid + kStepGather * kStepConsumers; f < TG; f += kStepConsumers) {
    const int s = f >= 2 * NG ? 2 : (f >= NG ? 1 : 0), g = f - s * NG;
    float4 x = ld_xchg_v4(reinterpret_cast<const float4*>(xs + size_t(s) * xs_stride) + g);
    for (unsigned it = 1; !tagged4(x, tag); ++it) {
      if ((it & 15u) == 0u && !poll_check(w, t0)) break;
      x = ld_xchg_v4(reinterpret_cast<const float4*>(xs + size_t(s) * xs_stride) + g);
    }
    store_digits_compact(planes + size_t(s) * 3 * K, g, x, s == 0 ? inv0 : (s == 1 ? inv1 : inv2));
  }
}

// The read side of a statistics exchange, called by all consumer threads: thread c < G gathers the
// record of CTA c (mean and centred sum of squares of its n_c elements), the records are combined in
// fp64 in a fixed order, and every thread gets mean and 1/sqrt(var + 1e-5) of the whole vector
// (modules/layernorm.py:11-20).  var = (sum_c M2_c + n_c mean_c^2  -  D mean^2) / D: the inputs are
// fp32 numbers, so the fp64 subtraction loses nothing that matters.  One named barrier inside.
__device__ __forceinline__ void gather_statistics(double* scratch, const float4* part, int G, int D, double inv_d, unsigned tag,
                                                  const StepWaitCtx& w, float& mean_out, float& rstd_out) {
  constexpr int kRecWarps = kStepPartPerLane;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  double a = 0.0, b = 0.0;
  if (warp < kRecWarps) {
    const bool has = tid < G;
    float4 p = make_float4(0.f, 0.f, 0.f, 0.f);
    if (has) {
      p = ld_xchg_v4(part + size_t(tid) * kRecStride);
      const unsigned long long t0 = globaltimer_ns();
      for (unsigned it = 1; !tagged4(p, tag); ++it) {
        if ((it & 15u) == 0u && !poll_check(w, t0)) break;
        __nanosleep(64);
        p = ld_xchg_v4(part + size_t(tid) * kRecStride);
      }
      const double n = double(int((long long)D * (tid + 1) / G) - int((long long)D * tid / G));
      a = n * double(p.x);
      b = double(p.y) + a * double(p.x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) { a += __shfl_xor_sync(0xffffffffu, a, o); b += __shfl_xor_sync(0xffffffffu, b, o); }
    if (lane == 0) { scratch[2 * warp] = a; scratch[2 * warp + 1] = b; }
  }
  named_bar_sync(1, kStepConsumers);
  a = 0.0; b = 0.0;
#pragma unroll
  for (int j = 0; j < kRecWarps; ++j) { a += scratch[2 * j]; b += scratch[2 * j + 1]; }
  const double mean = a * inv_d;
  mean_out = float(mean);
  rstd_out = 1.0f / sqrtf(fmaxf(float((b - a * mean) * inv_d), 0.f) + 1e-5f);
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
  volatile int* cons_abort = reinterpret_cast<volatile int*>(smem + kSOffConsAbort);
  SegScalars* scal = reinterpret_cast<SegScalars*>(smem + kOffScale);
  float* inv_s = reinterpret_cast<float*>(smem + kSOffInv);
  float* red = reinterpret_cast<float*>(smem + kSOffRed);
  float* bc = reinterpret_cast<float*>(smem + kSOffBc);
  float* x_own = reinterpret_cast<float*>(smem + P.off_own);   // this CTA's slice of the residual stream
  float* rf_own = x_own + P.own_rows;                          // ... of sigmoid(ffn receptance)
  int* rowsum = reinterpret_cast<int*>(smem + P.off_rows);
  unsigned char* planes = smem + P.off_planes;
  unsigned char* ring = smem + P.off_ring;
  const uint32_t full0 = smem_u32(smem + kOffFull), empty0 = smem_u32(smem + kOffEmpty);
  const unsigned long long limit = P.wait_limit_ns;

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, kStepConsumerWarps);
    }
    *abort_flag = 0;
    *issued_ptr = 0;
    *handoff = 1;
    *cons_abort = 0;
    inv_s[0] = inv_s[1] = inv_s[2] = 0.f;
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
          tma_load_3d(smem_u32(ring + size_t(slot) * P.slot_bytes), &M->tmap, 0, ic.r0 + ic.row, ch * (kc / 128),
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
    const int r0D = int((long long)D * cta / G), nrD = int((long long)D * (cta + 1) / G) - r0D;
    StepWaitCtx wctx;
    wctx.abort_flag = abort_flag; wctx.cons_abort = cons_abort; wctx.abort_word = P.abort_word; wctx.status = P.status; wctx.limit = limit;
    // use counts of the exchange buffers so far (the same in every CTA); the parity of a count tags the words of that use
    unsigned u_kvr = P.uses[0], u_att = P.uses[1], u_fkr = P.uses[2], u_ffn = P.uses[3], u_head = P.uses[4], u_st = P.uses[5];

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
              *cons_abort = 1;
              if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
              break;
            }
            const uint32_t a_addr = ring_s32 + uint32_t(slot) * uint32_t(P.slot_bytes) + a_lane;
            const uint32_t b_addr = b_seg + uint32_t(ch * kbpc) * 96u;
            consume_stage(c, a_addr, b_addr, gq < 3, kbn, warp);
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

    // ---- the write side of an xs exchange: one element of a next-matrix input, xs = v * ry with the
    // use's tag, and this thread's share of the slice's record
    struct XsAcc { float zp, sxs, sx, amax; };
    auto xs_emit = [&](XsAcc& a, float* dst, int n, float v, float ry, float my, unsigned tag) __attribute__((always_inline)) {
      const float xs = tag_f32(v * ry, tag);
      st_xchg_f32(dst + n, xs);
      a.amax = fmaxf(a.amax, fabsf(xs));
      a.zp += v * my;
      a.sxs += xs;
      a.sx += v;
    };
    // ... and the record itself, by the four threads that hold its fields after cta_reduce<3 * n, n>
    auto write_record = [&](float4* rec, int field, float v, unsigned tag) __attribute__((always_inline)) {
      st_xchg_f32(reinterpret_cast<float*>(rec) + field, tag_f32(v, tag));
    };

    // ---- operands a thread needs after a matrix has streamed (constants, or state only this thread
    // touches) are copied asynchronously (cp.async, no register) into a thread-private shared-memory
    // slot before the exchange in front of that matrix is read, so their latency is off the chain.
    // Slot j of thread t: park[j * park_stride + t], 13 slots.
    float* park = reinterpret_cast<float*>(smem + P.off_park);
    const int pstride = P.park_stride;
    const size_t rym_stride = size_t(12) * D + size_t(2) * P.F;
    auto vec_of = [&](int l, int id) __attribute__((always_inline)) -> const float* { return P.vpack + (size_t(l) * kStepVecs + id) * D; };
    // ry (which = 0) or my (1) of matrix m of block l: 0..5 the D-input matrices, 6 ffn value; l == L: the head
    auto rym_of = [&](int l, int m, int which) __attribute__((always_inline)) -> const float* {
      const float* base = P.rympack + size_t(l) * rym_stride;
      return m < 6 ? base + (size_t(m) * 2 + which) * D : base + size_t(12) * D + size_t(which) * P.F;
    };
    // operands of a layer-norm hop for this thread's element of the residual: w, b, carry, then per
    // following matrix mu, ry, my.  lv / lw, lb: block and ids of the layer norm; m0: first following matrix.
    auto hop_async = [&](int lv, int id_w, int id_b, int id_mix0, int nmix, const float* carry_row, int lm, int m0, int nseg) __attribute__((always_inline)) {
      if (tid < nrD) {
        const int n = r0D + tid;
        cp_async_f32(park + tid, (lv < 0 ? P.lnout_w : vec_of(lv, id_w)) + n);
        cp_async_f32(park + pstride + tid, (lv < 0 ? P.lnout_b : vec_of(lv, id_b)) + n);
        if (carry_row) cp_async_f32(park + 2 * pstride + tid, carry_row + n);
#pragma unroll
        for (int s = 0; s < kMaxSeg; ++s) {
          if (s < nseg) {
            if (s < nmix) cp_async_f32(park + (3 + 3 * s) * pstride + tid, vec_of(lv, id_mix0 + s) + n);
            cp_async_f32(park + (4 + 3 * s) * pstride + tid, rym_of(lm, m0 + s, 0) + n);
            cp_async_f32(park + (5 + 3 * s) * pstride + tid, rym_of(lm, m0 + s, 1) + n);
          }
        }
      }
    };
    // layer norm + token-shift mix of this CTA's slice of the residual for the nseg matrices that
    // follow (modules/layernorm.py:11-20, modules/block.py:58-67, :82-91): writes their xs slices,
    // the new carry, and the slice's record per matrix
    auto ln_hop = [&](float mean, float rstd, float* carry_row, int nseg, float* xs_dst, float4* part_dst, unsigned tag) __attribute__((always_inline)) {
      XsAcc acc[kMaxSeg];
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) { acc[s].zp = 0.f; acc[s].sxs = 0.f; acc[s].sx = 0.f; acc[s].amax = 0.f; }
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
            xs_emit(acc[s], xs_dst + size_t(s) * D, n, v, park[(4 + 3 * s) * pstride + tid], park[(5 + 3 * s) * pstride + tid], tag);
          }
        }
      }
      float v[9], m[3];
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) { v[3 * s] = acc[s].zp; v[3 * s + 1] = acc[s].sxs; v[3 * s + 2] = acc[s].sx; m[s] = acc[s].amax; }
      cta_reduce<9, 3>(v, m, red);
      if (tid < 3 * nseg) write_record(part_dst + (size_t(tid / 3) * G + cta) * kRecStride, 1 + tid % 3, v[0], tag);
      else if (tid >= 32 && tid < 32 + nseg) write_record(part_dst + (size_t(tid - 32) * G + cta) * kRecStride, 0, m[0], tag);
    };
    // the record of this CTA's slice of the residual for the next layer norm: mean and centred sum of squares
    auto publish_stats = [&](unsigned tag) __attribute__((always_inline)) {
      if (tid < 32) {
        float s = 0.f;
        for (int i = lane; i < nrD; i += 32) s += x_own[i];
        const float mc = warp_sum(s) / float(nrD);
        float q = 0.f;
        for (int i = lane; i < nrD; i += 32) { const float d = x_own[i] - mc; q += d * d; }
        q = warp_sum(q);
        if (lane == 0) st_xchg_v4(P.part_st + size_t(cta) * kRecStride, make_float4(tag_f32(mc, tag), tag_f32(q, tag), tag_f32(0.f, tag), tag_f32(0.f, tag)));
      }
    };

    // ================================================================== the step
    float mean = 0.f, rstd = 1.f;
    hop_async(0, VEC_LN1_W, VEC_LN1_B, VEC_MIX_K, 3, P.state, 0, 0, 3);   // operands of the first block's ln1 hop
    // ---- embedding row + ln0 (emb.py:8-9, opt.py:63-64).  Every CTA evaluates the whole vector: it
    // needs the statistics of ln0's output for the first block's layer norm and keeps its own slice.
    {
      long long tok = *P.token;
      tok = tok < 0 ? 0 : (tok >= P.V ? P.V - 1 : tok);
      const float* row = P.emb + size_t(tok) * D;
      auto block_sum = [&](float v) __attribute__((always_inline)) -> float {
        v = warp_sum(v);
        if (lane == 0) red[warp] = v;
        named_bar_sync(1, kStepConsumers);
        if (tid == 0) {
          float a = 0.f;
          for (int i = 0; i < kStepConsumerWarps; ++i) a += red[i];
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
      s = 0.f;
      for (int i = tid; i < D; i += kStepConsumers) {
        const float y = P.ln0_w[i] * ((row[i] - mean0) / sdev) + P.ln0_b[i];
        if (i >= r0D && i < r0D + nrD) x_own[i - r0D] = y;
        s += y;
      }
      mean = block_sum(s) / float(D);
      s = 0.f;
      for (int i = tid; i < D; i += kStepConsumers) {
        const float c = (P.ln0_w[i] * ((row[i] - mean0) / sdev) + P.ln0_b[i]) - mean;
        s += c * c;
      }
      rstd = 1.0f / sqrtf(block_sum(s) / float(D) + 1e-5f);
    }
    cp_async_wait_all();

    // ---- the launches: per block 0 key/value/receptance + WKV, 1 attention output, 2 ffn key +
    // receptance, 3 ffn value; then 4 = the head.  One copy of every stage of a launch; what differs
    // between the launch types is selected by `type`.
    const int nph = 4 * L + (P.logits ? 1 : 0);
    bool dead = false;
    for (int ph = 0; ph < nph; ++ph) {
      const int type = ph < 4 * L ? (ph & 3) : 4;
      const int l = ph < 4 * L ? (ph >> 2) : L - 1;
      const bool more = l + 1 < L;
      float* st = P.state + size_t(l) * 5 * D;
      const int mfirst = 7 * l + (type == 0 ? 0 : type == 1 ? 3 : type == 2 ? 4 : type == 3 ? 6 : 7);
      const int nseg = type == 0 ? 3 : (type == 2 ? 2 : 1);

      // ---- A. a layer norm in front of the matrices: normalise and mix this CTA's slice
      // (the named barriers inside the previous launch's epilogue already separate its reads of the row
      // sums from their zeroing in load_phase)
      if (type == 0) {
        ++u_kvr;
        ln_hop(mean, rstd, st, 3, P.xs_kvr, P.part_kvr, u_kvr & 1u);
        STEP_TRACE(ph, 5);
      } else if (type == 2) {
        ++u_fkr;
        ln_hop(mean, rstd, st + size_t(D), 2, P.xs_fkr, P.part_fkr, u_fkr & 1u);
        STEP_TRACE(ph, 5);
      } else if (type == 4) {
        ++u_head;
        ln_hop(mean, rstd, nullptr, 1, P.xs_head, P.part_head, u_head & 1u);
        STEP_TRACE(ph, 5);
      }
      load_phase(mfirst, nseg);

      // ---- B. operands for after the stream; the exchange read; digit planes
      if (type == 0) {          // WKV state and parameters; ry, my of the output projection
        if (tid < nrD) {
          const int n = r0D + tid;
          cp_async_f32(park + tid, st + 2 * size_t(D) + n);
          cp_async_f32(park + pstride + tid, st + 3 * size_t(D) + n);
          cp_async_f32(park + 2 * pstride + tid, st + 4 * size_t(D) + n);
          cp_async_f32(park + 3 * pstride + tid, vec_of(l, VEC_DECAY) + n);
          cp_async_f32(park + 4 * pstride + tid, vec_of(l, VEC_FIRST) + n);
          cp_async_f32(park + 5 * pstride + tid, rym_of(l, 3, 0) + n);
          cp_async_f32(park + 6 * pstride + tid, rym_of(l, 3, 1) + n);
        }
      } else if (type == 1) {   // the ln2 hop that follows this matrix
        hop_async(l, VEC_LN2_W, VEC_LN2_B, VEC_FMIX_K, 2, st + size_t(D), l, 4, 2);
      } else if (type == 2) {   // ry, my of the value projection at this thread's first ffn-key row
        if (tid < snr[0]) {
          cp_async_f32(park + tid, rym_of(l, 6, 0) + sr0[0] + tid);
          cp_async_f32(park + pstride + tid, rym_of(l, 6, 1) + sr0[0] + tid);
        }
      } else if (type == 3) {   // the next block's ln1 hop, or ln_out
        if (more) hop_async(l + 1, VEC_LN1_W, VEC_LN1_B, VEC_MIX_K, 3, st + size_t(5) * D, l + 1, 0, 3);
        else if (P.logits) hop_async(-1, 0, 0, 0, 0, nullptr, L, 0, 1);
      }
      {
        const unsigned tag = (type == 0 ? u_kvr : type == 1 ? u_att : type == 2 ? u_fkr : type == 3 ? u_ffn : u_head) & 1u;
        const float* xs_src = type == 0 ? P.xs_kvr : type == 1 ? P.xs_att : type == 2 ? P.xs_fkr : type == 3 ? P.xs_ffn : P.xs_head;
        const float4* part_src = type == 0 ? P.part_kvr : type == 1 ? P.part_att : type == 2 ? P.part_fkr : type == 3 ? P.part_ffn : P.part_head;
        gather_digit_planes(planes, scal, inv_s, red, xs_src, size_t(D), part_src, G, nseg, pK, tag, wctx);
      }
      named_bar_sync(1, kStepConsumers);      // planes, zeroed row sums, parked operands
      if (*cons_abort) { dead = true; break; }
      if (tid == 0) *handoff = 0;
      STEP_TRACE(ph, 1);
      stream_rows();
      cp_async_wait_all();                    // this thread's parked operands have landed
      named_bar_sync(1, kStepConsumers);
      if (*cons_abort) { dead = true; break; }
      if (tid == 0) *handoff = 1;
      STEP_TRACE(ph, 2);

      // ---- C. what follows the matrices in the block (modules/block.py:72-100)
      if (type == 0) {            // WKV update, sigmoid(r) * wkv -> input of the output projection
        ++u_att;
        XsAcc acc; acc.zp = 0.f; acc.sxs = 0.f; acc.sx = 0.f; acc.amax = 0.f;
        if (tid < nrD) {
          const int n = r0D + tid;
          const float k = value(0, tid), v = value(1, tid), r = sigmoidf_(value(2, tid));
          float aa = park[tid], bb = park[pstride + tid], pp = park[2 * pstride + tid];
          const float y = wkv_step(k, v, park[3 * pstride + tid], park[4 * pstride + tid], aa, bb, pp);
          st[2 * size_t(D) + n] = aa; st[3 * size_t(D) + n] = bb; st[4 * size_t(D) + n] = pp;
          xs_emit(acc, P.xs_att, n, r * y, park[5 * pstride + tid], park[6 * pstride + tid], u_att & 1u);
        }
        float v3[3] = {acc.zp, acc.sxs, acc.sx}, m1[1] = {acc.amax};
        cta_reduce<3, 1>(v3, m1, red);
        if (tid < 3) write_record(P.part_att + size_t(cta) * kRecStride, 1 + tid, v3[0], u_att & 1u);
        else if (tid == 32) write_record(P.part_att + size_t(cta) * kRecStride, 0, m1[0], u_att & 1u);
      } else if (type == 2) {     // relu(key)^2 -> input of the value projection; sigmoid(receptance) stays here
        ++u_ffn;
        XsAcc acc; acc.zp = 0.f; acc.sxs = 0.f; acc.sx = 0.f; acc.amax = 0.f;
        const float* vry = rym_of(l, 6, 0);
        const float* vmy = rym_of(l, 6, 1);
        for (int row = tid; row < snr[0]; row += kStepConsumers) {
          const int n = sr0[0] + row;
          float y = fmaxf(value(0, row), 0.f);
          y *= y;
          const bool parked = row < kStepConsumers;    // row == tid then: this thread parked them
          xs_emit(acc, P.xs_ffn, n, y, parked ? park[row] : __ldg(vry + n), parked ? park[pstride + row] : __ldg(vmy + n), u_ffn & 1u);
        }
        if (tid < nrD) rf_own[tid] = sigmoidf_(value(1, tid));
        float v3[3] = {acc.zp, acc.sxs, acc.sx}, m1[1] = {acc.amax};
        cta_reduce<3, 1>(v3, m1, red);
        if (tid < 3) write_record(P.part_ffn + size_t(cta) * kRecStride, 1 + tid, v3[0], u_ffn & 1u);
        else if (tid == 32) write_record(P.part_ffn + size_t(cta) * kRecStride, 0, m1[0], u_ffn & 1u);
      } else if (type == 4) {     // logits
        for (int row = tid; row < snr[0]; row += kStepConsumers) P.logits[sr0[0] + row] = value(0, row);
      } else {                    // residual update; a layer norm follows unless the step ends here
        if (tid < nrD) x_own[tid] = type == 1 ? value(0, tid) + x_own[tid] : value(0, tid) * rf_own[tid] + x_own[tid];
        if (type == 1 || more || P.logits) {
          named_bar_sync(1, kStepConsumers);    // x_own complete
          ++u_st;
          publish_stats(u_st & 1u);
          STEP_TRACE(ph, 3);
          gather_statistics(reinterpret_cast<double*>(smem + kSOffStat), P.part_st, G, D, P.inv_d, u_st & 1u, wctx, mean, rstd);
          if (*cons_abort) { dead = true; break; }
          STEP_TRACE(ph + 1, 4);
          continue;
        }
      }
      STEP_TRACE(ph, 3);
    }
    if (!dead && cta == 0 && tid == 0) {
      P.uses[0] = u_kvr; P.uses[1] = u_att; P.uses[2] = u_fkr; P.uses[3] = u_ffn; P.uses[4] = u_head; P.uses[5] = u_st;
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
  if (G > 32 * kStepPartPerLane) return false;             // a warp gathers the CTAs' partial results, kStepPartPerLane per lane
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
