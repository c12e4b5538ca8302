// Activation preparation for the streaming GEMV: one CTA per matrix turns the raw activation
// vector into the fixed-point digit planes and scalar terms that every GEMV CTA needs, ONCE,
// instead of every CTA recomputing them.  The CTAs run on the SMs the GEMV grid leaves free, so they
// can be resident while the previous GEMV still streams and load their parameter vectors before
// their dependency resolves.
//
// Per segment s (up to three matrices share one launch):
//   v_s[k]  = input of matrix s: either xin_s[k], or LayerNorm(ln_x)[k] mixed with the carried
//             previous-token vector (modules/block.py:58-67, :82-91; layernorm.py:11-20)
//   xs_s[k] = v_s[k] * ry_s[k];   inv_s = QMAX / max_k |xs_s[k]|;   X_s[k] = rint(xs_s[k] * inv_s)
//   planes  : signed base-256 digits of X_s, 128 bytes per 32 inputs: [a:32][b:32][c:32][0:32]
//   scalars : 1/inv_s (fp32), zp_s = sum_k v_s[k]*my_s[k], sum_k xs_s[k], sum_k v_s[k]
//
// To keep the chain between two GEMV launches short, whatever needs a reduction over ALL outputs of
// the previous launch is published by that launch's epilogue with order-independent integer
// atomics (PubSlot): the layer-norm sums, or - when the next matrix input is an element-wise
// function of the previous outputs - the already scaled xs with its max and sums.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kPrepThreads = 512;
constexpr int kPrepWarps = kPrepThreads / 32;
constexpr int kPrepRedBytes = (kPrepWarps + 1) * 16 * 4 + 64;  // reduction scratch, rounded to 128
constexpr int kMaxSeg = 3;
constexpr float kQMax = 8355000.0f;  // |X| <= QMAX keeps all three signed digits inside int8

// Fixed-point units of the published sums (int64 accumulators: exact, order-independent).  The
// ranges they leave: |sum x|, |sum v*my|, |sum v| < 2.1e9 and |sum xs| < 8.3e6.  Squares are carried
// in two limbs (see square_limbs): exact from 2^-60 to 2^55 per element, sums up to 3.6e16.
constexpr float kPubSumScale = 4294967296.0f;        // 2^32
constexpr float kPubSqHiScale = 256.0f;              // 2^8: high limb of a square
constexpr float kPubSqLoScale = 1099511627776.0f;    // 2^40 on top of the 2^8: low limb in 2^-48 units
constexpr float kPubXsScale = 1099511627776.0f;      // 2^40 (xs = v * ry is small: ry ~ 1e-3)

// What the epilogue of one launch publishes for the preparation of the next (zeroed once per step).
struct PubSlot {
  long long sum;              // sum_n x[n]   * 2^32   (x = the residual stream the launch wrote)
  long long sq;               // high limb of sum_n x[n]^2: units of 2^-8
  unsigned amax_bits;         // float bits of max_n |xs[n]|  (xs = next input, already times ry)
  unsigned pad;
  long long zp, sumxs, sumx;  // sum v*my * 2^32, sum xs * 2^40, sum v * 2^32
  long long sq_lo;            // low limb of sum_n x[n]^2: units of 2^-48
  long long reserved[9];
};
static_assert(sizeof(PubSlot) == 128, "PubSlot is one 128-byte line");

struct SegScalars {   // 32 bytes per segment, written by the prep kernel, read by every GEMV CTA
  float sd;           // fp32(1 / inv): value of one fixed-point unit
  float zp, sumxs, sumx;
  float pad[4];
};

enum PrepMode : int {
  PREP_PLAIN = 0,   // v_s = xin_s; statistics by block reduction
  PREP_LN = 1,      // v_s = mix(LayerNorm(ln_x), shift); mean/variance from pub->sum, pub->sq
  PREP_XS = 2,      // one segment; xin_0 already holds xs; max and sums from pub
};

struct PrepSeg {
  const float* ry;    // [K] per-input scale
  const float* my;    // [K] per-input offset
  const float* mix;   // [K] time-mix coefficient, or null (PREP_LN only)
  const float* xin;   // [K] input vector (PREP_PLAIN) or prepared xs (PREP_XS)
};

struct PrepParams {
  PrepSeg seg[kMaxSeg];
  int nseg, K;
  int mode;
  const float* ln_x;      // [K]
  const float* ln_w;
  const float* ln_b;
  const float* shift;     // [K] carried previous-token vector (the state row of modules/block.py:61-64)
  float* shift_out;       // [K] scratch that receives the layer-norm output = the next carry; the GEMV
                          // launch that follows copies it into the state row (may be null)
  int need_sums;          // also produce sum xs and sum v (only matrices with rx / mx / half need them)
  const PubSlot* pub;     // published statistics (PREP_LN, PREP_XS)
  unsigned char* planes;  // out: nseg * 4*K bytes
  SegScalars* scal;       // out: nseg entries
  unsigned long long* trace;  // optional: 4 stamps (entry, dependency resolved, statistics, done)
};

// y^2, exactly, as two integers added to hi (units of 2^-8) and lo (units of 2^-48): the rounded
// product p = fl(y*y) is split into rint(p * 2^8) and its remainder, and the rounding error of the
// product itself, e = fma(y, y, -p), goes to lo as well.  Every step is exact (power-of-two
// scalings; the remainder of a float against its rounding to an integer and the error of a product
// are floats), so sums of either limb are order-free and carry sum y^2 without any rounding for
// 2^-24 <= |y| < 2^27.
__device__ __forceinline__ void square_limbs(float y, long long& hi, long long& lo) {
  const float p = __fmul_rn(y, y);
  const float e = __fmaf_rn(y, y, -p);
  const float s = __fmul_rn(p, kPubSqHiScale);
  const float sh = rintf(s);
  hi += __float2ll_rn(sh);
  lo += __float2ll_rn(__fmul_rn(__fsub_rn(s, sh), kPubSqLoScale)) + __float2ll_rn(__fmul_rn(e, 281474976710656.0f));
}

// Mean and 1/sqrt(variance + 1e-5) of K values from their published sums.  var = E[x^2] - mean^2 is
// evaluated in fp64 on exact sums, so it does not cancel when |mean| is large against the spread
// (the reference centres first, modules/layernorm.py:11-20).  Multiplications only: fp64 division
// and square root are subroutines.
__device__ __forceinline__ void stats_from_sums(long long sum, long long sq_hi, long long sq_lo, int K, float& mean, float& rstd) {
  const double inv_k = double(1.0f / float(K)) * (2.0 - double(K) * double(1.0f / float(K)));   // one Newton step: 1/K to fp64 accuracy
  const double mu = double(sum) * (1.0 / 4294967296.0) * inv_k;
  const double q = double(sq_hi) * (1.0 / 256.0) + double(sq_lo) * (1.0 / 281474976710656.0);
  const double var = q * inv_k - mu * mu;
  mean = float(mu);
  rstd = 1.0f / sqrtf(fmaxf(float(var), 0.f) + 1e-5f);
}

// rint(v) for 0 <= v < 2^23 without the conversion pipe: the sum with 2^23 holds it in the mantissa.
__device__ __forceinline__ int rint_nonneg(float v) { return __float_as_int(__fadd_rn(v, 8388608.0f)) - 0x4B000000; }

// Digits of four inputs -> one word per plane, stored to the block layout.  X = a*65536 + b*256 + c
// with b, c in [-128,127]: the bytes of X + 0x8080 are (a, b+128, c+128), so flipping bit 7 of the
// two low bytes gives the signed digits.
__device__ __forceinline__ void store_digits(unsigned char* planes, int g, float4 xs, float inv) {
  const float v[4] = {xs.x, xs.y, xs.z, xs.w};
  uint32_t y[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int mag = rint_nonneg(__fmul_rn(fabsf(v[i]), inv));  // same value as cvt.rni of the fp32 product
    const int X = v[i] < 0.f ? -mag : mag;
    y[i] = uint32_t(X + 0x8080) ^ 0x8080u;
  }
  const uint32_t c01 = __byte_perm(y[0], y[1], 0x0040), c23 = __byte_perm(y[2], y[3], 0x0040);
  const uint32_t b01 = __byte_perm(y[0], y[1], 0x0051), b23 = __byte_perm(y[2], y[3], 0x0051);
  const uint32_t a01 = __byte_perm(y[0], y[1], 0x0062), a23 = __byte_perm(y[2], y[3], 0x0062);
  uint32_t* blk = reinterpret_cast<uint32_t*>(planes + size_t(g >> 3) * 128);
  const int j = g & 7;
  blk[j] = __byte_perm(a01, a23, 0x5410);
  blk[8 + j] = __byte_perm(b01, b23, 0x5410);
  blk[16 + j] = __byte_perm(c01, c23, 0x5410);
  blk[24 + j] = 0u;
}

// Block reduction of one segment's statistics (max|xs|, sum v*my, sum xs, sum v): warp partials ->
// shared memory -> every warp folds the 16 partials itself with shuffles (one barrier, no serial loop).
__device__ __forceinline__ void prep_reduce_stats(float& amax, float& szp, float& sxs, float& sx, float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  amax = warp_max(amax); szp = warp_sum(szp); sxs = warp_sum(sxs); sx = warp_sum(sx);
  if (lane == 0) reinterpret_cast<float4*>(red)[warp] = make_float4(amax, szp, sxs, sx);
  __syncthreads();
  static_assert(kPrepWarps == 16, "the fold below covers 16 warp partials");
  float4 t = reinterpret_cast<const float4*>(red)[lane & 15];
#pragma unroll
  for (int o = 8; o > 0; o >>= 1) {
    t.x = fmaxf(t.x, __shfl_xor_sync(0xffffffffu, t.x, o));
    t.y += __shfl_xor_sync(0xffffffffu, t.y, o);
    t.z += __shfl_xor_sync(0xffffffffu, t.z, o);
    t.w += __shfl_xor_sync(0xffffffffu, t.w, o);
  }
  amax = t.x; szp = t.y; sxs = t.z; sx = t.w;
}

// PREP_PLAIN and PREP_LN: CTA s prepares segment s (the segments share nothing but the layer norm,
// which every CTA evaluates for itself from the published sums).  GB = groups of four inputs a
// thread keeps in registers per batch.  xs is parked in shared memory (`stage`, 16 bytes per group)
// between the statistics pass and the digit pass.
template <int GB, bool LN>
__device__ __forceinline__ void prep_body(const PrepParams& P, unsigned char* stage, float* red) {
  const int tid = threadIdx.x;
  const int K = P.K, NG = K / 4;
  const int sidx = blockIdx.x;
  const PrepSeg& S = P.seg[sidx];
  const bool mixing = LN && S.mix != nullptr;

  // ---- parameter vectors of the first batch: loaded before the dependency wait
  float4 cw[LN ? GB : 1], cb[LN ? GB : 1], cmu[LN ? GB : 1], cry[GB], cmy[GB];
  auto load_consts = [&](int g0) {
#pragma unroll
    for (int i = 0; i < GB; ++i) {
      const int g = g0 + i * kPrepThreads;
      if (g < NG) {
        if (LN) {
          cw[i] = ld_param_v4(reinterpret_cast<const float4*>(P.ln_w) + g);
          cb[i] = ld_param_v4(reinterpret_cast<const float4*>(P.ln_b) + g);
          if (mixing) cmu[i] = ld_param_v4(reinterpret_cast<const float4*>(S.mix) + g);
        }
        cry[i] = ld_param_v4(reinterpret_cast<const float4*>(S.ry) + g);
        cmy[i] = ld_param_v4(reinterpret_cast<const float4*>(S.my) + g);
      }
    }
  };
  load_consts(tid);

  griddep_wait();  // everything below reads what earlier kernels wrote
  if (tid == 0 && P.trace && sidx == 0) P.trace[1] = globaltimer_ns();

  float mean = 0.f, rstd = 1.f;
  float amax = 0.f, szp = 0.f, sxs = 0.f, sx = 0.f;
  float4* park = reinterpret_cast<float4*>(stage);
  for (int g0 = tid, batch = 0; g0 < NG; g0 += GB * kPrepThreads, ++batch) {
    if (batch > 0) load_consts(g0);
    // activation loads of the batch go out together: one memory round trip
    float4 xv[GB], tc[LN ? GB : 1];
#pragma unroll
    for (int i = 0; i < GB; ++i) {
      const int g = g0 + i * kPrepThreads;
      if (g < NG) {
        if (LN) {
          xv[i] = ld_act_v4(reinterpret_cast<const float4*>(P.ln_x) + g);
          tc[i] = mixing && P.shift ? ld_act_v4(reinterpret_cast<const float4*>(P.shift) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
          xv[i] = ld_act_v4(reinterpret_cast<const float4*>(S.xin) + g);
        }
      }
    }
    if (LN && batch == 0) {
      // same round trip: the launch that wrote ln_x published its sum and sum of squares (exact
      // integer atomics); a handful of fp64 multiplications finish them
      stats_from_sums(__ldcg(&P.pub->sum), __ldcg(&P.pub->sq), __ldcg(&P.pub->sq_lo), K, mean, rstd);
      if (tid == 0 && P.trace && sidx == 0) P.trace[2] = globaltimer_ns();
    }
#pragma unroll
    for (int i = 0; i < GB; ++i) {
      const int g = g0 + i * kPrepThreads;
      if (g < NG) {
        float4 v = xv[i];
        if (LN) {
          const float4 x = xv[i];
          float4 xy;
          xy.x = cw[i].x * ((x.x - mean) * rstd) + cb[i].x;
          xy.y = cw[i].y * ((x.y - mean) * rstd) + cb[i].y;
          xy.z = cw[i].z * ((x.z - mean) * rstd) + cb[i].z;
          xy.w = cw[i].w * ((x.w - mean) * rstd) + cb[i].w;
          // the new carry cannot go to the state row in place (the other CTAs are reading it): CTA 0
          // parks it in shift_out and the GEMV launch that follows commits it
          if (sidx == 0 && P.shift_out) reinterpret_cast<float4*>(P.shift_out)[g] = xy;
          v = xy;
          if (mixing) {
            const float4 mu = cmu[i], t = tc[i];
            v.x = xy.x * mu.x + t.x * (1.f - mu.x);
            v.y = xy.y * mu.y + t.y * (1.f - mu.y);
            v.z = xy.z * mu.z + t.z * (1.f - mu.z);
            v.w = xy.w * mu.w + t.w * (1.f - mu.w);
          }
        }
        const float4 ry = cry[i], my = cmy[i];
        const float4 xs = make_float4(v.x * ry.x, v.y * ry.y, v.z * ry.z, v.w * ry.w);
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(xs.x), fabsf(xs.y)), fmaxf(fabsf(xs.z), fabsf(xs.w))));
        szp += (v.x * my.x + v.y * my.y) + (v.z * my.z + v.w * my.w);
        if (P.need_sums) {
          sxs += (xs.x + xs.y) + (xs.z + xs.w);
          sx += (v.x + v.y) + (v.z + v.w);
        }
        park[g] = xs;  // own slot, read back below
      }
    }
  }
  prep_reduce_stats(amax, szp, sxs, sx, red);

  // ---- digits, straight to global memory
  const float inv = amax > 0.f ? kQMax / amax : 0.f;
  if (tid == 0) {
    SegScalars sc;
    sc.sd = amax > 0.f ? __fdiv_rn(1.0f, inv) : 0.f;   // IEEE fp32 division, no fp64 on this path
    sc.zp = szp; sc.sumxs = sxs; sc.sumx = sx;
    sc.pad[0] = sc.pad[1] = sc.pad[2] = sc.pad[3] = 0.f;
    P.scal[sidx] = sc;
  }
  unsigned char* dst = P.planes + size_t(sidx) * 4 * K;
#pragma unroll 2
  for (int g = tid; g < NG; g += kPrepThreads) store_digits(dst, g, park[g], inv);
}

// PREP_XS: the previous epilogue already wrote xs and published max / sums; only digits remain, and
// they need no reduction, so the vector is cut into gridDim.x slices, one CTA (one free SM) each.
// The xs loads of the first batch and the loads of the published scalars go out together.
__device__ __forceinline__ void prep_xs(const PrepParams& P) {
  constexpr int GB = 8;
  const int tid = threadIdx.x;
  const int NG = P.K / 4;
  const int g_lo = int((long long)NG * blockIdx.x / gridDim.x), g_hi = int((long long)NG * (blockIdx.x + 1) / gridDim.x);
  griddep_wait();
  if (tid == 0 && P.trace && blockIdx.x == 0) P.trace[1] = globaltimer_ns();
  float4 xs[GB];
#pragma unroll
  for (int i = 0; i < GB; ++i) {
    const int g = g_lo + tid + i * kPrepThreads;
    if (g < g_hi) xs[i] = ld_act_v4(reinterpret_cast<const float4*>(P.seg[0].xin) + g);
  }
  const float amax = __uint_as_float(__ldcg(&P.pub->amax_bits));
  const float inv = amax > 0.f ? kQMax / amax : 0.f;
  if (tid == 0 && blockIdx.x == 0) {
    SegScalars sc;
    sc.sd = amax > 0.f ? __fdiv_rn(1.0f, inv) : 0.f;   // IEEE fp32 division, no fp64 on this path
    sc.zp = __ll2float_rn(__ldcg(&P.pub->zp)) * (1.0f / kPubSumScale);
    sc.sumxs = __ll2float_rn(__ldcg(&P.pub->sumxs)) * (1.0f / kPubXsScale);
    sc.sumx = __ll2float_rn(__ldcg(&P.pub->sumx)) * (1.0f / kPubSumScale);
    sc.pad[0] = sc.pad[1] = sc.pad[2] = sc.pad[3] = 0.f;
    P.scal[0] = sc;
    if (P.trace) P.trace[2] = globaltimer_ns();
  }
#pragma unroll
  for (int i = 0; i < GB; ++i) {
    const int g = g_lo + tid + i * kPrepThreads;
    if (g < g_hi) store_digits(P.planes, g, xs[i], inv);
  }
  for (int g = g_lo + tid + GB * kPrepThreads; g < g_hi; g += kPrepThreads)   // inputs beyond the first batch
    store_digits(P.planes, g, ld_act_v4(reinterpret_cast<const float4*>(P.seg[0].xin) + g), inv);
}

__global__ void __launch_bounds__(kPrepThreads, 1) vector_prep_kernel(const __grid_constant__ PrepParams P) {
  extern __shared__ __align__(128) unsigned char prep_smem[];
  float* red = reinterpret_cast<float*>(prep_smem);          // [16 warps + 1][4]
  unsigned char* stage = prep_smem + kPrepRedBytes;          // 4*K bytes: this CTA's fp32 xs
  if (threadIdx.x == 0 && P.trace && blockIdx.x == 0) P.trace[0] = globaltimer_ns();
  griddep_launch_dependents();
  if (P.mode == PREP_XS) prep_xs(P);
  else if (P.mode == PREP_LN) prep_body<4, true>(P, stage, red);
  else prep_body<8, false>(P, stage, red);
  if (threadIdx.x == 0 && P.trace && blockIdx.x == 0) P.trace[3] = globaltimer_ns();
}

inline size_t prep_smem_bytes(int K, int mode) { return size_t(kPrepRedBytes) + (mode == PREP_XS ? 0 : size_t(4) * K); }
inline int prep_grid(int nseg, int mode) { return mode == PREP_XS ? kMaxSeg : nseg; }   // one CTA per SM the GEMV grid leaves free

}  // namespace b200
