// Typical sampling on the device: one CTA per row of logits, no sort and no host round trip.
//
// What the reference's sampler computes on the host per token (samplers/typical.py:1-17):
//   p = softmax(logits); nl = -log p; ent = sum(nl * p) (NaN terms skipped); s = |nl - ent|;
//   sort by s, running sum of p in that order, cutoff = number of running sums < tau;
//   every p whose s is larger than the s at the cutoff position becomes 0; p <- p^(1/temp);
//   one draw from the resulting (unnormalised) distribution.
// The sort only serves to find one threshold: the smallest value t among the s_i for which the
// mass of {i : s_i <= t} reaches tau.  Here that threshold is found by a radix select over the
// bit pattern of s (s >= 0, so float order is unsigned-integer order) weighted by p: four passes
// of 256-bin mass histograms, each fixing one byte of t.  Masses are fixed point (p * 2^31 rounded to
// nearest, 32-bit shared-memory atomics, which are native; 64-bit totals): integer sums do not
// depend on arrival order, so every pass and every run sees the same totals, and the rounding
// (2.3e-10 per token) stays below what the reference's fp32 running sum resolves.  The draw
// is an inverse-CDF walk in index order with a uniform number the caller supplies, so a run is
// reproducible from its seed.
// The row (V floats, 200 KB at V = 50277) stays in L2; every pass recomputes p and s from the
// logits with the same instructions, so all passes see identical values.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kSampleThreads = 1024;
constexpr int kSampleHists = 16;   // mass histograms per CTA: lane l adds into histogram l % 16, so the
                                   // lanes of a warp that meet in one bin hit 16 addresses in 16 banks
constexpr int kSampleHistStride = 257;   // odd stride: equal bins of different histograms in different banks
constexpr float kMassScale = 2147483648.0f;   // 2^31

struct TypicalRow {
  float mx;       // largest logit
  float inv_z;    // 1 / sum exp(l - mx)
  float log_z;    // log of that sum
  float ent;      // entropy in nats
};

// The surprise -log p of a logit is log_z - (l - mx): one subtraction instead of a logarithm of an
// exponential (and exact where the reference's fp32 -log(softmax) carries the rounding of p).
__device__ __forceinline__ float typical_shift(float l, const TypicalRow& r) {
  return fabsf((r.log_z - (l - r.mx)) - r.ent);
}
__device__ __forceinline__ float typical_prob(float l, const TypicalRow& r) {
  return expf(l - r.mx) * r.inv_z;
}
// p and s of one logit; identical code in every pass.
__device__ __forceinline__ void typical_eval(float l, const TypicalRow& r, float& p, float& s) {
  p = typical_prob(l, r);
  s = typical_shift(l, r);
}

// The passes are bound by load latency (one CTA, a row that does not fit L1), so every loop
// fetches eight logits before it touches the first: f(index, logit) in increasing index order.
template <typename F>
__device__ __forceinline__ void for_each_strided(const float* __restrict__ row, int n, F&& f) {
  for (int base = threadIdx.x; base < n; base += 8 * kSampleThreads) {
    float l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = base + j * kSampleThreads;
      l[j] = i < n ? __ldg(row + i) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = base + j * kSampleThreads;
      if (i < n) f(i, l[j]);
    }
  }
}
template <typename F>
__device__ __forceinline__ void for_each_in_range(const float* __restrict__ row, int i0, int i1, F&& f) {
  for (int base = i0; base < i1; base += 8) {
    float l[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) l[j] = base + j < i1 ? __ldg(row + base + j) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
      if (base + j < i1) f(base + j, l[j]);
  }
}

__device__ __forceinline__ double block_sum_f64(double v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();                      // red may still be read from an earlier call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < kSampleThreads / 32; ++w) t += red[w];   // same order in every thread
  return t;
}

__device__ __forceinline__ float block_max_f32(float v, double* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  __syncthreads();
  if (lane == 0) red[warp] = double(v);
  __syncthreads();
  double t = red[0];
  for (int w = 1; w < kSampleThreads / 32; ++w) t = fmax(t, red[w]);
  return float(t);
}

// logits [rows][ldx]; u: one uniform number in [0,1) per draw, read at u[row + rows * step] where
// step = *history_count when a history is kept and 0 otherwise; out[row] = sampled id;
// probs_out (nullable) [rows][n]: the masked, tempered, unnormalised probabilities the draw used.
__global__ void __launch_bounds__(kSampleThreads)
sample_typical_kernel(const float* __restrict__ x, int n, long long ldx, float temp, float tau,
                      const float* __restrict__ u, long long* __restrict__ out, float* __restrict__ probs_out,
                      long long* __restrict__ hist, int* __restrict__ hist_count, int hist_cap) {
  __shared__ double red[kSampleThreads / 32];
  __shared__ unsigned int mass[kSampleHists][kSampleHistStride];
  __shared__ unsigned long long tot[256];
  __shared__ double part[kSampleThreads];
  __shared__ unsigned int sh_prefix;
  __shared__ unsigned long long sh_below;
  __shared__ int sh_keep_all, sh_chunk;
  __shared__ double sh_target, sh_before;

  const int tid = threadIdx.x, warp = tid >> 5;
  const int row_id = blockIdx.x;
  const float* row = x + size_t(row_id) * ldx;

  // ---- softmax statistics and entropy
  float mx = -INFINITY;
  for_each_strided(row, n, [&](int, float l) { mx = fmaxf(mx, l); });
  TypicalRow r;
  r.mx = block_max_f32(mx, red);
  // one pass for both sums: Z = sum e^d and sum d e^d (d = l - mx), entropy = log Z - (sum d e^d) / Z
  double z = 0.0, dz = 0.0;
  for_each_strided(row, n, [&](int, float l) {
    const float d = l - r.mx;
    const float e = expf(d);
    z += double(e);
    if (e > 0.f) dz += double(d * e);
  });
  z = block_sum_f64(z, red);
  dz = block_sum_f64(dz, red);
  r.inv_z = float(1.0 / z);
  r.log_z = float(log(z));
  r.ent = float(log(z) - dz / z);

  // ---- threshold: smallest s whose cumulative mass (in order of s) reaches tau
  if (tid == 0) { sh_prefix = 0u; sh_below = 0ull; sh_keep_all = 0; }
  const unsigned long long tau_fixed = __double2ull_ru(double(tau) * double(kMassScale));
  unsigned int known = 0u;                       // mask of the bits of the threshold fixed so far
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < kSampleHists * kSampleHistStride; i += kSampleThreads) (&mass[0][0])[i] = 0u;
    __syncthreads();
    const unsigned int prefix = sh_prefix;
    if (!sh_keep_all) {
      unsigned int* h = mass[tid & (kSampleHists - 1)];
      for_each_strided(row, n, [&](int, float l) {
        const unsigned int key = __float_as_uint(typical_shift(l, r));
        if ((key & known) == prefix) {           // the exponential only for logits still in the running
          const float p = typical_prob(l, r);
          if (p > 0.f) atomicAdd(&h[(key >> shift) & 255u], __float2uint_rn(p * kMassScale));
        }
      });
    }
    __syncthreads();
    if (tid < 256) {
      unsigned long long t = 0ull;
      for (int k = 0; k < kSampleHists; ++k) t += mass[k][tid];
      tot[tid] = t;
    }
    __syncthreads();
    if (warp == 0) {
      // lane l owns bins [8 l, 8 l + 8): running totals across the lanes, then inside one lane
      const int lane = tid;
      const int keep_all_now = sh_keep_all;
      const unsigned long long below = sh_below;
      unsigned long long loc[8], sum = 0ull;
#pragma unroll
      for (int k = 0; k < 8; ++k) { loc[k] = tot[lane * 8 + k]; sum += loc[k]; }
      unsigned long long inc = sum;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
      }
      const unsigned long long before = below + inc - sum;
      const unsigned hit = __ballot_sync(0xffffffffu, before + sum >= tau_fixed);
      if (!keep_all_now) {
        if (hit == 0u) {
          if (lane == 0) sh_keep_all = 1;        // the whole row has less mass than tau: nothing is cut
        } else if (lane == __ffs(hit) - 1) {
          unsigned long long run = before;
          int b = -1;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (b < 0) {
              if (run + loc[k] >= tau_fixed) b = k;
              else run += loc[k];
            }
          }
          sh_prefix = prefix | (unsigned(lane * 8 + b) << shift);
          sh_below = run;
        }
      }
    }
    known |= 255u << shift;
    __syncthreads();
  }
  const bool keep_all = sh_keep_all != 0;
  const float thresh = __uint_as_float(sh_prefix);

  // ---- the draw: inverse CDF over q_i = keep_i ? p_i^(1/temp) : 0 in index order
  const float inv_temp = 1.0f / temp;
  const bool tempered = temp != 1.0f;
  const int chunk = (n + kSampleThreads - 1) / kSampleThreads;
  const int i0 = tid * chunk, i1 = min(n, i0 + chunk);
  double mine = 0.0;
  for_each_in_range(row, i0, i1, [&](int i, float l) {
    float p, s;
    typical_eval(l, r, p, s);
    float q = (keep_all || s <= thresh) ? p : 0.f;
    if (tempered && q > 0.f) q = powf(q, inv_temp);
    if (probs_out) probs_out[size_t(row_id) * n + i] = q;
    mine += double(q);
  });
  part[tid] = mine;
  __syncthreads();
  if (warp == 0) {
    // lane l owns the partial sums of chunks [32 l, 32 l + 32): scan across lanes, then inside one lane
    const int lane = tid;
    double loc = 0.0;
    for (int k = 0; k < 32; ++k) loc += part[lane * 32 + k];
    double inc = loc;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const double t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    const double total = __shfl_sync(0xffffffffu, inc, 31);
    // u holds rows * history_capacity numbers when a history is kept: replays beyond the capacity reuse the last one
    int step = (hist && hist_count) ? *hist_count : 0;
    if (step >= hist_cap && hist_cap > 0) step = hist_cap - 1;
    const double target = double(u[row_id + size_t(gridDim.x) * step]) * total;
    const unsigned hit = __ballot_sync(0xffffffffu, loc > 0.0 && inc >= target);
    const unsigned nonzero = __ballot_sync(0xffffffffu, loc > 0.0);
    // rounding can leave the target past the end: then the last lane that holds any mass
    const int owner = hit ? __ffs(hit) - 1 : (nonzero ? 31 - __clz(nonzero) : 0);
    if (lane == owner) {
      double run = inc - loc;
      int c = -1, last = -1;
      for (int k = 0; k < 32; ++k) {
        const double v = part[lane * 32 + k];
        if (v > 0.0) {
          last = lane * 32 + k;
          if (run + v >= target) { c = last; break; }
        }
        run += v;
      }
      if (c < 0) {
        c = last < 0 ? lane * 32 : last;
        run = inc - loc;
        for (int k = lane * 32; k < c; ++k) run += part[k];
      }
      sh_chunk = c; sh_target = target; sh_before = run;
    }
  }
  __syncthreads();
  if (tid == sh_chunk) {
    double run = sh_before;
    long long pick = -1, last = -1;
    for_each_in_range(row, i0, i1, [&](int i, float l) {
      if (pick >= 0) return;
      float p, s;
      typical_eval(l, r, p, s);
      float q = (keep_all || s <= thresh) ? p : 0.f;
      if (tempered && q > 0.f) q = powf(q, inv_temp);
      if (q > 0.f) {
        last = i;
        run += double(q);
        if (run >= sh_target) pick = i;
      }
    });
    if (pick < 0) pick = last < 0 ? i0 : last;
    out[row_id] = pick;
    if (hist && hist_count && row_id == 0) {
      const int cnt = *hist_count;
      if (cnt < hist_cap) hist[cnt] = pick;
      *hist_count = cnt + 1;
    }
  }
}

}  // namespace b200
