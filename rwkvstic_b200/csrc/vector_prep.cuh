// Activation preparation for the streaming GEMV: one CTA turns the raw activation vector(s) into
// the fixed-point digit planes and scalar terms that every GEMV CTA needs, ONCE, instead of every
// CTA recomputing them.  It runs on the SM the GEMV grid leaves free, so it can be resident while
// the previous GEMV still streams and load its parameter vectors before its dependency resolves.
//
// Per segment s (up to three matrices share one launch):
//   v_s[k]  = input of matrix s: either xin_s[k], or LayerNorm(ln_x)[k] mixed with the carried
//             previous-token vector (modules/block.py:58-67, :82-91; layernorm.py:11-20)
//   xs_s[k] = v_s[k] * ry_s[k];   inv_s = QMAX / max_k |xs_s[k]|;   X_s[k] = rint(xs_s[k] * inv_s)
//   planes  : signed base-256 digits of X_s, 128 bytes per 32 inputs: [a:32][b:32][c:32][0:32]
//   scalars : 1/inv_s (fp64), zp_s = sum_k v_s[k]*my_s[k], sum_k xs_s[k], sum_k v_s[k]
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kPrepThreads = 512;
constexpr int kPrepWarps = kPrepThreads / 32;
constexpr int kPrepRedBytes = (kPrepWarps + 1) * 16 * 4 + 64;  // reduction scratch, rounded to 128
constexpr int kMaxSeg = 3;
constexpr float kQMax = 8355000.0f;  // |X| <= QMAX keeps all three signed digits inside int8

struct SegScalars {   // 32 bytes per segment, written by the prep kernel, read by every GEMV CTA
  double sd;          // 1 / inv
  float zp, sumxs, sumx, pad;
};

struct PrepSeg {
  const float* ry;    // [K] per-input scale
  const float* my;    // [K] per-input offset
  const float* mix;   // [K] time-mix coefficient, or null (layer-norm mode only)
  const float* xin;   // [K] input vector (plain mode only)
};

struct PrepParams {
  PrepSeg seg[kMaxSeg];
  int nseg, K;
  int ln;                 // 1: layer norm (+ mix) of ln_x; 0: plain inputs
  const float* ln_x;      // [K]
  const float* ln_w;
  const float* ln_b;
  float* shift;           // [K] carried previous-token vector: read, then overwritten with the
                          // layer-norm output (the state row of modules/block.py:61-64); may be null
  unsigned char* planes;  // out: nseg * 4*K bytes
  SegScalars* scal;       // out: nseg entries
  unsigned long long* trace;  // optional: 4 stamps (entry, dependency resolved, statistics, done)
};

// Sum of `v` over the whole CTA, result in every thread.  Two barriers; `red` row layout [warp][16],
// column `col` is used for the partials and red[256 + col] for the total.
__device__ __forceinline__ float prep_block_sum(float v, float* red, int col) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  v = warp_sum(v);
  if (lane == 0) red[warp * 16 + col] = v;
  __syncthreads();
  if (warp == 0) {
    float a = lane < kPrepWarps ? red[lane * 16 + col] : 0.f;
    a = warp_sum(a);
    if (lane == 0) red[kPrepWarps * 16 + col] = a;
  }
  __syncthreads();
  return red[kPrepWarps * 16 + col];
}

// GB = groups of four inputs a thread keeps in registers per batch; NS = segments compiled in.
template <int GB, int NS, bool LN>
__device__ __forceinline__ void prep_body(const PrepParams& P, unsigned char* stage, float* red) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int K = P.K, NG = K / 4;

  // ---- parameter vectors of the first batch: loaded before the dependency wait
  float4 cw[LN ? GB : 1], cb[LN ? GB : 1], cmu[GB][NS], cry[GB][NS], cmy[GB][NS];
  auto load_consts = [&](int g0) {
#pragma unroll
    for (int i = 0; i < GB; ++i) {
      const int g = g0 + i * kPrepThreads;
      if (g < NG) {
        if (LN) {
          cw[i] = ld_param_v4(reinterpret_cast<const float4*>(P.ln_w) + g);
          cb[i] = ld_param_v4(reinterpret_cast<const float4*>(P.ln_b) + g);
        }
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          if (s < P.nseg) {
            cry[i][s] = ld_param_v4(reinterpret_cast<const float4*>(P.seg[s].ry) + g);
            cmy[i][s] = ld_param_v4(reinterpret_cast<const float4*>(P.seg[s].my) + g);
            if (LN && P.seg[s].mix) cmu[i][s] = ld_param_v4(reinterpret_cast<const float4*>(P.seg[s].mix) + g);
          }
        }
      }
    }
  };
  load_consts(tid);

  griddep_wait();  // everything below reads what earlier kernels wrote
  if (tid == 0 && P.trace) P.trace[1] = globaltimer_ns();

  // Activation loads of the first batch go out together, right after the dependency resolves:
  // one memory round trip on the critical path.
  float4 dep0[GB][LN ? 1 : NS];  // LN: carried previous-token vector; else the input vectors
  auto load_deps = [&](float4 (&dep)[GB][LN ? 1 : NS], int g0) {
#pragma unroll
    for (int i = 0; i < GB; ++i) {
      const int g = g0 + i * kPrepThreads;
      if (g < NG) {
        if (LN) {
          dep[i][0] = P.shift ? ld_act_v4(reinterpret_cast<const float4*>(P.shift) + g) : make_float4(0.f, 0.f, 0.f, 0.f);
        } else {
#pragma unroll
          for (int s = 0; s < NS; ++s)
            if (s < P.nseg) dep[i][s] = ld_act_v4(reinterpret_cast<const float4*>(P.seg[s].xin) + g);
        }
      }
    }
  };
  // Until the digits are written, group g keeps its fp32 values at byte 16*g of its segment's
  // staging region; segment 0's region first holds the raw ln_x.
  float4* tmp0 = reinterpret_cast<float4*>(stage);
  float mean = 0.f, sdev = 1.f;
  if (LN) {
    float sum = 0.f;
    {
      float4 xv[GB];
#pragma unroll
      for (int i = 0; i < GB; ++i) {
        const int g = tid + i * kPrepThreads;
        if (g < NG) xv[i] = ld_act_v4(reinterpret_cast<const float4*>(P.ln_x) + g);
      }
      load_deps(dep0, tid);
#pragma unroll
      for (int i = 0; i < GB; ++i) {
        const int g = tid + i * kPrepThreads;
        if (g < NG) { tmp0[g] = xv[i]; sum += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w); }
      }
    }
    for (int g = tid + GB * kPrepThreads; g < NG; g += kPrepThreads) {  // inputs beyond the first batch
      const float4 x = ld_act_v4(reinterpret_cast<const float4*>(P.ln_x) + g);
      tmp0[g] = x;
      sum += (x.x + x.y) + (x.z + x.w);
    }
    mean = prep_block_sum(sum, red, 0) / float(K);
    float m2 = 0.f;
    for (int g = tid; g < NG; g += kPrepThreads) {
      const float4 x = tmp0[g];
      const float a = x.x - mean, b = x.y - mean, c = x.z - mean, d = x.w - mean;
      m2 += (a * a + b * b) + (c * c + d * d);
    }
    sdev = sqrtf(prep_block_sum(m2, red, 1) / float(K) + 1e-5f);
  } else {
    load_deps(dep0, tid);
  }
  if (tid == 0 && P.trace) P.trace[2] = globaltimer_ns();

  // ---- xs per segment and its statistics
  const float rstd = 1.0f / sdev;
  float amax[NS], szp[NS], sxs[NS], sx[NS];
#pragma unroll
  for (int s = 0; s < NS; ++s) { amax[s] = 0.f; szp[s] = 0.f; sxs[s] = 0.f; sx[s] = 0.f; }
  for (int g0 = tid, batch = 0; g0 < NG; g0 += GB * kPrepThreads, ++batch) {
    float4 dep[GB][LN ? 1 : NS];
    if (batch > 0) {
      load_consts(g0);
      load_deps(dep, g0);
    } else {
#pragma unroll
      for (int i = 0; i < GB; ++i)
#pragma unroll
        for (int j = 0; j < (LN ? 1 : NS); ++j) dep[i][j] = dep0[i][j];
    }
#pragma unroll
    for (int i = 0; i < GB; ++i) {
      const int g = g0 + i * kPrepThreads;
      if (g < NG) {
        float4 xy = make_float4(0.f, 0.f, 0.f, 0.f);
        if (LN) {
          const float4 x = tmp0[g];
          xy.x = cw[i].x * ((x.x - mean) * rstd) + cb[i].x;
          xy.y = cw[i].y * ((x.y - mean) * rstd) + cb[i].y;
          xy.z = cw[i].z * ((x.z - mean) * rstd) + cb[i].z;
          xy.w = cw[i].w * ((x.w - mean) * rstd) + cb[i].w;
          if (P.shift) reinterpret_cast<float4*>(P.shift)[g] = xy;  // this thread read it just above
        }
#pragma unroll
        for (int s = 0; s < NS; ++s) {
          if (s < P.nseg) {
            float4 v;
            if (LN) {
              v = xy;
              if (P.seg[s].mix) {
                const float4 mu = cmu[i][s], tc = dep[i][0];
                v.x = xy.x * mu.x + tc.x * (1.f - mu.x);
                v.y = xy.y * mu.y + tc.y * (1.f - mu.y);
                v.z = xy.z * mu.z + tc.z * (1.f - mu.z);
                v.w = xy.w * mu.w + tc.w * (1.f - mu.w);
              }
            } else {
              v = dep[i][s];
            }
            const float4 ry = cry[i][s], my = cmy[i][s];
            const float4 xs = make_float4(v.x * ry.x, v.y * ry.y, v.z * ry.z, v.w * ry.w);
            amax[s] = fmaxf(amax[s], fmaxf(fmaxf(fabsf(xs.x), fabsf(xs.y)), fmaxf(fabsf(xs.z), fabsf(xs.w))));
            szp[s] += (v.x * my.x + v.y * my.y) + (v.z * my.z + v.w * my.w);
            sxs[s] += (xs.x + xs.y) + (xs.z + xs.w);
            sx[s] += (v.x + v.y) + (v.z + v.w);
            reinterpret_cast<float4*>(stage + size_t(s) * 4 * K)[g] = xs;  // own slot
          }
        }
      }
    }
  }
  // block reduction of the 4*nseg statistics: warp partials -> shared memory -> warp 0 folds the
  // 16 rows (one lane per statistic) -> everyone reads the totals.  Columns 2.. of the scratch rows.
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    amax[s] = warp_max(amax[s]); szp[s] = warp_sum(szp[s]); sxs[s] = warp_sum(sxs[s]); sx[s] = warp_sum(sx[s]);
    if (lane == 0) {
      red[warp * 16 + 2 + s] = amax[s]; red[warp * 16 + 5 + s] = szp[s];
      red[warp * 16 + 8 + s] = sxs[s];  red[warp * 16 + 11 + s] = sx[s];
    }
  }
  __syncthreads();
  if (warp == 0 && lane >= 2 && lane < 14) {
    float a = red[lane];
    for (int w = 1; w < kPrepWarps; ++w) a = lane < 5 ? fmaxf(a, red[w * 16 + lane]) : a + red[w * 16 + lane];
    red[kPrepWarps * 16 + lane] = a;
  }
  __syncthreads();
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    amax[s] = red[kPrepWarps * 16 + 2 + s]; szp[s] = red[kPrepWarps * 16 + 5 + s];
    sxs[s] = red[kPrepWarps * 16 + 8 + s];  sx[s] = red[kPrepWarps * 16 + 11 + s];
  }

  // ---- digits.  The eight groups of one 32-input block are owned by eight neighbouring lanes.
#pragma unroll
  for (int s = 0; s < NS; ++s) {
    if (s < P.nseg) {
      const float inv = amax[s] > 0.f ? kQMax / amax[s] : 0.f;
      if (tid == 0) {
        SegScalars sc;
        sc.sd = amax[s] > 0.f ? 1.0 / double(inv) : 0.0;
        sc.zp = szp[s]; sc.sumxs = sxs[s]; sc.sumx = sx[s]; sc.pad = 0.f;
        P.scal[s] = sc;
      }
      unsigned char* pl = stage + size_t(s) * 4 * K;
      for (int gb = tid - lane; gb < NG; gb += kPrepThreads) {
        const int g = gb + lane;
        const bool act = g < NG;
        float4 xs = make_float4(0.f, 0.f, 0.f, 0.f);
        if (act) xs = reinterpret_cast<const float4*>(pl)[g];
        __syncwarp();
        if (act) {
          const int X[4] = {__float2int_rn(xs.x * inv), __float2int_rn(xs.y * inv), __float2int_rn(xs.z * inv),
                            __float2int_rn(xs.w * inv)};
          uint32_t wa = 0u, wb = 0u, wc = 0u;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int x1 = (X[i] + 128) >> 8;   // X = x1*256 + c, c in [-128,127]
            const int x2 = (x1 + 128) >> 8;     // x1 = x2*256 + b
            wc |= (uint32_t(X[i]) & 0xffu) << (8 * i);
            wb |= (uint32_t(x1) & 0xffu) << (8 * i);
            wa |= (uint32_t(x2) & 0xffu) << (8 * i);
          }
          uint32_t* blk = reinterpret_cast<uint32_t*>(pl + size_t(g >> 3) * 128);
          const int j = g & 7;
          blk[j] = wa; blk[8 + j] = wb; blk[16 + j] = wc; blk[24 + j] = 0u;
        }
      }
    }
  }
  __syncthreads();
  // ---- staging -> global, 16 bytes per thread per step
  const int n16 = P.nseg * K / 4;
  for (int i = tid; i < n16; i += kPrepThreads)
    reinterpret_cast<uint4*>(P.planes)[i] = reinterpret_cast<const uint4*>(stage)[i];
}

__global__ void __launch_bounds__(kPrepThreads, 1) vector_prep_kernel(const __grid_constant__ PrepParams P) {
  extern __shared__ __align__(128) unsigned char prep_smem[];
  float* red = reinterpret_cast<float*>(prep_smem);          // [16 warps + 1][16]
  unsigned char* stage = prep_smem + kPrepRedBytes;          // nseg * 4*K bytes
  if (threadIdx.x == 0 && P.trace) P.trace[0] = globaltimer_ns();
  griddep_launch_dependents();
  // Three specialisations (registers per thread differ): layer norm + mix for up to three matrices;
  // one plain matrix (long K); up to three plain matrices.
  if (P.ln) prep_body<2, kMaxSeg, true>(P, stage, red);
  else if (P.nseg == 1) prep_body<8, 1, false>(P, stage, red);
  else prep_body<2, kMaxSeg, false>(P, stage, red);
  if (threadIdx.x == 0 && P.trace) P.trace[3] = globaltimer_ns();
}

inline size_t prep_smem_bytes(int K, int nseg) { return size_t(kPrepRedBytes) + size_t(nseg) * 4 * K; }

}  // namespace b200
