// Streaming uint8 GEMV for sm_100a: the decode-time (one token) matrix-vector kernel.
//
// Data layout in HBM: every matrix is output-major bytes qt[N][K]; the rows a CTA owns are one
// contiguous byte range.  One launch covers up to three matrices ("segments") with the same K.
//
// Work split: CTA c owns rows [N*c/G, N*(c+1)/G) of every segment and reads each of its bytes
// exactly once.  A producer lane streams that range through a ring of shared-memory stages with
// 1-D TMA bulk copies (cp.async.bulk + mbarrier complete_tx); 16 consumer warps eat the stages.
//
// Arithmetic: the activation vector xs[k] = x[k]*ry[k] is turned, per segment, into 24-bit fixed
// point X[k] = rint(xs[k]*inv), inv = QMAX/max|xs|, split into three byte planes (X = a*65536 +
// b*256 + c, a signed).  The dot product with the uint8 weights is then pure integer work:
// three dp4a per four weight bytes, exact int64 row sums, exact (order-independent) reduction
// across lanes, warps and shared-memory atomics.  y = I/inv carries only the input rounding
// (2^-24 of the largest |xs|), comparable to fp32 accumulation but bit-reproducible for any
// partitioning.
//
// Fusion: the prologue builds xs from the raw activations (optionally layer norm + token-shift
// mix, the reference's modules/block.py:58-67 and :82-91), the epilogue applies the affine
// correction terms and the activation / gate / residual / WKV-state update that follows the
// matrix in modules/block.py:72-100, so a decode step is 4 launches per layer.
#pragma once

#include "common.cuh"

namespace b200 {

constexpr int kConsumers = 512;                 // consumer threads (16 warps)
constexpr int kGemvThreads = kConsumers + 32;   // + one producer warp
constexpr int kMaxSeg = 3;
constexpr int kMaxStages = 8;
constexpr int kStageTarget = 32 * 1024;         // preferred bytes per ring stage
constexpr int kStageLimit = 40 * 1024;          // hard upper bound per stage
constexpr int kSmemLimit = 227 * 1024;          // dynamic shared memory per CTA on sm_100
constexpr float kQMax = 8388352.0f;             // 2^23 - 256: |X| stays inside 24-bit signed after rounding

enum Act : int { ACT_NONE = 0, ACT_RELUSQ = 1, ACT_SIGMOID = 2 };
enum Prologue : int { PRO_VEC = 0, PRO_LNMIX = 1 };
enum Epilogue : int { EPI_GENERIC = 0, EPI_WKV = 1 };

struct GemvSeg {
  const uint8_t* qt;   // [N][K]
  const float* ry;     // [K]
  const float* my;     // [K]
  const float* rx;     // [N] or null
  const float* mx;     // [N] or null
  const float* xin;    // PRO_VEC: input vector [K]
  const float* mix;    // PRO_LNMIX: time-mix vector [K] or null (no mix: input = layer-norm output)
  float* out;          // EPI_GENERIC: destination [N]
  const float* res;    // EPI_GENERIC: residual added to the output, or null
  const float* gate;   // EPI_GENERIC: multiplies act(y), or null
  float half;
  int N;
  int act;
};

struct GemvParams {
  GemvSeg seg[kMaxSeg];
  int nseg, K;
  // geometry (derived from K on the host, see plan_gemv)
  int tpr;          // threads that share one row (multiple of 32)
  int rl;           // rows processed side by side = kConsumers / tpr
  int m, log_m;     // rows per thread per stage (power of two <= 8)
  int stages;       // ring depth
  int stage_bytes;  // ring slot size >= rl*m*K
  int rpc;          // max rows per CTA per segment
  // prologue
  int pro;
  const float* ln_x;       // PRO_LNMIX: vector to normalise [K]
  const float* ln_w;
  const float* ln_b;
  const float* shift_in;   // carried previous-token vector [K] (null when no segment mixes)
  float* shift_out;        // CTA 0 stores the layer-norm output here [K] (may be null)
  // deferred state commit done by CTA 0 after the dependency wait: dst[0..n) = src[0..n)
  const float* commit_src;
  float* commit_dst;
  int commit_n;
  // epilogue
  int epi;
  int accumulate;          // EPI_GENERIC: out += result instead of out = result
  const float* wkv_w;      // EPI_WKV: decay w = -exp(time_decay) [N]
  const float* wkv_u;      // time_first [N]
  float* aa;               // state rows, updated in place [N]
  float* bb;
  float* pp;
  float* wkv_out;          // sigmoid(r) * wkv [N]
  int* status;             // device status word or null
};

// Shared-memory map (byte offsets)
constexpr int kOffFull = 0;        // 8 x u64
constexpr int kOffEmpty = 64;      // 8 x u64
constexpr int kOffAbort = 128;     // int
constexpr int kOffRed = 256;       // float[16][16] block-reduction scratch
constexpr int kOffFinal = 1280;    // float[16] reduced values
constexpr int kOffScale = 1344;    // double sd[3]; float zp[3], sumxs[3], sumx[3]
constexpr int kOffRows = 1536;     // int64 rowsum[nseg*rpc], then planes, then ring

struct GemvPlan {
  int kch, tpr, rl, m, log_m, stages, stage_bytes, rpc, grid;
  size_t smem;
};

// Choose the thread geometry for a reduction length K.  Returns false when K is unsupported.
inline bool plan_gemv(int K, int nseg, int max_n, int num_sms, GemvPlan* p) {
  if (K <= 0 || (K % 16) != 0 || nseg < 1 || nseg > kMaxSeg || max_n <= 0) return false;
  const int cpr = K / 16;  // 16-byte chunks per row
  int best_kch = 0, best_tpr = 0, best_rl = 0;
  double best_util = -1.0;
  for (int kch = 1; kch <= 4; ++kch) {
    int tpr = ((cpr + kch - 1) / kch + 31) / 32 * 32;
    if (tpr > kConsumers) continue;
    int rl = kConsumers / tpr;
    double util = double(cpr) * rl / (double(kch) * kConsumers);
    if (util >= best_util - 1e-9) {  // ties go to the larger kch (fewer cross-lane reductions per byte)
      best_util = util; best_kch = kch; best_tpr = tpr; best_rl = rl;
    }
  }
  if (best_kch == 0) return false;
  if ((long long)best_rl * K > kStageLimit) return false;
  int m = 8;
  while (m > 1 && (long long)best_rl * m * K > kStageTarget) m >>= 1;
  int log_m = 0;
  while ((1 << log_m) < m) ++log_m;
  p->kch = best_kch; p->tpr = best_tpr; p->rl = best_rl; p->m = m; p->log_m = log_m;
  p->stage_bytes = (best_rl * m * K + 127) / 128 * 128;
  p->grid = num_sms < max_n ? num_sms : max_n;
  p->rpc = (max_n + p->grid - 1) / p->grid;
  size_t fixed = kOffRows + (size_t(nseg) * p->rpc * 8 + 127) / 128 * 128 + size_t(nseg) * 4 * K;
  fixed = (fixed + 127) / 128 * 128;
  if (fixed + 2 * size_t(p->stage_bytes) > size_t(kSmemLimit)) return false;
  int stages = int((size_t(kSmemLimit) - fixed) / p->stage_bytes);
  if (stages > kMaxStages) stages = kMaxStages;
  p->stages = stages;
  p->smem = fixed + size_t(stages) * p->stage_bytes;
  return true;
}

// Sum of up to NV values per thread over the 512 consumer threads; result broadcast to all.
// is_max[i] selects max instead of sum.  Uses named barrier 1.
template <int NV>
__device__ __forceinline__ void consumer_reduce(float (&v)[NV], unsigned max_mask, float* red, float* fin, int tid) {
  const int warp = tid >> 5, lane = tid & 31;
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = ((max_mask >> i) & 1u) ? warp_max(v[i]) : warp_sum(v[i]);
  if (lane == 0) {
#pragma unroll
    for (int i = 0; i < NV; ++i) red[warp * 16 + i] = v[i];
  }
  named_bar_sync(1, kConsumers);
  if (tid < NV) {
    float a = red[tid];
    const bool mx = (max_mask >> tid) & 1u;
    for (int w = 1; w < kConsumers / 32; ++w) a = mx ? fmaxf(a, red[w * 16 + tid]) : a + red[w * 16 + tid];
    fin[tid] = a;
  }
  named_bar_sync(1, kConsumers);
#pragma unroll
  for (int i = 0; i < NV; ++i) v[i] = fin[i];
  named_bar_sync(1, kConsumers);  // fin/red may be reused by the next call
}

template <int KCH>
__global__ void __launch_bounds__(kGemvThreads, 1) stream_gemv_kernel(const __grid_constant__ GemvParams P) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31;
  const int G = gridDim.x, cta = blockIdx.x;
  const int K = P.K;
  const int RS = P.rl * P.m;  // rows per full stage

  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + kOffAbort);
  volatile int* issued_ptr = reinterpret_cast<volatile int*>(smem + kOffAbort + 4);  // stages the producer issued
  float* red = reinterpret_cast<float*>(smem + kOffRed);
  float* fin = reinterpret_cast<float*>(smem + kOffFinal);
  double* sd = reinterpret_cast<double*>(smem + kOffScale);
  float* zp_s = reinterpret_cast<float*>(smem + kOffScale + 32);
  float* sumxs_s = zp_s + 4;
  float* sumx_s = zp_s + 8;
  unsigned long long* rowsum = reinterpret_cast<unsigned long long*>(smem + kOffRows);
  const size_t rows_bytes = (size_t(P.nseg) * P.rpc * 8 + 127) / 128 * 128;
  unsigned char* planes = smem + kOffRows + rows_bytes;  // per segment 4*K bytes: uint4 per 4 inputs
  const size_t ring_off = (kOffRows + rows_bytes + size_t(P.nseg) * 4 * K + 127) / 128 * 128;
  unsigned char* ring = smem + ring_off;
  const uint32_t full0 = smem_u32(smem + kOffFull), empty0 = smem_u32(smem + kOffEmpty);

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
  const int active_warps = P.rl * P.tpr / 32;

  if (tid == 0) {
    for (int i = 0; i < kMaxStages; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, active_warps);
    }
    *abort_flag = 0;
    *issued_ptr = 0;
    fence_mbar_init();
  }
  __syncthreads();
  griddep_launch_dependents();

  if (warp == kConsumers / 32) {
    // ------------------------------------------------------------------ producer: weights only,
    // which no earlier kernel writes, so it does not wait on the launch dependency.
    if (lane == 0) {
      int slot = 0, issued = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int s = 0; s < P.nseg && ok; ++s) {
        const uint8_t* base = P.seg[s].qt + size_t(r0[s]) * K;
        for (int row = 0; row < nr[s]; row += RS) {
          const int rows = nr[s] - row < RS ? nr[s] - row : RS;
          if (!mbar_wait_bounded(empty0 + 8 * slot, phase ^ 1u, abort_flag)) {
            if (P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_EMPTY);
            ok = false;
            break;
          }
          const uint32_t bytes = uint32_t(rows) * uint32_t(K);
          mbar_arrive_expect_tx(full0 + 8 * slot, bytes);
          bulk_g2s(smem_u32(ring + size_t(slot) * P.stage_bytes), base + size_t(row) * K, bytes, full0 + 8 * slot);
          ++issued;
          if (++slot == P.stages) { slot = 0; phase ^= 1u; }
        }
      }
      *issued_ptr = issued;
    }
  } else {
    // ------------------------------------------------------------------ consumers
    const int NG = K / 4;  // groups of four inputs
    for (int i = tid; i < P.nseg * P.rpc; i += kConsumers) rowsum[i] = 0ull;

    griddep_wait();  // everything below reads what earlier kernels wrote

    if (cta == 0 && P.commit_n > 0) {
      for (int i = tid; i < P.commit_n; i += kConsumers) P.commit_dst[i] = P.commit_src[i];
    }

    // ---- prologue: xs per segment -> fixed-point planes in shared memory
    float mean = 0.f, sdev = 1.f;
    if (P.pro == PRO_LNMIX) {
      float v1[1] = {0.f};
      for (int g = tid; g < NG; g += kConsumers) {
        const float4 x = reinterpret_cast<const float4*>(P.ln_x)[g];
        v1[0] += (x.x + x.y) + (x.z + x.w);
      }
      consumer_reduce<1>(v1, 0u, red, fin, tid);
      mean = v1[0] / float(K);
      v1[0] = 0.f;
      for (int g = tid; g < NG; g += kConsumers) {
        const float4 x = reinterpret_cast<const float4*>(P.ln_x)[g];
        const float a = x.x - mean, b = x.y - mean, c = x.z - mean, d = x.w - mean;
        v1[0] += (a * a + b * b) + (c * c + d * d);
      }
      consumer_reduce<1>(v1, 0u, red, fin, tid);
      sdev = sqrtf(v1[0] / float(K) + 1e-5f);
    }
    // stats: [0..2] max|xs|, [3..5] sum x*my, [6..8] sum xs, [9..11] sum x
    float st[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) st[i] = 0.f;
    for (int g = tid; g < NG; g += kConsumers) {
      float4 xy = make_float4(0.f, 0.f, 0.f, 0.f), tc = xy;
      if (P.pro == PRO_LNMIX) {
        const float4 x = reinterpret_cast<const float4*>(P.ln_x)[g];
        const float4 w = reinterpret_cast<const float4*>(P.ln_w)[g];
        const float4 b = reinterpret_cast<const float4*>(P.ln_b)[g];
        xy.x = w.x * ((x.x - mean) / sdev) + b.x;
        xy.y = w.y * ((x.y - mean) / sdev) + b.y;
        xy.z = w.z * ((x.z - mean) / sdev) + b.z;
        xy.w = w.w * ((x.w - mean) / sdev) + b.w;
        if (P.shift_in) tc = reinterpret_cast<const float4*>(P.shift_in)[g];
        if (cta == 0 && P.shift_out) reinterpret_cast<float4*>(P.shift_out)[g] = xy;
      }
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) {
        if (s < P.nseg) {
          float4 v;
          if (P.pro == PRO_LNMIX) {
            v = xy;
            if (P.seg[s].mix) {
              const float4 mu = reinterpret_cast<const float4*>(P.seg[s].mix)[g];
              v.x = xy.x * mu.x + tc.x * (1.f - mu.x);
              v.y = xy.y * mu.y + tc.y * (1.f - mu.y);
              v.z = xy.z * mu.z + tc.z * (1.f - mu.z);
              v.w = xy.w * mu.w + tc.w * (1.f - mu.w);
            }
          } else {
            v = reinterpret_cast<const float4*>(P.seg[s].xin)[g];
          }
          const float4 ry = reinterpret_cast<const float4*>(P.seg[s].ry)[g];
          const float4 my = reinterpret_cast<const float4*>(P.seg[s].my)[g];
          const float4 xs = make_float4(v.x * ry.x, v.y * ry.y, v.z * ry.z, v.w * ry.w);
          st[s] = fmaxf(st[s], fmaxf(fmaxf(fabsf(xs.x), fabsf(xs.y)), fmaxf(fabsf(xs.z), fabsf(xs.w))));
          st[3 + s] += (v.x * my.x + v.y * my.y) + (v.z * my.z + v.w * my.w);
          st[6 + s] += (xs.x + xs.y) + (xs.z + xs.w);
          st[9 + s] += (v.x + v.y) + (v.z + v.w);
          reinterpret_cast<float4*>(planes + size_t(s) * 4 * K)[g] = xs;  // own slot, quantised in place below
        }
      }
    }
    consumer_reduce<12>(st, 0x7u, red, fin, tid);
#pragma unroll
    for (int s = 0; s < kMaxSeg; ++s) {
      if (s < P.nseg) {
        const float amax = st[s];
        const float inv = amax > 0.f ? kQMax / amax : 0.f;
        if (tid == 0) {
          sd[s] = amax > 0.f ? 1.0 / double(inv) : 0.0;
          zp_s[s] = st[3 + s];
          sumxs_s[s] = st[6 + s];
          sumx_s[s] = st[9 + s];
        }
        uint4* pl = reinterpret_cast<uint4*>(planes + size_t(s) * 4 * K);
        for (int g = tid; g < NG; g += kConsumers) {
          const float4 xs = reinterpret_cast<const float4*>(pl)[g];
          const int X0 = __float2int_rn(xs.x * inv), X1 = __float2int_rn(xs.y * inv);
          const int X2 = __float2int_rn(xs.z * inv), X3 = __float2int_rn(xs.w * inv);
          uint4 o;
          o.x = (uint32_t(X0 >> 16) & 0xffu) | ((uint32_t(X1 >> 16) & 0xffu) << 8) | ((uint32_t(X2 >> 16) & 0xffu) << 16) |
                ((uint32_t(X3 >> 16) & 0xffu) << 24);
          o.y = (uint32_t(X0 >> 8) & 0xffu) | ((uint32_t(X1 >> 8) & 0xffu) << 8) | ((uint32_t(X2 >> 8) & 0xffu) << 16) |
                ((uint32_t(X3 >> 8) & 0xffu) << 24);
          o.z = (uint32_t(X0) & 0xffu) | ((uint32_t(X1) & 0xffu) << 8) | ((uint32_t(X2) & 0xffu) << 16) |
                ((uint32_t(X3) & 0xffu) << 24);
          o.w = 0u;
          pl[g] = o;
        }
      }
    }
    named_bar_sync(1, kConsumers);

    // ---- main loop: integer dot products over the streamed rows
    if (warp < active_warps) {
      const int cl = tid % P.tpr, rl = tid / P.tpr;
      const int cpr = K / 16;
      const int M = P.m, logM = P.log_m;
      int slot = 0;
      uint32_t phase = 0;
      bool dead = false;
      for (int s = 0; s < P.nseg && !dead; ++s) {
        const int nrows = nr[s];
        const int nst = (nrows + RS - 1) / RS;
        uint32_t xa[KCH][4], xb[KCH][4], xc[KCH][4];
        const uint4* pl = reinterpret_cast<const uint4*>(planes + size_t(s) * 4 * K);
#pragma unroll
        for (int i = 0; i < KCH; ++i) {
          const int c = cl + P.tpr * i;
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            uint4 t = make_uint4(0u, 0u, 0u, 0u);
            if (c < cpr) t = pl[c * 4 + w];
            xa[i][w] = t.x; xb[i][w] = t.y; xc[i][w] = t.z;
          }
        }
        for (int stb = 0; stb < nst && !dead; stb += (8 >> logM)) {
          int A[8];
          uint32_t B[8], C[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) { A[u] = 0; B[u] = 0u; C[u] = 0u; }
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int sidx = stb + (u >> logM);
            const int rin = u & (M - 1);
            const bool sv = (sidx < nst) && !dead;
            if (sv && rin == 0) {
              const bool ok = mbar_wait_bounded(full0 + 8 * slot, phase, abort_flag);
              if (!__all_sync(0xffffffffu, ok)) {
                dead = true;
                if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
              }
            }
            const int lrow = sidx * RS + rin * P.rl + rl;
            if (sv && !dead && lrow < nrows) {
              const unsigned char* p = ring + size_t(slot) * P.stage_bytes + size_t(rin * P.rl + rl) * K + cl * 16;
#pragma unroll
              for (int i = 0; i < KCH; ++i) {
                if (cl + P.tpr * i < cpr) {
                  const uint4 w = *reinterpret_cast<const uint4*>(p + size_t(i) * P.tpr * 16);
                  A[u] = dp4a_us(w.x, xa[i][0], A[u]); B[u] = dp4a_uu(w.x, xb[i][0], B[u]); C[u] = dp4a_uu(w.x, xc[i][0], C[u]);
                  A[u] = dp4a_us(w.y, xa[i][1], A[u]); B[u] = dp4a_uu(w.y, xb[i][1], B[u]); C[u] = dp4a_uu(w.y, xc[i][1], C[u]);
                  A[u] = dp4a_us(w.z, xa[i][2], A[u]); B[u] = dp4a_uu(w.z, xb[i][2], B[u]); C[u] = dp4a_uu(w.z, xc[i][2], C[u]);
                  A[u] = dp4a_us(w.w, xa[i][3], A[u]); B[u] = dp4a_uu(w.w, xb[i][3], B[u]); C[u] = dp4a_uu(w.w, xc[i][3], C[u]);
                }
              }
            }
            if (sv && !dead && rin == M - 1) {
              __syncwarp();
              if (lane == 0) mbar_arrive(empty0 + 8 * slot);
              if (++slot == P.stages) { slot = 0; phase ^= 1u; }
            }
          }
          // exact 64-bit partial row sums, then an 8-row transposed butterfly over the warp
          long long v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u)
            v[u] = ((long long)A[u] << 16) + (long long)(((unsigned long long)B[u] << 8) + (unsigned long long)C[u]);
          long long b4[4], c2[2], d;
          {
            const bool up = lane & 16;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const long long keep = up ? v[i + 4] : v[i], send = up ? v[i] : v[i + 4];
              b4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
            }
          }
          {
            const bool up = lane & 8;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const long long keep = up ? b4[i + 2] : b4[i], send = up ? b4[i] : b4[i + 2];
              c2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
          }
          {
            const bool up = lane & 4;
            const long long keep = up ? c2[1] : c2[0], send = up ? c2[0] : c2[1];
            d = keep + __shfl_xor_sync(0xffffffffu, send, 4);
          }
          d += __shfl_xor_sync(0xffffffffu, d, 2);
          d += __shfl_xor_sync(0xffffffffu, d, 1);
          if ((lane & 3) == 0) {
            const int u = ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
            const int sidx = stb + (u >> logM);
            const int lrow = sidx * RS + (u & (M - 1)) * P.rl + rl;
            if (sidx < nst && lrow < nrows) atomicAdd(&rowsum[s * P.rpc + lrow], (unsigned long long)d);
          }
        }
      }
    }
    named_bar_sync(1, kConsumers);

    // ---- epilogue: affine terms + the element-wise op that follows this matrix in the block
    auto value = [&](int s, int row, int n) -> float {
      const double main = double((long long)rowsum[s * P.rpc + row]) * sd[s];
      float y = float(main) + P.seg[s].half * sumxs_s[s];
      if (P.seg[s].rx) y *= P.seg[s].rx[n];
      y += zp_s[s];
      if (P.seg[s].mx) y += P.seg[s].mx[n] * sumx_s[s];
      return y;
    };
    if (P.epi == EPI_WKV) {
      for (int row = tid; row < nr[0]; row += kConsumers) {
        const int n = r0[0] + row;
        const float k = value(0, row, n), v = value(1, row, n), r = sigmoidf_(value(2, row, n));
        float aa = P.aa[n], bb = P.bb[n], pp = P.pp[n];
        const float y = wkv_step(k, v, P.wkv_w[n], P.wkv_u[n], aa, bb, pp);
        P.aa[n] = aa; P.bb[n] = bb; P.pp[n] = pp;
        P.wkv_out[n] = r * y;
      }
    } else {
#pragma unroll
      for (int s = 0; s < kMaxSeg; ++s) {
        if (s < P.nseg) {
          for (int row = tid; row < nr[s]; row += kConsumers) {
            const int n = r0[s] + row;
            float y = value(s, row, n);
            if (P.seg[s].act == ACT_RELUSQ) { y = fmaxf(y, 0.f); y *= y; }
            else if (P.seg[s].act == ACT_SIGMOID) y = sigmoidf_(y);
            if (P.seg[s].gate) y *= P.seg[s].gate[n];
            if (P.seg[s].res) y += P.seg[s].res[n];
            if (P.accumulate) y += P.seg[s].out[n];
            P.seg[s].out[n] = y;
          }
        }
      }
    }
  }

  __syncthreads();
  // After an aborted wait some bulk copies may still be in flight into this CTA's shared memory:
  // give every copy the producer issued a bounded chance to land before the CTA retires.
  if (tid == 0 && *abort_flag) {
    const int issued = *issued_ptr;
    const unsigned long long t0 = globaltimer_ns();
    for (int i = issued > P.stages ? issued - P.stages : 0; i < issued; ++i) {
      const uint32_t bar = full0 + 8 * (i % P.stages), parity = uint32_t(i / P.stages) & 1u;
      while (!mbar_try_wait(bar, parity) && globaltimer_ns() - t0 < kWaitLimitNs / 10) {
      }
    }
  }
}

// ---- host side ------------------------------------------------------------------------------------
cudaError_t launch_stream_gemv(GemvParams& P, int max_n, bool pdl, cudaStream_t stream, const char** why);

}  // namespace b200
