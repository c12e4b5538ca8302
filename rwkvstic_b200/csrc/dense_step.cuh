// One token through an RWKV-4 network with UNQUANTISED weights (the reference's TORCH mode:
// agnostic/agnosticRwkv.py:123-187 over the op table of agnostic/backends/torch.py:6-166).
// Matrices stay in their own type T (bf16 / fp16 / fp32, [out][in] as the checkpoint has them),
// vectors and the state are fp32.  The reference's matvec rounds the activation to T, multiplies
// in T and rounds the result to T (torch.py:162-164); everything else is fp32 element-wise work.
//
// Two kernels, chained with programmatic dependent launch:
//   dense_vec_kernel   one CTA: layer norm of the residual stream, token-shift mix against the
//                      carried row of the state, results rounded to T for the products that follow
//   dense_rows_kernel  the matrix rows, streamed once from HBM by warps (16-byte pieces, fp32 sums),
//                      with the activation vector(s) staged in shared memory as T and the rest of
//                      the block folded into the epilogue:
//                        key + value + receptance rows of one channel  -> WKV update, sigmoid gate
//                        attention output rows                         -> residual add
//                        ffn key rows -> relu^2 ; ffn receptance rows  -> sigmoid   (one launch)
//                        ffn value rows                                -> gated residual add
//                        head rows                                     -> logits
// Four row launches and two vector launches per block; each sum is formed in a fixed order, so the
// step is deterministic.
#pragma once

#include "dense_gemv.cuh"

namespace b200 {

constexpr int kDsWarps = 8;
constexpr int kDsThreads = kDsWarps * 32;
constexpr int kDsVecThreads = 1024;
constexpr int kDsMaxEmbd = 12160;          // the vector kernel keeps one fp32 row in its 48 KB of static shared memory
constexpr int kDsMaxStage = 200 * 1024;    // staged activation vectors per CTA of the rows kernel

enum DenseEpilogue { kEpStore = 0, kEpResid = 1, kEpRelu2 = 2, kEpSigmoid = 3, kEpGated = 4 };

__device__ __forceinline__ uint4 ld_act_u4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// torch.lerp(start, end, weight) as ATen evaluates it: the end point the weight is nearer to is the base.
__device__ __forceinline__ float lerp_like_torch(float start, float end, float weight) {
  const float diff = end - start;
  return fabsf(weight) < 0.5f ? fmaf(weight, diff, start) : fmaf(weight - 1.0f, diff, end);
}

// ------------------------------------------------------------------------------------ vector kernel
struct DenseVecParams {
  const float* x;           // residual stream [D]; nullptr: row `*token` of emb instead
  const float* emb;
  const long long* token;
  const float *ln_w, *ln_b;
  float* x_out;             // fp32 copy of the normalised row (embedding step), or nullptr
  float* carry;             // state row: previous normalised row in, this one out; nullptr: no token shift
  const float* mix[3];
  void* out[3];             // out[m] = T(lerp(carry, ln, mix[m])); with nmix == 0 and out[0] set: out[0] = T(ln)
  int nmix, D;
};

__device__ __forceinline__ float block_sum_1024(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();          // red may still be read by the previous call
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = red[lane];
  return warp_sum(t);
}

template <typename T>
__global__ void __launch_bounds__(kDsVecThreads)
dense_vec_kernel(const DenseVecParams P) {
  __shared__ float row[kDsMaxEmbd];
  __shared__ float red[32];
  griddep_launch_dependents();
  griddep_wait();
  const int tid = threadIdx.x, D = P.D;
  const float* src = P.x ? P.x : P.emb + size_t(*P.token) * D;
  float s = 0.f;
  for (int j = tid; j < D; j += kDsVecThreads) {
    const float v = P.x ? ld_act_f32(src + j) : ld_param_f32(src + j);
    row[j] = v;
    s += v;
  }
  const float mean = block_sum_1024(s, red) / float(D);
  float q = 0.f;
  for (int j = tid; j < D; j += kDsVecThreads) {
    const float c = row[j] - mean;
    q = fmaf(c, c, q);
  }
  const float sd = sqrtf(block_sum_1024(q, red) / float(D) + 1e-5f);
  for (int j = tid; j < D; j += kDsVecThreads) {
    const float y = P.ln_w[j] * ((row[j] - mean) / sd) + P.ln_b[j];      // torch.py:102-110
    if (P.x_out) P.x_out[j] = y;
    if (P.carry) {
      const float prev = ld_act_f32(P.carry + j);
#pragma unroll
      for (int m = 0; m < 3; ++m)
        if (m < P.nmix) static_cast<T*>(P.out[m])[j] = DenseType<T>::from_f32(lerp_like_torch(prev, y, P.mix[m][j]));
      P.carry[j] = y;
    } else if (P.out[0]) {
      static_cast<T*>(P.out[0])[j] = DenseType<T>::from_f32(y);
    }
  }
}

// ------------------------------------------------------------------------------------ rows kernel
struct DenseSeg {
  const void* w;        // [n][ldw] of T
  const void* x;        // [K] of T, written by an earlier kernel of the step
  void* out;            // kEpStore / kEpSigmoid: float[n]; kEpRelu2: T[n]; the residual epilogues use `resid`
  long long ldw;
  int n, ep;
};

struct DenseRowsParams {
  DenseSeg seg[3];
  int nseg, K, tasks, split;
  float* resid;            // fp32 residual stream [n] (kEpResid, kEpGated)
  const float* gate;       // sigmoid(ffn receptance) [n] (kEpGated)
  float* state;            // WKV launch: this block's [5][n] rows
  const float *decay, *first;
  void* wkv_out;           // WKV launch: T[n] = sigmoid(r) * wkv
};

// R == 3: task o = row o of the key, value and receptance matrices (segments 0..2, each with its own
//         activation vector); the epilogue advances channel o of the WKV state.
// R == 2: task t = rows 2t, 2t+1 of the segments laid end to end (every segment but the last has an
//         even row count); the rows of a pair share their activation vector.
// `split` warps (1, 2, 4 or 8) share the K range of a task; their sums meet in shared memory in part order.
template <typename T, int R>
__global__ void __launch_bounds__(kDsThreads, R == 3 ? 2 : 3)
dense_rows_kernel(const DenseRowsParams P) {
  constexpr int VEC = 16 / int(sizeof(T));
  constexpr int U = R == 3 ? 4 : 6;                  // 16-byte pieces of each row in flight per lane
  extern __shared__ __align__(16) unsigned char ds_smem[];
  __shared__ float partial[kDsWarps][R];
  uint4* xs = reinterpret_cast<uint4*>(ds_smem);     // [nx][K / VEC]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pieces = P.K / VEC;
  const int nx = R == 3 ? 3 : P.nseg;

  griddep_launch_dependents();
  griddep_wait();
  for (int v = 0; v < nx; ++v) {
    const uint4* src = static_cast<const uint4*>(P.seg[v].x);
    for (int c = tid; c < pieces; c += kDsThreads) xs[v * pieces + c] = ld_act_u4(src + c);
  }
  __syncthreads();

  const int split = P.split, per_pass = kDsWarps / split;
  const int slot = warp / split, part = warp - slot * split;
  const int c_begin = int((long long)pieces * part / split), c_end = int((long long)pieces * (part + 1) / split);

  for (int base = blockIdx.x * per_pass; base < P.tasks; base += gridDim.x * per_pass) {
    const int task = base + slot;
    const bool live = task < P.tasks;
    const int tk = live ? task : P.tasks - 1;          // idle slots re-read the last task and store nothing
    const uint4* row[R];
    const uint4* xv[R];
    int sidx = 0, local = tk;                          // R == 2: segment and row inside it of the pair's first row
    if constexpr (R == 3) {
#pragma unroll
      for (int r = 0; r < 3; ++r) {
        row[r] = reinterpret_cast<const uint4*>(static_cast<const T*>(P.seg[r].w) + size_t(tk) * P.seg[r].ldw);
        xv[r] = xs + r * pieces;
      }
    } else {
      local = 2 * tk;
      while (sidx + 1 < P.nseg && local >= P.seg[sidx].n) { local -= P.seg[sidx].n; ++sidx; }
      const DenseSeg& S = P.seg[sidx];
      const T* W = static_cast<const T*>(S.w);
      row[0] = reinterpret_cast<const uint4*>(W + size_t(local) * S.ldw);
      row[1] = reinterpret_cast<const uint4*>(W + size_t(min(local + 1, S.n - 1)) * S.ldw);
      xv[0] = xv[1] = xs + sidx * pieces;
    }
    float sum[R];
#pragma unroll
    for (int r = 0; r < R; ++r) sum[r] = 0.f;

    int c = c_begin + lane;
    for (; c + (U - 1) * 32 < c_end; c += U * 32) {
      uint4 w[R][U];
#pragma unroll
      for (int r = 0; r < R; ++r)
#pragma unroll
        for (int j = 0; j < U; ++j) w[r][j] = __ldcs(row[r] + c + j * 32);
#pragma unroll
      for (int j = 0; j < U; ++j) {
        if constexpr (R == 3) {
#pragma unroll
          for (int r = 0; r < 3; ++r) {
            const uint4 a = xv[r][c + j * 32];
            const T* xe = reinterpret_cast<const T*>(&a);
            const T* we = reinterpret_cast<const T*>(&w[r][j]);
#pragma unroll
            for (int i = 0; i < VEC; ++i) sum[r] = fmaf(DenseType<T>::to_f32(xe[i]), DenseType<T>::to_f32(we[i]), sum[r]);
          }
        } else {
          const uint4 a = xv[0][c + j * 32];
          const T* xe = reinterpret_cast<const T*>(&a);
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const T* we = reinterpret_cast<const T*>(&w[r][j]);
#pragma unroll
            for (int i = 0; i < VEC; ++i) sum[r] = fmaf(DenseType<T>::to_f32(xe[i]), DenseType<T>::to_f32(we[i]), sum[r]);
          }
        }
      }
    }
    for (; c < c_end; c += 32) {
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const uint4 wv = __ldcs(row[r] + c);
        const uint4 a = xv[r][c];
        const T* xe = reinterpret_cast<const T*>(&a);
        const T* we = reinterpret_cast<const T*>(&wv);
#pragma unroll
        for (int i = 0; i < VEC; ++i) sum[r] = fmaf(DenseType<T>::to_f32(xe[i]), DenseType<T>::to_f32(we[i]), sum[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) sum[r] = warp_sum(sum[r]);
    if (split > 1) {                                   // uniform over the CTA
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) partial[warp][r] = sum[r];
      }
      __syncthreads();
      if (lane == 0 && part == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
          float t = 0.f;
          for (int q = 0; q < split; ++q) t += partial[warp + q][r];
          sum[r] = t;
        }
      }
      __syncthreads();
    }
    if (lane != 0 || part != 0 || !live) continue;

    if constexpr (R == 3) {
      const int n = P.seg[0].n, o = tk;
      const float k = DenseType<T>::round(sum[0]), v = DenseType<T>::round(sum[1]), r = DenseType<T>::round(sum[2]);
      float aa = ld_act_f32(P.state + 2 * size_t(n) + o), bb = ld_act_f32(P.state + 3 * size_t(n) + o);
      float pp = ld_act_f32(P.state + 4 * size_t(n) + o);
      const float y = wkv_step(k, v, P.decay[o], P.first[o], aa, bb, pp);      // agnosticRwkv.py:68-103
      P.state[2 * size_t(n) + o] = aa; P.state[3 * size_t(n) + o] = bb; P.state[4 * size_t(n) + o] = pp;
      static_cast<T*>(P.wkv_out)[o] = DenseType<T>::from_f32(sigmoidf_(r) * y);
    } else {
      const DenseSeg& S = P.seg[sidx];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int o = local + i;
        if (o >= S.n) break;
        const float v = DenseType<T>::round(sum[i]);
        switch (S.ep) {
          case kEpStore: static_cast<float*>(S.out)[o] = v; break;
          case kEpResid: P.resid[o] = __fadd_rn(ld_act_f32(P.resid + o), v); break;
          case kEpRelu2: { const float t = fmaxf(v, 0.f); static_cast<T*>(S.out)[o] = DenseType<T>::from_f32(__fmul_rn(t, t)); break; }
          case kEpSigmoid: static_cast<float*>(S.out)[o] = sigmoidf_(v); break;
          default: P.resid[o] = __fadd_rn(ld_act_f32(P.resid + o), __fmul_rn(v, ld_act_f32(P.gate + o))); break;
        }
      }
    }
  }
}

}  // namespace b200
