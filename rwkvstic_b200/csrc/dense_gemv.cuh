// Unquantised weights: y[o] = round_T( sum_j round_T(x[j]) * W[o][j] ) for W of type
// T in {bf16, fp16, fp32} - the reference's TORCH-mode `matvec`
// (agnostic/backends/torch.py:162-164: x.to(W.dtype).matmul(W).to(x.dtype)).  The reference keeps
// a matrix as the transposed VIEW of the checkpoint's [out][in] tensor (initTensor, torch.py:146-152),
// so in memory a row of W is one output's weights with the input index contiguous; that is the
// layout read here.  HBM-bound: N*K*sizeof(T) bytes per call.
//
// One warp per output row or pair of rows (grid-stride): the lanes walk the row in 16-byte
// pieces, eight pieces in flight per lane, the matching x values come from L1 (and are shared by
// the rows of a pair); fp32 sums, a shuffle reduction per row, one rounded store.  Every output
// is computed by one warp in a fixed order, so results do not depend on scheduling and no scratch
// is needed.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

constexpr int kDenseWarps = 8;
constexpr int kDenseThreads = kDenseWarps * 32;
// Output rows per warp pass x 16-byte pieces of each row in flight per lane: (2, 4) when there
// are rows enough to keep every SM's warps busy that way, (1, 8) for matrices with fewer rows.

template <typename T> struct DenseType;
template <> struct DenseType<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};
template <> struct DenseType<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};
template <> struct DenseType<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};

struct DenseParams {
  const void* w;        // [N][ldw] of T
  const float* x;       // [K]
  float* y;             // [N]
  long long ldw;        // elements between rows of W (>= K)
  int K, N;
  int vector_ok;        // rows of W start on 16-byte boundaries and x on a 16-byte boundary
};

template <typename T, int kDenseRows, int kDenseUnroll>
__global__ void __launch_bounds__(kDenseThreads)
dense_gemv_kernel(const DenseParams P) {
  constexpr int VEC = 16 / int(sizeof(T));
  const int lane = threadIdx.x & 31;
  const int warp_global = blockIdx.x * kDenseWarps + (threadIdx.x >> 5);
  const int warps_total = gridDim.x * kDenseWarps;
  const T* W = static_cast<const T*>(P.w);
  const int pieces = P.vector_ok ? P.K / VEC : 0;     // whole 16-byte pieces per row
  const int tail0 = pieces * VEC;

  for (int o0 = warp_global * kDenseRows; o0 < P.N; o0 += warps_total * kDenseRows) {
    const T* row[kDenseRows];
    float sum[kDenseRows];
#pragma unroll
    for (int r = 0; r < kDenseRows; ++r) {
      row[r] = W + size_t(min(o0 + r, P.N - 1)) * P.ldw;   // a pass past the end re-reads the last row
      sum[r] = 0.f;
    }
    int c = lane;
    for (; c + (kDenseUnroll - 1) * 32 < pieces; c += kDenseUnroll * 32) {
      uint4 v[kDenseRows][kDenseUnroll];
#pragma unroll
      for (int r = 0; r < kDenseRows; ++r)
#pragma unroll
        for (int j = 0; j < kDenseUnroll; ++j)
          v[r][j] = __ldcs(reinterpret_cast<const uint4*>(row[r]) + c + j * 32);
#pragma unroll
      for (int j = 0; j < kDenseUnroll; ++j) {
        float xv[VEC];
        const float4* xp = reinterpret_cast<const float4*>(P.x + size_t(c + j * 32) * VEC);
#pragma unroll
        for (int q = 0; q < VEC / 4; ++q) {
          const float4 t = __ldg(xp + q);
          xv[4 * q] = DenseType<T>::round(t.x); xv[4 * q + 1] = DenseType<T>::round(t.y);
          xv[4 * q + 2] = DenseType<T>::round(t.z); xv[4 * q + 3] = DenseType<T>::round(t.w);
        }
#pragma unroll
        for (int r = 0; r < kDenseRows; ++r) {
          const T* e = reinterpret_cast<const T*>(&v[r][j]);
#pragma unroll
          for (int i = 0; i < VEC; ++i) sum[r] = fmaf(xv[i], DenseType<T>::to_f32(e[i]), sum[r]);
        }
      }
    }
    for (; c < pieces; c += 32) {
#pragma unroll
      for (int r = 0; r < kDenseRows; ++r) {
        const uint4 v = __ldcs(reinterpret_cast<const uint4*>(row[r]) + c);
        const T* e = reinterpret_cast<const T*>(&v);
#pragma unroll
        for (int i = 0; i < VEC; ++i)
          sum[r] = fmaf(DenseType<T>::round(__ldg(P.x + size_t(c) * VEC + i)), DenseType<T>::to_f32(e[i]), sum[r]);
      }
    }
    // what is left of K, or all of it when rows do not start on 16-byte boundaries: element loads
    for (int j = tail0 + lane; j < P.K; j += 32) {
      const float xv = DenseType<T>::round(__ldg(P.x + j));
#pragma unroll
      for (int r = 0; r < kDenseRows; ++r) sum[r] = fmaf(xv, DenseType<T>::to_f32(row[r][j]), sum[r]);
    }
#pragma unroll
    for (int r = 0; r < kDenseRows; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], o);
      if (lane == 0 && o0 + r < P.N) P.y[o0 + r] = DenseType<T>::round(sum[r]);
    }
  }
}

}  // namespace b200
