// Unquantised weights: y[o] = round_T( sum_j round_T(x[j]) * W[o][j] ) for W of type
// T in {bf16, fp16, fp32} - the reference's TORCH-mode `matvec`
// (agnostic/backends/torch.py:162-164: x.to(W.dtype).matmul(W).to(x.dtype)).  The reference keeps
// a matrix as the transposed VIEW of the checkpoint's [out][in] tensor (initTensor, torch.py:146-152),
// so in memory a row of W is one output's weights with the input index contiguous; that is the
// layout read here.  HBM-bound: N*K*sizeof(T) bytes per call.
//
// One warp per output row or pair of rows (grid-stride): the lanes walk the row in 16-byte
// pieces, eight pieces in flight per lane, the matching x values come from L1 (and are shared by
// the rows of a pair); fp32 sums, a shuffle reduction per row, one rounded store.  Matrices with
// few long rows give a row to two or four warps of a CTA, whose sums meet in shared memory in a
// fixed order.  Results do not depend on scheduling and no scratch in global memory is needed.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"

namespace b200 {

constexpr int kDenseWarps = 8;
constexpr int kDenseThreads = kDenseWarps * 32;
// Template arguments: output rows per warp pass, 16-byte pieces of each row in flight per lane,
// warps that share one row's K.  (2, 8, 1) when there are rows enough to keep every SM's warps busy
// that way, (1, 8, 1) for fewer rows, (1, 8, 2 or 4) when even one warp per row leaves SMs short.

template <typename T> struct DenseType;
template <> struct DenseType<__nv_bfloat16> {
  static __device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ float round(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
  static __device__ __forceinline__ __nv_bfloat16 from_f32(float v) { return __float2bfloat16_rn(v); }
};
template <> struct DenseType<__half> {
  static __device__ __forceinline__ float to_f32(__half v) { return __half2float(v); }
  static __device__ __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
  static __device__ __forceinline__ __half from_f32(float v) { return __float2half_rn(v); }
};
template <> struct DenseType<float> {
  static __device__ __forceinline__ float to_f32(float v) { return v; }
  static __device__ __forceinline__ float round(float v) { return v; }
  static __device__ __forceinline__ float from_f32(float v) { return v; }
};

struct DenseParams {
  const void* w;        // [N][ldw] of T
  const float* x;       // [K]
  float* y;             // [N]
  long long ldw;        // elements between rows of W (>= K)
  int K, N;
  int vector_ok;        // rows of W start on 16-byte boundaries and x on a 16-byte boundary
};

template <typename T, int kDenseRows, int kDenseUnroll, int kDenseSplit>
__global__ void __launch_bounds__(kDenseThreads)
dense_gemv_kernel(const DenseParams P) {
  static_assert(kDenseSplit == 1 || kDenseRows == 1, "K is split only in the one-row variant");
  constexpr int VEC = 16 / int(sizeof(T));
  constexpr int kRowsPerCta = kDenseWarps / kDenseSplit * kDenseRows;
  __shared__ float partial[kDenseWarps];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int slot = warp / kDenseSplit, part = warp % kDenseSplit;   // which row of the CTA's pass, which K range
  const T* W = static_cast<const T*>(P.w);
  const int pieces = P.vector_ok ? P.K / VEC : 0;     // whole 16-byte pieces per row
  const int tail0 = pieces * VEC;
  // this warp's share of the pieces and of the element tail (contiguous ranges, in part order)
  const int c_begin = int((long long)pieces * part / kDenseSplit), c_end = int((long long)pieces * (part + 1) / kDenseSplit);
  const int t_begin = tail0 + int((long long)(P.K - tail0) * part / kDenseSplit);
  const int t_end = tail0 + int((long long)(P.K - tail0) * (part + 1) / kDenseSplit);

  // the loop bounds are the same for every warp of a CTA, so the barriers below are reached by all
  for (int base = blockIdx.x * kRowsPerCta; base < P.N; base += gridDim.x * kRowsPerCta) {
    const int o0 = base + slot * kDenseRows;
    const T* row[kDenseRows];
    float sum[kDenseRows];
#pragma unroll
    for (int r = 0; r < kDenseRows; ++r) {
      row[r] = W + size_t(min(o0 + r, P.N - 1)) * P.ldw;   // a pass past the end re-reads the last row
      sum[r] = 0.f;
    }
    int c = c_begin + lane;
    for (; c + (kDenseUnroll - 1) * 32 < c_end; c += kDenseUnroll * 32) {
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
    for (; c < c_end; c += 32) {
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
    for (int j = t_begin + lane; j < t_end; j += 32) {
      const float xv = DenseType<T>::round(__ldg(P.x + j));
#pragma unroll
      for (int r = 0; r < kDenseRows; ++r) sum[r] = fmaf(xv, DenseType<T>::to_f32(row[r][j]), sum[r]);
    }
#pragma unroll
    for (int r = 0; r < kDenseRows; ++r) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum[r] += __shfl_xor_sync(0xffffffffu, sum[r], o);
    }
    if constexpr (kDenseSplit == 1) {
#pragma unroll
      for (int r = 0; r < kDenseRows; ++r)
        if (lane == 0 && o0 + r < P.N) P.y[o0 + r] = DenseType<T>::round(sum[r]);
    } else {
      // the K ranges of a row meet in shared memory and are added in range order
      if (lane == 0) partial[warp] = sum[0];
      __syncthreads();
      if (lane == 0 && part == 0 && o0 < P.N) {
        float t = 0.f;
#pragma unroll
        for (int q = 0; q < kDenseSplit; ++q) t += partial[warp + q];
        P.y[o0] = DenseType<T>::round(t);
      }
      __syncthreads();
    }
  }
}

}  // namespace b200
