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

#include <type_traits>

#include "dense_gemv.cuh"

namespace b200 {

constexpr int kDsVecThreads = 1024;
constexpr int kDsMaxEmbd = 12160;          // the vector kernel keeps one fp32 row in its 48 KB of static shared memory

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
  int V;                    // rows of emb: a token outside 0..V-1 is clamped into the table
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
__device__ __forceinline__ void store_t4(T* dst, float a, float b, float c, float d) {
  if constexpr (sizeof(T) == 4) {
    *reinterpret_cast<float4*>(dst) = make_float4(a, b, c, d);
  } else {
    T v[4] = {DenseType<T>::from_f32(a), DenseType<T>::from_f32(b), DenseType<T>::from_f32(c), DenseType<T>::from_f32(d)};
    *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(v);
  }
}

// One CTA of 1024 threads; thread t owns the float4 groups t, t + 1024, ... (NV of them cover D).
// The parameter vectors are requested before the dependency wait, the row and the carried row
// right after it, so that every load of the kernel is in flight at once.
template <typename T, int NV>
__global__ void __launch_bounds__(kDsVecThreads)
dense_vec_kernel(const DenseVecParams P) {
  __shared__ float red[32];
  griddep_launch_dependents();
  const int tid = threadIdx.x, D4 = P.D >> 2;
  float4 lw[NV], lb[NV], xv[NV], cv[NV];
  const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int g = tid + i * kDsVecThreads;
    const bool in = g < D4;
    lw[i] = in ? ld_param_v4(reinterpret_cast<const float4*>(P.ln_w) + g) : zero;
    lb[i] = in ? ld_param_v4(reinterpret_cast<const float4*>(P.ln_b) + g) : zero;
  }
  griddep_wait();
  long long tok = P.x ? 0 : *P.token;
  tok = tok < 0 ? 0 : (tok >= P.V ? P.V - 1 : tok);
  const float4* src = reinterpret_cast<const float4*>(P.x ? P.x : P.emb + size_t(tok) * P.D);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int g = tid + i * kDsVecThreads;
    const bool in = g < D4;
    xv[i] = in ? ld_act_v4(src + g) : zero;
    cv[i] = in && P.carry ? ld_act_v4(reinterpret_cast<const float4*>(P.carry) + g) : zero;
  }
#pragma unroll
  for (int i = 0; i < NV; ++i) s += (xv[i].x + xv[i].y) + (xv[i].z + xv[i].w);
  const float mean = block_sum_1024(s, red) / float(P.D);
  float q = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    if (tid + i * kDsVecThreads < D4) {
      xv[i].x -= mean; xv[i].y -= mean; xv[i].z -= mean; xv[i].w -= mean;
      q = fmaf(xv[i].x, xv[i].x, q); q = fmaf(xv[i].y, xv[i].y, q); q = fmaf(xv[i].z, xv[i].z, q); q = fmaf(xv[i].w, xv[i].w, q);
    }
  }
  const float sd = sqrtf(block_sum_1024(q, red) / float(P.D) + 1e-5f);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int g = tid + i * kDsVecThreads;
    if (g >= D4) continue;
    float4 y;                                                            // torch.py:102-110
    y.x = lw[i].x * (xv[i].x / sd) + lb[i].x; y.y = lw[i].y * (xv[i].y / sd) + lb[i].y;
    y.z = lw[i].z * (xv[i].z / sd) + lb[i].z; y.w = lw[i].w * (xv[i].w / sd) + lb[i].w;
    if (P.x_out) reinterpret_cast<float4*>(P.x_out)[g] = y;
    if (P.carry) {
#pragma unroll
      for (int m = 0; m < 3; ++m) {
        if (m < P.nmix) {
          const float4 w = ld_param_v4(reinterpret_cast<const float4*>(P.mix[m]) + g);
          store_t4(static_cast<T*>(P.out[m]) + 4 * size_t(g), lerp_like_torch(cv[i].x, y.x, w.x), lerp_like_torch(cv[i].y, y.y, w.y),
                   lerp_like_torch(cv[i].z, y.z, w.z), lerp_like_torch(cv[i].w, y.w, w.w));
        }
      }
      reinterpret_cast<float4*>(P.carry)[g] = y;
    } else if (P.out[0]) {
      store_t4(static_cast<T*>(P.out[0]) + 4 * size_t(g), y.x, y.y, y.z, y.w);
    }
  }
}

// ------------------------------------------------------------------------------------ rows kernel
constexpr int kDrWarps = 16;
constexpr int kDrThreads = kDrWarps * 32;
constexpr int kDrSlots = 2;                            // ring slots per warp
constexpr int kDrStages = kDrWarps * kDrSlots;
#ifndef B200_DR_EARLY
#define B200_DR_EARLY 2
#endif
constexpr int kDrEarly = B200_DR_EARLY;               // slots per warp requested before the dependency wait
constexpr int kDrOffFull = 0, kDrOffAbort = 512, kDrOffData = 1024;
constexpr int kDrSmemLimit = 227 * 1024;

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
  int max_local;           // most tasks one CTA owns
  int row_stride;          // bytes between the rows of one ring slot (>= the longest K range, multiple of 16)
  int stage_bytes;         // R * row_stride rounded up to 128
  float* resid;            // fp32 residual stream [n] (kEpResid, kEpGated)
  const float* gate;       // sigmoid(ffn receptance) [n] (kEpGated)
  float* state;            // WKV launch: this block's [5][n] rows
  const float *decay, *first;
  void* wkv_out;           // WKV launch: T[n] = sigmoid(r) * wkv
  int* status;             // device status word (B200RWKV_STATUS_* bits)
  unsigned long long wait_limit_ns;   // bound of every wait of the kernel (0: the library default of one second)
  int withhold_copies;     // testing the time-out path: slots are announced but never filled, so every wait expires
#ifdef B200_DENSE_TRACE
  unsigned long long* trace;   // profiling builds: CTA 0, [warp][item 0..63][8] %globaltimer stamps
#endif
};

#ifdef B200_DENSE_TRACE
#define B200_DENSE_STAMP(i) do { if (lane == 0 && blockIdx.x == 0 && P.trace && k < 64) P.trace[(size_t(warp) * 64 + k) * 8 + (i)] = globaltimer_ns(); } while (0)
#else
#define B200_DENSE_STAMP(i) do { } while (0)
#endif

// Shared memory after the barriers: activation vectors, partial sums + arrival counters, epilogue
// operands of the CTA's tasks, one 16-byte record per task (R == 2: address of its first row, segment
// and row index inside it), ring.
struct DenseRowsLayout { size_t x_off, part_off, arrived_off, ep_off, table_off, ring_off, total; };
__host__ __device__ inline DenseRowsLayout dense_rows_layout(int nx, int K, int elem_bytes, int max_local, int split, int R, int stage_bytes) {
  DenseRowsLayout l;
  l.x_off = kDrOffData;
  l.part_off = (l.x_off + size_t(nx) * K * elem_bytes + 127) / 128 * 128;
  l.arrived_off = l.part_off + size_t(max_local) * split * R * 4;
  l.ep_off = l.arrived_off + size_t(max_local) * 4;
  l.table_off = (l.ep_off + size_t(max_local) * (R == 3 ? 5 : 4) * 4 + 15) / 16 * 16;
  l.ring_off = (l.table_off + size_t(max_local) * 16 + 127) / 128 * 128;
  l.total = l.ring_off + size_t(kDrStages) * stage_bytes;
  return l;
}

__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Sixteen bytes of activations times sixteen bytes of weights, added to two running sums (even and
// odd elements).  bf16 widens to fp32 with a shift or a mask: the conversion instruction runs at a
// fraction of the FMA rate and would bound the kernel.
template <typename T>
__device__ __forceinline__ void dot_piece(const uint4& a, const uint4& b, float& s0, float& s1) {
  if constexpr (sizeof(T) == 4) {
    s0 = fmaf(__uint_as_float(a.x), __uint_as_float(b.x), s0); s1 = fmaf(__uint_as_float(a.y), __uint_as_float(b.y), s1);
    s0 = fmaf(__uint_as_float(a.z), __uint_as_float(b.z), s0); s1 = fmaf(__uint_as_float(a.w), __uint_as_float(b.w), s1);
  } else {
    const uint32_t xa[4] = {a.x, a.y, a.z, a.w}, wb[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        s0 = fmaf(__uint_as_float(xa[i] << 16), __uint_as_float(wb[i] << 16), s0);
        s1 = fmaf(__uint_as_float(xa[i] & 0xffff0000u), __uint_as_float(wb[i] & 0xffff0000u), s1);
      } else {
        const float2 xf = __half22float2(*reinterpret_cast<const __half2*>(&xa[i]));
        const float2 wf = __half22float2(*reinterpret_cast<const __half2*>(&wb[i]));
        s0 = fmaf(xf.x, wf.x, s0);
        s1 = fmaf(xf.y, wf.y, s1);
      }
    }
  }
}

// One CTA of 16 warps per SM.  CTA b owns the contiguous tasks [tasks*b/grid, tasks*(b+1)/grid):
//   R == 3: task o = row o of the key, value and receptance matrices (segments 0..2, each with its own
//           activation vector); the epilogue advances channel o of the WKV state.
//   R == 2: task t = rows 2t, 2t+1 of the segments laid end to end (every segment but the last has an
//           even row count); the rows of a pair share their activation vector.
// A task is cut into `split` K ranges; item i = (task, range) in order; warp w takes items w, w + 16, ...
// Every warp runs its own two-slot ring: lane 0 requests an item's weight bytes with bulk copies that
// complete on the slot's mbarrier, the warp multiplies the landed slot against the activation vector
// staged in shared memory, and lane 0 refills the slot with the warp's item after next.  The first two
// items of every warp are requested before the dependency wait (no kernel writes weights), so the
// whole ring is in flight while the previous kernel drains.  Partial sums of a task meet in shared
// memory; whichever warp completes the task adds them in range order and runs the epilogue.  Warps
// never wait for one another, and every sum is formed in a fixed order.
template <typename T, int R>
__global__ void __launch_bounds__(kDrThreads, 1)
dense_rows_kernel(const DenseRowsParams P) {
  constexpr int VEC = 16 / int(sizeof(T));
  extern __shared__ __align__(128) unsigned char ds_smem[];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int pieces = P.K / VEC;
  const int nx = R == 3 ? 3 : P.nseg;
  const int split = P.split;
  const DenseRowsLayout lay = dense_rows_layout(nx, P.K, int(sizeof(T)), P.max_local, split, R, P.stage_bytes);
  const uint32_t full0 = smem_u32(ds_smem + kDrOffFull) + uint32_t(warp * kDrSlots) * 8u;     // this warp's barriers
  volatile int* abort_flag = reinterpret_cast<volatile int*>(ds_smem + kDrOffAbort);
  uint4* xs = reinterpret_cast<uint4*>(ds_smem + lay.x_off);                     // [nx][pieces]
  float* partial = reinterpret_cast<float*>(ds_smem + lay.part_off);             // [max_local * split][R]
  int* arrived = reinterpret_cast<int*>(ds_smem + lay.arrived_off);              // [max_local]
  float* eps = reinterpret_cast<float*>(ds_smem + lay.ep_off);                   // R == 3: [5][max_local]; R == 2: [2][2 * max_local]
  ulonglong2* table = reinterpret_cast<ulonglong2*>(ds_smem + lay.table_off);    // [max_local]: {row address, segment | row << 2}
  unsigned char* ring = ds_smem + lay.ring_off + size_t(warp * kDrSlots) * P.stage_bytes;   // this warp's slots

  griddep_launch_dependents();
  const unsigned long long wait_limit = P.wait_limit_ns ? P.wait_limit_ns : kWaitLimitNs;
  const int t0 = int((long long)P.tasks * blockIdx.x / gridDim.x);
  const int t1 = int((long long)P.tasks * (blockIdx.x + 1) / gridDim.x);
  if (tid == 0) *abort_flag = 0;
  if (lane == 0) {
    for (int i = 0; i < kDrSlots; ++i) mbar_init(full0 + 8 * i, 1);
    fence_mbar_init();
  }
  if constexpr (R == 2) {
    for (int i = tid; i < t1 - t0; i += kDrThreads) {
      int sidx = 0, local = 2 * (t0 + i);
      while (sidx + 1 < P.nseg && local >= P.seg[sidx].n) { local -= P.seg[sidx].n; ++sidx; }
      const T* W = static_cast<const T*>(P.seg[sidx].w) + size_t(local) * P.seg[sidx].ldw;
      // the second row of the pair follows ldw elements later; a pair past the end repeats its first row
      table[i] = make_ulonglong2(reinterpret_cast<unsigned long long>(W),
                                 (unsigned long long)(unsigned(sidx) | (unsigned(local) << 2) | (local + 1 < P.seg[sidx].n ? 0x80000000u : 0u)));
    }
    __syncthreads();
  } else {
    __syncwarp();
  }

  // K ranges are `range` pieces long (the last one of a row may be shorter); item -> (task, range)
  // indices advance by kDrWarps items without divisions.
  const int range = P.row_stride >> 4;
  const int adv_lt = kDrWarps / split, adv_part = kDrWarps % split;
  auto advance = [&](int& lt, int& part) __attribute__((always_inline)) {
    lt += adv_lt; part += adv_part;
    if (part >= split) { part -= split; ++lt; }
  };
  // lane 0: request item (lt, part), the warp's k-th, into slot k % 2
  auto request = [&](int k, int lt, int part) __attribute__((always_inline)) {
    if (lt >= t1 - t0) return;
    const int task = t0 + lt;
    const int c0 = part * range, c1 = min(c0 + range, pieces);
    const uint32_t bytes = uint32_t(c1 - c0) * 16u;
    const uint32_t bar = full0 + 8 * (k % kDrSlots);
    const uint32_t dst = smem_u32(ring + size_t(k % kDrSlots) * P.stage_bytes);
    mbar_arrive_expect_tx(bar, bytes * R);
    if constexpr (R == 3) {
#pragma unroll
      for (int r = 0; r < 3; ++r)
        if (!P.withhold_copies)
          bulk_g2s(dst + r * P.row_stride,
                   reinterpret_cast<const uint4*>(static_cast<const T*>(P.seg[r].w) + size_t(task) * P.seg[r].ldw) + c0, bytes, bar);
    } else {
      const ulonglong2 rec = table[lt];
      const unsigned meta = unsigned(rec.y);
      const T* W = reinterpret_cast<const T*>(rec.x);
      if (!P.withhold_copies) {
        bulk_g2s(dst, reinterpret_cast<const uint4*>(W) + c0, bytes, bar);
        bulk_g2s(dst + P.row_stride, reinterpret_cast<const uint4*>(W + ((meta >> 31) ? P.seg[meta & 3u].ldw : 0)) + c0, bytes, bar);
      }
    }
  };
  int lt = warp / split, part = warp % split;          // the item being consumed
  int rlt = lt, rpart = part;                          // the next item to request
  if (lane == 0) {
#pragma unroll
    for (int k = 0; k < kDrEarly; ++k) {
      request(k, rlt, rpart);
      advance(rlt, rpart);
    }
  }

  griddep_wait();
  for (int i = tid; i < t1 - t0; i += kDrThreads) arrived[i] = 0;
  // Operands of the epilogues of all the CTA's tasks, fetched now in one latency: a load issued
  // later would queue behind the megabytes of weight requests in flight.
  if constexpr (R == 3) {
    const int n = P.seg[0].n;
    for (int i = tid; i < 5 * (t1 - t0); i += kDrThreads) {
      const int a = i / (t1 - t0), j = i - a * (t1 - t0);
      eps[a * P.max_local + j] = a < 3 ? ld_act_f32(P.state + size_t(2 + a) * n + t0 + j)
                                       : ld_param_f32((a == 3 ? P.decay : P.first) + t0 + j);
    }
  } else if (P.resid) {                   // residual epilogues: one segment, outputs 2*t0 .. 2*t1-1
    const int n = P.seg[0].n, cnt = min(2 * t1, n) - 2 * t0;
    for (int i = tid; i < cnt; i += kDrThreads) {
      eps[i] = ld_act_f32(P.resid + 2 * t0 + i);
      if (P.gate) eps[2 * P.max_local + i] = ld_act_f32(P.gate + 2 * t0 + i);
    }
  }
  for (int v = 0; v < nx; ++v) {
    const uint4* src = static_cast<const uint4*>(P.seg[v].x);
    for (int c = tid; c < pieces; c += kDrThreads) xs[v * pieces + c] = ld_act_u4(src + c);
  }
  __syncthreads();
  if (lane == 0) {
#pragma unroll
    for (int k = kDrEarly; k < kDrSlots; ++k) {
      request(k, rlt, rpart);
      advance(rlt, rpart);
    }
  }

  int k = 0;
  bool dead = false;
  for (; lt < t1 - t0; advance(lt, part), ++k) {
    const int task = t0 + lt, item = lt * split + part;
    const int c0 = part * range, c1 = min(c0 + range, pieces);
    int sidx = 0, local = task;
    if constexpr (R == 2) {
      const unsigned meta = unsigned(table[lt].y);
      sidx = int(meta & 3u);
      local = int((meta & 0x7fffffffu) >> 2);
    }
    const int slot = k % kDrSlots;
    B200_DENSE_STAMP(0);
    const bool ok = mbar_wait_limited(full0 + 8 * slot, uint32_t(k / kDrSlots) & 1u, abort_flag, wait_limit);
    if (!__all_sync(0xffffffffu, ok)) {
      if (lane == 0 && P.status) atomicOr(P.status, B200RWKV_STATUS_WAIT_FULL);
      dead = true;
      break;
    }
    B200_DENSE_STAMP(1);
    const uint4* st = reinterpret_cast<const uint4*>(ring + size_t(slot) * P.stage_bytes);
    const int rs = P.row_stride >> 4, n = c1 - c0;
    float acc[R][2];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r][0] = acc[r][1] = 0.f;
    const uint4* x0 = xs + (R == 3 ? 0 : sidx * pieces) + c0;
#pragma unroll 4
    for (int p = lane; p < n; p += 32) {
      uint4 a = x0[p];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        if (R == 3 && r > 0) a = x0[r * pieces + p];
        dot_piece<T>(a, st[r * rs + p], acc[r][0], acc[r][1]);
      }
    }
    __syncwarp();
    B200_DENSE_STAMP(2);
    if (lane == 0) {                       // the slot has been read: refill it with the item after next
      fence_proxy_async_smem();
      request(k + kDrSlots, rlt, rpart);
      advance(rlt, rpart);
    }
    B200_DENSE_STAMP(4);
    float sum[R];
    if constexpr (R == 2) {
      // both rows in five shuffles: the lower half of the warp ends up with row 0's total, the upper with row 1's
      const float mine = acc[0][0] + acc[0][1], other = acc[1][0] + acc[1][1];
      const bool up = lane >= 16;
      float v = (up ? other : mine) + __shfl_xor_sync(0xffffffffu, up ? mine : other, 16);
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      sum[0] = __shfl_sync(0xffffffffu, v, 0);
      sum[1] = __shfl_sync(0xffffffffu, v, 16);
    } else {
#pragma unroll
      for (int r = 0; r < R; ++r) sum[r] = warp_sum(acc[r][0] + acc[r][1]);
    }
    B200_DENSE_STAMP(5);
    // Lane 0 runs the shared-memory hand-over of the partial sums; lane 1 does the epilogue's global
    // stores, so that lane 0's fences never wait for a store on its way to L2.
    int last = 1;
    if (split > 1) {
      if (lane == 0) {
#pragma unroll
        for (int r = 0; r < R; ++r) partial[size_t(item) * R + r] = sum[r];
        __threadfence_block();
        last = atomicAdd(&arrived[lt], 1) == split - 1;
        if (last) {
          __threadfence_block();
#pragma unroll
          for (int r = 0; r < R; ++r) {
            float t = 0.f;
            for (int q = 0; q < split; ++q) t += partial[(size_t(lt) * split + q) * R + r];
            sum[r] = t;
          }
        }
      }
      last = __shfl_sync(0xffffffffu, last, 0);
#pragma unroll
      for (int r = 0; r < R; ++r) sum[r] = __shfl_sync(0xffffffffu, sum[r], 0);
    }
    if (last && lane == 1) {
      if constexpr (R == 3) {
        const int nn = P.seg[0].n, o = local;
        const float kk = DenseType<T>::round(sum[0]), v = DenseType<T>::round(sum[1]), r = DenseType<T>::round(sum[2]);
        float aa = eps[lt], bb = eps[P.max_local + lt], pp = eps[2 * P.max_local + lt];
        const float y = wkv_step(kk, v, eps[3 * P.max_local + lt], eps[4 * P.max_local + lt], aa, bb, pp);   // agnosticRwkv.py:68-103
        P.state[2 * size_t(nn) + o] = aa; P.state[3 * size_t(nn) + o] = bb; P.state[4 * size_t(nn) + o] = pp;
        static_cast<T*>(P.wkv_out)[o] = DenseType<T>::from_f32(sigmoidf_(r) * y);
      } else {
        const DenseSeg& S = P.seg[sidx];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const int o = local + i;
          if (o < S.n) {
            const float v = DenseType<T>::round(sum[i]);
            switch (S.ep) {
              case kEpStore: static_cast<float*>(S.out)[o] = v; break;
              case kEpResid: P.resid[o] = __fadd_rn(eps[2 * lt + i], v); break;
              case kEpRelu2: { const float t = fmaxf(v, 0.f); static_cast<T*>(S.out)[o] = DenseType<T>::from_f32(__fmul_rn(t, t)); break; }
              case kEpSigmoid: static_cast<float*>(S.out)[o] = sigmoidf_(v); break;
              default: P.resid[o] = __fadd_rn(eps[2 * lt + i], __fmul_rn(v, eps[2 * P.max_local + 2 * lt + i])); break;
            }
          }
        }
      }
    }
    B200_DENSE_STAMP(3);
    __syncwarp();
  }
  // After an abandoned wait the warp's requests may still be in flight into its slots: give each a
  // bounded chance to land before the CTA retires.
  if (dead && lane == 0) {
    const unsigned long long t_start = globaltimer_ns();
    for (int j = k; j < k + kDrSlots; ++j) {
      if (warp + j * kDrWarps >= (t1 - t0) * split) break;
      while (!mbar_try_wait(full0 + 8 * (j % kDrSlots), uint32_t(j / kDrSlots) & 1u) && globaltimer_ns() - t_start < wait_limit / 10) {
      }
    }
  }
}

}  // namespace b200
