// C ABI of the library (declarations and per-function contracts: include/b200rwkv.h) and the small
// vector kernels that sit between the streaming GEMV launches.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <vector>

#include "stream_gemv.cuh"
#include "tile_gemm.cuh"
#include "sampling.cuh"
#include "dense_gemv.cuh"
#include "decode_step.cuh"
#include "dense_step.cuh"
#include "dense_gemm.cuh"

namespace b200 {

// ---------------------------------------------------------------------------------------- errors
static thread_local char g_err[512] = "";

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int device_sms() {
  static int cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    cached[dev] = n;
  }
  return cached[dev];
}

// ---------------------------------------------------------------------------------------- GEMV launch
static cudaError_t launch_planned(const GemvParams& P, const GemvPlan& plan, bool pdl, cudaStream_t stream) {
  static bool configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(stream_gemv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(plan.grid);
  cfg.blockDim = dim3(kGemvThreads);
  cfg.dynamicSmemBytes = plan.smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, stream_gemv_kernel, P);
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no link against libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Describe a byte matrix p[rows][K] to TMA as [K/128][rows][128 bytes]; one box =
// [box_chunks][box_rows][128 bytes], 128-byte swizzle.
static bool encode_byte_map(CUtensorMap* map, const void* p, unsigned long long rows, int K, int box_rows, int box_chunks) {
  EncodeTiledFn enc = encode_tiled_fn();
  if (!enc) return false;
  const cuuint64_t gdim[3] = {128, cuuint64_t(rows), cuuint64_t(K / 128)};
  const cuuint64_t gstr[2] = {cuuint64_t(K), 128};
  const cuuint32_t box[3] = {128, cuuint32_t(box_rows), cuuint32_t(box_chunks)};
  const cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(p), gdim, gstr, box, estr,
             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static bool encode_weight_map(CUtensorMap* map, const uint8_t* qt, int N, int K, int kc) {
  return encode_byte_map(map, qt, (unsigned long long)N, K, kTileRows, kc / 128);
}

cudaError_t launch_stream_gemv(GemvParams& P, int max_n, bool pdl, cudaStream_t stream, const char** why) {
  const int sms = device_sms();
  GemvPlan plan;
  if (sms <= 0 || !plan_gemv(P.K, P.nseg, max_n, sms, &plan)) {
    *why = "unsupported GEMV shape (k_in must be a multiple of 128 and at most 65536; 1..3 matrices)";
    return cudaErrorInvalidValue;
  }
  P.kc = plan.kc; P.nchunks = plan.nchunks;
  P.stages = plan.stages; P.stage_bytes = plan.stage_bytes; P.rpc16 = plan.rpc16;
  for (int s = 0; s < P.nseg; ++s) {
    if (!encode_weight_map(&P.tmap[s], P.seg[s].qt, P.seg[s].N, P.K, plan.kc)) {
      *why = "cuTensorMapEncodeTiled failed for a weight matrix";
      return cudaErrorInvalidValue;
    }
  }
  *why = "kernel launch failed";
  return launch_planned(P, plan, pdl, stream);
}

cudaError_t launch_vector_prep(const PrepParams& P, bool pdl, cudaStream_t stream, const char** why) {
  static bool configured[64];
  *why = "vector_prep launch failed";
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(vector_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const size_t smem = prep_smem_bytes(P.K, P.mode);
  if (smem > 200 * 1024) {
    *why = "unsupported shape: activation planes do not fit the preparation kernel's shared memory";
    return cudaErrorInvalidValue;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(prep_grid(P.nseg, P.mode));
  cfg.blockDim = dim3(kPrepThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pdl ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, vector_prep_kernel, P);
}

static int check_matrix(const b200rwkv_matrix& m, const char* name) {
  if (!m.qt || !m.ry || !m.my) return fail(B200RWKV_EINVAL, "%s: null qt/ry/my", name);
  if (m.n_out <= 0 || m.k_in <= 0 || (m.k_in % 128) != 0)
    return fail(B200RWKV_EINVAL, "%s: n_out=%d k_in=%d (k_in must be a positive multiple of 128)", name, m.n_out, m.k_in);
  if (!aligned16(m.qt) || !aligned16(m.ry) || !aligned16(m.my))
    return fail(B200RWKV_EINVAL, "%s: qt/ry/my must be 16-byte aligned", name);
  return B200RWKV_OK;
}

static void fill_seg(GemvSeg& s, const b200rwkv_matrix& m) {
  memset(&s, 0, sizeof(s));
  s.qt = m.qt; s.rx = m.rx; s.mx = m.mx;
  s.half = m.half; s.N = m.n_out; s.act = ACT_NONE;
}

constexpr int kNextPrefetchBytes = 384 * 1024;  // per CTA; x147 CTAs = 56 MB of the 126 MB L2

// Tell launch P which matrices the following launch streams (same k_in for all of them).
static void set_next(GemvParams& P, const b200rwkv_matrix* const* next, int n) {
  P.next_nseg = n; P.next_k = n > 0 ? next[0]->k_in : 0; P.next_prefetch = n > 0 ? kNextPrefetchBytes : 0;
  for (int i = 0; i < n; ++i) { P.next_qt[i] = next[i]->qt; P.next_n[i] = next[i]->n_out; }
}

static void fill_prep_seg(PrepSeg& s, const b200rwkv_matrix& m, const float* mix, const float* xin) {
  s.ry = m.ry; s.my = m.my; s.mix = mix; s.xin = xin;
}

static bool wants_sums(const b200rwkv_matrix& m) { return m.rx || m.mx || m.half != 0.f; }

// ---------------------------------------------------------------------------------------- small kernels
// x = LayerNorm(emb[token]) (the reference's emb.py:8-9 gather followed by ln_in, opt.py:63-64).
// First kernel of a decode step: it also clears the step's publication slots and publishes the sum
// and sum of squares of x for the first block's layer norm (slot 0).  With x_in set (a pipeline stage
// behind the first one) the row is the residual stream handed over by the previous stage, taken as it is.
__global__ void __launch_bounds__(512, 1)
embed_ln0_kernel(const float* __restrict__ emb, const long long* __restrict__ token, int D, int V,
                 const float* __restrict__ w, const float* __restrict__ b, float* __restrict__ out,
                 PubSlot* __restrict__ pub, int npub, const float* __restrict__ x_in) {
  __shared__ float red[16];
  __shared__ long long redl[48];
  __shared__ float bc;
  griddep_launch_dependents();
  griddep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < npub * 16; i += 512) reinterpret_cast<long long*>(pub)[i] = 0;
  long long tok = x_in ? 0 : *token;
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const float* row = x_in ? x_in : emb + size_t(tok) * D;
  auto block_sum = [&](float v) -> float {
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (tid == 0) {
      float a = 0.f;
      for (int i = 0; i < 16; ++i) a += red[i];
      bc = a;
    }
    __syncthreads();
    const float r = bc;
    __syncthreads();
    return r;
  };
  float mean = 0.f, sdev = 1.f;
  if (!x_in) {
    float s = 0.f;
    for (int i = tid; i < D; i += 512) s += row[i];
    mean = block_sum(s) / float(D);
    s = 0.f;
    for (int i = tid; i < D; i += 512) { const float c = row[i] - mean; s += c * c; }
    sdev = sqrtf(block_sum(s) / float(D) + 1e-5f);
  }
  long long p_sum = 0, p_sq = 0, p_sqlo = 0;
  for (int i = tid; i < D; i += 512) {
    const float y = x_in ? __ldcg(x_in + i) : w[i] * ((row[i] - mean) / sdev) + b[i];
    out[i] = y;
    p_sum += __float2ll_rn(y * kPubSumScale);
    square_limbs(y, p_sq, p_sqlo);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    p_sum += __shfl_xor_sync(0xffffffffu, p_sum, o); p_sq += __shfl_xor_sync(0xffffffffu, p_sq, o); p_sqlo += __shfl_xor_sync(0xffffffffu, p_sqlo, o);
  }
  if (lane == 0) { redl[warp * 3] = p_sum; redl[warp * 3 + 1] = p_sq; redl[warp * 3 + 2] = p_sqlo; }
  __syncthreads();                      // also orders the zeroing of slot 0 before the store below
  if (tid < 3) {
    long long a = 0;
    for (int i = 0; i < 16; ++i) a += redl[i * 3 + tid];
    if (tid == 0) pub[0].sum = a; else if (tid == 1) pub[0].sq = a; else pub[0].sq_lo = a;
  }
}

// WKV-4 recurrence, one thread per (stream, channel), sequential over T; k/v/y are [B][T][C] so a
// warp reads 32 consecutive channels of one time step.
template <int CONV>
__global__ void __launch_bounds__(128)
wkv_scan_kernel(int B, int T, int C, const float* __restrict__ w, const float* __restrict__ u,
                const float* __restrict__ k, const float* __restrict__ v, float* __restrict__ y,
                float* __restrict__ aa, float* __restrict__ bb, float* __restrict__ pp) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * C) return;
  const int b = idx / C, c = idx - b * C;
  const float wv = w[c], uv = u[c];
  float a = aa[idx], q = bb[idx], p;
  if (CONV == 1) {
    // reference state: a = exp(w) * A, q = exp(w) * Bsum.  In max-trick terms (A = a_m * exp(p_m))
    // that is a_m = a, p_m = -w; an all-zero state maps to the empty max-trick state.
    p = (a == 0.f && q == 0.f) ? -1e30f : -wv;
  } else {
    p = pp[idx];
  }
  const size_t base = size_t(b) * T * C + c;
  for (int t = 0; t < T; ++t) {
    const size_t o = base + size_t(t) * C;
    y[o] = wkv_step(k[o], v[o], wv, uv, a, q, p);
  }
  if (CONV == 1) {
    const float e = expf(wv + p);  // back to the reference convention; pp is left untouched
    aa[idx] = a * e;
    bb[idx] = q * e;
  } else {
    aa[idx] = a; bb[idx] = q; pp[idx] = p;
  }
}

constexpr size_t kTraceStride = 1024 * 8;  // u64 slots per GEMV launch in a decode-step trace

struct Workspace {
  int* status;
  float *xa, *xb, *xs_att, *rf, *xs_ffn, *shift_new;
  unsigned char* planes;
  SegScalars* scal;
  PubSlot* pub;      // one slot per GEMV launch of a step
  size_t bytes;
};

static size_t align256(size_t n) { return (n + 255) / 256 * 256; }

static Workspace carve(const b200rwkv_model* m, void* base) {
  Workspace w;
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t n) { char* r = p ? p + off : nullptr; off += align256(n); return r; };
  const size_t D = size_t(m->n_embd) * 4, F = size_t(m->n_ffn) * 4;
  w.status = reinterpret_cast<int*>(take(256));
  w.xa = reinterpret_cast<float*>(take(D));
  w.xb = reinterpret_cast<float*>(take(D));
  w.xs_att = reinterpret_cast<float*>(take(D));    // sigmoid(r)*wkv, already times the output matrix's ry
  w.rf = reinterpret_cast<float*>(take(D));
  w.shift_new = reinterpret_cast<float*>(take(D));  // next token-shift carry, committed by the following GEMV launch
  w.xs_ffn = reinterpret_cast<float*>(take(F));    // relu(k)^2, already times the value matrix's ry
  w.planes = reinterpret_cast<unsigned char*>(take(3 * D > F ? 3 * D : F));  // 4*K bytes per matrix
  w.scal = reinterpret_cast<SegScalars*>(take(sizeof(SegScalars) * kMaxSeg));
  w.pub = reinterpret_cast<PubSlot*>(take(sizeof(PubSlot) * (4 * size_t(m->n_layer) + 1)));
  w.bytes = off;
  return w;
}

// Scratch of the stand-alone GEMV entry point: [status 256 B][planes nmat*4*K][scalars].
static size_t gemv_workspace_bytes(int k_in, int nmat) {
  return 256 + align256(size_t(nmat) * 4 * k_in) + align256(sizeof(SegScalars) * kMaxSeg);
}


// ---------------------------------------------------------------------------------------- many-rows path
// x[r] = LayerNorm(emb[token[r]]) for R rows (emb.py:8-9 + ln_in, opt.py:63-64); one CTA per row.
__global__ void __launch_bounds__(256)
embed_ln0_rows_kernel(const float* __restrict__ emb, const long long* __restrict__ tokens, int D, int V,
                      const float* __restrict__ w, const float* __restrict__ b, float* __restrict__ out) {
  __shared__ float red[8];
  __shared__ float bc;
  griddep_launch_dependents();
  griddep_wait();
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  long long tok = tokens[blockIdx.x];
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const float* row = emb + size_t(tok) * D;
  float* o = out + size_t(blockIdx.x) * D;
  auto block_sum = [&](float v) -> float {
    v = warp_sum(v);
    if (lane == 0) red[warp] = v;
    __syncthreads();
    if (tid == 0) {
      float a = 0.f;
      for (int i = 0; i < 8; ++i) a += red[i];
      bc = a;
    }
    __syncthreads();
    const float r = bc;
    __syncthreads();
    return r;
  };
  float s = 0.f;
  for (int i = tid; i < D; i += 256) s += row[i];
  const float mean = block_sum(s) / float(D);
  s = 0.f;
  for (int i = tid; i < D; i += 256) { const float c = row[i] - mean; s += c * c; }
  const float sdev = sqrtf(block_sum(s) / float(D) + 1e-5f);
  for (int i = tid; i < D; i += 256) o[i] = w[i] * ((row[i] - mean) / sdev) + b[i];
}

// WKV-4 over rows laid out [stream][T][C]: one thread per (stream, channel), sequential over T,
// max-trick state rows of stream s at aa/bb/pp + s * state_stride; y = gate * wkv written over k.
__global__ void __launch_bounds__(128)
wkv_rows_kernel(int B, int T, int C, const float* __restrict__ w, const float* __restrict__ u, float* __restrict__ k,
                const float* __restrict__ v, const float* __restrict__ gate, float* __restrict__ aa,
                float* __restrict__ bb, float* __restrict__ pp, long long state_stride) {
  griddep_launch_dependents();
  griddep_wait();
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= B * C) return;
  const int s = idx / C, c = idx - s * C;
  const float wv = w[c], uv = u[c];
  const size_t so = size_t(s) * state_stride + c;
  float a = aa[so], q = bb[so], p = pp[so];
  const size_t base = size_t(s) * T * C + c;
  // The recurrence is sequential in t but its inputs are not: fetch eight steps at a time so the
  // chain waits for memory once per eight steps instead of once per step.
  constexpr int U = 8;
  int t = 0;
  for (; t + U <= T; t += U) {
    float kv[U], vv[U], gv[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const size_t o = base + size_t(t + i) * C;
      kv[i] = __ldcg(k + o); vv[i] = __ldcg(v + o); gv[i] = __ldcg(gate + o);
    }
#pragma unroll
    for (int i = 0; i < U; ++i) k[base + size_t(t + i) * C] = gv[i] * wkv_step(kv[i], vv[i], wv, uv, a, q, p);
  }
  for (; t < T; ++t) {
    const size_t o = base + size_t(t) * C;
    k[o] = gate[o] * wkv_step(k[o], v[o], wv, uv, a, q, p);
  }
  aa[so] = a; bb[so] = q; pp[so] = p;
}


// ---- WKV over long rows: T cut into chunks that run in parallel (the recurrence is a scan whose
// state composes: after n steps without input the max-trick state (aa, bb, pp) is (aa, bb, pp + n*w),
// and two states add after bringing them to a common exponent).
constexpr int kWkvChunk = 64;

// Pass 1: thread (stream, chunk j, channel) runs chunk j from the EMPTY state and stores the
// resulting local state (no outputs); the last chunk is not needed.  The thread of chunk 0 also
// copies the stream's state into the scratch (behind the local states): pass 2 reads that snapshot,
// because its last-chunk thread overwrites the state while the other chunks' threads may not have
// started yet.
__global__ void __launch_bounds__(128)
wkv_chunk_state_kernel(int B, int T, int C, int NC, const float* __restrict__ w, const float* __restrict__ k,
                       const float* __restrict__ v, float* __restrict__ loc, const float* __restrict__ aa,
                       const float* __restrict__ bb, const float* __restrict__ pp, long long state_stride) {
  griddep_launch_dependents();
  griddep_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * (NC - 1) * C) return;
  const int c = int(idx % C);
  const int j = int((idx / C) % (NC - 1)), s = int(idx / ((long long)C * (NC - 1)));
  const float wv = w[c];
  float a = 0.f, q = 0.f, p = -1e30f;
  const size_t base = (size_t(s) * T + size_t(j) * kWkvChunk) * C + c;
  constexpr int U = 8;
  for (int t = 0; t < kWkvChunk; t += U) {   // chunks before the last are full
    float kv[U], vv[U];
#pragma unroll
    for (int i = 0; i < U; ++i) { kv[i] = __ldcg(k + base + size_t(t + i) * C); vv[i] = __ldcg(v + base + size_t(t + i) * C); }
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const float ww2 = p + wv, p2 = fmaxf(ww2, kv[i]);
      const float f1 = expf(ww2 - p2), f2 = expf(kv[i] - p2);
      a = f1 * a + f2 * vv[i]; q = f1 * q + f2; p = p2;
    }
  }
  float* o = loc + (size_t(s) * (NC - 1) + j) * 3 * C + c;
  o[0] = a; o[size_t(C)] = q; o[2 * size_t(C)] = p;
  if (j == 0) {
    const size_t so = size_t(s) * state_stride + c;
    float* snap = loc + (size_t(B) * (NC - 1) + s) * 3 * C + c;
    snap[0] = aa[so]; snap[size_t(C)] = bb[so]; snap[2 * size_t(C)] = pp[so];
  }
}

// Pass 2: thread (stream, chunk j, channel) rebuilds the state at the start of chunk j from the
// stream's state and the local states of chunks 0..j-1, then runs chunk j with outputs
// (y = gate * wkv written over k).  The thread of the last chunk stores the stream's new state.
__global__ void __launch_bounds__(128)
wkv_chunk_output_kernel(int B, int T, int C, int NC, const float* __restrict__ w, const float* __restrict__ u,
                        float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ gate,
                        const float* __restrict__ loc, float* __restrict__ aa, float* __restrict__ bb,
                        float* __restrict__ pp, long long state_stride) {
  griddep_launch_dependents();
  griddep_wait();
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)B * NC * C) return;
  const int c = int(idx % C);
  const int j = int((idx / C) % NC), s = int(idx / ((long long)C * NC));
  const float wv = w[c], uv = u[c];
  const size_t so = size_t(s) * state_stride + c;
  const float* snap = loc + (size_t(B) * (NC - 1) + s) * 3 * C + c;   // the state as pass 1 found it
  float a = __ldcg(snap), q = __ldcg(snap + size_t(C)), p = __ldcg(snap + 2 * size_t(C));
  const float wn = wv * float(kWkvChunk);
  for (int i = 0; i < j; ++i) {
    const float* l = loc + (size_t(s) * (NC - 1) + i) * 3 * C + c;
    const float la = __ldcg(l), lq = __ldcg(l + size_t(C)), lp = __ldcg(l + 2 * size_t(C));
    const float pd = p + wn, pm = fmaxf(pd, lp);
    const float e1 = expf(pd - pm), e2 = expf(lp - pm);
    a = e1 * a + e2 * la; q = e1 * q + e2 * lq; p = pm;
  }
  const int t0 = j * kWkvChunk, t1 = t0 + kWkvChunk < T ? t0 + kWkvChunk : T;
  const size_t base = size_t(s) * T * C + c;
  constexpr int U = 8;
  int t = t0;
  for (; t + U <= t1; t += U) {
    float kv[U], vv[U], gv[U];
#pragma unroll
    for (int i = 0; i < U; ++i) {
      const size_t o = base + size_t(t + i) * C;
      kv[i] = __ldcg(k + o); vv[i] = __ldcg(v + o); gv[i] = __ldcg(gate + o);
    }
#pragma unroll
    for (int i = 0; i < U; ++i) k[base + size_t(t + i) * C] = gv[i] * wkv_step(kv[i], vv[i], wv, uv, a, q, p);
  }
  for (; t < t1; ++t) {
    const size_t o = base + size_t(t) * C;
    k[o] = gate[o] * wkv_step(k[o], v[o], wv, uv, a, q, p);
  }
  if (j == NC - 1) { aa[so] = a; bb[so] = q; pp[so] = p; }
}

struct RowsWorkspace {
  int* status;
  float *xa, *xb, *kb, *vb, *rb, *kk, *shift_new, *wkv_loc;
  int* sk_acc;
  unsigned* sk_count;
  signed char* digits;
  SegScalars* scal;
  size_t bytes;
};


static RowsWorkspace carve_rows(const b200rwkv_model* m, int B, int T, void* base) {
  RowsWorkspace w;
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t n) { char* r = p ? p + off : nullptr; off += align256(n); return r; };
  const size_t R = size_t(B) * T, Rpad = size_t(gemm_padded_rows(int(R)));
  const size_t D = size_t(m->n_embd), F = size_t(m->n_ffn);
  w.status = reinterpret_cast<int*>(take(256));
  w.xa = reinterpret_cast<float*>(take(R * D * 4));
  w.xb = reinterpret_cast<float*>(take(R * D * 4));
  w.kb = reinterpret_cast<float*>(take(R * D * 4));
  w.vb = reinterpret_cast<float*>(take(R * D * 4));
  w.rb = reinterpret_cast<float*>(take(R * D * 4));
  w.kk = reinterpret_cast<float*>(take(R * F * 4));
  w.shift_new = reinterpret_cast<float*>(take(size_t(B) * D * 4));
  w.wkv_loc = reinterpret_cast<float*>(take(size_t(B) * size_t((T + kWkvChunk - 1) / kWkvChunk) * 3 * D * 4));   // local chunk states
  w.sk_acc = reinterpret_cast<int*>(take(kSplitAccBytes));        // split-K scratch, zero between launches
  w.sk_count = reinterpret_cast<unsigned*>(take(size_t(kSplitMaxTiles) * 4));
  w.digits = reinterpret_cast<signed char*>(take(kDigits * Rpad * (3 * D > F ? 3 * D : F)));
  w.scal = reinterpret_cast<SegScalars*>(take(sizeof(SegScalars) * kMaxSeg * R));
  w.bytes = off;
  return w;
}

static size_t gemm_workspace_bytes(int k_in, int nmat, int rows) {
  const size_t Rpad = size_t(gemm_padded_rows(rows));
  return 256 + align256(kSplitAccBytes) + align256(size_t(kSplitMaxTiles) * 4) + align256(size_t(nmat) * kDigits * Rpad * k_in) +
         align256(sizeof(SegScalars) * size_t(nmat) * rows);
}

// Launch with programmatic stream serialisation: the kernel may start while its predecessor on the
// stream is still running; every kernel launched this way calls griddepcontrol.wait before it
// touches global memory.
static thread_local bool g_chain_rows = true;   // set per call by forward_rows_impl / gemm_u8

template <typename Kernel, typename... Args>
static cudaError_t launch_chained(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args... args) {
  if (!g_chain_rows) {
    kernel<<<grid, block, smem, stream>>>(args...);
    return cudaGetLastError();
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, args...);
}

template <int NT, int MODE, int G>
static cudaError_t launch_rows_prep_as(const RowsPrepParams& P, dim3 grid, size_t smem, cudaStream_t stream) {
  return launch_chained(rows_prep_kernel<NT, MODE, G>, grid, dim3(NT), smem, stream, P);
}

static cudaError_t launch_rows_prep(const RowsPrepParams& P_in, cudaStream_t stream, const char** why) {
  static bool configured[64];
  static int sm_count[64];
  *why = "rows_prep launch failed";
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  if (!configured[dev]) {
    e = cudaFuncSetAttribute(rows_prep_long_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sm_count[dev], cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  RowsPrepParams P = P_in;
  rows_prep_grouping(P.nseg, P.K, P.mode, P.R, sm_count[dev], &P.segs_per_cta, &P.rows_per_cta);
  const size_t smem = rows_prep_smem(P.K, P.mode);
  const int groups = (P.R + P.rows_per_cta - 1) / P.rows_per_cta;
  if (smem > 200 * 1024 || groups > 65535) {
    *why = "unsupported shape: k_in too large for the row preparation kernel, or more than 65535 rows";
    return cudaErrorInvalidValue;
  }
  const dim3 grid(P.segs_per_cta == 1 ? P.nseg : 1, groups);
  const bool ln = P.mode == ROWS_LN;
  const int threads = rows_prep_threads(P.K, P.mode);
  if (!rows_prep_in_regs(P.K, P.mode, threads)) return launch_chained(rows_prep_long_kernel, grid, dim3(512), smem, stream, P);
  const int G = rows_prep_groups(P.K, threads);
  if (ln) {
    if (threads == 256) switch (G) {
      case 1: return launch_rows_prep_as<256, ROWS_LN, 1>(P, grid, smem, stream);
      case 2: return launch_rows_prep_as<256, ROWS_LN, 2>(P, grid, smem, stream);
      case 3: return launch_rows_prep_as<256, ROWS_LN, 3>(P, grid, smem, stream);
      default: return launch_rows_prep_as<256, ROWS_LN, 4>(P, grid, smem, stream);
    }
    return G <= 3 ? launch_rows_prep_as<512, ROWS_LN, 3>(P, grid, smem, stream) : launch_rows_prep_as<512, ROWS_LN, 4>(P, grid, smem, stream);
  }
  if (threads == 256) switch (G) {
    case 1: return launch_rows_prep_as<256, ROWS_PLAIN, 1>(P, grid, smem, stream);
    case 2: return launch_rows_prep_as<256, ROWS_PLAIN, 2>(P, grid, smem, stream);
    case 3: return launch_rows_prep_as<256, ROWS_PLAIN, 3>(P, grid, smem, stream);
    case 4: return launch_rows_prep_as<256, ROWS_PLAIN, 4>(P, grid, smem, stream);
    case 5: case 6: return launch_rows_prep_as<256, ROWS_PLAIN, 6>(P, grid, smem, stream);
    default: return launch_rows_prep_as<256, ROWS_PLAIN, 8>(P, grid, smem, stream);
  }
  switch (G) {
    case 5: return launch_rows_prep_as<512, ROWS_PLAIN, 5>(P, grid, smem, stream);
    case 6: return launch_rows_prep_as<512, ROWS_PLAIN, 6>(P, grid, smem, stream);
    default: return launch_rows_prep_as<512, ROWS_PLAIN, 8>(P, grid, smem, stream);
  }
}

// Fills the tensor maps of P (weights and digit rows) and launches the tile GEMM.  digits: [nseg][3][Rpad][K].
static cudaError_t launch_tile_gemm(GemmParams& P, const b200rwkv_matrix* const* mats, const signed char* digits,
                                    cudaStream_t stream, const char** why) {
  static bool configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  *why = "tile_gemm launch failed";
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(tile_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kGemmSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  // Tile shape.  The kernel is bound by operand bytes entering each SM (128 bytes of K per step for
  // mt weight rows and 3*Rt digit rows) plus a fixed cost per tile; the launch takes as many rounds
  // as the busiest CTA has tiles.  Few rows want small tiles (many CTAs, every weight byte still
  // read once per row tile from L2); many rows want the 256 x 80 tile (most MACs per byte).
  {
    const long long sms = device_sms() > 0 ? device_sms() : 1;
    const double fixed = 225.0 * 1024;   // ~3 us of a tile (start, accumulator hand-off, epilogue tail) in ingest bytes
    const int nk = P.K / 128;
    double best = 0.0;
    P.mt = 128; P.Rt = 16; P.ksplit = 1;
    for (int mt = 128; mt <= kGemmM; mt += 128) {
      for (int rt = 16; rt <= kGemmRowsMax; rt += 16) {
        long long tiles = 0;
        for (int s = 0; s < P.nseg; ++s) tiles += (long long)((P.R + rt - 1) / rt) * ((P.seg[s].N + mt - 1) / mt);
        for (int ks = 1; ks <= 8; ks *= 2) {
          // K slices: only where the scratch exists and fits, and where they create CTAs the launch lacks
          if (ks > 1 && (!P.sk_acc || mt != 128 || rt > kSplitMaxRt || tiles > kSplitMaxTiles || nk % ks != 0 ||
                         nk / ks < 4 || tiles * (ks / 2) >= sms))
            continue;
          const double rounds = double((tiles * ks + sms - 1) / sms);
          const double reduce = ks > 1 ? 2.0 * mt * kDigits * rt * 4 + 100.0 * 1024 : 0.0;   // atomics out, totals back, ticket
          const double cost = rounds * (double(nk / ks) * 128.0 * (mt + kDigits * rt) + fixed + reduce);
          if (best == 0.0 || cost < best) { best = cost; P.mt = mt; P.Rt = rt; P.ksplit = ks; }
        }
      }
    }
  }
  for (int s = 0; s < P.nseg; ++s) {
    GemmSeg& S = P.seg[s];
    if (!encode_byte_map(&S.wmap, mats[s]->qt, (unsigned long long)S.N, P.K, P.mt, 1) ||
        !encode_byte_map(&S.xmap, digits + size_t(s) * kDigits * P.Rpad * P.K, (unsigned long long)kDigits * P.Rpad, P.K,
                         P.Rt, 1)) {
      *why = "cuTensorMapEncodeTiled failed";
      return cudaErrorInvalidValue;
    }
  }
  P.row_tiles = (P.R + P.Rt - 1) / P.Rt;
  P.block_tiles = gemm_block_tiles(P.row_tiles, P.Rt, P.K);
  P.ntiles = 0;
  for (int s = 0; s < P.nseg; ++s) {
    P.tiles_seg[s] = P.row_tiles * ((P.seg[s].N + P.mt - 1) / P.mt);
    P.ntiles += P.tiles_seg[s];
  }
  const int items = P.ntiles * P.ksplit;
  const dim3 grid(items < device_sms() ? items : device_sms());
  return launch_chained(tile_gemm_kernel, grid, dim3(kGemmThreads), size_t(kGemmSmem), stream, P);
}

static void fill_gemm_seg(GemmSeg& s, const b200rwkv_matrix& m, const SegScalars* scal, float* out, long long ldo) {
  memset(&s, 0, sizeof(s));
  s.rx = m.rx; s.mx = m.mx; s.half = m.half; s.N = m.n_out; s.act = ACT_NONE;
  s.scal = scal; s.out = out; s.ldo = ldo;
}


// Greedy sampling on the device: index of the largest of n values per row (ties: lowest index, as
// torch.argmax on a CPU tensor gives); optionally appended to a history buffer so that a decode
// loop can run without the host reading anything until it ends.
__global__ void __launch_bounds__(1024)
argmax_rows_kernel(const float* __restrict__ x, int n, long long ldx, long long* __restrict__ out,
                   long long* __restrict__ hist, int* __restrict__ hist_count, int hist_cap) {
  __shared__ float sv[32];
  __shared__ int si[32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float* row = x + size_t(blockIdx.x) * ldx;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = tid; i < n; i += 1024) {
    const float v = __ldcg(row + i);
    if (v > best || (v == best && i < bi) || bi == 0x7fffffff) { best = v; bi = i; }
  }
  auto better = [](float v, int i, float w, int j) { return j != 0x7fffffff && (i == 0x7fffffff || w > v || (w == v && j < i)); };
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float w = __shfl_xor_sync(0xffffffffu, best, o);
    const int j = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(best, bi, w, j)) { best = w; bi = j; }
  }
  if (lane == 0) { sv[warp] = best; si[warp] = bi; }
  __syncthreads();
  if (warp == 0) {
    best = sv[lane]; bi = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float w = __shfl_xor_sync(0xffffffffu, best, o);
      const int j = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(best, bi, w, j)) { best = w; bi = j; }
    }
    if (lane == 0) {
      out[blockIdx.x] = bi;
      if (hist && hist_count && blockIdx.x == 0) {
        const int c = *hist_count;
        if (c < hist_cap) hist[c] = bi;
        *hist_count = c + 1;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------- static scratch
// Scratch of b200rwkv_gemv_u8_static: digit planes (up to kStaticPlaneBytes) followed by the
// per-matrix scalars.  Lives in every GPU's memory from the moment the library is loaded there.
constexpr size_t kStaticPlaneBytes = 192 * 1024;   // = 3 matrices x 4 x k_in(16384), or 1 x 4 x 49152
constexpr size_t kStaticScratchBytes = kStaticPlaneBytes + 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];


// ---- whole decode step as one persistent kernel ------------------------------------------------------
// Plan buffer (device, caller-owned): [status 256 B][use counts, abort word 256 B][exchange vectors]
// [per-CTA records][matrix table][vector table].
struct StepLayout {
  size_t off_uses, off_xs_kvr, off_xs_att, off_xs_fkr, off_xs_ffn, off_xs_head;
  size_t off_part_kvr, off_part_att, off_part_fkr, off_part_ffn, off_part_head, off_part_st, off_mats, off_vpack, off_rym, bytes;
};

static StepLayout step_layout(const b200rwkv_model* m) {
  StepLayout o;
  const size_t D = size_t(m->n_embd), F = size_t(m->n_ffn), L = size_t(m->n_layer);
  const size_t G = size_t(32) * kStepPartPerLane * kRecStride;   // records of the largest grid the kernel supports, one 128-byte line each
  size_t off = 256;
  o.off_uses = off; off += 256;
  o.off_xs_kvr = off; off += align256(3 * D * 4);
  o.off_xs_att = off; off += align256(D * 4);
  o.off_xs_fkr = off; off += align256(2 * D * 4);
  o.off_xs_ffn = off; off += align256(F * 4);
  o.off_xs_head = off; off += align256(D * 4);
  o.off_part_kvr = off; off += align256(3 * G * 16);
  o.off_part_att = off; off += align256(G * 16);
  o.off_part_fkr = off; off += align256(2 * G * 16);
  o.off_part_ffn = off; off += align256(G * 16);
  o.off_part_head = off; off += align256(G * 16);
  o.off_part_st = off; off += align256(G * 16);
  o.off_mats = off; off += align256((7 * L + 1) * sizeof(StepMat));
  o.off_vpack = off; off += align256(L * kStepVecs * D * 4);
  o.off_rym = off; off += align256((L * (12 * D + 2 * F) + 2 * D) * 4);
  o.bytes = off;
  return o;
}

static int check_step_model(const b200rwkv_model* m, const char* who) {
  if (!m || !m->layers || !m->emb || !m->ln0_w || !m->ln0_b) return fail(B200RWKV_EINVAL, "%s: null model field", who);
  const int D = m->n_embd, F = m->n_ffn, V = m->n_vocab, L = m->n_layer;
  if (D <= 0 || (D % 128) != 0 || F <= 0 || (F % 128) != 0 || V <= 0 || L <= 0)
    return fail(B200RWKV_EINVAL, "%s: n_embd=%d n_ffn=%d must be positive multiples of 128", who, D, F);
  for (int l = 0; l < L; ++l) {
    const b200rwkv_layer& ly = m->layers[l];
    const b200rwkv_matrix* chk[7] = {&ly.att_key, &ly.att_value, &ly.att_receptance, &ly.att_output,
                                     &ly.ffn_key, &ly.ffn_receptance, &ly.ffn_value};
    const int want_n[7] = {D, D, D, D, F, D, D}, want_k[7] = {D, D, D, D, D, D, F};
    for (int i = 0; i < 7; ++i) {
      if (int rc = check_matrix(*chk[i], who)) return rc;
      if (chk[i]->n_out != want_n[i] || chk[i]->k_in != want_k[i])
        return fail(B200RWKV_EINVAL, "%s: layer %d matrix %d is %dx%d, expected %dx%d", who, l, i, chk[i]->n_out, chk[i]->k_in,
                    want_n[i], want_k[i]);
    }
  }
  if (m->head.qt) {
    if (int rc = check_matrix(m->head, who)) return rc;
    if (m->head.n_out != V || m->head.k_in != D || !m->ln_out_w || !m->ln_out_b)
      return fail(B200RWKV_EINVAL, "%s: head is %dx%d or ln_out missing", who, m->head.n_out, m->head.k_in);
  }
  return B200RWKV_OK;
}

static bool fill_step_mat(StepMat& o, const b200rwkv_matrix& m) {
  memset(&o, 0, sizeof(o));
  o.qt = m.qt; o.ry = m.ry; o.my = m.my; o.rx = m.rx; o.mx = m.mx; o.half = m.half;
  o.N = m.n_out; o.K = m.k_in; o.need_sums = wants_sums(m) ? 1 : 0;
  step_mat_geometry(m.k_in, &o.kc, &o.nchunks);
  return encode_weight_map(&o.tmap, m.qt, m.n_out, m.k_in, o.kc);
}

}  // namespace b200

using namespace b200;

static int dense_elem_bytes(int dtype) { return dtype == B200RWKV_F32 ? 4 : (dtype == B200RWKV_BF16 || dtype == B200RWKV_F16) ? 2 : 0; }

// ---- unquantised weights: one token through the network -------------------------------------------
// Testing the time-out path (b200rwkv_debug_expire_waits): while enabled, the rows launches of the
// unquantised step announce their ring slots but withhold the copies, with this bound on every wait.
static int g_expire_waits = 0;
static unsigned long long g_expire_limit_ns = 0;

// A wait that nothing satisfies: one mbarrier expecting bytes that never come, every thread waits for it
// with the given bound and reports the expiry.
__global__ void __launch_bounds__(64) wait_selftest_kernel(unsigned long long limit_ns, int* status) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t b = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(b, 1);
    abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_arrive_expect_tx(b, 16);
  __syncthreads();
  const bool ok = mbar_wait_limited(b, 0, &abort_flag, limit_ns);
  if (!ok && threadIdx.x == 0 && status) atomicOr(status, B200RWKV_STATUS_WAIT_FULL);
}

struct DenseWorkspace {
  int* status;
  float *x, *gate;
  void *xk, *xv, *xr, *rw, *fk, *fr, *kk, *hx;
  size_t bytes;
};

static DenseWorkspace dense_carve(const b200rwkv_dense_model* m, void* base) {
  DenseWorkspace w;
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t n) { char* r = p ? p + off : nullptr; off += align256(n); return r; };
  const size_t D = size_t(m->n_embd) * 4, F = size_t(m->n_ffn) * 4;    // sized for the widest type
  w.status = reinterpret_cast<int*>(take(256));
  w.x = reinterpret_cast<float*>(take(D));
  w.gate = reinterpret_cast<float*>(take(D));
  w.xk = take(D); w.xv = take(D); w.xr = take(D); w.rw = take(D);
  w.fk = take(D); w.fr = take(D); w.hx = take(D);
  w.kk = take(F);
  w.bytes = off;
  return w;
}

template <typename T>
static cudaError_t dense_launch_vec(const DenseVecParams& P, bool chained, cudaStream_t stream) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(1); cfg.blockDim = dim3(kDsVecThreads); cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = chained ? 1 : 0;
  // Same shared-memory carve-out as the rows kernels it alternates with: an SM whose split between L1
  // and shared memory has to change first drains, which would serialise the chain.
  static bool configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(dense_vec_kernel<T, 1>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dense_vec_kernel<T, 2>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(dense_vec_kernel<T, 3>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int groups = (P.D / 4 + kDsVecThreads - 1) / kDsVecThreads;    // float4 groups per thread
  if (groups <= 1) return cudaLaunchKernelEx(&cfg, dense_vec_kernel<T, 1>, P);
  if (groups == 2) return cudaLaunchKernelEx(&cfg, dense_vec_kernel<T, 2>, P);
  return cudaLaunchKernelEx(&cfg, dense_vec_kernel<T, 3>, P);
}

// Geometry of one rows launch: one CTA per SM, each owning an equal share of the tasks.  A task is cut
// into the fewest K ranges for which 32 ring slots fit beside the staged activation vectors (so the
// ring is as deep in bytes as shared memory allows), and into more while a CTA would have fewer than
// 64 items and a range still has two 16-byte pieces per lane.
static bool dense_rows_geometry(DenseRowsParams& P, int R, int elem_bytes, int sms, int* grid, size_t* smem) {
  const int nx = R == 3 ? 3 : P.nseg;
  const int pieces = P.K * elem_bytes / 16;
  *grid = sms < P.tasks ? sms : P.tasks;
  if (*grid < 1 || pieces < 1) return false;
  P.max_local = (P.tasks + *grid - 1) / *grid;
  const int want = (64 + P.max_local - 1) / P.max_local;
  for (int split = 1; split <= pieces; ++split) {
    const int range = (pieces + split - 1) / split;
    if ((split - 1) * range >= pieces) continue;            // a split whose last range would be empty
    P.row_stride = range * 16;
    P.stage_bytes = (R * P.row_stride + 127) / 128 * 128;
    const DenseRowsLayout lay = dense_rows_layout(nx, P.K, elem_bytes, P.max_local, split, R, P.stage_bytes);
    if (lay.total > size_t(kDrSmemLimit)) continue;
    if (split < want && range >= 128) continue;
    P.split = split;
    *smem = lay.total;
    return true;
  }
  return false;
}

template <typename T, int R>
static cudaError_t dense_launch_rows(DenseRowsParams& P, cudaStream_t stream) {
  static bool configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaErrorInvalidDevice;
  auto kernel = dense_rows_kernel<T, R>;
  if (!configured[dev]) {
    e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDrSmemLimit);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  int grid = 0;
  size_t smem = 0;
  if (!dense_rows_geometry(P, R, int(sizeof(T)), device_sms(), &grid, &smem)) return cudaErrorInvalidValue;
  P.withhold_copies = g_expire_waits;
  P.wait_limit_ns = g_expire_waits ? g_expire_limit_ns : 0;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid); cfg.blockDim = dim3(kDrThreads);
  cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, P);
}

template <typename T>
static int dense_step_impl(const b200rwkv_dense_model* m, int l0, int l1, const int64_t* token, float* state, float* logits,
                           const DenseWorkspace& ws, cudaStream_t st) {
  const int D = m->n_embd, F = m->n_ffn, V = m->n_vocab;
  cudaError_t e;
#define B200_DS_CHECK(call, what)                                                        \
  do {                                                                                   \
    e = (call);                                                                          \
    if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "dense_step: %s: %s", what, cudaGetErrorString(e)); \
  } while (0)
  DenseVecParams vp;
  memset(&vp, 0, sizeof(vp));
  vp.emb = m->emb; vp.token = reinterpret_cast<const long long*>(token);
  vp.ln_w = m->ln0_w; vp.ln_b = m->ln0_b; vp.x_out = ws.x; vp.D = D; vp.V = V;
  if (l0 == 0) B200_DS_CHECK(dense_launch_vec<T>(vp, false, st), "embedding");
  for (int l = l0; l < l1; ++l) {
    const b200rwkv_dense_layer& Lr = m->layers[l];
    float* sl = state + size_t(l) * 5 * D;
    memset(&vp, 0, sizeof(vp));
    vp.x = ws.x; vp.ln_w = Lr.ln1_w; vp.ln_b = Lr.ln1_b; vp.carry = sl; vp.D = D; vp.nmix = 3;
    vp.mix[0] = Lr.att_mix_k; vp.mix[1] = Lr.att_mix_v; vp.mix[2] = Lr.att_mix_r;
    vp.out[0] = ws.xk; vp.out[1] = ws.xv; vp.out[2] = ws.xr;
    B200_DS_CHECK(dense_launch_vec<T>(vp, true, st), "attention mix");

    DenseRowsParams rp;
    memset(&rp, 0, sizeof(rp));
    rp.status = ws.status;
    rp.nseg = 3; rp.K = D; rp.tasks = D;
    rp.seg[0] = DenseSeg{Lr.att_key, ws.xk, nullptr, D, D, 0};
    rp.seg[1] = DenseSeg{Lr.att_value, ws.xv, nullptr, D, D, 0};
    rp.seg[2] = DenseSeg{Lr.att_receptance, ws.xr, nullptr, D, D, 0};
    rp.state = sl; rp.decay = Lr.time_decay; rp.first = Lr.time_first; rp.wkv_out = ws.rw;
    B200_DS_CHECK((dense_launch_rows<T, 3>(rp, st)), "key/value/receptance rows");

    memset(&rp, 0, sizeof(rp));
    rp.status = ws.status;
    rp.nseg = 1; rp.K = D; rp.tasks = (D + 1) / 2;
    rp.seg[0] = DenseSeg{Lr.att_output, ws.rw, nullptr, D, D, kEpResid};
    rp.resid = ws.x;
    B200_DS_CHECK((dense_launch_rows<T, 2>(rp, st)), "attention output rows");

    memset(&vp, 0, sizeof(vp));
    vp.x = ws.x; vp.ln_w = Lr.ln2_w; vp.ln_b = Lr.ln2_b; vp.carry = sl + D; vp.D = D; vp.nmix = 2;
    vp.mix[0] = Lr.ffn_mix_k; vp.mix[1] = Lr.ffn_mix_r;
    vp.out[0] = ws.fk; vp.out[1] = ws.fr;
    B200_DS_CHECK(dense_launch_vec<T>(vp, true, st), "ffn mix");

    memset(&rp, 0, sizeof(rp));
    rp.status = ws.status;
    rp.nseg = 2; rp.K = D; rp.tasks = (F + D + 1) / 2;
    rp.seg[0] = DenseSeg{Lr.ffn_key, ws.fk, ws.kk, D, F, kEpRelu2};
    rp.seg[1] = DenseSeg{Lr.ffn_receptance, ws.fr, ws.gate, D, D, kEpSigmoid};
    B200_DS_CHECK((dense_launch_rows<T, 2>(rp, st)), "ffn key and receptance rows");

    memset(&rp, 0, sizeof(rp));
    rp.status = ws.status;
    rp.nseg = 1; rp.K = F; rp.tasks = (D + 1) / 2;
    rp.seg[0] = DenseSeg{Lr.ffn_value, ws.kk, nullptr, F, D, kEpGated};
    rp.resid = ws.x; rp.gate = ws.gate;
    B200_DS_CHECK((dense_launch_rows<T, 2>(rp, st)), "ffn value rows");
  }
  if (logits && l1 == m->n_layer) {
    memset(&vp, 0, sizeof(vp));
    vp.x = ws.x; vp.ln_w = m->ln_out_w; vp.ln_b = m->ln_out_b; vp.D = D; vp.out[0] = ws.hx;
    B200_DS_CHECK(dense_launch_vec<T>(vp, true, st), "output layer norm");
    DenseRowsParams rp;
    memset(&rp, 0, sizeof(rp));
    rp.status = ws.status;
    rp.nseg = 1; rp.K = D; rp.tasks = (V + 1) / 2;
    rp.seg[0] = DenseSeg{m->head, ws.hx, logits, D, V, kEpStore};
    B200_DS_CHECK((dense_launch_rows<T, 2>(rp, st)), "head rows");
  }
#undef B200_DS_CHECK
  return B200RWKV_OK;
}

// ---- unquantised weights: many rows ------------------------------------------------------------------
struct DenseRowsWorkspace {
  int* status;
  float *xa, *xb, *kb, *vb, *rb, *carry_new, *wkv_loc;
  unsigned short *t0, *t1, *t2, *kk, *hx;
  float* sk_part;        // partial sums of K slices (launches with few rows)
  unsigned* sk_count;    // their tickets, zero between launches
  size_t bytes;
};

static DenseRowsWorkspace dense_carve_rows(const b200rwkv_dense_model* m, int B, int T, void* base) {
  DenseRowsWorkspace w;
  char* p = static_cast<char*>(base);
  size_t off = 0;
  auto take = [&](size_t n) { char* r = p ? p + off : nullptr; off += align256(n); return r; };
  const size_t R = size_t(B) * T, Rpad = size_t(gemm_padded_rows(int(R))), Bpad = size_t(gemm_padded_rows(B));
  const size_t D = size_t(m->n_embd), F = size_t(m->n_ffn);
  w.status = reinterpret_cast<int*>(take(256));
  w.xa = reinterpret_cast<float*>(take(R * D * 4));
  w.xb = reinterpret_cast<float*>(take(R * D * 4));
  w.kb = reinterpret_cast<float*>(take(R * D * 4));
  w.vb = reinterpret_cast<float*>(take(R * D * 4));
  w.rb = reinterpret_cast<float*>(take(R * D * 4));
  w.carry_new = reinterpret_cast<float*>(take(size_t(B) * D * 4));
  w.wkv_loc = reinterpret_cast<float*>(take(size_t(B) * size_t((T + kWkvChunk - 1) / kWkvChunk) * 3 * D * 4));
  w.t0 = reinterpret_cast<unsigned short*>(take(Rpad * D * 2));
  w.t1 = reinterpret_cast<unsigned short*>(take(Rpad * D * 2));
  w.t2 = reinterpret_cast<unsigned short*>(take(Rpad * D * 2));
  w.kk = reinterpret_cast<unsigned short*>(take(Rpad * F * 2));
  w.hx = reinterpret_cast<unsigned short*>(take(Bpad * D * 2));
  w.sk_count = reinterpret_cast<unsigned*>(take(size_t(kDgSplitMaxItems) * 4));
  w.sk_part = reinterpret_cast<float*>(take(R <= size_t(kDgSplitMaxRows) ? kDgSplitBytes : 0));   // only calls with few rows split K
  w.bytes = off;
  return w;
}

// Picks the tile, encodes the tensor maps and launches.  w[s]: [N_s][K] of the 16-bit
// type; x[s]: [rows_alloc][K] of the same type.
static cudaError_t launch_dense_gemm(DGemmParams& P, const void* const* w, const unsigned short* const* x, int K, int rows_alloc,
                                     cudaStream_t stream, const char** why) {
  static bool configured[64];
  *why = "dense_tile_gemm launch failed";
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(dense_tile_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDgSmem);
    if (e != cudaSuccess) return e;
    configured[dev] = true;
  }
  const int sms = device_sms();
  P.ksteps = K * 2 / 128;
  // Tile: rounds of tiles per CTA x (operand bytes of a tile + a fixed cost per tile), over both tile
  // widths and every height that splits the rows evenly.
  double best = 0.0;
  for (int mt = 128; mt <= 256; mt += 128) {
    for (int rt_rows = 1; rt_rows <= (P.R + 15) / 16; ++rt_rows) {
      const int rt = gemm_padded_rows((P.R + rt_rows - 1) / rt_rows);
      if (rt > kDgRowsMax) continue;
      const int row_tiles = (P.R + rt - 1) / rt;
      if (row_tiles != rt_rows) continue;
      long long tiles = 0;
      for (int s = 0; s < P.nseg; ++s) tiles += (long long)row_tiles * ((P.seg[s].N + mt - 1) / mt);
      for (int ks = 1; ks <= 8; ks *= 2) {     // K slices: only where few tiles would leave most SMs idle
        if (ks > 1 && (!P.sk_part || mt != 128 || tiles * ks > kDgSplitMaxItems || tiles * ks * rt > kDgSplitMaxCells ||
                       P.ksteps % ks != 0 || P.ksteps / ks < 4))
          continue;
        const double rounds = double((tiles * ks + sms - 1) / sms);
        const double reduce = ks > 1 ? 2.0 * rt * 128 * 4 + 64.0 * 1024 : 0.0;   // partial sums out and back, ticket
        const double cost = rounds * (double(P.ksteps / ks) * 128.0 * (mt + rt) + 48.0 * 1024 + reduce);
        if (best == 0.0 || cost < best) { best = cost; P.mt = mt; P.Rt = rt; P.ksplit = ks; }
      }
    }
  }
  if (best == 0.0) { *why = "no tile fits"; return cudaErrorInvalidValue; }
  P.row_tiles = (P.R + P.Rt - 1) / P.Rt;
  P.stage_bytes = (P.mt + P.Rt) * 128;
  P.stages = kDgRingBytes / P.stage_bytes < kDgMaxStages ? kDgRingBytes / P.stage_bytes : kDgMaxStages;
  P.ntiles = 0;
  for (int s = 0; s < P.nseg; ++s) {
    if (!encode_byte_map(&P.seg[s].wmap, w[s], (unsigned long long)P.seg[s].N, K * 2, P.mt, 1) ||
        !encode_byte_map(&P.seg[s].xmap, x[s], (unsigned long long)rows_alloc, K * 2, P.Rt, 1)) {
      *why = "cuTensorMapEncodeTiled failed";
      return cudaErrorInvalidValue;
    }
    P.tiles_seg[s] = P.row_tiles * ((P.seg[s].N + P.mt - 1) / P.mt);
    P.ntiles += P.tiles_seg[s];
  }
  const int items = P.ntiles * P.ksplit;
  const dim3 grid(items < sms ? items : sms);
  return launch_chained(dense_tile_gemm_kernel, grid, dim3(kGemmThreads), size_t(kDgSmem), stream, P);
}

static void fill_dgemm_seg(DGemmSeg& s, int N, void* out, long long ldo, int act, int out_t) {
  memset(&s, 0, sizeof(s));
  s.N = N; s.out = out; s.ldo = ldo; s.act = act; s.out_t = out_t;
}

static const char* dense_model_problem(const b200rwkv_dense_model* m) {
  if (!m || !m->layers || !m->emb || !m->head || !m->ln0_w || !m->ln0_b || !m->ln_out_w || !m->ln_out_b) return "null pointer in the model";
  if (m->n_layer < 1 || m->n_vocab < 1 || m->n_embd < 8 || m->n_ffn < 8) return "bad dimensions";
  if (m->n_embd % 8 || m->n_ffn % 8) return "n_embd and n_ffn must be multiples of 8";
  if (m->n_embd > kDsMaxEmbd) return "n_embd above 12160";
  const int eb = dense_elem_bytes(m->dtype);
  if (!eb) return "unknown dtype";
  if (size_t(3) * m->n_embd * eb > size_t(160) * 1024 || size_t(m->n_ffn) * eb > size_t(160) * 1024) return "rows too long to stage in shared memory";
  if (!aligned16(m->head)) return "head not 16-byte aligned";
  for (int l = 0; l < m->n_layer; ++l) {
    const b200rwkv_dense_layer& L = m->layers[l];
    const void* ptrs[] = {L.ln1_w, L.ln1_b, L.ln2_w, L.ln2_b, L.att_mix_k, L.att_mix_v, L.att_mix_r, L.ffn_mix_k, L.ffn_mix_r,
                          L.time_decay, L.time_first, L.att_key, L.att_value, L.att_receptance, L.att_output, L.ffn_key,
                          L.ffn_receptance, L.ffn_value};
    for (const void* q : ptrs) if (!q) return "null pointer in a layer";
    const void* mats[] = {L.att_key, L.att_value, L.att_receptance, L.att_output, L.ffn_key, L.ffn_receptance, L.ffn_value};
    for (const void* q : mats) if (!aligned16(q)) return "a matrix is not 16-byte aligned";
  }
  return nullptr;
}

extern "C" {

int b200rwkv_version(void) { return 100; }

const char* b200rwkv_last_error(void) { return g_err; }

static int gemv_u8_impl(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y, int accumulate,
                        void* workspace, size_t workspace_bytes, unsigned long long* trace, void* stream) {
  if (nmat < 1 || nmat > kMaxSeg || !mats || !x || !y || !workspace)
    return fail(B200RWKV_EINVAL, "gemv_u8: nmat=%d or null argument", nmat);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(B200RWKV_EINVAL, "gemv_u8: workspace must be 256-byte aligned");
  GemvParams P;
  PrepParams Q;
  memset(&P, 0, sizeof(P));
  memset(&Q, 0, sizeof(Q));
  int max_n = 0;
  for (int i = 0; i < nmat; ++i) {
    if (int rc = check_matrix(mats[i], "gemv_u8 matrix")) return rc;
    if (mats[i].k_in != mats[0].k_in) return fail(B200RWKV_EINVAL, "gemv_u8: matrices must share k_in");
    if (!x[i] || !y[i] || !aligned16(x[i])) return fail(B200RWKV_EINVAL, "gemv_u8: x/y null or x not 16-byte aligned");
    fill_seg(P.seg[i], mats[i]);
    P.seg[i].out = y[i];
    fill_prep_seg(Q.seg[i], mats[i], nullptr, x[i]);
    if (mats[i].n_out > max_n) max_n = mats[i].n_out;
  }
  const int K = mats[0].k_in;
  if (workspace_bytes < gemv_workspace_bytes(K, nmat))
    return fail(B200RWKV_EINVAL, "gemv_u8: workspace %zu < %zu bytes", workspace_bytes, gemv_workspace_bytes(K, nmat));
  char* wsb = static_cast<char*>(workspace);
  int* status = reinterpret_cast<int*>(wsb);
  unsigned char* planes = reinterpret_cast<unsigned char*>(wsb + 256);
  SegScalars* scal = reinterpret_cast<SegScalars*>(wsb + 256 + align256(size_t(nmat) * 4 * K));
  Q.nseg = nmat; Q.K = K; Q.mode = PREP_PLAIN; Q.planes = planes; Q.scal = scal; Q.need_sums = 1;
  Q.trace = trace ? trace + 1023 * 8 : nullptr;
  P.nseg = nmat; P.K = K; P.epi = EPI_GENERIC; P.accumulate = accumulate ? 1 : 0;
  P.planes = planes; P.scal = scal; P.status = status; P.trace = trace;
  const char* why = "";
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = launch_vector_prep(Q, false, s, &why);
  if (e == cudaSuccess) e = launch_stream_gemv(P, max_n, true, s, &why);
  if (e != cudaSuccess) return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "gemv_u8: %s (%s)", why, cudaGetErrorString(e));
  return B200RWKV_OK;
}

size_t b200rwkv_gemv_workspace_bytes(int k_in, int nmat) {
  if (k_in <= 0 || nmat < 1 || nmat > kMaxSeg) return 0;
  return gemv_workspace_bytes(k_in, nmat);
}

int b200rwkv_gemv_u8(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y, int accumulate,
                     void* workspace, size_t workspace_bytes, void* stream) {
  return gemv_u8_impl(nmat, mats, x, y, accumulate, workspace, workspace_bytes, nullptr, stream);
}

int b200rwkv_gemv_u8_traced(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y,
                            int accumulate, void* workspace, size_t workspace_bytes, uint64_t* trace, void* stream) {
  if (!trace) return fail(B200RWKV_EINVAL, "gemv_u8_traced: null trace buffer");
  return gemv_u8_impl(nmat, mats, x, y, accumulate, workspace, workspace_bytes,
                      reinterpret_cast<unsigned long long*>(trace), stream);
}

int b200rwkv_gemv_u8_static(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y,
                            int accumulate, int* status, void* stream) {
  if (nmat < 1 || nmat > kMaxSeg || !mats || !x || !y) return fail(B200RWKV_EINVAL, "gemv_u8_static: nmat=%d or null argument", nmat);
  // In host code the name of a __device__ array is only a handle.  Its device address is looked up
  // once per device, with that device current, and cached; the kernels are given the address.
  static unsigned char* scratch_of_device[64];
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) return fail(B200RWKV_ECUDA, "gemv_u8_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (!scratch_of_device[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || !p) return fail(B200RWKV_ECUDA, "gemv_u8_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    scratch_of_device[dev] = static_cast<unsigned char*>(p);
  }
  GemvParams P;
  PrepParams Q;
  memset(&P, 0, sizeof(P));
  memset(&Q, 0, sizeof(Q));
  int max_n = 0;
  for (int i = 0; i < nmat; ++i) {
    if (int rc = check_matrix(mats[i], "gemv_u8_static matrix")) return rc;
    if (mats[i].k_in != mats[0].k_in) return fail(B200RWKV_EINVAL, "gemv_u8_static: matrices must share k_in");
    if (!x[i] || !y[i] || !aligned16(x[i])) return fail(B200RWKV_EINVAL, "gemv_u8_static: x/y null or x not 16-byte aligned");
    fill_seg(P.seg[i], mats[i]);
    P.seg[i].out = y[i];
    fill_prep_seg(Q.seg[i], mats[i], nullptr, x[i]);
    if (mats[i].n_out > max_n) max_n = mats[i].n_out;
  }
  const int K = mats[0].k_in;
  const size_t need = size_t(nmat) * 4 * K;
  if (need > kStaticPlaneBytes)
    return fail(B200RWKV_EINVAL, "gemv_u8_static: nmat * 4 * k_in = %zu bytes exceeds the built-in scratch of %zu bytes "
                "(use b200rwkv_gemv_u8 with a caller-provided workspace)", need, kStaticPlaneBytes);
  unsigned char* planes = scratch_of_device[dev];
  SegScalars* scal = reinterpret_cast<SegScalars*>(planes + kStaticPlaneBytes);
  Q.nseg = nmat; Q.K = K; Q.mode = PREP_PLAIN; Q.planes = planes; Q.scal = scal; Q.need_sums = 1;
  P.nseg = nmat; P.K = K; P.epi = EPI_GENERIC; P.accumulate = accumulate ? 1 : 0;
  P.planes = planes; P.scal = scal; P.status = status;
  const char* why = "";
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  e = launch_vector_prep(Q, false, s, &why);
  if (e == cudaSuccess) e = launch_stream_gemv(P, max_n, true, s, &why);
  if (e != cudaSuccess) return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "gemv_u8_static: %s (%s)", why, cudaGetErrorString(e));
  return B200RWKV_OK;
}

int b200rwkv_wkv_scan(int B, int T, int C, const float* w, const float* u, const float* k, const float* v, float* y,
                      float* aa, float* bb, float* pp, int convention, void* stream) {
  if (B <= 0 || T < 0 || C <= 0 || !w || !u || !k || !v || !y || !aa || !bb || (convention == 0 && !pp))
    return fail(B200RWKV_EINVAL, "wkv_scan: bad shape B=%d T=%d C=%d or null pointer", B, T, C);
  if (convention != 0 && convention != 1) return fail(B200RWKV_EINVAL, "wkv_scan: convention must be 0 or 1");
  if ((long long)B * C > 0x7fffffffLL) return fail(B200RWKV_EINVAL, "wkv_scan: B*C too large");
  const int n = B * C, block = 128, grid = (n + block - 1) / block;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (convention == 0) wkv_scan_kernel<0><<<grid, block, 0, s>>>(B, T, C, w, u, k, v, y, aa, bb, pp);
  else wkv_scan_kernel<1><<<grid, block, 0, s>>>(B, T, C, w, u, k, v, y, aa, bb, pp);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "wkv_scan: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

int b200rwkv_gemv_plan(int k_in, int nmat, int max_n_out, int num_sms, int64_t* out) {
  GemvPlan p;
  if (!out || num_sms <= 0 || !plan_gemv(k_in, nmat, max_n_out, num_sms, &p))
    return fail(B200RWKV_EINVAL, "gemv_plan: unsupported shape k_in=%d nmat=%d n_out=%d sms=%d", k_in, nmat, max_n_out, num_sms);
  const int64_t v[10] = {p.kc, p.nchunks, 128, kTileRows, p.stages, p.stage_bytes, p.rpc16, p.grid, (int64_t)p.smem, kConsumers};
  for (int i = 0; i < 10; ++i) out[i] = v[i];
  return B200RWKV_OK;
}

size_t b200rwkv_decode_workspace_bytes(const b200rwkv_model* m) {
  if (!m || m->n_embd <= 0 || m->n_ffn <= 0) return 0;
  return carve(m, nullptr).bytes;
}

// x_io: null for a whole model.  Else the step is one pipeline stage: without `token` the residual stream
// is read from x_io instead of the embedding, and in any case the stage's result is left in x_io.
static int decode_step_impl(const b200rwkv_model* m, const int64_t* token, float* x_io, float* state, float* logits, void* workspace,
                            size_t workspace_bytes, unsigned long long* trace, void* stream) {
  if (!m || (!token && !x_io) || !state || !workspace || !m->layers || (token && !m->emb))
    return fail(B200RWKV_EINVAL, "decode_step: null argument");
  if (x_io && !aligned16(x_io)) return fail(B200RWKV_EINVAL, "decode_step: x must be 16-byte aligned");
  const int D = m->n_embd, F = m->n_ffn, V = m->n_vocab, L = m->n_layer;
  if (D <= 0 || (D % 128) != 0 || F <= 0 || (F % 128) != 0 || ((token || logits) && V <= 0) || L <= 0)
    return fail(B200RWKV_EINVAL, "decode_step: n_embd=%d n_ffn=%d must be positive multiples of 128", D, F);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || !aligned16(state))
    return fail(B200RWKV_EINVAL, "decode_step: workspace must be 256-byte and state 16-byte aligned");
  Workspace ws = carve(m, workspace);
  if (workspace_bytes < ws.bytes) return fail(B200RWKV_EINVAL, "decode_step: workspace %zu < %zu bytes", workspace_bytes, ws.bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char* why = "";
  cudaError_t e;
  int li = 0;  // GEMV launch index, selects the slice of the optional trace buffer
  auto trace_slice = [&]() -> unsigned long long* { return trace ? trace + size_t(li++) * kTraceStride : nullptr; };

  {  // embedding gather + ln0, chained like every other launch
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(512); cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, embed_ln0_kernel, m->emb, reinterpret_cast<const long long*>(token), D, V, m->ln0_w,
                           m->ln0_b, ws.xa, ws.pub, 4 * L + 1, token ? static_cast<const float*>(nullptr) : static_cast<const float*>(x_io));
    if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "decode_step: embed launch: %s", cudaGetErrorString(e));
  }

  for (int l = 0; l < L; ++l) {
    const b200rwkv_layer& ly = m->layers[l];
    float* st = state + size_t(l) * 5 * D;
    const b200rwkv_matrix* chk[7] = {&ly.att_key, &ly.att_value, &ly.att_receptance, &ly.att_output,
                                     &ly.ffn_key, &ly.ffn_receptance, &ly.ffn_value};
    const int want_n[7] = {D, D, D, D, F, D, D}, want_k[7] = {D, D, D, D, D, D, F};
    for (int i = 0; i < 7; ++i) {
      if (int rc = check_matrix(*chk[i], "decode_step layer matrix")) return rc;
      if (chk[i]->n_out != want_n[i] || chk[i]->k_in != want_k[i])
        return fail(B200RWKV_EINVAL, "decode_step: layer %d matrix %d is %dx%d, expected %dx%d", l, i, chk[i]->n_out,
                    chk[i]->k_in, want_n[i], want_k[i]);
    }
    GemvParams P;
    PrepParams Q;
    PubSlot* pub = ws.pub + 4 * size_t(l);   // slot j feeds the preparation of GEMV launch j of the step
    // 1. ln1 + token-shift mix (carry = state row 0) -> key/value/receptance -> WKV update ->
    //    sigmoid(r)*wkv, written already scaled for the output projection
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.att_key, ly.att_mix_k, nullptr);
    fill_prep_seg(Q.seg[1], ly.att_value, ly.att_mix_v, nullptr);
    fill_prep_seg(Q.seg[2], ly.att_receptance, ly.att_mix_r, nullptr);
    Q.nseg = 3; Q.K = D; Q.mode = PREP_LN; Q.ln_x = ws.xa; Q.ln_w = ly.ln1_w; Q.ln_b = ly.ln1_b; Q.shift = st; Q.shift_out = ws.shift_new;
    Q.need_sums = wants_sums(ly.att_key) || wants_sums(ly.att_value) || wants_sums(ly.att_receptance);
    Q.pub = pub + 0;
    Q.planes = ws.planes; Q.scal = ws.scal; Q.trace = trace ? trace + size_t(li) * kTraceStride + 1023 * 8 : nullptr;
    if ((e = launch_vector_prep(Q, true, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.att_key); fill_seg(P.seg[1], ly.att_value); fill_seg(P.seg[2], ly.att_receptance);
    P.nseg = 3; P.K = D; P.planes = ws.planes; P.scal = ws.scal;
    P.epi = EPI_WKV; P.wkv_w = ly.time_decay; P.wkv_u = ly.time_first;
    P.aa = st + 2 * size_t(D); P.bb = st + 3 * size_t(D); P.pp = st + 4 * size_t(D);
    P.commit_src = ws.shift_new; P.commit_dst = st; P.commit_n = D;
    P.seg[0].xs_out = ws.xs_att; P.seg[0].xs_ry = ly.att_output.ry; P.seg[0].xs_my = ly.att_output.my; P.seg[0].pub_xs = pub + 1;
    { const b200rwkv_matrix* nx[1] = {&ly.att_output}; set_next(P, nx, 1); }
    P.status = ws.status; P.trace = trace_slice();
    if ((e = launch_stream_gemv(P, D, true, s, &why)) != cudaSuccess) goto launch_failed;
    // 2. attention output projection + residual; publishes the layer-norm sums of the new residual
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.att_output, nullptr, ws.xs_att);
    Q.nseg = 1; Q.K = D; Q.mode = PREP_XS; Q.pub = pub + 1; Q.planes = ws.planes; Q.scal = ws.scal;
    Q.trace = trace ? trace + size_t(li) * kTraceStride + 1023 * 8 : nullptr;
    if ((e = launch_vector_prep(Q, true, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.att_output); P.seg[0].out = ws.xb; P.seg[0].res = ws.xa;
    P.nseg = 1; P.K = D; P.planes = ws.planes; P.scal = ws.scal; P.epi = EPI_GENERIC; P.pub_ln = pub + 2;
    { const b200rwkv_matrix* nx[2] = {&ly.ffn_key, &ly.ffn_receptance}; set_next(P, nx, 2); }
    P.status = ws.status; P.trace = trace_slice();
    if ((e = launch_stream_gemv(P, D, true, s, &why)) != cudaSuccess) goto launch_failed;
    // 3. ln2 + token-shift mix (carry = state row 1) -> ffn key (relu^2, written already scaled for
    //    the value projection) and ffn receptance (sigmoid)
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.ffn_key, ly.ffn_mix_k, nullptr);
    fill_prep_seg(Q.seg[1], ly.ffn_receptance, ly.ffn_mix_r, nullptr);
    Q.nseg = 2; Q.K = D; Q.mode = PREP_LN; Q.ln_x = ws.xb; Q.ln_w = ly.ln2_w; Q.ln_b = ly.ln2_b; Q.shift = st + size_t(D); Q.shift_out = ws.shift_new;
    Q.need_sums = wants_sums(ly.ffn_key) || wants_sums(ly.ffn_receptance);
    Q.pub = pub + 2;
    Q.planes = ws.planes; Q.scal = ws.scal; Q.trace = trace ? trace + size_t(li) * kTraceStride + 1023 * 8 : nullptr;
    if ((e = launch_vector_prep(Q, true, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.ffn_key);        P.seg[0].act = ACT_RELUSQ;
    P.seg[0].xs_out = ws.xs_ffn; P.seg[0].xs_ry = ly.ffn_value.ry; P.seg[0].xs_my = ly.ffn_value.my; P.seg[0].pub_xs = pub + 3;
    fill_seg(P.seg[1], ly.ffn_receptance); P.seg[1].act = ACT_SIGMOID; P.seg[1].out = ws.rf;
    P.nseg = 2; P.K = D; P.planes = ws.planes; P.scal = ws.scal; P.epi = EPI_GENERIC;
    P.commit_src = ws.shift_new; P.commit_dst = st + size_t(D); P.commit_n = D;
    { const b200rwkv_matrix* nx[1] = {&ly.ffn_value}; set_next(P, nx, 1); }
    P.status = ws.status; P.trace = trace_slice();
    if ((e = launch_stream_gemv(P, F > D ? F : D, true, s, &why)) != cudaSuccess) goto launch_failed;
    // 4. ffn value projection, gated by the receptance, + residual; publishes the layer-norm sums
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.ffn_value, nullptr, ws.xs_ffn);
    Q.nseg = 1; Q.K = F; Q.mode = PREP_XS; Q.pub = pub + 3; Q.planes = ws.planes; Q.scal = ws.scal;
    Q.trace = trace ? trace + size_t(li) * kTraceStride + 1023 * 8 : nullptr;
    if ((e = launch_vector_prep(Q, true, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.ffn_value); P.seg[0].out = ws.xa; P.seg[0].res = ws.xb; P.seg[0].gate = ws.rf;
    P.nseg = 1; P.K = F; P.planes = ws.planes; P.scal = ws.scal; P.epi = EPI_GENERIC; P.pub_ln = pub + 4;
    if (l + 1 < L) {
      const b200rwkv_layer& nl = m->layers[l + 1];
      const b200rwkv_matrix* nx[3] = {&nl.att_key, &nl.att_value, &nl.att_receptance};
      set_next(P, nx, 3);
    } else if (logits) {
      const b200rwkv_matrix* nx[1] = {&m->head};
      set_next(P, nx, 1);
    }
    P.status = ws.status; P.trace = trace_slice();
    if ((e = launch_stream_gemv(P, D, true, s, &why)) != cudaSuccess) goto launch_failed;
  }
  if (logits) {
    if (int rc = check_matrix(m->head, "decode_step head")) return rc;
    if (m->head.n_out != V || m->head.k_in != D) return fail(B200RWKV_EINVAL, "decode_step: head is %dx%d", m->head.n_out, m->head.k_in);
    GemvParams P;
    PrepParams Q;
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], m->head, nullptr, nullptr);
    Q.nseg = 1; Q.K = D; Q.mode = PREP_LN; Q.ln_x = ws.xa; Q.ln_w = m->ln_out_w; Q.ln_b = m->ln_out_b;
    Q.need_sums = wants_sums(m->head);
    Q.pub = ws.pub + 4 * size_t(L);
    Q.planes = ws.planes; Q.scal = ws.scal; Q.trace = trace ? trace + size_t(li) * kTraceStride + 1023 * 8 : nullptr;
    if ((e = launch_vector_prep(Q, true, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], m->head); P.seg[0].out = logits;
    P.nseg = 1; P.K = D; P.planes = ws.planes; P.scal = ws.scal; P.epi = EPI_GENERIC;
    {  // the next decode step starts with layer 0's key/value/receptance
      const b200rwkv_matrix* nx[3] = {&m->layers[0].att_key, &m->layers[0].att_value, &m->layers[0].att_receptance};
      set_next(P, nx, 3);
    }
    P.status = ws.status; P.trace = trace_slice();
    if ((e = launch_stream_gemv(P, V, true, s, &why)) != cudaSuccess) goto launch_failed;
  }
  if (x_io) {      // hand the residual stream to the next stage
    why = "copy of the residual stream";
    if ((e = cudaMemcpyAsync(x_io, ws.xa, size_t(D) * 4, cudaMemcpyDeviceToDevice, s)) != cudaSuccess) goto launch_failed;
  }
  return B200RWKV_OK;
launch_failed:
  return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "decode_step: %s (%s)", why, cudaGetErrorString(e));
}

int b200rwkv_decode_step(const b200rwkv_model* m, const int64_t* token, float* state, float* logits, void* workspace,
                         size_t workspace_bytes, void* stream) {
  if (!token) return fail(B200RWKV_EINVAL, "decode_step: null argument");
  return decode_step_impl(m, token, nullptr, state, logits, workspace, workspace_bytes, nullptr, stream);
}

int b200rwkv_decode_step_stage(const b200rwkv_model* m, const int64_t* token, float* x, float* state, float* logits,
                               void* workspace, size_t workspace_bytes, void* stream) {
  if (!x) return fail(B200RWKV_EINVAL, "decode_step_stage: null x");
  return decode_step_impl(m, token, x, state, logits, workspace, workspace_bytes, nullptr, stream);
}

int b200rwkv_decode_step_traced(const b200rwkv_model* m, const int64_t* token, float* state, float* logits,
                                void* workspace, size_t workspace_bytes, uint64_t* trace, void* stream) {
  if (!trace) return fail(B200RWKV_EINVAL, "decode_step_traced: null trace buffer");
  if (!token) return fail(B200RWKV_EINVAL, "decode_step_traced: null argument");
  return decode_step_impl(m, token, nullptr, state, logits, workspace, workspace_bytes, reinterpret_cast<unsigned long long*>(trace), stream);
}


// ---- persistent decode step --------------------------------------------------------------------------
size_t b200rwkv_step_plan_bytes(const b200rwkv_model* m) {
  if (!m || m->n_embd <= 0 || m->n_ffn <= 0 || m->n_layer <= 0) return 0;
  return step_layout(m).bytes;
}

int b200rwkv_step_geometry(const b200rwkv_model* m, int num_sms, int64_t* out) {
  StepPlan p;
  if (!m || !out || !plan_step(m->n_embd, m->n_ffn, m->n_vocab, m->head.qt != nullptr, num_sms, &p))
    return fail(B200RWKV_EINVAL, "step_geometry: unsupported shape");
  const int64_t v[8] = {p.grid, p.stages, p.slot_bytes, (int64_t)p.smem, p.off_rows, p.off_planes, p.off_ring, kStepThreads};
  for (int i = 0; i < 8; ++i) out[i] = v[i];
  return B200RWKV_OK;
}

int b200rwkv_step_plan_init(const b200rwkv_model* m, void* plan, size_t plan_bytes) {
  if (int rc = check_step_model(m, "step_plan_init")) return rc;
  if (!plan || (reinterpret_cast<uintptr_t>(plan) & 255u) != 0) return fail(B200RWKV_EINVAL, "step_plan_init: plan must be 256-byte aligned");
  const StepLayout lay = step_layout(m);
  if (plan_bytes < lay.bytes) return fail(B200RWKV_EINVAL, "step_plan_init: plan %zu < %zu bytes", plan_bytes, lay.bytes);
  StepPlan geo;
  if (device_sms() <= 0 || !plan_step(m->n_embd, m->n_ffn, m->n_vocab, m->head.qt != nullptr, device_sms(), &geo))
    return fail(B200RWKV_EINVAL, "step_plan_init: the shape does not fit the step kernel's shared memory");
  const int L = m->n_layer;
  std::vector<StepMat> mats(static_cast<size_t>(7 * L + 1));
  memset(mats.data(), 0, mats.size() * sizeof(StepMat));
  char* base = static_cast<char*>(plan);
  cudaError_t e = cudaMemset(base, 0, lay.bytes);
  const size_t D = size_t(m->n_embd), F = size_t(m->n_ffn);
  float* vpack = reinterpret_cast<float*>(base + lay.off_vpack);
  float* rym = reinterpret_cast<float*>(base + lay.off_rym);
  const size_t rym_stride = 12 * D + 2 * F;
  auto copy_vec = [&](float* dst, const float* src, size_t n) {
    if (e == cudaSuccess) e = cudaMemcpy(dst, src, n * sizeof(float), cudaMemcpyDeviceToDevice);
  };
  for (int l = 0; l < L; ++l) {
    const b200rwkv_layer& ly = m->layers[l];
    const b200rwkv_matrix* ms[7] = {&ly.att_key, &ly.att_value, &ly.att_receptance, &ly.att_output,
                                    &ly.ffn_key, &ly.ffn_receptance, &ly.ffn_value};
    for (int i = 0; i < 7; ++i)
      if (!fill_step_mat(mats[size_t(7) * l + i], *ms[i])) return fail(B200RWKV_ECUDA, "step_plan_init: cuTensorMapEncodeTiled failed");
    const float* vec[kStepVecs] = {ly.ln1_w, ly.ln1_b, ly.ln2_w, ly.ln2_b, ly.att_mix_k, ly.att_mix_v, ly.att_mix_r,
                                   ly.ffn_mix_k, ly.ffn_mix_r, ly.time_decay, ly.time_first};
    for (int i = 0; i < kStepVecs; ++i) {
      if (!vec[i]) return fail(B200RWKV_EINVAL, "step_plan_init: layer %d has a null vector parameter", l);
      copy_vec(vpack + (size_t(l) * kStepVecs + i) * D, vec[i], D);
    }
    // D-input matrices in the order key, value, receptance, output, ffn key, ffn receptance; then ffn value
    const b200rwkv_matrix* dm[6] = {&ly.att_key, &ly.att_value, &ly.att_receptance, &ly.att_output, &ly.ffn_key, &ly.ffn_receptance};
    for (int i = 0; i < 6; ++i) {
      copy_vec(rym + size_t(l) * rym_stride + (size_t(i) * 2 + 0) * D, dm[i]->ry, D);
      copy_vec(rym + size_t(l) * rym_stride + (size_t(i) * 2 + 1) * D, dm[i]->my, D);
    }
    copy_vec(rym + size_t(l) * rym_stride + 12 * D, ly.ffn_value.ry, F);
    copy_vec(rym + size_t(l) * rym_stride + 12 * D + F, ly.ffn_value.my, F);
  }
  if (m->head.qt) {
    if (!fill_step_mat(mats[size_t(7) * L], m->head)) return fail(B200RWKV_ECUDA, "step_plan_init: cuTensorMapEncodeTiled failed");
    copy_vec(rym + size_t(L) * rym_stride, m->head.ry, D);
    copy_vec(rym + size_t(L) * rym_stride + D, m->head.my, D);
  }
  if (e == cudaSuccess) e = cudaMemcpy(base + lay.off_mats, mats.data(), mats.size() * sizeof(StepMat), cudaMemcpyHostToDevice);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "step_plan_init: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

int b200rwkv_decode_step_persistent(const b200rwkv_model* m, void* plan, size_t plan_bytes, const int64_t* token, float* state,
                                    float* logits, const int32_t* tuning, uint64_t* trace, void* stream) {
  if (!m || !plan || !token || !state) return fail(B200RWKV_EINVAL, "decode_step_persistent: null argument");
  if ((reinterpret_cast<uintptr_t>(plan) & 255u) != 0 || !aligned16(state))
    return fail(B200RWKV_EINVAL, "decode_step_persistent: plan must be 256-byte and state 16-byte aligned");
  if (logits && !m->head.qt) return fail(B200RWKV_EINVAL, "decode_step_persistent: logits wanted but the model has no head");
  const StepLayout lay = step_layout(m);
  if (plan_bytes < lay.bytes) return fail(B200RWKV_EINVAL, "decode_step_persistent: plan %zu < %zu bytes", plan_bytes, lay.bytes);
  StepPlan geo;
  if (device_sms() <= 0 || !plan_step(m->n_embd, m->n_ffn, m->n_vocab, m->head.qt != nullptr, device_sms(), &geo))
    return fail(B200RWKV_EINVAL, "decode_step_persistent: the shape does not fit the step kernel's shared memory");
  static bool configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "decode_step_persistent: %s", cudaGetErrorString(e));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
    if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "decode_step_persistent: %s", cudaGetErrorString(e));
    configured[dev] = true;
  }
  char* base = static_cast<char*>(plan);
  StepParams P;
  memset(&P, 0, sizeof(P));
  P.mats = reinterpret_cast<const StepMat*>(base + lay.off_mats);
  P.vpack = reinterpret_cast<const float*>(base + lay.off_vpack);
  P.rympack = reinterpret_cast<const float*>(base + lay.off_rym);
  P.L = m->n_layer; P.D = m->n_embd; P.F = m->n_ffn; P.V = m->n_vocab; P.inv_d = 1.0 / double(m->n_embd);
  P.emb = m->emb; P.ln0_w = m->ln0_w; P.ln0_b = m->ln0_b; P.lnout_w = m->ln_out_w; P.lnout_b = m->ln_out_b;
  P.token = reinterpret_cast<const long long*>(token); P.state = state; P.logits = logits;
  P.xs_kvr = reinterpret_cast<float*>(base + lay.off_xs_kvr);
  P.xs_att = reinterpret_cast<float*>(base + lay.off_xs_att);
  P.xs_fkr = reinterpret_cast<float*>(base + lay.off_xs_fkr);
  P.xs_ffn = reinterpret_cast<float*>(base + lay.off_xs_ffn);
  P.xs_head = reinterpret_cast<float*>(base + lay.off_xs_head);
  P.part_kvr = reinterpret_cast<float4*>(base + lay.off_part_kvr);
  P.part_att = reinterpret_cast<float4*>(base + lay.off_part_att);
  P.part_fkr = reinterpret_cast<float4*>(base + lay.off_part_fkr);
  P.part_ffn = reinterpret_cast<float4*>(base + lay.off_part_ffn);
  P.part_head = reinterpret_cast<float4*>(base + lay.off_part_head);
  P.part_st = reinterpret_cast<float4*>(base + lay.off_part_st);
  P.uses = reinterpret_cast<unsigned*>(base + lay.off_uses);
  P.abort_word = reinterpret_cast<unsigned*>(base + lay.off_uses + 128);
  P.status = reinterpret_cast<int*>(base);
  P.trace = reinterpret_cast<unsigned long long*>(trace);
  P.slot_bytes = geo.slot_bytes; P.stages = geo.stages; P.off_own = geo.off_own; P.own_rows = geo.own_rows;
  P.off_park = geo.off_park; P.park_stride = geo.park_stride;
  P.off_rows = geo.off_rows; P.off_planes = geo.off_planes; P.off_ring = geo.off_ring;
  P.window = tuning && tuning[0] > 0 ? tuning[0] : geo.stages;
  P.window_handoff = tuning && tuning[1] > 0 ? tuning[1] : geo.stages;
  P.pf_bytes = tuning && tuning[2] >= 0 ? tuning[2] : kStepPrefetchDefault;
  P.wait_limit_ns = (tuning && tuning[3] > 0 ? (unsigned long long)tuning[3] : 1000ull) * 1000000ull;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(geo.grid); cfg.blockDim = dim3(kStepThreads); cfg.dynamicSmemBytes = geo.smem; cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;     // all CTAs resident at once, or the launch fails
  attr[0].val.cooperative = 1;
  cfg.attrs = attr; cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, decode_step_kernel, P);
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "decode_step_persistent: launch: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

size_t b200rwkv_gemm_workspace_bytes(int k_in, int nmat, int rows) {
  if (k_in <= 0 || nmat < 1 || nmat > kMaxSeg || rows < 1) return 0;
  return gemm_workspace_bytes(k_in, nmat, rows);
}

int b200rwkv_gemm_u8(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y, int rows,
                     void* workspace, size_t workspace_bytes, void* stream) {
  if (nmat < 1 || nmat > kMaxSeg || !mats || !x || !y || !workspace || rows < 1 || rows > 65535)
    return fail(B200RWKV_EINVAL, "gemm_u8: nmat=%d rows=%d (1..3 matrices, 1..65535 rows) or null argument", nmat, rows);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0) return fail(B200RWKV_EINVAL, "gemm_u8: workspace must be 256-byte aligned");
  const int K = mats[0].k_in;
  for (int i = 0; i < nmat; ++i) {
    if (int rc = check_matrix(mats[i], "gemm_u8 matrix")) return rc;
    if (mats[i].k_in != K) return fail(B200RWKV_EINVAL, "gemm_u8: matrices must share k_in");
    if (!x[i] || !y[i] || !aligned16(x[i])) return fail(B200RWKV_EINVAL, "gemm_u8: x/y null or x not 16-byte aligned");
  }
  if (workspace_bytes < gemm_workspace_bytes(K, nmat, rows))
    return fail(B200RWKV_EINVAL, "gemm_u8: workspace %zu < %zu bytes", workspace_bytes, gemm_workspace_bytes(K, nmat, rows));
  const int Rpad = gemm_padded_rows(rows);
  char* wsb = static_cast<char*>(workspace);
  int* sk_acc = reinterpret_cast<int*>(wsb + 256);
  unsigned* sk_count = reinterpret_cast<unsigned*>(wsb + 256 + align256(kSplitAccBytes));
  char* after = wsb + 256 + align256(kSplitAccBytes) + align256(size_t(kSplitMaxTiles) * 4);
  signed char* digits = reinterpret_cast<signed char*>(after);
  SegScalars* scal = reinterpret_cast<SegScalars*>(after + align256(size_t(nmat) * kDigits * Rpad * K));
  RowsPrepParams Q;
  GemmParams P;
  memset(&Q, 0, sizeof(Q));
  memset(&P, 0, sizeof(P));
  const b200rwkv_matrix* mp[kMaxSeg];
  for (int i = 0; i < nmat; ++i) {
    fill_prep_seg(Q.seg[i], mats[i], nullptr, x[i]);
    fill_gemm_seg(P.seg[i], mats[i], scal + size_t(i) * rows, y[i], mats[i].n_out);
    mp[i] = &mats[i];
  }
  Q.nseg = nmat; Q.K = K; Q.R = rows; Q.T = 1; Q.Rpad = Rpad; Q.mode = ROWS_PLAIN; Q.need_sums = 1; Q.ldx = K;
  Q.digits = digits; Q.scal = scal;
  P.nseg = nmat; P.K = K; P.R = rows; P.Rpad = Rpad; P.status = reinterpret_cast<int*>(wsb); P.sk_acc = sk_acc; P.sk_count = sk_count;
  const char* why = "";
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  g_chain_rows = rows <= 1024;
  cudaError_t e = launch_rows_prep(Q, s, &why);
  if (e == cudaSuccess) e = launch_tile_gemm(P, mp, digits, s, &why);
  if (e != cudaSuccess) return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "gemm_u8: %s (%s)", why, cudaGetErrorString(e));
  return B200RWKV_OK;
}

size_t b200rwkv_rows_workspace_bytes(const b200rwkv_model* m, int streams, int tokens_per_stream) {
  if (!m || m->n_embd <= 0 || m->n_ffn <= 0 || streams < 1 || tokens_per_stream < 1) return 0;
  if ((long long)streams * tokens_per_stream > 65535) return 0;
  return carve_rows(m, streams, tokens_per_stream, nullptr).bytes;
}

// tokens != null: embedding + ln0 produce the rows; else the rows arrive in x_ext.  x_ext != null: the
// residual stream lives there (and is left there for the next pipeline stage) instead of the workspace.
static int forward_rows_impl(const b200rwkv_model* m, const int64_t* tokens, float* x_ext, int streams, int tokens_per_stream,
                             float* state, int64_t state_stride, float* logits, void* workspace, size_t workspace_bytes,
                             void* stream) {
  if (!m || !state || !workspace || !m->layers || (!tokens && !x_ext) || (tokens && !m->emb))
    return fail(B200RWKV_EINVAL, "forward_rows: null argument");
  if (x_ext && !aligned16(x_ext)) return fail(B200RWKV_EINVAL, "forward_rows: x must be 16-byte aligned");
  const int D = m->n_embd, F = m->n_ffn, V = m->n_vocab, L = m->n_layer, B = streams, T = tokens_per_stream;
  if (D <= 0 || (D % 128) != 0 || F <= 0 || (F % 128) != 0 || L <= 0 || ((tokens || logits) && V <= 0))
    return fail(B200RWKV_EINVAL, "forward_rows: n_embd=%d n_ffn=%d must be positive multiples of 128", D, F);
  if (B < 1 || T < 1 || (long long)B * T > 65535) return fail(B200RWKV_EINVAL, "forward_rows: streams=%d x tokens=%d must be 1..65535 rows", B, T);
  if (state_stride < (int64_t)L * 5 * D || (state_stride % 4) != 0)
    return fail(B200RWKV_EINVAL, "forward_rows: state_stride %lld < n_layer*5*n_embd or not a multiple of 4", (long long)state_stride);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || !aligned16(state))
    return fail(B200RWKV_EINVAL, "forward_rows: workspace must be 256-byte and state 16-byte aligned");
  RowsWorkspace ws = carve_rows(m, B, T, workspace);
  if (workspace_bytes < ws.bytes) return fail(B200RWKV_EINVAL, "forward_rows: workspace %zu < %zu bytes", workspace_bytes, ws.bytes);
  const int R = B * T, Rpad = gemm_padded_rows(R);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char* why = "";
  cudaError_t e;

  // Chaining pays when the kernels are short (decode, short prompts: 10-15 % per step); with thousands
  // of rows per launch it measured 9 % slower than plain stream order (3B shape, 4096 rows), so it is off there.
  g_chain_rows = B * T <= 1024;
  if (x_ext) ws.xa = x_ext;
  if (tokens) {
    e = launch_chained(embed_ln0_rows_kernel, dim3(R), dim3(256), 0, s, m->emb, reinterpret_cast<const long long*>(tokens), D, V,
                       m->ln0_w, m->ln0_b, ws.xa);
    if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "forward_rows: embed launch: %s", cudaGetErrorString(e));
  }

  RowsPrepParams Q;
  GemmParams P;
  auto prep_common = [&](int nseg, int K, int mode, const float* ln_x, const float* ln_w, const float* ln_b,
                         const float* shift, bool need_sums) {
    Q.nseg = nseg; Q.K = K; Q.R = R; Q.T = T; Q.Rpad = Rpad; Q.mode = mode; Q.need_sums = need_sums ? 1 : 0; Q.ldx = K;
    Q.ln_x = ln_x; Q.ln_w = ln_w; Q.ln_b = ln_b; Q.shift = shift; Q.shift_stride = state_stride;
    Q.shift_out = mode == ROWS_LN ? ws.shift_new : nullptr; Q.digits = ws.digits; Q.scal = ws.scal;
  };
  auto gemm_common = [&](int nseg, int K) {
    P.nseg = nseg; P.K = K; P.R = R; P.Rpad = Rpad; P.status = ws.status; P.sk_acc = ws.sk_acc; P.sk_count = ws.sk_count;
  };
  // new token-shift carry of every stream -> its state row, done by the NEXT preparation launch
  // (the launch that parked it had sibling CTAs still reading the old row)
  auto commit_carry = [&](float* dst_row) {
    Q.commit_src = ws.shift_new; Q.commit_dst = dst_row; Q.commit_stride = state_stride; Q.commit_n = D;
  };

  for (int l = 0; l < L; ++l) {
    const b200rwkv_layer& ly = m->layers[l];
    float* st = state + size_t(l) * 5 * D;
    const b200rwkv_matrix* chk[7] = {&ly.att_key, &ly.att_value, &ly.att_receptance, &ly.att_output,
                                     &ly.ffn_key, &ly.ffn_receptance, &ly.ffn_value};
    const int want_n[7] = {D, D, D, D, F, D, D}, want_k[7] = {D, D, D, D, D, D, F};
    for (int i = 0; i < 7; ++i) {
      if (int rc = check_matrix(*chk[i], "forward_rows layer matrix")) return rc;
      if (chk[i]->n_out != want_n[i] || chk[i]->k_in != want_k[i])
        return fail(B200RWKV_EINVAL, "forward_rows: layer %d matrix %d is %dx%d, expected %dx%d", l, i, chk[i]->n_out,
                    chk[i]->k_in, want_n[i], want_k[i]);
    }
    // 1. ln1 + token-shift mix -> key, value, sigmoid(receptance)
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.att_key, ly.att_mix_k, nullptr);
    fill_prep_seg(Q.seg[1], ly.att_value, ly.att_mix_v, nullptr);
    fill_prep_seg(Q.seg[2], ly.att_receptance, ly.att_mix_r, nullptr);
    prep_common(3, D, ROWS_LN, ws.xa, ly.ln1_w, ly.ln1_b, st,
                wants_sums(ly.att_key) || wants_sums(ly.att_value) || wants_sums(ly.att_receptance));
    if ((e = launch_rows_prep(Q, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_gemm_seg(P.seg[0], ly.att_key, ws.scal, ws.kb, D);
    fill_gemm_seg(P.seg[1], ly.att_value, ws.scal + size_t(R), ws.vb, D);
    fill_gemm_seg(P.seg[2], ly.att_receptance, ws.scal + 2 * size_t(R), ws.rb, D);
    P.seg[2].act = ACT_SIGMOID;
    gemm_common(3, D);
    { const b200rwkv_matrix* mp[3] = {&ly.att_key, &ly.att_value, &ly.att_receptance};
      if ((e = launch_tile_gemm(P, mp, ws.digits, s, &why)) != cudaSuccess) goto launch_failed; }
    // 2. WKV recurrence over each stream's rows; kb <- sigmoid(r) * wkv
    why = "wkv_rows launch failed";
    if (T <= 2 * kWkvChunk) {
      e = launch_chained(wkv_rows_kernel, dim3((B * D + 127) / 128), dim3(128), 0, s, B, T, D, ly.time_decay, ly.time_first, ws.kb,
                         (const float*)ws.vb, (const float*)ws.rb, st + 2 * size_t(D), st + 3 * size_t(D), st + 4 * size_t(D),
                         (long long)state_stride);
    } else {   // long rows: chunks of 64 steps in parallel, two passes
      const int NC = (T + kWkvChunk - 1) / kWkvChunk;
      const long long n1 = (long long)B * (NC - 1) * D, n2 = (long long)B * NC * D;
      e = launch_chained(wkv_chunk_state_kernel, dim3((unsigned)((n1 + 127) / 128)), dim3(128), 0, s, B, T, D, NC, ly.time_decay,
                         (const float*)ws.kb, (const float*)ws.vb, ws.wkv_loc, (const float*)(st + 2 * size_t(D)),
                         (const float*)(st + 3 * size_t(D)), (const float*)(st + 4 * size_t(D)), (long long)state_stride);
      if (e == cudaSuccess)
        e = launch_chained(wkv_chunk_output_kernel, dim3((unsigned)((n2 + 127) / 128)), dim3(128), 0, s, B, T, D, NC, ly.time_decay,
                           ly.time_first, ws.kb, (const float*)ws.vb, (const float*)ws.rb, (const float*)ws.wkv_loc,
                           st + 2 * size_t(D), st + 3 * size_t(D), st + 4 * size_t(D), (long long)state_stride);
    }
    if (e != cudaSuccess) goto launch_failed;
    // 3. attention output projection + residual -> xb
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.att_output, nullptr, ws.kb);
    prep_common(1, D, ROWS_PLAIN, nullptr, nullptr, nullptr, nullptr, wants_sums(ly.att_output));
    commit_carry(st);                 // ln1 output of each stream's last row -> state row 0
    if ((e = launch_rows_prep(Q, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_gemm_seg(P.seg[0], ly.att_output, ws.scal, ws.xb, D);
    P.seg[0].res = ws.xa; P.seg[0].ldres = D;
    gemm_common(1, D);
    { const b200rwkv_matrix* mp[1] = {&ly.att_output};
      if ((e = launch_tile_gemm(P, mp, ws.digits, s, &why)) != cudaSuccess) goto launch_failed; }
    // 4. ln2 + token-shift mix -> relu(key)^2, sigmoid(receptance)
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.ffn_key, ly.ffn_mix_k, nullptr);
    fill_prep_seg(Q.seg[1], ly.ffn_receptance, ly.ffn_mix_r, nullptr);
    prep_common(2, D, ROWS_LN, ws.xb, ly.ln2_w, ly.ln2_b, st + size_t(D), wants_sums(ly.ffn_key) || wants_sums(ly.ffn_receptance));
    if ((e = launch_rows_prep(Q, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_gemm_seg(P.seg[0], ly.ffn_key, ws.scal, ws.kk, F);
    P.seg[0].act = ACT_RELUSQ;
    fill_gemm_seg(P.seg[1], ly.ffn_receptance, ws.scal + size_t(R), ws.rb, D);
    P.seg[1].act = ACT_SIGMOID;
    gemm_common(2, D);
    { const b200rwkv_matrix* mp[2] = {&ly.ffn_key, &ly.ffn_receptance};
      if ((e = launch_tile_gemm(P, mp, ws.digits, s, &why)) != cudaSuccess) goto launch_failed; }
    // 5. ffn value projection, gated, + residual -> xa
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], ly.ffn_value, nullptr, ws.kk);
    prep_common(1, F, ROWS_PLAIN, nullptr, nullptr, nullptr, nullptr, wants_sums(ly.ffn_value));
    commit_carry(st + size_t(D));     // ln2 output of each stream's last row -> state row 1
    if ((e = launch_rows_prep(Q, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_gemm_seg(P.seg[0], ly.ffn_value, ws.scal, ws.xa, D);
    P.seg[0].res = ws.xb; P.seg[0].ldres = D; P.seg[0].gate = ws.rb; P.seg[0].ldgate = D;
    gemm_common(1, F);
    { const b200rwkv_matrix* mp[1] = {&ly.ffn_value};
      if ((e = launch_tile_gemm(P, mp, ws.digits, s, &why)) != cudaSuccess) goto launch_failed; }
  }
  if (logits) {
    // ln_out + head on the last row of every stream (opt.py:73-75)
    if (int rc = check_matrix(m->head, "forward_rows head")) return rc;
    if (m->head.n_out != V || m->head.k_in != D) return fail(B200RWKV_EINVAL, "forward_rows: head is %dx%d", m->head.n_out, m->head.k_in);
    const int Bpad = gemm_padded_rows(B);
    memset(&Q, 0, sizeof(Q));
    fill_prep_seg(Q.seg[0], m->head, nullptr, nullptr);
    Q.nseg = 1; Q.K = D; Q.R = B; Q.T = 1; Q.Rpad = Bpad; Q.mode = ROWS_LN; Q.need_sums = wants_sums(m->head) ? 1 : 0;
    Q.ldx = (long long)T * D; Q.ln_x = ws.xa + size_t(T - 1) * D; Q.ln_w = m->ln_out_w; Q.ln_b = m->ln_out_b;
    Q.digits = ws.digits; Q.scal = ws.scal;
    if ((e = launch_rows_prep(Q, s, &why)) != cudaSuccess) goto launch_failed;
    memset(&P, 0, sizeof(P));
    fill_gemm_seg(P.seg[0], m->head, ws.scal, logits, V);
    P.nseg = 1; P.K = D; P.R = B; P.Rpad = Bpad; P.status = ws.status; P.sk_acc = ws.sk_acc; P.sk_count = ws.sk_count;
    { const b200rwkv_matrix* mp[1] = {&m->head};
      if ((e = launch_tile_gemm(P, mp, ws.digits, s, &why)) != cudaSuccess) goto launch_failed; }
  }
  return B200RWKV_OK;
launch_failed:
  return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "forward_rows: %s (%s)", why, cudaGetErrorString(e));
}

int b200rwkv_forward_rows(const b200rwkv_model* m, const int64_t* tokens, int streams, int tokens_per_stream, float* state,
                          int64_t state_stride, float* logits, void* workspace, size_t workspace_bytes, void* stream) {
  if (!tokens) return fail(B200RWKV_EINVAL, "forward_rows: null tokens");
  return forward_rows_impl(m, tokens, nullptr, streams, tokens_per_stream, state, state_stride, logits, workspace,
                           workspace_bytes, stream);
}

int b200rwkv_forward_rows_stage(const b200rwkv_model* m, const int64_t* tokens, float* x, int streams, int tokens_per_stream,
                                float* state, int64_t state_stride, float* logits, void* workspace, size_t workspace_bytes,
                                void* stream) {
  if (!x) return fail(B200RWKV_EINVAL, "forward_rows_stage: null x");
  return forward_rows_impl(m, tokens, x, streams, tokens_per_stream, state, state_stride, logits, workspace, workspace_bytes,
                           stream);
}

int b200rwkv_argmax(const float* x, int rows, int n, int64_t ldx, int64_t* out, int64_t* history, int* history_count,
                    int history_capacity, void* stream) {
  if (!x || !out || rows < 1 || n < 1 || ldx < n || (history && (!history_count || history_capacity < 1)))
    return fail(B200RWKV_EINVAL, "argmax: bad argument (rows=%d n=%d)", rows, n);
  argmax_rows_kernel<<<rows, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      x, n, ldx, reinterpret_cast<long long*>(out), reinterpret_cast<long long*>(history), history_count, history_capacity);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "argmax: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

int b200rwkv_sample_typical(const float* x, int rows, int n, int64_t ldx, float temp, float tau, const float* u, int64_t* out,
                            float* probs_out, int64_t* history, int* history_count, int history_capacity, void* stream) {
  if (!x || !u || !out || rows < 1 || n < 1 || ldx < n || !(temp > 0.f) || !(tau > 0.f) ||
      (history && (!history_count || history_capacity < 1 || rows != 1)))
    return fail(B200RWKV_EINVAL, "sample_typical: bad argument (rows=%d n=%d temp=%g tau=%g)", rows, n, double(temp), double(tau));
  sample_typical_kernel<<<rows, kSampleThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      x, n, ldx, temp, tau, u, reinterpret_cast<long long*>(out), probs_out, reinterpret_cast<long long*>(history),
      history_count, history_capacity);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "sample_typical: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

// ---- unquantised weights (TORCH-mode matvec) -----------------------------------------------------

int b200rwkv_gemv_dense(const void* w, int dtype, int k_in, int n_out, int64_t ldw, const float* x, float* y, void* stream) {
  const int eb = dense_elem_bytes(dtype);
  if (!w || !x || !y || k_in < 1 || n_out < 1 || ldw < k_in || !eb)
    return fail(B200RWKV_EINVAL, "gemv_dense: bad argument (k_in=%d n_out=%d dtype=%d)", k_in, n_out, dtype);
  DenseParams P;
  memset(&P, 0, sizeof(P));
  P.w = w; P.x = x; P.y = y; P.ldw = ldw; P.K = k_in; P.N = n_out;
  P.vector_ok = reinterpret_cast<uintptr_t>(w) % 16 == 0 && (size_t(ldw) * eb) % 16 == 0 &&
                reinterpret_cast<uintptr_t>(x) % 16 == 0;
  // four CTAs fit an SM in the two-row variant (56 registers x 256 threads), eight in the others;
  // pairs of rows only when that still fills them, shared rows when one warp per row does not
  const int warps_full = device_sms() * 8 * kDenseWarps;
  const bool pairs = n_out >= warps_full;
  // a warp's share of a row should still be one or two passes of eight 16-byte pieces per lane (4 KB each)
  const size_t row_bytes = size_t(k_in) * eb;
  const int split = pairs ? 1 : (n_out * 2 <= warps_full && row_bytes >= 32768) ? 4 : (row_bytes >= 8192) ? 2 : 1;
  const int most = device_sms() * (pairs ? 4 : 8);
  const int per_cta = pairs ? kDenseWarps * 2 : kDenseWarps / split;
  const int passes = (n_out + per_cta - 1) / per_cta;
  const dim3 grid(passes < most ? passes : most);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
#define B200_DENSE_LAUNCH(T)                                                            \
  do {                                                                                  \
    if (pairs) dense_gemv_kernel<T, 2, 8, 1><<<grid, kDenseThreads, 0, st>>>(P);        \
    else if (split == 4) dense_gemv_kernel<T, 1, 8, 4><<<grid, kDenseThreads, 0, st>>>(P); \
    else if (split == 2) dense_gemv_kernel<T, 1, 8, 2><<<grid, kDenseThreads, 0, st>>>(P); \
    else dense_gemv_kernel<T, 1, 8, 1><<<grid, kDenseThreads, 0, st>>>(P);              \
  } while (0)
  if (dtype == B200RWKV_BF16) B200_DENSE_LAUNCH(__nv_bfloat16);
  else if (dtype == B200RWKV_F16) B200_DENSE_LAUNCH(__half);
  else B200_DENSE_LAUNCH(float);
#undef B200_DENSE_LAUNCH
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "gemv_dense: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

// ---- unquantised weights: one token through the network (entry points; helpers above the C block)
size_t b200rwkv_dense_workspace_bytes(const b200rwkv_dense_model* m) {
  if (!m || m->n_embd < 1 || m->n_ffn < 1) return 0;
  return dense_carve(m, nullptr).bytes;
}

int b200rwkv_dense_step_layers(const b200rwkv_dense_model* m, int layer_begin, int layer_end, const int64_t* token, float* state,
                               float* logits, void* workspace, size_t workspace_bytes, void* stream) {
  if (const char* why = dense_model_problem(m)) return fail(B200RWKV_EINVAL, "dense_step: %s", why);
  if (!token || !state || !workspace || !aligned16(workspace))
    return fail(B200RWKV_EINVAL, "dense_step: token, state and a 16-byte aligned workspace are required");
  if (layer_begin < 0 || layer_begin > layer_end || layer_end > m->n_layer)
    return fail(B200RWKV_EINVAL, "dense_step: layers [%d, %d) outside 0..%d", layer_begin, layer_end, m->n_layer);
  const DenseWorkspace ws = dense_carve(m, workspace);
  if (workspace_bytes < ws.bytes)
    return fail(B200RWKV_EINVAL, "dense_step: workspace of %zu bytes, %zu needed", workspace_bytes, ws.bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (m->dtype == B200RWKV_BF16) return dense_step_impl<__nv_bfloat16>(m, layer_begin, layer_end, token, state, logits, ws, st);
  if (m->dtype == B200RWKV_F16) return dense_step_impl<__half>(m, layer_begin, layer_end, token, state, logits, ws, st);
  return dense_step_impl<float>(m, layer_begin, layer_end, token, state, logits, ws, st);
}

int b200rwkv_dense_step(const b200rwkv_dense_model* m, const int64_t* token, float* state, float* logits,
                        void* workspace, size_t workspace_bytes, void* stream) {
  return b200rwkv_dense_step_layers(m, 0, m ? m->n_layer : 0, token, state, logits, workspace, workspace_bytes, stream);
}


size_t b200rwkv_dense_rows_workspace_bytes(const b200rwkv_dense_model* m, int streams, int tokens_per_stream) {
  if (!m || m->n_embd < 1 || m->n_ffn < 1 || streams < 1 || tokens_per_stream < 1) return 0;
  if ((long long)streams * tokens_per_stream > 65535) return 0;
  return dense_carve_rows(m, streams, tokens_per_stream, nullptr).bytes;
}

int b200rwkv_dense_forward_rows(const b200rwkv_dense_model* m, const int64_t* tokens, int streams, int tokens_per_stream,
                                float* state, int64_t state_stride, float* logits, void* workspace, size_t workspace_bytes,
                                void* stream) {
  return b200rwkv_dense_forward_rows_layers(m, 0, m ? m->n_layer : 0, tokens, streams, tokens_per_stream, state, state_stride, logits,
                                            workspace, workspace_bytes, stream);
}

int b200rwkv_dense_forward_rows_layers(const b200rwkv_dense_model* m, int layer_begin, int layer_end, const int64_t* tokens,
                                       int streams, int tokens_per_stream, float* state, int64_t state_stride, float* logits,
                                       void* workspace, size_t workspace_bytes, void* stream) {
  if (const char* why = dense_model_problem(m)) return fail(B200RWKV_EINVAL, "dense_forward_rows: %s", why);
  if (layer_begin < 0 || layer_begin > layer_end || layer_end > m->n_layer)
    return fail(B200RWKV_EINVAL, "dense_forward_rows: layers [%d, %d) outside 0..%d", layer_begin, layer_end, m->n_layer);
  if (m->dtype != B200RWKV_BF16 && m->dtype != B200RWKV_F16)
    return fail(B200RWKV_EINVAL, "dense_forward_rows: the tensor-core rows path takes bf16 or fp16 matrices (fp32: feed tokens one by one)");
  const int D = m->n_embd, F = m->n_ffn, V = m->n_vocab, L = m->n_layer, B = streams, T = tokens_per_stream;
  if (!tokens || !state || !workspace) return fail(B200RWKV_EINVAL, "dense_forward_rows: null argument");
  if ((D % 64) != 0 || (F % 64) != 0) return fail(B200RWKV_EINVAL, "dense_forward_rows: n_embd and n_ffn must be multiples of 64");
  if (B < 1 || T < 1 || (long long)B * T > 65535) return fail(B200RWKV_EINVAL, "dense_forward_rows: streams x tokens must be 1..65535 rows");
  if (state_stride < (int64_t)L * 5 * D) return fail(B200RWKV_EINVAL, "dense_forward_rows: state_stride below n_layer*5*n_embd");
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || !aligned16(state))
    return fail(B200RWKV_EINVAL, "dense_forward_rows: workspace must be 256-byte and state 16-byte aligned");
  DenseRowsWorkspace ws = dense_carve_rows(m, B, T, workspace);
  if (workspace_bytes < ws.bytes) return fail(B200RWKV_EINVAL, "dense_forward_rows: workspace %zu < %zu bytes", workspace_bytes, ws.bytes);
  const int R = B * T, Rpad = gemm_padded_rows(R), bf = m->dtype == B200RWKV_BF16 ? 1 : 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char* why = "";
  cudaError_t e;
  g_chain_rows = R <= 1024;
  static bool prep_configured[64];
  static int prep_sms[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail(B200RWKV_ECUDA, "dense_forward_rows: no current device");
  if (!prep_configured[dev]) {
    if (cudaFuncSetAttribute(dense_rows_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kDsMaxEmbd * 4) != cudaSuccess ||
        cudaDeviceGetAttribute(&prep_sms[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
      return fail(B200RWKV_ECUDA, "dense_forward_rows: cannot size the preparation kernel's shared memory");
    prep_configured[dev] = true;
  }
  // preparation CTAs resident at once (registers, and two rows of shared memory each)
  int prep_per_sm = 1;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&prep_per_sm, dense_rows_prep_kernel, 256, size_t(2) * D * 4) != cudaSuccess || prep_per_sm < 1)
    prep_per_sm = 1;
  const int prep_slots = prep_sms[dev] * prep_per_sm;
#define B200_DR_CHECK(call, what)                                                                      \
  do {                                                                                                 \
    e = (call);                                                                                        \
    if (e != cudaSuccess)                                                                              \
      return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "dense_forward_rows: %s: %s (%s)", what, why, \
                  cudaGetErrorString(e));                                                              \
  } while (0)
  if (layer_begin == 0)
    B200_DR_CHECK(launch_chained(embed_ln0_rows_kernel, dim3(R), dim3(256), 0, s, m->emb, reinterpret_cast<const long long*>(tokens),
                                 D, V, m->ln0_w, m->ln0_b, ws.xa), "embedding");
  DRowsPrepParams Q;
  DGemmParams P;
  auto prep = [&](const float* x, const float* lw, const float* lb, const float* carry, int nmix, const float* const* mix,
                  unsigned short* const* out, int last_only) -> cudaError_t {
    memset(&Q, 0, sizeof(Q));
    Q.x = x; Q.ln_w = lw; Q.ln_b = lb; Q.carry = carry; Q.carry_stride = state_stride;
    Q.carry_out = !carry ? nullptr : (T == 1 ? const_cast<float*>(carry) : ws.carry_new);
    Q.carry_out_stride = T == 1 ? state_stride : D;
    Q.nmix = nmix; Q.D = D; Q.Tn = T; Q.last_only = last_only; Q.is_bf16 = bf;
    for (int i = 0; i < (nmix > 0 ? nmix : 1); ++i) { Q.mix[i] = mix ? mix[i] : nullptr; Q.out[i] = out[i]; }
    // one row per CTA while that fits the GPU at once; beyond, a CTA walks consecutive rows and takes each layer norm once
    Q.R = last_only ? B : R;
    Q.rows_per_cta = (Q.R + prep_slots - 1) / prep_slots;
    return launch_chained(dense_rows_prep_kernel, dim3((Q.R + Q.rows_per_cta - 1) / Q.rows_per_cta), dim3(256), size_t(2) * D * 4, s, Q);
  };
  auto commit = [&](float* row) -> cudaError_t {      // parked layer norm of every stream's last row -> its state row
    if (T == 1) return cudaSuccess;                    // one row per stream: the preparation kernel wrote the state row itself
    return cudaMemcpy2DAsync(row, size_t(state_stride) * 4, ws.carry_new, size_t(D) * 4, size_t(D) * 4, size_t(B),
                             cudaMemcpyDeviceToDevice, s);
  };
  for (int l = layer_begin; l < layer_end; ++l) {
    const b200rwkv_dense_layer& ly = m->layers[l];
    float* st = state + size_t(l) * 5 * D;
    // 1. ln1 + token-shift mix -> key, value, sigmoid(receptance)
    { const float* mix[3] = {ly.att_mix_k, ly.att_mix_v, ly.att_mix_r};
      unsigned short* out[3] = {ws.t0, ws.t1, ws.t2};
      B200_DR_CHECK(prep(ws.xa, ly.ln1_w, ly.ln1_b, st, 3, mix, out, 0), "attention mix"); }
    B200_DR_CHECK(commit(st), "attention carry");
    memset(&P, 0, sizeof(P));
    P.nseg = 3; P.R = R; P.is_bf16 = bf; P.status = ws.status; P.sk_part = R <= kDgSplitMaxRows ? ws.sk_part : nullptr; P.sk_count = ws.sk_count;
    fill_dgemm_seg(P.seg[0], D, ws.kb, D, ACT_NONE, 0);
    fill_dgemm_seg(P.seg[1], D, ws.vb, D, ACT_NONE, 0);
    fill_dgemm_seg(P.seg[2], D, ws.rb, D, ACT_SIGMOID, 0);
    { const void* w[3] = {ly.att_key, ly.att_value, ly.att_receptance};
      const unsigned short* x[3] = {ws.t0, ws.t1, ws.t2};
      B200_DR_CHECK(launch_dense_gemm(P, w, x, D, Rpad, s, &why), "key/value/receptance"); }
    // 2. WKV recurrence over each stream's rows; kb <- sigmoid(r) * wkv
    why = "wkv launch";
    if (T <= 2 * kWkvChunk) {
      e = launch_chained(wkv_rows_kernel, dim3((B * D + 127) / 128), dim3(128), 0, s, B, T, D, ly.time_decay, ly.time_first, ws.kb,
                         (const float*)ws.vb, (const float*)ws.rb, st + 2 * size_t(D), st + 3 * size_t(D), st + 4 * size_t(D),
                         (long long)state_stride);
    } else {
      const int NC = (T + kWkvChunk - 1) / kWkvChunk;
      const long long n1 = (long long)B * (NC - 1) * D, n2 = (long long)B * NC * D;
      e = launch_chained(wkv_chunk_state_kernel, dim3((unsigned)((n1 + 127) / 128)), dim3(128), 0, s, B, T, D, NC, ly.time_decay,
                         (const float*)ws.kb, (const float*)ws.vb, ws.wkv_loc, (const float*)(st + 2 * size_t(D)),
                         (const float*)(st + 3 * size_t(D)), (const float*)(st + 4 * size_t(D)), (long long)state_stride);
      if (e == cudaSuccess)
        e = launch_chained(wkv_chunk_output_kernel, dim3((unsigned)((n2 + 127) / 128)), dim3(128), 0, s, B, T, D, NC, ly.time_decay,
                           ly.time_first, ws.kb, (const float*)ws.vb, (const float*)ws.rb, (const float*)ws.wkv_loc,
                           st + 2 * size_t(D), st + 3 * size_t(D), st + 4 * size_t(D), (long long)state_stride);
    }
    B200_DR_CHECK(e, "wkv");
    // 3. attention output + residual -> xb
    B200_DR_CHECK(launch_chained(dense_rows_cast_kernel, dim3(unsigned(std::min<long long>((long long)R * D / 4 / 256 + 1, 4096))), dim3(256), 0, s,
                                 (const float*)ws.kb, ws.t0, (long long)R * D / 4, bf), "cast");
    memset(&P, 0, sizeof(P));
    P.nseg = 1; P.R = R; P.is_bf16 = bf; P.status = ws.status; P.sk_part = R <= kDgSplitMaxRows ? ws.sk_part : nullptr; P.sk_count = ws.sk_count;
    fill_dgemm_seg(P.seg[0], D, ws.xb, D, ACT_NONE, 0);
    P.seg[0].res = ws.xa; P.seg[0].ldres = D;
    { const void* w[1] = {ly.att_output};
      const unsigned short* x[1] = {ws.t0};
      B200_DR_CHECK(launch_dense_gemm(P, w, x, D, Rpad, s, &why), "attention output"); }
    // 4. ln2 + token-shift mix -> relu(key)^2 (kept in the matrices' type), sigmoid(receptance)
    { const float* mix[2] = {ly.ffn_mix_k, ly.ffn_mix_r};
      unsigned short* out[2] = {ws.t0, ws.t1};
      B200_DR_CHECK(prep(ws.xb, ly.ln2_w, ly.ln2_b, st + D, 2, mix, out, 0), "ffn mix"); }
    B200_DR_CHECK(commit(st + D), "ffn carry");
    memset(&P, 0, sizeof(P));
    P.nseg = 2; P.R = R; P.is_bf16 = bf; P.status = ws.status; P.sk_part = R <= kDgSplitMaxRows ? ws.sk_part : nullptr; P.sk_count = ws.sk_count;
    fill_dgemm_seg(P.seg[0], F, ws.kk, F, ACT_RELUSQ, 1);
    fill_dgemm_seg(P.seg[1], D, ws.rb, D, ACT_SIGMOID, 0);
    { const void* w[2] = {ly.ffn_key, ly.ffn_receptance};
      const unsigned short* x[2] = {ws.t0, ws.t1};
      B200_DR_CHECK(launch_dense_gemm(P, w, x, D, Rpad, s, &why), "ffn key and receptance"); }
    // 5. ffn value, gated, + residual -> xa
    memset(&P, 0, sizeof(P));
    P.nseg = 1; P.R = R; P.is_bf16 = bf; P.status = ws.status; P.sk_part = R <= kDgSplitMaxRows ? ws.sk_part : nullptr; P.sk_count = ws.sk_count;
    fill_dgemm_seg(P.seg[0], D, ws.xa, D, ACT_NONE, 0);
    P.seg[0].res = ws.xb; P.seg[0].ldres = D; P.seg[0].gate = ws.rb; P.seg[0].ldgate = D;
    { const void* w[1] = {ly.ffn_value};
      const unsigned short* x[1] = {ws.kk};
      B200_DR_CHECK(launch_dense_gemm(P, w, x, F, Rpad, s, &why), "ffn value"); }
  }
  if (logits && layer_end == L) {
    unsigned short* out[1] = {ws.hx};
    B200_DR_CHECK(prep(ws.xa, m->ln_out_w, m->ln_out_b, nullptr, 0, nullptr, out, 1), "output layer norm");
    memset(&P, 0, sizeof(P));
    P.nseg = 1; P.R = B; P.is_bf16 = bf; P.status = ws.status; P.sk_part = R <= kDgSplitMaxRows ? ws.sk_part : nullptr; P.sk_count = ws.sk_count;
    fill_dgemm_seg(P.seg[0], V, logits, V, ACT_NONE, 0);
    const void* w[1] = {m->head};
    const unsigned short* x[1] = {ws.hx};
    B200_DR_CHECK(launch_dense_gemm(P, w, x, D, gemm_padded_rows(B), s, &why), "head");
  }
#undef B200_DR_CHECK
  return B200RWKV_OK;
}

// ---- time-out path under test ----------------------------------------------------------------------------
int b200rwkv_debug_expire_waits(int enable, uint64_t limit_ns) {
  if (enable && (limit_ns < 1000ull || limit_ns > 1000ull * 1000ull * 1000ull))
    return fail(B200RWKV_EINVAL, "debug_expire_waits: limit must be between 1 us and 1 s");
  g_expire_waits = enable ? 1 : 0;
  g_expire_limit_ns = enable ? limit_ns : 0;
  return B200RWKV_OK;
}

int b200rwkv_wait_selftest(uint64_t limit_ns, int* status, void* stream) {
  if (!status || limit_ns < 1000ull || limit_ns > 1000ull * 1000ull * 1000ull)
    return fail(B200RWKV_EINVAL, "wait_selftest: status pointer and a limit between 1 us and 1 s are required");
  wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, status);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B200RWKV_ECUDA, "wait_selftest: %s", cudaGetErrorString(e));
  return B200RWKV_OK;
}

}  // extern "C"
