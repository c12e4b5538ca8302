// C ABI of the library (declarations and per-function contracts: include/b200rwkv.h) and the small
// vector kernels that sit between the streaming GEMV launches.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "stream_gemv.cuh"

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
template <int KCH>
static cudaError_t launch_kch(const GemvParams& P, const GemvPlan& plan, bool pdl, cudaStream_t stream) {
  static bool configured[64];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    e = cudaFuncSetAttribute(stream_gemv_kernel<KCH>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemLimit);
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
  return cudaLaunchKernelEx(&cfg, stream_gemv_kernel<KCH>, P);
}

cudaError_t launch_stream_gemv(GemvParams& P, int max_n, bool pdl, cudaStream_t stream, const char** why) {
  const int sms = device_sms();
  GemvPlan plan;
  if (sms <= 0 || !plan_gemv(P.K, P.nseg, max_n, sms, &plan)) {
    *why = "unsupported GEMV shape (k_in must be a multiple of 16 and at most 40960; 1..3 matrices)";
    return cudaErrorInvalidValue;
  }
  P.tpr = plan.tpr; P.rl = plan.rl; P.m = plan.m; P.log_m = plan.log_m;
  P.stages = plan.stages; P.stage_bytes = plan.stage_bytes; P.rpc = plan.rpc;
  *why = "kernel launch failed";
  switch (plan.kch) {
    case 1: return launch_kch<1>(P, plan, pdl, stream);
    case 2: return launch_kch<2>(P, plan, pdl, stream);
    case 3: return launch_kch<3>(P, plan, pdl, stream);
    default: return launch_kch<4>(P, plan, pdl, stream);
  }
}

static int check_matrix(const b200rwkv_matrix& m, const char* name) {
  if (!m.qt || !m.ry || !m.my) return fail(B200RWKV_EINVAL, "%s: null qt/ry/my", name);
  if (m.n_out <= 0 || m.k_in <= 0 || (m.k_in % 16) != 0)
    return fail(B200RWKV_EINVAL, "%s: n_out=%d k_in=%d (k_in must be a positive multiple of 16)", name, m.n_out, m.k_in);
  if (!aligned16(m.qt) || !aligned16(m.ry) || !aligned16(m.my))
    return fail(B200RWKV_EINVAL, "%s: qt/ry/my must be 16-byte aligned", name);
  return B200RWKV_OK;
}

static void fill_seg(GemvSeg& s, const b200rwkv_matrix& m) {
  memset(&s, 0, sizeof(s));
  s.qt = m.qt; s.ry = m.ry; s.my = m.my; s.rx = m.rx; s.mx = m.mx;
  s.half = m.half; s.N = m.n_out; s.act = ACT_NONE;
}

// ---------------------------------------------------------------------------------------- small kernels
// x = LayerNorm(emb[token]) (the reference's emb.py:8-9 gather followed by ln_in, opt.py:63-64).
__global__ void __launch_bounds__(512, 1)
embed_ln0_kernel(const float* __restrict__ emb, const long long* __restrict__ token, int D, int V,
                 const float* __restrict__ w, const float* __restrict__ b, float* __restrict__ out) {
  __shared__ float red[16];
  __shared__ float bc;
  griddep_launch_dependents();
  griddep_wait();
  long long tok = *token;
  tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
  const float* row = emb + size_t(tok) * D;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
  float s = 0.f;
  for (int i = tid; i < D; i += 512) s += row[i];
  const float mean = block_sum(s) / float(D);
  s = 0.f;
  for (int i = tid; i < D; i += 512) { const float c = row[i] - mean; s += c * c; }
  const float sdev = sqrtf(block_sum(s) / float(D) + 1e-5f);
  for (int i = tid; i < D; i += 512) out[i] = w[i] * ((row[i] - mean) / sdev) + b[i];
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

struct Workspace {
  int* status;
  float *xa, *xb, *rwkv, *s_att, *s_ffn, *rf, *kk;
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
  w.rwkv = reinterpret_cast<float*>(take(D));
  w.s_att = reinterpret_cast<float*>(take(D));
  w.s_ffn = reinterpret_cast<float*>(take(D));
  w.rf = reinterpret_cast<float*>(take(D));
  w.kk = reinterpret_cast<float*>(take(F));
  w.bytes = off;
  return w;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200rwkv_version(void) { return 100; }

const char* b200rwkv_last_error(void) { return g_err; }

int b200rwkv_gemv_u8(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y, int accumulate,
                     int* status, void* stream) {
  if (nmat < 1 || nmat > kMaxSeg || !mats || !x || !y) return fail(B200RWKV_EINVAL, "gemv_u8: nmat=%d or null argument", nmat);
  GemvParams P;
  memset(&P, 0, sizeof(P));
  int max_n = 0;
  for (int i = 0; i < nmat; ++i) {
    if (int rc = check_matrix(mats[i], "gemv_u8 matrix")) return rc;
    if (mats[i].k_in != mats[0].k_in) return fail(B200RWKV_EINVAL, "gemv_u8: matrices must share k_in");
    if (!x[i] || !y[i] || !aligned16(x[i])) return fail(B200RWKV_EINVAL, "gemv_u8: x/y null or x not 16-byte aligned");
    fill_seg(P.seg[i], mats[i]);
    P.seg[i].xin = x[i];
    P.seg[i].out = y[i];
    if (mats[i].n_out > max_n) max_n = mats[i].n_out;
  }
  P.nseg = nmat; P.K = mats[0].k_in; P.pro = PRO_VEC; P.epi = EPI_GENERIC; P.accumulate = accumulate ? 1 : 0;
  P.status = status;
  const char* why = "";
  cudaError_t e = launch_stream_gemv(P, max_n, false, static_cast<cudaStream_t>(stream), &why);
  if (e != cudaSuccess) return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "gemv_u8: %s (%s)", why, cudaGetErrorString(e));
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
  const int64_t v[10] = {p.kch, p.tpr, p.rl, p.m, p.stages, p.stage_bytes, p.rpc, p.grid, (int64_t)p.smem, kConsumers};
  for (int i = 0; i < 10; ++i) out[i] = v[i];
  return B200RWKV_OK;
}

size_t b200rwkv_decode_workspace_bytes(const b200rwkv_model* m) {
  if (!m || m->n_embd <= 0 || m->n_ffn <= 0) return 0;
  return carve(m, nullptr).bytes;
}

int b200rwkv_decode_step(const b200rwkv_model* m, const int64_t* token, float* state, float* logits, void* workspace,
                         size_t workspace_bytes, void* stream) {
  if (!m || !token || !state || !workspace || !m->layers || !m->emb)
    return fail(B200RWKV_EINVAL, "decode_step: null argument");
  const int D = m->n_embd, F = m->n_ffn, V = m->n_vocab, L = m->n_layer;
  if (D <= 0 || (D % 16) != 0 || F <= 0 || (F % 16) != 0 || V <= 0 || L <= 0)
    return fail(B200RWKV_EINVAL, "decode_step: n_embd=%d n_ffn=%d must be positive multiples of 16", D, F);
  if ((reinterpret_cast<uintptr_t>(workspace) & 255u) != 0 || !aligned16(state))
    return fail(B200RWKV_EINVAL, "decode_step: workspace must be 256-byte and state 16-byte aligned");
  Workspace ws = carve(m, workspace);
  if (workspace_bytes < ws.bytes) return fail(B200RWKV_EINVAL, "decode_step: workspace %zu < %zu bytes", workspace_bytes, ws.bytes);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const char* why = "";
  cudaError_t e;

  {  // embedding gather + ln0, chained like every other launch
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(1); cfg.blockDim = dim3(512); cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, embed_ln0_kernel, m->emb, reinterpret_cast<const long long*>(token), D, V, m->ln0_w,
                           m->ln0_b, ws.xa);
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
    // 1. ln1 + token-shift mix -> key/value/receptance -> WKV state update -> sigmoid(r)*wkv
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.att_key);        P.seg[0].mix = ly.att_mix_k;
    fill_seg(P.seg[1], ly.att_value);      P.seg[1].mix = ly.att_mix_v;
    fill_seg(P.seg[2], ly.att_receptance); P.seg[2].mix = ly.att_mix_r;
    P.nseg = 3; P.K = D; P.pro = PRO_LNMIX; P.ln_x = ws.xa; P.ln_w = ly.ln1_w; P.ln_b = ly.ln1_b;
    P.shift_in = st; P.shift_out = ws.s_att;
    P.epi = EPI_WKV; P.wkv_w = ly.time_decay; P.wkv_u = ly.time_first;
    P.aa = st + 2 * size_t(D); P.bb = st + 3 * size_t(D); P.pp = st + 4 * size_t(D); P.wkv_out = ws.rwkv;
    P.status = ws.status;
    if ((e = launch_stream_gemv(P, D, true, s, &why)) != cudaSuccess) goto launch_failed;
    // 2. attention output projection + residual; commits the att token-shift carry
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.att_output); P.seg[0].xin = ws.rwkv; P.seg[0].out = ws.xb; P.seg[0].res = ws.xa;
    P.nseg = 1; P.K = D; P.pro = PRO_VEC; P.epi = EPI_GENERIC;
    P.commit_src = ws.s_att; P.commit_dst = st; P.commit_n = D; P.status = ws.status;
    if ((e = launch_stream_gemv(P, D, true, s, &why)) != cudaSuccess) goto launch_failed;
    // 3. ln2 + token-shift mix -> ffn key (relu^2) and ffn receptance (sigmoid)
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.ffn_key);        P.seg[0].mix = ly.ffn_mix_k; P.seg[0].act = ACT_RELUSQ;  P.seg[0].out = ws.kk;
    fill_seg(P.seg[1], ly.ffn_receptance); P.seg[1].mix = ly.ffn_mix_r; P.seg[1].act = ACT_SIGMOID; P.seg[1].out = ws.rf;
    P.nseg = 2; P.K = D; P.pro = PRO_LNMIX; P.ln_x = ws.xb; P.ln_w = ly.ln2_w; P.ln_b = ly.ln2_b;
    P.shift_in = st + size_t(D); P.shift_out = ws.s_ffn; P.epi = EPI_GENERIC; P.status = ws.status;
    if ((e = launch_stream_gemv(P, F > D ? F : D, true, s, &why)) != cudaSuccess) goto launch_failed;
    // 4. ffn value projection, gated by the receptance, + residual; commits the ffn carry
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], ly.ffn_value); P.seg[0].xin = ws.kk; P.seg[0].out = ws.xa; P.seg[0].res = ws.xb; P.seg[0].gate = ws.rf;
    P.nseg = 1; P.K = F; P.pro = PRO_VEC; P.epi = EPI_GENERIC;
    P.commit_src = ws.s_ffn; P.commit_dst = st + size_t(D); P.commit_n = D; P.status = ws.status;
    if ((e = launch_stream_gemv(P, D, true, s, &why)) != cudaSuccess) goto launch_failed;
  }
  if (logits) {
    if (int rc = check_matrix(m->head, "decode_step head")) return rc;
    if (m->head.n_out != V || m->head.k_in != D) return fail(B200RWKV_EINVAL, "decode_step: head is %dx%d", m->head.n_out, m->head.k_in);
    GemvParams P;
    memset(&P, 0, sizeof(P));
    fill_seg(P.seg[0], m->head); P.seg[0].out = logits;
    P.nseg = 1; P.K = D; P.pro = PRO_LNMIX; P.ln_x = ws.xa; P.ln_w = m->ln_out_w; P.ln_b = m->ln_out_b;
    P.epi = EPI_GENERIC; P.status = ws.status;
    if ((e = launch_stream_gemv(P, V, true, s, &why)) != cudaSuccess) goto launch_failed;
  }
  return B200RWKV_OK;
launch_failed:
  return fail(e == cudaErrorInvalidValue ? B200RWKV_EINVAL : B200RWKV_ECUDA, "decode_step: %s (%s)", why, cudaGetErrorString(e));
}

}  // extern "C"
