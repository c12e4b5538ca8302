/*
 * b200rwkv - C ABI of the sm_100a RWKV-4 uint8 inference kernels.
 *
 * Plain C: pointers and sizes only, no torch types.  Every pointer named "device"
 * is a CUDA device pointer on the current device; `stream` is a cudaStream_t passed as
 * void*.  Functions return 0 or a negative B200RWKV_E* code and never abort; the text
 * of the last error on the calling thread is available from b200rwkv_last_error().
 * Unless a comment says otherwise a function allocates nothing, launches
 * asynchronously on `stream`, and the caller owns every buffer.
 *
 * "Reference" below is rwkvstic 3.0.0; paths are relative to its
 * src/rwkvstic/agnostic/backends/ folder.
 */
#ifndef B200RWKV_H
#define B200RWKV_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200RWKV_OK 0
#define B200RWKV_EINVAL (-1)   /* null/misaligned pointer, unsupported shape */
#define B200RWKV_ECUDA (-2)    /* a CUDA runtime call failed */
#define B200RWKV_ETIMEOUT (-3) /* a bounded device-side wait expired (see b200rwkv_status_*) */

/* Bits a kernel may set in the caller's device status word (an int the caller zeroes). */
#define B200RWKV_STATUS_WAIT_FULL 1    /* consumer gave up waiting for a weight stage   */
#define B200RWKV_STATUS_WAIT_EMPTY 2   /* producer gave up waiting for a free ring slot */
#define B200RWKV_STATUS_WAIT_PEER 4    /* a CTA of the persistent decode step gave up waiting for another CTA's data */

/*
 * One quantised matrix, used as y = x @ W with W[k_in, n_out].  Bytes are stored
 * output-major, `qt[n_out][k_in]` with k contiguous (the transpose of the reference's
 * MM8.weight u8[in,out], modules/matmul.py:15-21), 16-byte aligned, k_in % 128 == 0.
 *
 *   y[n] = rx[n] * ( sum_k (x[k]*ry[k]) * qt[n][k] + half * sum_k x[k]*ry[k] )
 *          + sum_k x[k]*my[k] + mx[n] * sum_k x[k]
 *
 * FASTQUANT (modules/matmul.py:26-40): ry = range, my = offset, rx = mx = NULL, half = 0.
 * Two-axis scheme "(q+0.5)*ry*rx+my+mx": all four vectors, half = 0.5.
 */
typedef struct b200rwkv_matrix {
  const uint8_t* qt; /* device u8 [n_out][k_in] */
  const float* ry;   /* device f32 [k_in] */
  const float* my;   /* device f32 [k_in] */
  const float* rx;   /* device f32 [n_out] or NULL (= 1) */
  const float* mx;   /* device f32 [n_out] or NULL (= 0) */
  float half;
  int32_t n_out;
  int32_t k_in;
} b200rwkv_matrix;

/* Parameters of one RWKV-4 block (modules/block.py:7-50). All device f32 [n_embd]. */
typedef struct b200rwkv_layer {
  const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
  const float *att_mix_k, *att_mix_v, *att_mix_r; /* time_mix_* (block.py:35-37) */
  const float *ffn_mix_k, *ffn_mix_r;             /* block.py:46-47 */
  const float* time_decay;                        /* w = -exp(raw time_decay) (block.py:41) */
  const float* time_first;                        /* u, raw (block.py:39) */
  b200rwkv_matrix att_key, att_value, att_receptance, att_output;
  b200rwkv_matrix ffn_key, ffn_receptance, ffn_value;
} b200rwkv_layer;

/* A whole model (opt.py:25-58).  `layers` is a HOST array of n_layer entries. */
typedef struct b200rwkv_model {
  int32_t n_layer, n_embd, n_ffn, n_vocab;
  const float* emb; /* device f32 [n_vocab][n_embd] */
  const float *ln0_w, *ln0_b, *ln_out_w, *ln_out_b;
  b200rwkv_matrix head;
  const b200rwkv_layer* layers;
} b200rwkv_model;

/* Library version (major*10000 + minor*100 + patch). */
int b200rwkv_version(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* b200rwkv_last_error(void);

/* Bytes of device scratch b200rwkv_gemv_u8 needs for `nmat` matrices of reduction length k_in. */
size_t b200rwkv_gemv_workspace_bytes(int k_in, int nmat);

/*
 * uint8 GEMV, 1 to 3 matrices of equal k_in:  y_i = contract(mats[i], x[i]).
 * Replaces rwkv::mm8_one / rwkv::mm8_three (cuda/wrapper.cpp:52-129, kernels
 * cuda/operators32.cu:18-115) together with the offset term the reference adds on the
 * host side (modules/matmul.py:58-62, :95-102).  x[i]: device f32 [k_in]; y[i]: device
 * f32 [n_out_i], overwritten, or added to when `accumulate` is non-zero (the reference
 * op accumulates onto a zero-filled y).  Two launches: a one-CTA kernel turns the x[i] into
 * fixed-point digit planes, then the streaming kernel reads every weight byte once.
 * `workspace`: device scratch of b200rwkv_gemv_workspace_bytes(k_in, nmat), 256-byte
 * aligned; its first int is a status word the kernels OR B200RWKV_STATUS_* bits into (zero
 * it once).  Calls that share a workspace must be ordered on one stream.
 */
int b200rwkv_gemv_u8(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y,
                     int accumulate, void* workspace, size_t workspace_bytes, void* stream);

/*
 * b200rwkv_gemv_u8 with a per-CTA phase timeline for profiling.  `trace`: device u64
 * [1024][8], filled with %globaltimer nanoseconds.  Row c < grid (grid from
 * b200rwkv_gemv_plan) belongs to CTA c of the streaming kernel: 0 kernel entry, 1 launch
 * dependency resolved, 4 digit planes in shared memory (first weight stage may be consumed),
 * 5 all rows done, 6 epilogue done, 7 producer issued its last bulk copy.  Row 1023 belongs to
 * the preparation kernel: 0 entry, 1 dependency resolved, 2 layer-norm statistics done, 3 done.
 * No counterpart in the reference.
 */
int b200rwkv_gemv_u8_traced(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y,
                            int accumulate, void* workspace, size_t workspace_bytes, uint64_t* trace,
                            void* stream);

/*
 * b200rwkv_gemv_u8 for callers that cannot allocate device memory: plugin hosts whose memory
 * pool is closed to extensions, code running while a stream capture is in progress, or a
 * C program that never touches cudaMalloc at all.  Same arithmetic and same two launches as
 * b200rwkv_gemv_u8 (results are bit-identical), but the scratch for the activation digits lives
 * in a 192.25 KB array compiled into the library, which every GPU that loads the library
 * holds until the process exits.  The call itself never allocates or frees anything.
 *   limit     nmat * 4 * k_in <= 196608 bytes (three matrices up to k_in = 16384, one up to
 *             49152); larger requests return B200RWKV_EINVAL and a message naming the limit.
 *   status    optional caller-owned device int for the B200RWKV_STATUS_* bits, or NULL.
 *   set-up    the first call on each device looks up the array's device address; make that
 *             call before starting any stream capture.
 *   sharing   all calls on a device use the same array and find the previous call's contents
 *             in it (nothing in it needs clearing: each call overwrites what it reads).  Two
 *             calls that can overlap on the GPU (different streams, no event between them) race
 *             on it - order them.
 * No counterpart in the reference.
 */
int b200rwkv_gemv_u8_static(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y,
                            int accumulate, int* status, void* stream);

/*
 * WKV-4 recurrence, B independent streams x C channels, sequential over T
 * (replaces rwkv::wkv_forward, cuda/wrapper.cpp:45-50 / cuda/operators.cu:6-44, and
 * TorchWKV, modules/wkv.py:23-40).  k, v, y: device f32 [B][T][C]; w (= -exp(decay)),
 * u: device f32 [C]; aa, bb, pp: device f32 [B][C] updated in place.
 * convention 0: max-trick state (agnosticRwkv.py:68-103): sums are scaled by exp(-pp),
 *               decay applied at the start of the next step; empty state (0, 0, -1e30).
 * convention 1: the reference FASTQUANT state (modules/wkv.py:31-39): aa, bb already
 *               multiplied by exp(w), pp untouched.  Computed with the same max-trick
 *               arithmetic internally and converted on entry and exit.
 */
int b200rwkv_wkv_scan(int B, int T, int C, const float* w, const float* u, const float* k, const float* v,
                      float* y, float* aa, float* bb, float* pp, int convention, void* stream);

/*
 * Host-only introspection of the GEMV launch geometry for reduction length k_in, `nmat`
 * matrices, the largest n_out, and a GPU with `num_sms` SMs.  Fills
 * out[0..9] = {chunk_bytes (bytes of one row per ring stage), chunks_per_row, swizzle_bytes,
 * rows_per_stage, ring_stages, stage_bytes, max_rows_per_cta (rounded up to 16), grid,
 * shared_memory_bytes, consumer_threads}.
 * Returns B200RWKV_EINVAL for an unsupported shape.  No counterpart in the reference (its
 * launch shape is fixed: cuda/operators32.cu:86-115); used by tests and the roofline report.
 */
int b200rwkv_gemv_plan(int k_in, int nmat, int max_n_out, int num_sms, int64_t* out);

/* Bytes of device scratch that b200rwkv_decode_step needs for this model. */
size_t b200rwkv_decode_workspace_bytes(const b200rwkv_model* m);

/*
 * One decode step (T = 1) of the whole network for one stream: the fused replacement for
 * myRWKV.forward (opt.py:61-76) with Block.forward (modules/block.py:56-102) at T == 1.
 *   token     device int64[1]
 *   state     device f32 [n_layer][5][n_embd], updated in place: rows 0/1 the att/ffn
 *             token-shift carries (block.py:61-64, :85-88), rows 2..4 aa, bb, pp in the
 *             max-trick convention; the empty state is (0,0,0,0,-1e30) as opt.py:31-32.
 *   logits    device f32 [n_vocab], or NULL to skip ln_out + head (prompt tokens whose
 *             logits nobody reads)
 *   workspace device scratch of b200rwkv_decode_workspace_bytes(m), 256-byte aligned; its
 *             first int is the status word the kernels OR error bits into (zero it once).
 * Launches 8*n_layer + 3 kernels (per matrix group one activation-preparation CTA and one
 * streaming GEMV grid) chained by programmatic dependent launch; safe to capture in a CUDA graph.
 */
int b200rwkv_decode_step(const b200rwkv_model* m, const int64_t* token, float* state, float* logits,
                         void* workspace, size_t workspace_bytes, void* stream);

/*
 * b200rwkv_decode_step with the per-CTA phase timeline of every GEMV launch (profiling).
 * `trace`: device u64 [4*n_layer + 1][1024][8]; GEMV launch i (in issue order: per layer key/value/
 * receptance, attention output, ffn key+receptance, ffn value; then the head) and the preparation
 * kernel in front of it fill trace[i] as described at b200rwkv_gemv_u8_traced.  No counterpart in the reference.
 */
/*
 * One pipeline stage of the step above, for a model object that holds a contiguous range of blocks
 * only (blocks placed on different devices: the TORCH_SPLIT placement; in-tree the hop between
 * devices is modules/matmul.py:154-163).  The one-row streaming path for a single row, where
 * b200rwkv_forward_rows_stage would run the tensor-core tiles.
 *   token   device int64[1] on the first stage (m->emb set): embedding + ln0 produce the row; NULL on
 *           later stages, where the row is read from x
 *   x       device f32 [n_embd], 16-byte aligned: the residual stream handed over by the previous
 *           stage (read when token is NULL) and, on return, this stage's result for the next one
 *   logits  device f32 [n_vocab] on the last stage (m->head set), else NULL
 * Same workspace, state rows and error convention as b200rwkv_decode_step; results are bit-identical
 * to the unsplit step (same kernels on the same values).
 */
int b200rwkv_decode_step_stage(const b200rwkv_model* m, const int64_t* token, float* x, float* state, float* logits,
                               void* workspace, size_t workspace_bytes, void* stream);
int b200rwkv_decode_step_traced(const b200rwkv_model* m, const int64_t* token, float* state, float* logits,
                                void* workspace, size_t workspace_bytes, uint64_t* trace, void* stream);

/*
 * The decode step as ONE persistent kernel (same contract as b200rwkv_decode_step: the fused
 * replacement for myRWKV.forward, opt.py:61-76, with Block.forward, modules/block.py:56-102, at
 * T == 1).  One CTA per SM stays resident for the whole step; its weight ring runs on from matrix
 * to matrix, and the CTAs exchange activations (six exchanges per block) through words in L2 that
 * carry the parity of their buffer's use count, so there is no barrier, atomic or fence between
 * them.  On a B200 the chained path (b200rwkv_decode_step) is the faster of the two; this one is
 * kept because it is a single launch per token.
 * The step needs a "plan": a caller-owned device buffer that holds the table of matrices (with
 * their TMA descriptors), copies of the vector parameters at fixed offsets, the exchange buffers,
 * their use counts and the status word.
 *
 * b200rwkv_step_plan_bytes   size of the plan buffer for this model
 * b200rwkv_step_plan_init    fills it (synchronous: cudaMemset / cudaMemcpy; call it once, outside any
 *                            stream capture, with the device current; 256-byte aligned).  The model
 *                            needs emb/ln0; ln_out/head only if logits will be asked for.  The vector
 *                            parameters are COPIED: call it again if they change.
 * b200rwkv_decode_step_persistent
 *   token, state, logits  as b200rwkv_decode_step (logits NULL skips ln_out + head)
 *   tuning   NULL, or int32[4] = {weight stages a CTA may have in flight (0: the whole ring), the same
 *            while its consumers are between two matrices (0: the whole ring), bytes per CTA requested
 *            from L2 beyond the ring (-1: default), limit of every device-side wait in ms (0: 1000)}
 *   trace    NULL, or device u64 [4*n_layer + 1][grid][8] of %globaltimer stamps per launch and CTA:
 *            1 exchange read and digit planes built, 2 rows summed, 3 epilogue done, 4 layer-norm
 *            statistics gathered, 5 normalised slice published
 *   One cooperative kernel launch; allocation-free; safe to capture in a CUDA graph.  Steps that
 *   share a plan must be ordered on one stream.  When B200RWKV_STATUS_* bits appear in the status
 *   word (first int of the plan) the state is undefined and the plan must be initialised again.
 * b200rwkv_step_geometry  host-only: out[0..7] = {grid, ring_stages, slot_bytes, shared_memory_bytes,
 *   row_sum_offset, plane_offset, ring_offset, threads} for a GPU with num_sms SMs.
 * No counterpart in the reference (it launches ~45 kernels per block and token).
 */
size_t b200rwkv_step_plan_bytes(const b200rwkv_model* m);
int b200rwkv_step_plan_init(const b200rwkv_model* m, void* plan, size_t plan_bytes);
int b200rwkv_decode_step_persistent(const b200rwkv_model* m, void* plan, size_t plan_bytes, const int64_t* token,
                                    float* state, float* logits, const int32_t* tuning, uint64_t* trace, void* stream);
int b200rwkv_step_geometry(const b200rwkv_model* m, int num_sms, int64_t* out);

/* Bytes of device scratch b200rwkv_gemm_u8 needs (digit rows: 3 bytes per input per row, rows
 * rounded up to 16; plus 32 bytes per row and matrix). */
size_t b200rwkv_gemm_workspace_bytes(int k_in, int nmat, int rows);

/*
 * uint8 GEMM, 1 to 3 matrices of equal k_in applied to `rows` activation rows each:
 *   y_i[r][:] = contract(mats[i], x_i[r][:])        x_i: device f32 [rows][k_in], y_i: [rows][n_out_i]
 * The many-rows form of b200rwkv_gemv_u8: replaces the reference's sequence-mode matmul, which
 * dequantises the whole matrix and calls a float GEMM (modules/matmul.py:64-68, :103-114), and its
 * batched decode.  Same arithmetic per row as the one-row kernel (24-bit fixed-point activations,
 * exact integer dot products, the same affine terms), so a row's result does not depend on
 * which of the two entry points computed it beyond the fp32 summation order of sum_k x*my.
 * Two launches: a row-wise preparation kernel, then a tcgen05 (kind::i8) tensor-core kernel with
 * TMA-fed operands and TMEM accumulators: persistent CTAs over tiles of 128 or 256 outputs x
 * 16..80 rows, the shape picked per launch.  rows <= 65535.
 * `workspace`: b200rwkv_gemm_workspace_bytes(k_in, nmat, rows), 256-byte aligned, ZERO-FILLED once
 * before its first use (first int = status word; it also holds the integer scratch in which launches
 * with few rows combine their K slices, which every launch leaves zero again).
 */
int b200rwkv_gemm_u8(int nmat, const b200rwkv_matrix* mats, const float* const* x, float* const* y, int rows,
                     void* workspace, size_t workspace_bytes, void* stream);

/* Bytes of device scratch b200rwkv_forward_rows needs (0 if streams * tokens_per_stream > 65535);
 * zero-fill it once before its first use (status word and K-slice scratch, see b200rwkv_gemm_u8). */
size_t b200rwkv_rows_workspace_bytes(const b200rwkv_model* m, int streams, int tokens_per_stream);

/*
 * The whole network over `streams` independent streams of `tokens_per_stream` tokens each, every
 * matrix applied to all streams * tokens rows at once (b200rwkv_gemm_u8's kernels): prompt
 * ingestion (one stream, many tokens; myRWKV.forward with T > 1, opt.py:61-76, Block.forward
 * modules/block.py:56-102) and batched decode (many streams, one token).
 *   tokens   device int64 [streams][tokens_per_stream]
 *   state    device f32: stream s at state + s * state_stride, each [n_layer][5][n_embd] as in
 *            b200rwkv_decode_step, updated in place
 *   logits   device f32 [streams][n_vocab]: logits after the LAST token of every stream, or NULL
 * Rows = streams * tokens_per_stream <= 65535; longer prompts are fed in pieces (the state carries).
 */
int b200rwkv_forward_rows(const b200rwkv_model* m, const int64_t* tokens, int streams, int tokens_per_stream,
                          float* state, int64_t state_stride, float* logits, void* workspace,
                          size_t workspace_bytes, void* stream);

/*
 * One pipeline stage of b200rwkv_forward_rows for a model whose blocks are partitioned
 * contiguously over several GPUs (the layer split: each GPU holds the blocks of its stage, as the
 * reference's TORCH_SPLIT strategy places whole layers on devices).  `m` describes THIS stage:
 * n_layer and `layers` are the stage's blocks; emb/ln0 are needed only by the first stage, ln_out/head
 * only by the last.
 *   tokens   first stage: device int64 [streams][tokens_per_stream]; later stages: NULL
 *   x        device f32 [streams*tokens_per_stream][n_embd], 16-byte aligned: the residual stream.
 *            Later stages read it (as received from the previous stage); every stage leaves its
 *            output in it for the caller to hand to the next GPU (peer copy / NCCL send).
 *   state    the stage's own blocks only: stream s at state + s*state_stride, [n_layer][5][n_embd]
 *   logits   last stage: device f32 [streams][n_vocab] (or NULL); other stages: NULL
 * Workspace size: b200rwkv_rows_workspace_bytes of the stage's model.
 * The handoff itself is the caller's (rwkvstic_b200/layer_split.py uses torch.distributed P2P).
 */
int b200rwkv_forward_rows_stage(const b200rwkv_model* m, const int64_t* tokens, float* x, int streams,
                                int tokens_per_stream, float* state, int64_t state_stride, float* logits,
                                void* workspace, size_t workspace_bytes, void* stream);

/*
 * Greedy sampling on the device (replaces the host-side argmax of the reference's sampler for
 * temperature 0, rwkvMaster.py:32-45, which reads the whole logits vector back per token).
 * out[r] = index of the largest of x[r*ldx .. r*ldx+n), lowest index on ties.  `history`
 * (optional, with its device counter and capacity): row 0's result is also appended at
 * history[*history_count] and the counter incremented, so a decode loop can feed `out` straight
 * back as the next token and read all generated ids once at the end.
 */
int b200rwkv_argmax(const float* x, int rows, int n, int64_t ldx, int64_t* out, int64_t* history,
                    int* history_count, int history_capacity, void* stream);

/*
 * Typical sampling on the device (replaces the reference's host-side sampler,
 * samplers/typical.py:1-17, called per token from rwkvMaster.py:39-45 after the whole logits
 * vector has been read back).  Per row: p = softmax(x), s = | -log p - entropy |, the tokens are
 * kept in order of s until their mass reaches `tau`, kept probabilities are raised to 1/temp and
 * one token is drawn by inverse CDF in index order with the caller's uniform number.
 *   x         device f32 [rows][ldx], n values used per row
 *   temp,tau  > 0 (tau >= 1 keeps every token)
 *   u         device f32, uniform in [0,1): row r reads u[r + rows*step], step = *history_count
 *             when a history is given and 0 otherwise (so a captured decode loop draws a fresh
 *             number per replay from a buffer filled once); with a history u must hold
 *             rows * history_capacity numbers, and steps beyond the capacity reuse the last one
 *   out       device int64 [rows]
 *   probs_out optional device f32 [rows][n]: the masked, tempered, unnormalised probabilities
 *   history   as b200rwkv_argmax; needs rows == 1
 * The reference draws with torch.multinomial, whose random stream cannot be matched; what is
 * matched is the distribution it draws from (same kept set, same weights).
 */
int b200rwkv_sample_typical(const float* x, int rows, int n, int64_t ldx, float temp, float tau, const float* u,
                            int64_t* out, float* probs_out, int64_t* history, int* history_count,
                            int history_capacity, void* stream);

/*
 * Unquantised weights: the TORCH-mode matrix-vector product of the reference
 * (agnostic/backends/torch.py:162-164, `x.to(W.dtype).matmul(W).to(x.dtype)`).
 *   y[o] = round_T( sum_j round_T(x[j]) * W[o][j] ),  T = the weights' type, fp32 accumulation
 *   w      device, [n_out][ldw] elements of `dtype` (B200RWKV_BF16 / _F16 / _F32), ldw >= k_in:
 *          the checkpoint's own [out][in] tensor, which the reference keeps and addresses through a
 *          transposed view (initTensor, torch.py:146-152).  Rows that start on 16-byte boundaries
 *          (w and ldw * sizeof(T) multiples of 16, x 16-byte aligned) take the fast path.
 *   x, y   device f32 [k_in], [n_out]; y is overwritten
 * No workspace; every output is summed by one warp in a fixed order (deterministic).
 */
#define B200RWKV_F32 0
#define B200RWKV_BF16 1
#define B200RWKV_F16 2
int b200rwkv_gemv_dense(const void* w, int dtype, int k_in, int n_out, int64_t ldw, const float* x, float* y,
                        void* stream);


/*
 * Unquantised weights: one token through the whole network, the reference's TORCH mode
 * (helpers/loadWeights.py:11-85 with agnostic/backends/torch.py:125-166 as the op table, network
 * agnostic/agnosticRwkv.py:123-187).  Matrices are the checkpoint's own [out][in] tensors in `dtype`
 * (rows contiguous, every row on a 16-byte boundary); vectors are f32, time_decay already
 * -exp(raw) as loadWeights leaves it (loadWeights.py:63-64).  Every product rounds the activation to
 * `dtype`, sums in f32 and rounds the result to `dtype` (torch.py:162-164); the rest is f32.
 */
typedef struct b200rwkv_dense_layer {
  const float *ln1_w, *ln1_b, *ln2_w, *ln2_b;
  const float *att_mix_k, *att_mix_v, *att_mix_r, *ffn_mix_k, *ffn_mix_r;
  const float *time_decay, *time_first;
  const void *att_key, *att_value, *att_receptance, *att_output;   /* [n_embd][n_embd] */
  const void *ffn_key;                                             /* [n_ffn][n_embd] */
  const void *ffn_receptance;                                      /* [n_embd][n_embd] */
  const void *ffn_value;                                           /* [n_embd][n_ffn] */
} b200rwkv_dense_layer;

typedef struct b200rwkv_dense_model {
  int32_t n_layer, n_embd, n_ffn, n_vocab;
  int32_t dtype;                       /* B200RWKV_F32 / _BF16 / _F16: the matrices' type */
  const float* emb;                    /* device f32 [n_vocab][n_embd] */
  const float *ln0_w, *ln0_b, *ln_out_w, *ln_out_b;
  const void* head;                    /* [n_vocab][n_embd] */
  const b200rwkv_dense_layer* layers;  /* HOST array of n_layer entries (device pointers inside) */
} b200rwkv_dense_model;

size_t b200rwkv_dense_workspace_bytes(const b200rwkv_dense_model* m);

/*
 * forward(token, state) -> (logits, state) for one token (agnosticRwkv.py:171-187 with T = 1).
 *   token   device int64[1]
 *   state   device f32 [n_layer][5][n_embd] in the reference's own convention (base.py:61-62 and
 *           agnosticRwkv.py:68-103): rows 0, 1 the token-shift carries, rows 2, 3 the WKV sums scaled
 *           by exp(-row 4), row 4 the running maximum exponent (-1e30 when empty); updated in place
 *   logits  device f32 [n_vocab], or NULL to advance the state only
 * n_embd and n_ffn multiples of 8, n_embd <= 12160.  Enqueues 6 * n_layer + 3 kernels on `stream`
 * (capturable in a CUDA graph), no allocation, no host synchronisation; deterministic.
 */
int b200rwkv_dense_step(const b200rwkv_dense_model* m, const int64_t* token, float* state, float* logits,
                        void* workspace, size_t workspace_bytes, void* stream);

/*
 * The same network for `streams` independent sequences of `tokens_per_stream` tokens each (row r =
 * stream r / tokens_per_stream): every matrix is applied to all rows at once on the tensor cores, as
 * AgnosticRWKV does with a sequence (agnosticRwkv.py:123-187; matvec of a [T, D] input, torch.py:162-164).
 * bf16 and fp16 matrices only (an fp32 product has no exact tensor-core form; feed such a model
 * token by token).  n_embd and n_ffn multiples of 64.
 *   tokens  device int64 [streams][tokens_per_stream]
 *   state   device f32, stream b at state + b * state_stride, [n_layer][5][n_embd] each, updated in place
 *   logits  device f32 [streams][n_vocab] after each stream's last token, or NULL
 * Enqueues about 12 kernels per block on `stream`; no allocation, no host synchronisation.
 */
size_t b200rwkv_dense_rows_workspace_bytes(const b200rwkv_dense_model* m, int streams, int tokens_per_stream);
/*
 * The two calls above for the blocks [layer_begin, layer_end) only, so that a host can keep some blocks'
 * matrices in pinned host memory and bring them to the device while earlier blocks compute (the
 * reference README's TORCH_STREAM mode: "matrixes will be stored in ram and moved to the GPU as needed").
 * The embedding (+ ln0) runs when layer_begin == 0, the head when layer_end == n_layer and logits is
 * not NULL; the residual stream stays in the workspace between calls, which must therefore be the same
 * buffer (and, for rows, the same streams x tokens_per_stream) for all ranges of one token / one call.
 * Only the layers of the range are dereferenced on the device; all entries of m->layers must still be
 * filled in (they are checked for NULL and alignment).
 */
int b200rwkv_dense_step_layers(const b200rwkv_dense_model* m, int layer_begin, int layer_end, const int64_t* token, float* state,
                               float* logits, void* workspace, size_t workspace_bytes, void* stream);
int b200rwkv_dense_forward_rows_layers(const b200rwkv_dense_model* m, int layer_begin, int layer_end, const int64_t* tokens,
                                       int streams, int tokens_per_stream, float* state, int64_t state_stride, float* logits,
                                       void* workspace, size_t workspace_bytes, void* stream);
int b200rwkv_dense_forward_rows(const b200rwkv_dense_model* m, const int64_t* tokens, int streams, int tokens_per_stream,
                                float* state, int64_t state_stride, float* logits, void* workspace, size_t workspace_bytes,
                                void* stream);

/*
 * The time-out path under test.  Every device-side wait of the library is bounded; these two calls let a
 * test make a bound run out without faulting anything.  No counterpart in the reference (its kernels do
 * not wait on one another).
 *   b200rwkv_wait_selftest: one small kernel waits, with the given bound, for bytes that are announced to
 *     an mbarrier and never delivered; on expiry it ORs B200RWKV_STATUS_WAIT_FULL into *status (device
 *     int) and returns.  The kernel ends limit_ns after it started.
 *   b200rwkv_debug_expire_waits(1, limit_ns): process-wide switch; while on, the rows kernels of
 *     b200rwkv_dense_step* announce their ring slots but withhold the copies, with limit_ns as the bound of
 *     every wait: each launch gives up after limit_ns, sets the status word of the workspace and runs to
 *     its end (results of such a step are undefined).  b200rwkv_debug_expire_waits(0, 0) switches it off.
 * limit_ns between 1 us and 1 s.
 */
int b200rwkv_wait_selftest(uint64_t limit_ns, int* status, void* stream);
int b200rwkv_debug_expire_waits(int enable, uint64_t limit_ns);

#ifdef __cplusplus
}
#endif
#endif /* B200RWKV_H */
