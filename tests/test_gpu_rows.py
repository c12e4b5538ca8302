"""GPU parity tests of the many-rows (tensor-core) path: the tile GEMM through the C ABI, then the
whole network in sequence mode and as batched decode, against the reference goldens and against
the one-row streaming path."""
import numpy as np
import pytest
import torch

from oracle import fastquant_oracle as O
from rwkvstic_b200 import ops
from rwkvstic_b200.model import B200RWKV
from rwkvstic_b200.quant import quantize_fastquant, quantize_two_axis
from rwkvstic_b200.synth import synth_checkpoint, synth_tokens

from kernel_contract import fixed_point_gemv
from test_gpu_kernels import random_matrix

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3
CANARY = 12345.678


def t64(a):
    return torch.from_numpy(np.asarray(a)).double()


def run_gemm(mats, xs):
    """Outputs live inside canary-padded buffers so that a write outside the matrix is seen."""
    rows = xs[0].shape[0]
    bufs = [torch.full((rows + 2, m.n_out), CANARY, dtype=torch.float32, device=DEV) for m in mats]
    views = [b[1:1 + rows] for b in bufs]
    ops.gemm_u8([m.to(DEV) for m in mats], [x.to(DEV).contiguous() for x in xs], views)
    torch.cuda.synchronize()
    for b in bufs:
        assert bool((b[0] == CANARY).all()) and bool((b[-1] == CANARY).all())
    return [v.cpu() for v in views]


# (rows, n_out, k_in): partial row tiles, partial output tiles, one and many K steps, the 7B shapes
GEMM_SHAPES = [(1, 80, 128), (64, 128, 128), (3, 19, 384), (65, 257, 768), (130, 3072, 768), (100, 768, 3072),
               (256, 4096, 4096), (96, 16384, 4096), (70, 4096, 16384), (33, 50277, 1024)]


@pytest.mark.parametrize("rows,n,k", GEMM_SHAPES)
def test_gemm_integer_part_is_bit_exact(rows, n, k):
    m = random_matrix(n, k, seed=n + k, zero_offset=True)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows + k)) * 3
    x[rows // 2] *= 1e-3                       # rows of very different magnitude: scaling is per row
    got = run_gemm([m], [x])[0]
    for r in sorted({0, rows // 2, rows - 1}):
        assert torch.equal(got[r], fixed_point_gemv(x[r], m, with_affine=False)), f"row {r}"
    # every row equals what the one-row streaming kernel computes for it
    for r in sorted({0, rows - 1}):
        one = ops.gemv_u8([m.to(DEV)], [x[r].to(DEV).contiguous()])[0].cpu()
        assert torch.equal(got[r], one)


@pytest.mark.parametrize("rows,n,k", [(5, 512, 4096), (20, 4096, 4096), (32, 300, 16384), (2, 2560, 10240)])
def test_gemm_few_rows_split_k_is_bit_exact_and_leaves_its_scratch_clean(rows, n, k):
    """Few rows and a long K: the launch is cut into K slices whose integer sums meet in a scratch
    buffer; the result must stay bit-exact and a second and third call must see a clean scratch."""
    m = random_matrix(n, k, seed=n + k, zero_offset=True)
    x = torch.randn(rows, k, generator=torch.Generator().manual_seed(rows + k)) * 3
    first = run_gemm([m], [x])[0]
    for r in range(rows):
        assert torch.equal(first[r], fixed_point_gemv(x[r], m, with_affine=False)), f"row {r}"
    x2 = torch.randn(rows, k, generator=torch.Generator().manual_seed(99)) * 0.1
    second = run_gemm([m], [x2])[0]
    assert torch.equal(second[0], fixed_point_gemv(x2[0], m, with_affine=False))
    assert torch.equal(run_gemm([m], [x])[0], first)


def test_gemm_fastquant_vs_oracle():
    g = torch.Generator().manual_seed(5)
    w = torch.randn(1000, 1024, generator=g) * 0.02
    m = quantize_fastquant(w)
    x = torch.randn(150, 1024, generator=g)
    got = run_gemm([m], [x])[0]
    om = O.Matrix(w)
    want = om(x.double())                       # the oracle's sequence-mode matmul: [T, in] -> [T, out]
    assert float((got.double() - want).abs().max()) < 1e-4 * max(1.0, float(want.abs().max()))


def test_gemm_three_matrices_of_different_width_and_two_axis():
    g = torch.Generator().manual_seed(6)
    mats = [random_matrix(n, 512, seed=n) for n in (512, 2048, 130)]
    xs = [torch.randn(77, 512, generator=g) for _ in mats]
    together = run_gemm(mats, xs)
    for m, x, y in zip(mats, xs, together):
        assert torch.equal(run_gemm([m], [x])[0], y)                      # grouping never changes the arithmetic
        assert torch.allclose(y[5], fixed_point_gemv(x[5], m), rtol=1e-5, atol=1e-5)
    w = torch.randn(300, 256, generator=g) * 0.05
    m2 = quantize_two_axis(w)
    x = torch.randn(40, 256, generator=g)
    got = run_gemm([m2], [x])[0]
    want = x.double() @ m2.dequant().t()
    assert float((got.double() - want).abs().max()) < 1e-4


def test_gemm_zero_rows_and_determinism():
    m = random_matrix(300, 256, seed=1)
    x = torch.randn(66, 256, generator=torch.Generator().manual_seed(2))
    x[7] = 0
    a = run_gemm([m], [x])[0]
    assert torch.equal(a[7], torch.zeros(300))
    for _ in range(3):
        assert torch.equal(run_gemm([m], [x])[0], a)


def test_gemm_rejects_bad_shapes():
    m = random_matrix(64, 128, seed=3).to(DEV)
    with pytest.raises(ValueError):
        ops.gemm_u8([m], [torch.zeros(4, 64, device=DEV)])
    with pytest.raises(RuntimeError):
        ops.gemm_u8([random_matrix(64, 128, seed=3)], [torch.zeros(4, 128)])


# ---------------------------------------------------------------------------------------- whole network
@pytest.fixture(scope="module")
def tiny():
    return B200RWKV.from_checkpoint(synth_checkpoint(2, 128, vocab=257, seed=31), device=DEV)


@pytest.fixture(scope="module")
def m169():
    return B200RWKV.from_checkpoint(synth_checkpoint(12, 768, seed=1234), device=DEV)


def test_rows_sequence_mode_matches_reference_goldens(tiny, golden):
    g = golden("model_tiny.npz")
    toks = torch.from_numpy(g["tokens"]).reshape(1, -1)
    st = tiny.empty_batch_state(1)
    lg = tiny.forward_rows(toks, st)
    assert float((lg[0].cpu().double() - t64(g["logits_seq"])).abs().max()) < TOL
    ref = t64(g["state_seq"])
    mine = tiny.to_reference_state(st[0]).cpu()
    assert torch.allclose(mine[:, :4], ref[:, :4], rtol=1e-3, atol=1e-4)
    # in two pieces: the state carries
    st = tiny.empty_batch_state(1)
    tiny.forward_rows(toks[:, :5], st)
    lg = tiny.forward_rows(toks[:, 5:], st)
    assert float((lg[0].cpu().double() - t64(g["logits_chunk"])).abs().max()) < TOL


def test_rows_path_agrees_with_one_row_path(tiny):
    B, T = 5, 23
    toks = synth_tokens(B * T, seed=9, vocab=257).reshape(B, T)
    st_rows, st_seq = tiny.empty_batch_state(B), tiny.empty_batch_state(B)
    lg_rows, _ = tiny.forward_batch(toks, st_rows, rows=True)
    lg_seq, _ = tiny.forward_batch(toks, st_seq, rows=False)
    assert float((lg_rows - lg_seq).abs().max()) < 2e-4
    assert torch.allclose(st_rows[:, :, :4], st_seq[:, :, :4], rtol=1e-4, atol=1e-4)
    assert torch.allclose(st_rows[:, :, 4], st_seq[:, :, 4], rtol=1e-5, atol=1e-4)
    # batched decode: many streams, one token each, several steps on the carried states
    for step in range(3):
        nxt = lg_seq.argmax(dim=1).reshape(B, 1).cpu()
        lg_rows, _ = tiny.forward_batch(nxt, st_rows, rows=True)
        lg_seq, _ = tiny.forward_batch(nxt, st_seq, rows=False)
        assert float((lg_rows - lg_seq).abs().max()) < 2e-4
    # a stream's result does not depend on which other streams share the call
    st_one = tiny.empty_batch_state(1)
    lg_one = tiny.forward_rows(toks[3:4], st_one)
    st_all = tiny.empty_batch_state(B)
    lg_all = tiny.forward_rows(toks, st_all)
    assert torch.equal(lg_one[0], lg_all[3]) and torch.equal(st_one[0], st_all[3])


def test_rows_long_rows_use_the_chunked_scan_and_agree_with_the_one_row_path(tiny):
    B, T = 2, 200                                  # > 128 tokens per stream: WKV runs as parallel 64-step chunks
    toks = synth_tokens(B * T, seed=13, vocab=257).reshape(B, T)
    st_rows, st_seq = tiny.empty_batch_state(B), tiny.empty_batch_state(B)
    lg_rows, _ = tiny.forward_batch(toks, st_rows, rows=True)
    lg_seq, _ = tiny.forward_batch(toks, st_seq, rows=False)
    assert float((lg_rows - lg_seq).abs().max()) < 5e-4
    assert torch.allclose(st_rows[:, :, :4], st_seq[:, :, :4], rtol=1e-3, atol=1e-4)
    assert torch.allclose(st_rows[:, :, 4], st_seq[:, :, 4], rtol=1e-5, atol=1e-4)


def test_rows_long_prompt_in_pieces_and_via_forward(tiny):
    toks = synth_tokens(300, seed=11, vocab=257)
    keep = tiny.rows_per_call
    try:
        tiny.rows_per_call = 128                  # 300 tokens -> pieces of 128, 128, 44
        st_a = tiny.empty_batch_state(1)
        a = tiny.forward_rows(toks.reshape(1, -1), st_a)
        tiny.rows_per_call = 4096
        st_b = tiny.empty_batch_state(1)
        b = tiny.forward_rows(toks.reshape(1, -1), st_b)
    finally:
        tiny.rows_per_call = keep
    assert float((a - b).abs().max()) < 2e-4
    lg, st = tiny.forward(toks, tiny.emptyState.clone())   # forward() routes long prompts to the rows path
    assert torch.equal(lg, b[0]) and torch.equal(st, st_b[0])


def test_169m_prompt_rows_path_vs_reference_and_one_row_path(m169, golden):
    g = golden("model_169m.npz")
    prompt = torch.from_numpy(g["prompt"])
    assert prompt.numel() >= m169.rows_threshold           # forward() sends this prompt down the rows path
    st_rows = m169.empty_batch_state(1)
    lg_rows = m169.forward_rows(prompt.reshape(1, -1), st_rows)[0]
    assert float((lg_rows.cpu().double() - t64(g["logits_first"])).abs().max()) < TOL
    keep = m169.rows_threshold
    try:
        m169.rows_threshold = 1 << 30
        lg_one, st_one = m169.forward(prompt, m169.emptyState.clone())
    finally:
        m169.rows_threshold = keep
    assert float((lg_rows - lg_one).abs().max()) < 5e-4
    assert torch.allclose(st_rows[0][:, :4], st_one[:, :4], rtol=1e-3, atol=1e-4)
    # 64 streams decoding in lock step from the same state give 64 times the same logits
    st64 = st_rows.repeat(64, 1, 1, 1).contiguous()
    tok = int(torch.argmax(lg_rows))
    lg64 = m169.forward_rows(torch.full((64, 1), tok, dtype=torch.int64), st64)
    assert bool((lg64 == lg64[0]).all())
    lg1, _ = m169.forward(torch.tensor([tok]), st_one)
    assert float((lg64[0] - lg1).abs().max()) < 5e-4
    assert int(torch.argmax(lg64[0])) == int(g["tokens"][1])


def test_rows_entry_points_reject_bad_shapes(tiny):
    st = tiny.empty_batch_state(2)
    with pytest.raises(ValueError):
        tiny.forward_rows(torch.zeros(3, 4, dtype=torch.int64), st)            # 3 streams, state for 2
    with pytest.raises(ValueError):
        tiny.forward_rows(torch.zeros(2, 0, dtype=torch.int64), st)
    with pytest.raises(ValueError):
        tiny.forward_rows(torch.zeros(2, 4, dtype=torch.int64), st.double())
    with pytest.raises(ValueError):
        tiny.forward_rows_stage(None, torch.zeros(7, 128, device=DEV), st, False)   # 7 rows do not split over 2 streams
    # out-of-range token ids are clamped like the one-row path (never an out-of-bounds gather)
    lg = tiny.forward_rows(torch.tensor([[5, 100000], [-3, 7]]), st)
    assert torch.isfinite(lg).all()


def test_rows_path_agrees_with_one_row_path_at_the_1b5_shape():
    """Full-size shapes (D=2048, F=8192, V=50277, 24 blocks): every tile shape the launcher picks for
    few rows (K slices), a prompt piece and a batch of streams must reproduce the one-row path."""
    model = B200RWKV.synthetic(24, 2048, seed=5, device=DEV)
    toks = synth_tokens(3 * 40, seed=21).reshape(3, 40)
    st_rows = model.empty_batch_state(3)
    lg_rows = model.forward_rows(toks, st_rows)                      # 120 rows
    keep = model.rows_threshold
    try:
        model.rows_threshold = 1 << 30
        st_one = model.empty_batch_state(1)
        lg_one, _ = model.forward(toks[1], st_one[0])                # 40 one-row steps
    finally:
        model.rows_threshold = keep
    assert float((lg_rows[1] - lg_one).abs().max()) < 1e-3
    assert torch.allclose(st_rows[1][:, :4], st_one[0][:, :4], rtol=2e-3, atol=2e-4)
    nxt = lg_rows.argmax(dim=1, keepdim=True)
    lg3 = model.forward_rows(nxt, st_rows)                           # 3 rows: K slices
    lg1, _ = model.forward(nxt[1].cpu(), st_one[0])
    assert float((lg3[1] - lg1).abs().max()) < 1e-3
    st64 = st_rows[1:2].repeat(64, 1, 1, 1).contiguous()             # 64 rows in lock step
    tok = lg3[1].argmax().reshape(1, 1).repeat(64, 1)
    lg64 = model.forward_rows(tok, st64)
    assert bool((lg64 == lg64[0]).all())
    model.check_status()


@pytest.mark.parametrize("embed", [512, 2048, 4096, 5120])
def test_row_preparation_gives_the_same_bits_however_rows_are_grouped(embed):
    """With thousands of rows a preparation CTA walks several consecutive rows for all matrices and keeps the
    layer norm of a row as the next row's token-shift partner; with few rows there is one CTA per (matrix, row).
    Six streams of 280 tokens in one call (1680 rows: groups of rows that straddle the stream boundaries)
    must give exactly the logits and states of the same streams run one per call.  The widths cover every
    instantiation family: 1, 2 and 4 register groups per thread at 256 threads, 512 threads at 5120 inputs,
    and for the ffn value input (4 x embed) 256 threads, 512 threads and the rows too long for registers."""
    model = B200RWKV.synthetic(2, embed, vocab=1000, seed=9, device=DEV)
    B, T = 6, 280
    toks = synth_tokens(B * T, seed=44, vocab=1000).reshape(B, T)
    start = model.empty_batch_state(B)
    start[:, :, :2] = torch.randn(B, model.n_layer, 2, model.n_embd, device=DEV)      # token-shift carries in use
    st_all = start.clone()
    lg_all = model.forward_rows(toks, st_all)
    for b in range(B):
        st = start[b:b + 1].clone()
        lg = model.forward_rows(toks[b:b + 1], st)
        assert torch.equal(lg[0], lg_all[b]), b
        assert torch.equal(st[0], st_all[b]), b
    model.check_status()
