"""The time-out path of the bounded device-side waits, exercised without faulting anything: a wait whose
bytes never arrive gives up after its bound, the kernel returns, a status bit tells the host, and the
next normal call computes the same bits as before."""
import time

import pytest
import torch

from rwkvstic_b200 import _lib
from rwkvstic_b200.dense_model import B200DenseRWKV
from rwkvstic_b200.synth import synth_tokens

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_a_wait_that_nothing_satisfies_expires_and_reports():
    L = _lib.lib()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    _lib.check(L.b200rwkv_wait_selftest(2_000_000, status.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert int(status[0]) == _lib.STATUS_WAIT_FULL
    assert 0.002 <= elapsed < 0.5, elapsed
    assert L.b200rwkv_wait_selftest(10, status.data_ptr(), None) == _lib.EINVAL            # bound below 1 us
    assert L.b200rwkv_wait_selftest(2_000_000, None, None) == _lib.EINVAL
    assert L.b200rwkv_debug_expire_waits(1, 5_000_000_000) == _lib.EINVAL                  # above 1 s


def test_rows_kernel_gives_up_when_its_copies_are_withheld_and_recovers():
    L = _lib.lib()
    m = B200DenseRWKV.synthetic(2, 256, vocab=300, seed=4, dtype=torch.float16, device=DEV, use_graph=False)
    toks = synth_tokens(3, seed=1, vocab=300)
    good_state = m.emptyState.clone()
    for t in toks:
        m._tok.copy_(t.reshape(1))
        m._step(good_state, True)
    good = m._logits.clone()
    m.check_status()
    try:
        _lib.check(L.b200rwkv_debug_expire_waits(1, 2_000_000))
        scratch = m.emptyState.clone()
        m._tok.copy_(toks[0].reshape(1))
        t0 = time.perf_counter()
        m._step(scratch, True)                     # every rows launch waits 2 ms for bytes that are never requested
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
    finally:
        _lib.check(L.b200rwkv_debug_expire_waits(0, 0))
    assert elapsed < 2.0, elapsed
    with pytest.raises(_lib.B200RWKVError) as err:
        m.check_status()
    assert err.value.code == _lib.ETIMEOUT
    m.check_status()                               # the status word was cleared by the failed check
    again = m.emptyState.clone()
    for t in toks:
        m._tok.copy_(t.reshape(1))
        m._step(again, True)
    torch.cuda.synchronize()
    assert torch.equal(m._logits, good) and torch.equal(again, good_state)
    m.check_status()
