"""A pipeline wait that runs out becomes a status bit and an exception, never a hang.

The kernels' bounded wait is exercised through `nsa_selftest_wait_timeout`: one warp polls a barrier that nobody arrives
on (nothing else is in flight), gives up after the poll limit, ORs its bit into the status word and returns.  Checked
here: the kernel returns, the bit is set, the second wait of the same kernel gave up on the shortened budget (the drain
path), `check_status()` raises and clears the word, the non-blocking poll used by NSACore.forward raises too, and an
ordinary launch afterwards still matches the oracle."""
import ctypes

import pytest
import torch

from oracle import nsa_oracle as O

pytestmark = pytest.mark.gpu


def _fire(polls=64):
    from flash_nsa import _lib
    from flash_nsa.ops._common import status_word
    word = status_word(torch.device("cuda", torch.cuda.current_device()))
    info = torch.zeros(1, dtype=torch.int32, device="cuda")
    rc = _lib.lib().nsa_selftest_wait_timeout(ctypes.c_void_p(word.data_ptr()), ctypes.c_int32(polls), ctypes.c_void_p(info.data_ptr()),
                                              ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 0
    return word, info


def test_a_wait_that_runs_out_sets_the_status_bit_and_the_context_stays_usable():
    import flash_nsa
    from flash_nsa import _lib
    word, info = _fire()
    torch.cuda.synchronize()                       # the kernel returned
    assert int(word.item()) & 512
    assert int(info.item()) == 2 * 1000 + 8        # both waits gave up; the budget was cut to the drain value after the first
    with pytest.raises(_lib.NsaError, match="wait self-test"):
        flash_nsa.check_status()
    assert int(word.item()) == 0                   # cleared by the check
    flash_nsa.check_status()                       # and clean now

    # the next ordinary launch still works: compressed attention on a small case against the oracle
    from flash_nsa import NSAHelper
    from flash_nsa.ops import mean_pooling, compress_attn
    torch.manual_seed(0)
    T, QH, KH, D = 300, 8, 2, 64
    q, k, v = [torch.randn(T, h, D).bfloat16() for h in (QH, KH, KH)]
    NSAHelper.reset_context_parallel()
    NSAHelper.set_hyperparameters()
    NSAHelper.init_cu_seqlens(torch.tensor([0, T], dtype=torch.int32, device="cuda"))
    ck, cv = mean_pooling(k.cuda()), mean_pooling(v.cuda())
    o, _ = compress_attn(q.cuda(), ck, cv)
    ref, _ = O.cmp_attn(q.float(), ck.float().cpu(), cv.float().cpu(), [0, T])
    assert (o.float().cpu() - ref).abs().max().item() <= 2e-2


def test_the_next_forward_reports_a_time_out_of_the_previous_call_without_synchronising():
    import flash_nsa
    from flash_nsa import _lib
    from flash_nsa.ops._common import post_status
    torch.manual_seed(1)
    T, QH, KH, D = 200, 8, 2, 64
    q, k, v = [torch.randn(T, h, D).bfloat16().cuda() for h in (QH, KH, KH)]
    w = torch.randn(T, QH, 3).bfloat16().cuda()
    cu = torch.tensor([0, T], dtype=torch.int32, device="cuda")
    flash_nsa.NSAHelper.reset_context_parallel()
    core = flash_nsa.NSACore(flash_nsa.NSAConfig(head_dim=D, num_heads=QH, num_kv_heads=KH))
    core(q, k, v, w, cu)                           # clean call: posts a clean word
    torch.cuda.synchronize()
    core(q, k, v, w, cu)                           # still clean
    torch.cuda.synchronize()                       # (its own status copy has landed, so the next one is not skipped)
    _fire()                                        # a kernel "of this call" gives up ...
    post_status(q.device)                          # ... and the word goes to the host behind it, as at the end of a forward
    torch.cuda.synchronize()
    with pytest.raises(_lib.NsaError, match="gave up waiting"):
        core(q, k, v, w, cu)
    torch.cuda.synchronize()
    flash_nsa.check_status()                       # the poll cleared the word
    core(q, k, v, w, cu)
    torch.cuda.synchronize()
    flash_nsa.check_status()
