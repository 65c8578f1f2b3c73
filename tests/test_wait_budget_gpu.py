"""The give-up path of the attention kernels, driven without faulting the GPU.

Every wait inside the kernels is bounded by a cycle budget.  Setting the budget to one cycle makes the
first wait that is not already satisfied run out: the CTA stops, waits for its own copies in flight,
frees tensor memory, fills its output rows with NaN and reports {code, CTA} through the status word.
The context stays usable and the next normal call is correct.
"""
import pytest
import torch

from gpu_util import cuda_or_fail, make_qkv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", ["fp32", "fp16+fp32"])       # the two-tile and the one-tile kernel
def test_wait_budget_runs_out_then_the_next_call_is_correct(mode, monkeypatch):
    import sageattention
    from sageattention import _capi as C
    from sageattention import core
    cuda_or_fail()
    q, k, v = make_qkv(1, 4, 2, 700, 128, torch.float16, "HND", seed=81, k_bias=1.0)
    kw = dict(tensor_layout="HND", is_causal=True, pv_accum_dtype=mode)
    good = sageattention.sageattn(q, k, v, **kw)
    torch.cuda.synchronize()
    previous = C.lib().sage_b200_set_wait_budget(1)
    try:
        assert previous > 1_000_000
        with pytest.raises(C.SageB200Error) as err:
            sageattention.sageattn(q, k, v, **kw)               # SAGE_B200_CHECK=1: synchronises and checks
        assert "gave up waiting (code " in str(err.value)
        # without the synchronous check the failure surfaces at the next launch on the device
        monkeypatch.setenv("SAGE_B200_CHECK", "0")
        bad = sageattention.sageattn(q, k, v, **kw)
        torch.cuda.synchronize()
        assert bool(torch.isnan(bad.float()).any())
        with pytest.raises(C.SageB200Error):
            core.check_device_status(q.device)
    finally:
        C.lib().sage_b200_set_wait_budget(0)
    monkeypatch.setenv("SAGE_B200_CHECK", "1")
    again = sageattention.sageattn(q, k, v, **kw)
    torch.cuda.synchronize()
    assert torch.equal(again, good)
    core.check_device_status(q.device)
