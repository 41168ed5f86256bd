"""moe_q2::run's two options (kernels/cuda/moe_q2.h:26-30) in both prefill forms: bf16 output rows
equal the float rows rounded to nearest; activation scale blocks of 64 stay within the bound the
reference's own test puts on that mode (tests/test_moe_q2.cpp:139-141, 3e-2 relative) of the
per-32 result. Needs a GPU."""
import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from helpers import Experts, cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("form", ["stream", "umma"])
def test_bf16_rows_and_block64(port, form):
    n, ff, E, K, T = 512, 256, 8, 3, 150
    ex = Experts(port, n, ff, E, shared=False)
    x = synth.activations(T, n)
    ids, _, _ = port.route(synth.router_logits(T, E), K)
    base = moe.moe_q2.run(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), form=form)
    b16 = moe.moe_q2.run_ex(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), yd_bf16=True, form=form)
    assert b16.dtype == torch.bfloat16 and torch.equal(b16, base.to(torch.bfloat16))
    b64 = moe.moe_q2.run_ex(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), block64=True, form=form)
    a, b = b64.double(), base.double()
    rel = float(((a - b) ** 2).sum().sqrt() / (b ** 2).sum().sqrt())
    assert 0 < rel < 3e-2, rel
    both = moe.moe_q2.run_ex(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), block64=True, yd_bf16=True, form=form)
    assert torch.equal(both, b64.to(torch.bfloat16))


def test_block64_forms_agree(port):
    n, ff, E, K, T = 512, 256, 8, 3, 150
    ex = Experts(port, n, ff, E, shared=False)
    x = synth.activations(T, n)
    ids, _, _ = port.route(synth.router_logits(T, E), K)
    a = moe.moe_q2.run_ex(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), block64=True, form="stream")
    b = moe.moe_q2.run_ex(ex.base, ex.stride, E, n, ff, cuda(x), cuda(ids), block64=True, form="umma")
    assert torch.equal(a, b)
