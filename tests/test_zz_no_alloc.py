"""frx_moe_decode_static, the entry point for callers that cannot allocate device memory, against
frx_moe_decode with a caller-owned workspace: same kernels, so the outputs must be identical.

Two calls in a row with different shapes and inputs, because every call shares one built-in
scratch array that still holds what the previous call left there. Collected last on purpose (a run
that stops at the first failure has then already run every other test). Needs a GPU."""
import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from flashrt_b200.lib import check, lib
from helpers import Experts, cuda

pytestmark = pytest.mark.gpu


def test_static_scratch_matches_workspace_entry_twice(port):
    n, ff, E = 512, 256, 16
    ex = Experts(port, n, ff, E)
    # The first call on a device looks up the scratch array (the CUDA runtime may load that part of
    # the library image, array included, only then): made here, before device memory is watched.
    z = torch.zeros(1, n, device="cuda")
    moe.moe_decode_static(ex.base, ex.stride, E, None, n, ff, z, torch.zeros(1, 1, dtype=torch.int32, device="cuda"),
                          torch.ones(1, 1, device="cuda"), None, torch.empty_like(z))
    torch.cuda.synchronize()
    for call, (T, K, seed) in enumerate([(7, 4, 1), (3, 6, 2)]):
        x = synth.activations(T, n, seed=seed)
        ids, wts, _ = port.route(synth.router_logits(T, E, seed=seed + 10), K)
        gate = np.linspace(-1.5, 1.5, T).astype(np.float32)
        want = moe.moe_decode(ex.base, ex.stride, E, ex.shared_ptr, n, ff, cuda(x), cuda(ids), cuda(wts), cuda(gate))
        dx, di, dw, dg = cuda(x), cuda(ids), cuda(wts), cuda(gate)
        out = torch.full((T, n), float("nan"), device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()        # cudaMemGetInfo: also sees a cudaMalloc made inside the library
        moe.moe_decode_static(ex.base, ex.stride, E, ex.shared_ptr, n, ff, dx, di, dw, dg, out)
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        assert torch.cuda.memory_allocated() == before, "the call must not allocate through torch"
        assert free_after >= free_before, f"the call took {free_before - free_after} bytes of device memory"
        check(lib.frx_moe_decode_static_status(moe._stream()))
        got, ref = out.cpu().numpy(), want.cpu().numpy()
        assert np.isfinite(got).all()
        assert np.array_equal(got, ref), f"call {call}: static-scratch output differs from the workspace entry"
        ref_cpu = port.moe_layer(ex.routed_planar(), ex.blob_bytes, ex.shared_planar, n, ff, x, ids, wts, gate)
        assert np.abs(got - ref_cpu).max() / np.sqrt(np.mean(ref_cpu.astype(np.float64) ** 2)) < 1e-5


def test_static_scratch_rejects_sizes_beyond_its_maximum():
    T, K, n, ff = 64, 10, 2048, 512            # needs about 7.9 MB, the built-in scratch holds 4 MiB
    z = torch.zeros(T, n, device="cuda")
    ids = torch.zeros(T, K, dtype=torch.int32, device="cuda")
    with pytest.raises(moe.FrxError, match="built-in scratch holds"):
        moe.moe_decode_static(z.data_ptr(), 884736, 512, None, n, ff, z, ids, torch.zeros(T, K, device="cuda"), None, torch.empty_like(z))
