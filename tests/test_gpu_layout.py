"""Q2_0 storage on the device against the oracle: bit-exact repack, relayout round trip and
dequantised weights. Needs a GPU."""
import numpy as np
import pytest
import torch

from flashrt_b200 import moe, synth
from helpers import Experts, cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,cols", [(8, 4096), (96, 2560), (512, 2048), (1, 64)])
def test_repack_bit_exact(port, rows, cols):
    g = synth.ggml_blocks(np.random.default_rng(20260927), rows, cols)
    got = moe.repack(cuda(g.reshape(-1)), rows, cols).cpu().numpy()
    assert np.array_equal(got, port.repack(g, rows, cols))


@pytest.mark.parametrize("n,ff", [(256, 128), (2048, 512), (2560, 640), (128, 384)])
def test_tile_untile_round_trip_and_dequant(port, n, ff):
    ex = Experts(port, n, ff, 3, shared=False)
    back = moe.untile_experts(ex.tiled, n, ff, 3).cpu().numpy().reshape(3, -1)
    assert np.array_equal(back, ex.planar)
    # the tiled blob is a permutation of the planar one: same multiset of bytes
    tiled = ex.tiled.cpu().numpy().reshape(3, ex.stride)[:, :ex.blob_bytes]
    assert np.array_equal(np.sort(tiled[1]), np.sort(ex.planar[1]))
    gu = port.mat_bytes(ff, n)
    for e in range(3):
        blob = ex.tiled[e * ex.stride:(e + 1) * ex.stride]
        g, u, d = moe.dequant_expert(blob, n, ff)
        assert np.array_equal(g.cpu().numpy(), port.dequant_planar(ex.planar[e][:gu], ff, n))
        assert np.array_equal(u.cpu().numpy(), port.dequant_planar(ex.planar[e][gu:2 * gu], ff, n))
        assert np.array_equal(d.cpu().numpy(), port.dequant_planar(ex.planar[e][2 * gu:], n, ff))


def test_dequant_edge_scales(port):
    # zero, subnormal, largest finite and negative scales decode exactly
    n, ff = 128, 128
    rng = np.random.default_rng(1)
    g, u, d = synth.expert_ggml(rng, n, ff)
    for blocks in (g, u, d):
        blocks[0, 0:2] = np.array([0x0000], np.uint16).view(np.uint8)
        blocks[1, 0:2] = np.array([0x0001], np.uint16).view(np.uint8)
        blocks[2, 0:2] = np.array([0x7BFF], np.uint16).view(np.uint8)
        blocks[3, 0:2] = np.array([0x8400], np.uint16).view(np.uint8)
    planar = port.repack_expert(g, u, d, n, ff)
    tiled = moe.tile_experts(cuda(planar), n, ff, 1)
    gg, uu, dd = moe.dequant_expert(tiled, n, ff)
    gu = port.mat_bytes(ff, n)
    assert np.array_equal(gg.cpu().numpy(), port.dequant_planar(planar[:gu], ff, n))
    assert np.array_equal(dd.cpu().numpy(), port.dequant_planar(planar[2 * gu:], n, ff))


def test_arena_addressing_and_load(port):
    n, ff, L, E = 256, 128, 2, 5
    ex = Experts(port, n, ff, L * E, shared=False)
    arena = moe.ExpertArena(L, E, n, ff)
    assert arena.stride == moe.expert_stride(n, ff) and arena.stride % 4096 == 0
    assert arena.blob(1, 2) == arena.base() + (1 * E + 2) * arena.stride      # ExpertArena::blob
    assert arena.total_bytes() == L * E * arena.stride
    with pytest.raises(moe.FrxError):
        arena.blob(2, 0)
    host = torch.from_numpy(ex.planar.reshape(-1))
    arena.load_planar(0, 0, E, host[:E * ex.blob_bytes])                       # from host memory
    arena.load_planar(1, 0, E, host[E * ex.blob_bytes:].cuda())                # from device memory
    torch.cuda.synchronize()
    import ctypes
    # read the arena back through an untile of its own memory
    back = torch.empty(L * E * ex.blob_bytes, dtype=torch.uint8, device="cuda")
    moe.check(moe.lib.frx_q2_untile_experts(ctypes.c_void_p(arena.base()), arena.stride, ctypes.c_void_p(back.data_ptr()),
                                            ex.blob_bytes, L * E, n, ff, None))
    torch.cuda.synchronize()
    assert np.array_equal(back.cpu().numpy().reshape(L * E, -1), ex.planar)
    arena.close()
