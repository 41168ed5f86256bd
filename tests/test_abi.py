"""The C-ABI library loads on a machine without a GPU, exports every symbol include/frx.h
declares, answers its size queries and rejects bad arguments before touching CUDA. CPU only."""
import ctypes as C
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L():
    from flashrt_b200 import lib
    return lib


def declared():
    text = open(os.path.join(ROOT, "include", "frx.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(frx_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(L):
    names = declared()
    assert len(names) >= 25
    for name in names:
        assert hasattr(L.lib, name), f"{name} declared in frx.h but not exported"
        assert name in L.SIGNATURES, f"{name} has no ctypes signature"
    assert set(L.SIGNATURES) == set(names)


def test_sizes(L):
    assert L.lib.frx_q2_mat_bytes(512, 2048) == 294912
    assert L.lib.frx_q2_expert_bytes(2048, 512) == 884736
    assert L.lib.frx_q2_expert_bytes(2560, 640) == 1382400      # tests/test_q2_0.cpp:141
    assert L.lib.frx_q2_expert_stride(2560, 640) == 1384448     # rounded up to 4 KiB
    assert L.lib.frx_moe_decode_workspace_bytes(64, 10, 2048, 512) > 0
    assert L.lib.frx_moe_decode_workspace_bytes(0, 10, 2048, 512) == 0
    assert L.lib.frx_moe_prefill_workspace_bytes(4096, 10, 2048, 512, 512) > 4096 * 10 * 512 * 4
    assert L.lib.frx_moe_hits_scratch_bytes(10, 2560, 640, 3) > 0
    assert L.lib.frx_moe_layer_workspace_bytes(8, 10, 2048, 512) > L.lib.frx_moe_decode_workspace_bytes(8, 10, 2048, 512)
    # the many-layer host form adds four staging slots, whatever the number of layers
    assert (L.lib.frx_moe_layers_host_workspace_bytes(64, 10, 2048, 512, 512) - L.lib.frx_moe_layer_workspace_bytes(64, 10, 2048, 512)
            >= 4 * 64 * (2 * 2048 + 512 + 1) * 4)
    # expert-parallel buffer: two slots of partial sums, one flag word per (rank, block), counters
    assert L.lib.frx_ep_flags_offset(64, 2048) == 2 * 64 * 2048 * 4
    assert L.lib.frx_ep_buffer_bytes(64, 2048) == 2 * 64 * 2048 * 4 + 8 * 1024 * 4 + 256
    assert L.lib.frx_ep_buffer_bytes(0, 2048) == 0


def test_bad_arguments_are_rejected_with_a_message(L):
    one = C.c_void_p(256)   # never dereferenced: validation fails first
    assert L.lib.frx_q2_repack(None, 4, 256, one, None) == L.ERR_ARG
    assert "null" in L.last_error()
    assert L.lib.frx_q2_repack(one, 4, 100, one, None) == L.ERR_SHAPE
    assert L.lib.frx_q2_tile_experts(one, 1 << 20, one, 1 << 20, 1, 2048, 500, None) == L.ERR_SHAPE
    assert L.lib.frx_route_topk(None, one, 4, 2048, 10, one, one, None, None, 0) == L.ERR_SHAPE
    assert "unsupported shape" in L.last_error()
    assert L.lib.frx_route_topk(None, one, 4, 512, 40, one, one, None, None, 0) == L.ERR_SHAPE
    assert L.lib.frx_quantize_q8(None, one, 4, 48, one, one) == L.ERR_SHAPE
    assert L.lib.frx_moe_decode(one, 884736, 512, None, 2048, 500, one, one, one, None, 1, 10, one, None, one, 1 << 30, None) == L.ERR_SHAPE
    assert L.lib.frx_moe_decode(one, 1000, 512, None, 2048, 512, one, one, one, None, 1, 10, one, None, one, 1 << 30, None) == L.ERR_ARG
    assert L.lib.frx_moe_decode(one, 884736, 512, None, 2048, 512, one, one, one, None, 1, 10, one, None, one, 16, None) == L.ERR_WORKSPACE
    assert "workspace" in L.last_error()
    assert L.lib.frx_moe_prefill(one, 884736, 512, 2048, 512, one, one, 8, 10, one, one, 16, None) == L.ERR_WORKSPACE
    assert L.lib.frx_moe_hits(one, one, 10, one, 2560, 640, one, 1 << 30, one, None, 200) == L.ERR_SHAPE
    assert L.lib.frx_moe_layer_ep_allreduce(one, 884736, 512, 0, 256, None, 2048, 512, one, one, None, 8, 10, one, None, None, None, one, 1 << 30,
                                            None) == L.ERR_ARG   # no communication state
    assert L.lib.frx_moe_layers_host(None, 884736, 512, None, 2048, 512, one, one, None, 2, 8, 10, one, one, 1 << 30, None) == L.ERR_ARG
    with pytest.raises(L.FrxError):
        L.check(L.ERR_SHAPE)


def test_cpp_shim_compiles_against_the_header():
    # include/frx_shim.hpp re-declares the reference's C++ signatures over the C ABI
    import shutil
    import subprocess
    import tempfile
    gxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime.h")):
        pytest.skip("needs g++ and the CUDA headers")
    src = ('#include "frx_shim.hpp"\n'
           "void f(cudaStream_t s, const uint8_t* e, const float* x, const int32_t* ids, void* yd, void* ws, int32_t* o, float* w) {\n"
           "  flashrt::moe_q2::run(e, 884736, 512, 2048, 512, x, ids, 8, 10, yd, ws, flashrt::moe_q2::workspace_bytes(8, 10, 2048, 512, 512), s);\n"
           "  flashrt::qwen4exp::moe_route_topk(s, x, 8, 512, 10, o, w, nullptr);\n"
           "  flashrt::qwen4exp::moe_hits(nullptr, ids, 10, x, 2560, 640, ws, w, s, 3);\n"
           "  flashrt::moe_q2::run(e, 884736, 512, 2048, 512, x, ids, 8, 10, yd, ws, 1 << 20, s, true, true);\n"
           # the draft head's MoE as arch/qwen4exp/mtp.cu:636-666 writes it
           "  const int64_t gu = flashrt::gemv::row_bytes(42, 2048) * 512;\n"
           "  flashrt::gemv::quantize_q8_1(x, 2048, 3, ws, s);\n"
           "  flashrt::gemv::moe_q(42, e, e, ws, ids, w, 3, 10, 2048, 512, gu, false, s);\n"
           "  const flashrt::gemm::MoePlan p = flashrt::gemm::moe_prepare(42, 512, x, false, ids, 64, 10, 2048, ws, flashrt::gemm::workspace_bytes(2048, 640), s);\n"
           "  flashrt::gemm::moe_run(p, e, gu, w, 512, s);\n}\n")
    with tempfile.NamedTemporaryFile("w", suffix=".cpp") as f:
        f.write(src)
        f.flush()
        r = subprocess.run([gxx, "-std=c++17", "-fsyntax-only", "-I" + os.path.join(ROOT, "include"), "-I" + cuda_inc, f.name],
                           capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
