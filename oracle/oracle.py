"""ctypes access to the CPU checkers. TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the benchmark's CPU-baseline leg may import this module; the
product (the ``flashrt_b200`` package and ``libfrx``) never does.

``port``  : ``liboracle.so``, the scalar C restatement in ``q2_oracle.c``.
``ref``   : ``_ref/libfrx_ref.so``, the reference's own CPU sources compiled unmodified, or
            ``None`` when it has not been built (it can only be built where the reference tree is).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_PORT = os.path.join(_HERE, "liboracle.so")
_REF = os.path.join(_HERE, "_ref", "libfrx_ref.so")


def find_reference() -> str | None:
    """The reference source tree: $FRX_REF_ROOT, else a directory named "reference" beside the
    repository. None when there is none (then only a prebuilt _ref library can be used)."""
    cands = [os.environ.get("FRX_REF_ROOT"), os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")]
    for c in cands:
        if c and os.path.exists(os.path.join(c, "quant", "q2_0", "q2_0.cpp")):
            return c
    return None


def build(ref_root: str | None = None) -> None:
    """Compiles both checkers (the reference one only if the reference tree is present)."""
    ref_root = ref_root or find_reference()
    cmd = ["make", "-C", _HERE] + ([f"REF={ref_root}"] if ref_root else [])
    subprocess.run(cmd, check=True, capture_output=True)


def _p(a: np.ndarray | None):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


def _load(path):
    return C.CDLL(path) if os.path.exists(path) else None


class Port:
    """The scalar oracle. All arrays are C-contiguous numpy arrays."""

    def __init__(self):
        if not os.path.exists(_PORT):
            build()
        self.lib = lib = C.CDLL(_PORT)
        lib.orc_fp16_to_fp32.restype = C.c_float
        lib.orc_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.orc_fp32_to_fp16.restype = C.c_uint16
        lib.orc_fp32_to_fp16.argtypes = [C.c_float]
        lib.orc_mat_bytes.restype = C.c_size_t
        lib.orc_expert_bytes.restype = C.c_size_t
        lib.orc_dot_ggml.restype = C.c_float
        lib.orc_dot_ggml.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        lib.orc_dot_q2_0_q8_1.restype = C.c_double
        lib.orc_dot_q2_0_q8_1.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        lib.orc_quantize_q8_1.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_void_p]
        lib.orc_moe_q2_0.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int,
                                     C.c_size_t, C.c_int]
        lib.orc_convert_q8_0_to_q2_0.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        lib.orc_moe_layer.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_int,
                                      C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                                      C.c_int]

    def fp16_to_fp32(self, h: int) -> float:
        return float(self.lib.orc_fp16_to_fp32(h))

    def fp32_to_fp16(self, f: float) -> int:
        return int(self.lib.orc_fp32_to_fp16(C.c_float(f)))

    def mat_bytes(self, rows, cols) -> int:
        return int(self.lib.orc_mat_bytes(rows, cols))

    def expert_bytes(self, n, ff) -> int:
        return int(self.lib.orc_expert_bytes(n, ff))

    def repack(self, ggml: np.ndarray, rows, cols) -> np.ndarray:
        out = np.empty(self.mat_bytes(rows, cols), np.uint8)
        self.lib.orc_repack(_p(ggml), rows, cols, _p(out))
        return out

    def repack_expert(self, gate, up, down, n, ff) -> np.ndarray:
        out = np.empty(self.expert_bytes(n, ff), np.uint8)
        self.lib.orc_repack_expert(_p(gate), _p(up), _p(down), n, ff, _p(out))
        return out

    def dequant_planar(self, mat: np.ndarray, rows, cols) -> np.ndarray:
        out = np.empty((rows, cols), np.float32)
        self.lib.orc_dequant_planar(_p(mat), rows, cols, _p(out))
        return out

    def dequant_ggml(self, ggml: np.ndarray, rows, cols) -> np.ndarray:
        out = np.empty((rows, cols), np.float32)
        self.lib.orc_dequant_ggml(_p(ggml), rows, cols, _p(out))
        return out

    def quantize_q8(self, x: np.ndarray):
        x = np.ascontiguousarray(x, np.float32)
        n = x.shape[-1]
        flat = x.reshape(-1, n)
        q = np.empty(flat.shape, np.int8)
        d = np.empty((flat.shape[0], n // 32), np.float32)
        for t in range(flat.shape[0]):
            self.lib.orc_quantize_q8(_p(flat[t]), n, _p(q[t]), _p(d[t]))
        return q.reshape(x.shape), d.reshape(x.shape[:-1] + (n // 32,))

    def matvec(self, mat: np.ndarray, rows, cols, q: np.ndarray, d: np.ndarray, r0=0, r1=None) -> np.ndarray:
        r1 = rows if r1 is None else r1
        y = np.zeros(rows, np.float32)
        self.lib.orc_matvec(_p(mat), rows, cols, _p(q), _p(d), r0, r1, _p(y))
        return y[r0:r1]

    def dot_ggml(self, ggml_row: np.ndarray, cols, q, d) -> float:
        return float(self.lib.orc_dot_ggml(_p(ggml_row), cols, _p(q), _p(d)))

    def expert_ffn(self, blob: np.ndarray, n, ff, xq, xd, want_hidden=False):
        out = np.empty(n, np.float32)
        h = np.empty(ff, np.float32)
        hq = np.empty(ff, np.int8)
        hd = np.empty(ff // 32, np.float32)
        self.lib.orc_expert_ffn(_p(blob), n, ff, _p(xq), _p(xd), _p(out), _p(h), _p(hq), _p(hd))
        return (out, h, hq, hd) if want_hidden else out

    def chain_rmsnorm_unit(self, x: np.ndarray, y: np.ndarray) -> np.ndarray:
        x, y = np.ascontiguousarray(x, np.float32), np.ascontiguousarray(y, np.float32)
        out = np.empty_like(x)
        self.lib.orc_chain_rmsnorm_unit(_p(x), _p(y), _p(out), x.shape[0], x.shape[1])
        return out

    # ---- ggml-layout pieces
    @staticmethod
    def q8_1_row_bytes(ncols: int) -> int:
        return (ncols + 511) // 512 * 512 // 32 * 36

    def quantize_q8_1(self, x: np.ndarray) -> np.ndarray:
        """x [n_tok][ncols] -> uint8 [n_tok][q8_1_row_bytes]."""
        x = np.ascontiguousarray(x, np.float32)
        n_tok, ncols = x.shape
        out = np.zeros((n_tok, self.q8_1_row_bytes(ncols)), np.uint8)
        self.lib.orc_quantize_q8_1(_p(x), ncols, n_tok, _p(out))
        return out

    def moe_q2_0(self, w: np.ndarray, gate: np.ndarray | None, xq: np.ndarray, ids: np.ndarray, ncols: int, nrows: int,
                 expert_stride: int, act_per_expert: bool) -> np.ndarray:
        """gemv::moe_q for Q2_0: dst [n_tok][k][nrows]."""
        ids = np.ascontiguousarray(ids, np.int32)
        n_tok, k = ids.shape
        dst = np.empty((n_tok, k, nrows), np.float32)
        self.lib.orc_moe_q2_0(_p(w), _p(gate), _p(xq), _p(ids), _p(dst), n_tok, k, ncols, nrows, expert_stride, int(act_per_expert))
        return dst

    def convert_q8_0_to_q2_0(self, src: np.ndarray) -> np.ndarray:
        n = src.size // 68
        dst = np.zeros(n * 18, np.uint8)
        self.lib.orc_convert_q8_0_to_q2_0(_p(src), _p(dst), n)
        return dst

    def route(self, logits: np.ndarray, K: int):
        logits = np.ascontiguousarray(logits, np.float32)
        T, E = logits.shape
        ids = np.empty((T, K), np.int32)
        wts = np.empty((T, K), np.float32)
        probs = np.empty((T, K), np.float32)
        self.lib.orc_route(_p(logits), T, E, K, _p(ids), _p(wts), _p(probs))
        return ids, wts, probs

    def moe_layer(self, experts: np.ndarray, stride, shared, n, ff, x, ids, wts, gate_logit=None, n_threads=1,
                  want_slots=False):
        """experts: uint8 array of planar blobs at e * stride. Returns out [T][n] (and the per-slot
        expert outputs [T*K][n] and shared-expert outputs [T][n] with want_slots)."""
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = np.ascontiguousarray(wts, np.float32)
        T, K = ids.shape
        out = np.empty((T, n), np.float32)
        ys = np.empty((T * K, n), np.float32) if want_slots else None
        ysh = np.empty((T, n), np.float32) if (want_slots and shared is not None) else None
        gl = None if gate_logit is None else np.ascontiguousarray(gate_logit, np.float32)
        self.lib.orc_moe_layer(_p(experts), stride, _p(shared), n, ff, _p(x), T, _p(ids), _p(wts), K, _p(gl), _p(out),
                               _p(ys), _p(ysh), n_threads)
        return (out, ys, ysh) if want_slots else out


class Ref:
    """The reference's own CPU path (compiled from the reference tree)."""

    def __init__(self, lib):
        self.lib = lib
        lib.ref_fp16_to_fp32.restype = C.c_float
        lib.ref_fp16_to_fp32.argtypes = [C.c_uint16]
        lib.ref_fp32_to_fp16.restype = C.c_uint16
        lib.ref_fp32_to_fp16.argtypes = [C.c_float]
        lib.ref_mat_bytes.restype = C.c_size_t
        lib.ref_expert_bytes.restype = C.c_size_t
        lib.ref_dot_ggml.restype = C.c_float
        lib.ref_moe_cpu.argtypes = [C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p,
                                    C.c_void_p, C.c_int, C.c_void_p, C.c_int]
        lib.ref_moe_cpu_timed.restype = C.c_double
        lib.ref_moe_cpu_timed.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_int, C.c_int, C.c_int, C.c_int,
                                          C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_int,
                                          C.c_int]

    def moe_cpu_times(self, experts, stride, layer_stride, n_layers, E, n, ff, x, ids, wts, workers, reps) -> np.ndarray:
        """Seconds of each of `reps` moe_cpu calls (quantize + entry list + moe_cpu), cycling over n_layers."""
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = np.ascontiguousarray(wts, np.float32)
        T, K = ids.shape[-2], ids.shape[-1]
        out = np.empty((T, n), np.float32)
        secs = np.zeros(reps, np.float64)
        self.lib.ref_moe_cpu_times(_p(experts), C.c_size_t(stride), C.c_size_t(layer_stride), n_layers, E, n, ff, _p(x), T, _p(ids), _p(wts), K,
                                   _p(out), workers, reps, _p(secs))
        return secs

    def matvec_timed(self, mats: np.ndarray, n_mats: int, rows: int, cols: int, x: np.ndarray, avx: bool, reps: int):
        """(seconds per call, y) of one planar matrix x one token on one thread, cycling over n_mats matrices."""
        x = np.ascontiguousarray(x, np.float32)
        y = np.zeros(rows, np.float32)
        fn = self.lib.ref_matvec_timed
        fn.restype = C.c_double
        sec = fn(_p(mats), n_mats, rows, cols, _p(x), _p(y), int(avx), reps)
        return float(sec), y

    def have_avx512(self) -> bool:
        return bool(self.lib.ref_have_avx512())

    def physical_cpus(self) -> int:
        return int(self.lib.ref_physical_cpus())

    def fp16_to_fp32(self, h):
        return float(self.lib.ref_fp16_to_fp32(h))

    def fp32_to_fp16(self, f):
        return int(self.lib.ref_fp32_to_fp16(C.c_float(f)))

    def mat_bytes(self, rows, cols):
        return int(self.lib.ref_mat_bytes(rows, cols))

    def expert_bytes(self, n, ff):
        return int(self.lib.ref_expert_bytes(n, ff))

    def repack(self, ggml, rows, cols):
        out = np.empty(self.mat_bytes(rows, cols), np.uint8)
        self.lib.ref_repack(_p(ggml), rows, cols, _p(out))
        return out

    def repack_expert(self, gate, up, down, n, ff):
        out = np.empty(self.expert_bytes(n, ff), np.uint8)
        self.lib.ref_repack_expert(_p(gate), _p(up), _p(down), n, ff, _p(out))
        return out

    def quantize_q8(self, x):
        x = np.ascontiguousarray(x, np.float32)
        n = x.shape[-1]
        q = np.empty(n, np.int8)
        d = np.empty(n // 32, np.float32)
        self.lib.ref_quantize_q8(_p(x), n, _p(q), _p(d))
        return q, d

    def matvec(self, mat, rows, cols, x, r0=0, r1=None, avx=False):
        r1 = rows if r1 is None else r1
        x = np.ascontiguousarray(x, np.float32)
        y = np.empty(r1 - r0, np.float32)
        self.lib.ref_matvec(_p(mat), rows, cols, _p(x), r0, r1, _p(y), int(avx))
        return y

    def dot_ggml(self, ggml_row, cols, x):
        x = np.ascontiguousarray(x, np.float32)
        return float(self.lib.ref_dot_ggml(_p(ggml_row), cols, _p(x)))

    def expert_ffn(self, blob, n, ff, x, avx=False):
        x = np.ascontiguousarray(x, np.float32).reshape(-1, n)
        out = np.empty(x.shape, np.float32)
        self.lib.ref_expert_ffn(_p(blob), n, ff, _p(x), x.shape[0], _p(out), int(avx))
        return out

    def moe_cpu(self, experts, stride, E, n, ff, x, ids, wts, workers=1):
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = np.ascontiguousarray(wts, np.float32)
        T, K = ids.shape
        out = np.empty((T, n), np.float32)
        self.lib.ref_moe_cpu(_p(experts), stride, E, n, ff, _p(x), T, _p(ids), _p(wts), K, _p(out), workers)
        return out

    def moe_cpu_timed(self, experts, stride, layer_stride, n_layers, E, n, ff, x, ids, wts, workers, reps) -> float:
        """Seconds per moe_cpu call (quantize + entry list + moe_cpu), cycling over n_layers."""
        x = np.ascontiguousarray(x, np.float32)
        ids = np.ascontiguousarray(ids, np.int32)
        wts = np.ascontiguousarray(wts, np.float32)
        T, K = ids.shape[-2], ids.shape[-1]
        out = np.empty((T, n), np.float32)
        return float(self.lib.ref_moe_cpu_timed(_p(experts), stride, layer_stride, n_layers, E, n, ff, _p(x), T, _p(ids),
                                                _p(wts), K, _p(out), workers, reps))

    def release(self):
        self.lib.ref_pool_release()


_port = None
_ref = None


def router_logits(w_bf16: np.ndarray, x: np.ndarray) -> np.ndarray:
    """CPU restatement of the router projection (arch/qwen4exp/blocks.cu:83-120, k_bf16_multi with
    no epilogue): y[t][r] = sum_k bf16(w[r][k]) * x[t][k]. w_bf16: uint16 [R][n], the bf16 bit
    patterns; x: float32 [T][n]. The reference adds in fp32 in an order fixed by its launch shape;
    this restatement adds in float64 and is what a tolerance is measured against. Parity unpinned:
    the reference's tests hold no vector for this kernel."""
    w = (w_bf16.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    return x.astype(np.float64) @ w.T


_REF_MTP = os.path.join(_HERE, "_ref", "libfrx_ref_mtp.so")
_ref_mtp = None


def ref_convert_q8_0_to_q2_0(src: np.ndarray, threads: int = 4) -> np.ndarray | None:
    """The reference's own requantizer (arch/qwen4exp/mtp.cu compiled unmodified), or None when that
    library has not been built."""
    global _ref_mtp
    if _ref_mtp is None:
        if not os.path.exists(_REF_MTP):
            return None
        _ref_mtp = C.CDLL(_REF_MTP, mode=os.RTLD_LAZY)
    n = src.size // 68
    dst = np.zeros(n * 18, np.uint8)
    _ref_mtp.ref_convert_q8_0_to_q2_0(_p(src), _p(dst), C.c_size_t(n), threads)
    return dst


def port() -> Port:
    global _port
    if _port is None:
        _port = Port()
    return _port


def ref() -> Ref | None:
    global _ref
    if _ref is None:
        lib = _load(_REF)
        _ref = Ref(lib) if lib is not None else None
    return _ref
