"""TEST INFRASTRUCTURE ONLY - ctypes bindings of the CPU oracle (oracle/libverify_oracle.so) and, where
it has been built, of the unmodified reference library (oracle/_ref/libedge_ref.so).

Only tests/, __graft_entry__.smoke() and bench.py's CPU-baseline legs load this module.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

HERE = Path(__file__).resolve().parent
ORACLE_LIB = HERE / "libverify_oracle.so"
REF_LIB = HERE / "_ref" / "libedge_ref.so"

DENSE, QWEIGHT, SCALES, ZEROS = 0, 1, 2, 3


class _Config(C.Structure):
    _fields_ = [("vocab", C.c_uint64), ("layers", C.c_uint64), ("heads", C.c_uint64), ("kv_heads", C.c_uint64),
                ("hidden", C.c_uint64), ("head_dim", C.c_uint64), ("ffn", C.c_uint64), ("max_pos", C.c_uint64),
                ("eps", C.c_float), ("theta", C.c_float), ("qk_norm", C.c_int32)]


class _RefConfig(C.Structure):
    _fields_ = [("vocab", C.c_uint64), ("layers", C.c_uint64), ("heads", C.c_uint64), ("kv_heads", C.c_uint64),
                ("hidden", C.c_uint64), ("head_dim", C.c_uint64), ("ffn", C.c_uint64), ("max_pos", C.c_uint64),
                ("eps", C.c_float), ("theta", C.c_float), ("qk_norm", C.c_int32), ("group_size", C.c_int32),
                ("eos", C.c_uint32)]


class _RefTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("shape", C.c_uint64 * 2), ("rank", C.c_int32),
                ("transposed", C.c_int32)]


_oracle = None
_ref = None


def oracle_library() -> C.CDLL:
    global _oracle
    if _oracle is None:
        if not ORACLE_LIB.exists():
            subprocess.run(["make", "-C", str(HERE), "oracle"], check=True, capture_output=True)
        lib = C.CDLL(str(ORACLE_LIB))
        lib.vo_last_error.restype = C.c_char_p
        lib.vo_create.restype = C.c_void_p
        lib.vo_create.argtypes = [C.POINTER(_Config), C.c_uint64]
        lib.vo_destroy.argtypes = [C.c_void_p]
        lib.vo_set_dense.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_uint64, C.c_uint64]
        lib.vo_set_awq.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64,
                                   C.c_int32, C.c_int32, C.c_int32]
        lib.vo_size.restype = C.c_uint64
        lib.vo_size.argtypes = [C.c_void_p]
        lib.vo_resize.argtypes = [C.c_void_p, C.c_uint64]
        lib.vo_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p]
        lib.vo_read_kv.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
        lib.vo_argmax.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]
        lib.vo_top2_gap.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_void_p]
        lib.vo_accept.restype = C.c_int32
        lib.vo_accept.argtypes = [C.c_void_p, C.c_void_p, C.c_int32]
        lib.vo_round_bf16_inplace.argtypes = [C.c_void_p, C.c_uint64]
        lib.vo_op_linear.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_void_p]
        lib.vo_op_rms_norm.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_float, C.c_void_p]
        lib.vo_op_rope.argtypes = [C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64, C.c_uint64, C.c_float, C.c_uint64]
        lib.vo_op_rope_table.argtypes = [C.c_void_p, C.c_uint64, C.c_float, C.c_uint64]
        lib.vo_op_silu_multiply.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        lib.vo_op_add.argtypes = [C.c_void_p, C.c_void_p, C.c_uint64, C.c_void_p]
        lib.vo_op_attention.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint64, C.c_uint64, C.c_uint64,
                                        C.c_uint64, C.c_uint64, C.c_int32, C.c_void_p]
        _oracle = lib
    return _oracle


def reference_available() -> bool:
    return REF_LIB.exists()


def reference_library() -> C.CDLL:
    global _ref
    if _ref is None:
        lib = C.CDLL(str(REF_LIB))
        lib.ref_last_error.restype = C.c_char_p
        lib.ref_cpu_create.restype = C.c_void_p
        lib.ref_cpu_create.argtypes = [C.POINTER(_RefConfig), C.POINTER(_RefTensor), C.c_int, C.c_uint64]
        lib.ref_cpu_destroy.argtypes = [C.c_void_p]
        lib.ref_cpu_size.restype = C.c_uint64
        lib.ref_cpu_size.argtypes = [C.c_void_p]
        lib.ref_cpu_resize.argtypes = [C.c_void_p, C.c_uint64]
        lib.ref_cpu_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        lib.ref_cpu_greedy.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
        lib.ref_cpu_read_kv.argtypes = [C.c_void_p, C.c_uint64, C.c_void_p, C.c_void_p]
        lib.ref_cuda_create.restype = C.c_void_p
        lib.ref_cuda_create.argtypes = [C.POINTER(_RefConfig), C.POINTER(_RefTensor), C.c_int, C.POINTER(_RefTensor),
                                        C.c_int, C.POINTER(_RefTensor), C.c_int, C.POINTER(_RefTensor), C.c_int,
                                        C.c_uint64]
        lib.ref_cuda_destroy.argtypes = [C.c_void_p]
        lib.ref_cuda_size.restype = C.c_uint64
        lib.ref_cuda_size.argtypes = [C.c_void_p]
        lib.ref_cuda_resize.argtypes = [C.c_void_p, C.c_uint64]
        lib.ref_cuda_forward.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]
        # direct operators on device pointers (absent from a library built before they were added)
        if hasattr(lib, "ref_op_rms_norm"):
            P, U = C.c_void_p, C.c_uint64
            lib.ref_op_rms_norm.argtypes = [P, P, P, U, U, C.c_float]
            lib.ref_op_add.argtypes = [P, P, P, U]
            lib.ref_op_silu_multiply.argtypes = [P, P, P, U]
            lib.ref_op_rope_precomputed.argtypes = [P, U, U, U, P, U, U]
            lib.ref_op_store_kv.argtypes = [P, P, U, U, U, U]
            lib.ref_op_awq_linear.argtypes = [P, U, U, U, P, P, U, P, U, P, P]
            lib.ref_op_linear.argtypes = [P, U, U, U, P, P, P]
            lib.ref_op_attention_prefill.argtypes = [P, P, P, P, U, U, U, U, U, U]
        _ref = lib
    return _ref


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def bf16_to_float(bits: np.ndarray) -> np.ndarray:
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------ model-level oracle
class OracleModel:
    """The CPU restatement over a synthetic model. `tensors`: name -> [(kind, numpy array)] with BF16 payloads
    as uint16 (the layout edge_infer_b200.synthetic.make_model produces)."""

    def __init__(self, shape, tensors: Dict[str, List[Tuple[int, np.ndarray]]], capacity: int,
                 round_awq_weights: bool = True):
        self.lib = oracle_library()
        self.shape = shape
        cfg = _Config(shape.vocab_size, shape.n_layers, shape.n_heads, shape.n_kv_heads, shape.hidden_size,
                      shape.head_dim, shape.intermediate_size, shape.max_position_embeddings, shape.rms_norm_eps,
                      shape.rope_theta, 1 if shape.qk_norm else 0)
        self.handle = C.c_void_p(self.lib.vo_create(C.byref(cfg), capacity))
        for name, items in tensors.items():
            kinds = {kind: data for kind, data in items}
            if QWEIGHT in kinds:
                q, s, z = kinds[QWEIGHT], kinds[SCALES], kinds[ZEROS]
                inp = q.shape[1] * 8
                self._check(self.lib.vo_set_awq(self.handle, name.encode(), _ptr(np.ascontiguousarray(q)),
                                                _ptr(np.ascontiguousarray(s)), _ptr(np.ascontiguousarray(z)),
                                                q.shape[0], inp, shape.group_size, s.shape[1],
                                                1 if round_awq_weights else 0))
            else:
                data = _f32(bf16_to_float(kinds[DENSE]))
                rows, cols = (data.shape[0], data.shape[1]) if data.ndim == 2 else (1, data.shape[0])
                self._check(self.lib.vo_set_dense(self.handle, name.encode(), _ptr(data), rows, cols))
        if shape.tied_embeddings:
            data = _f32(bf16_to_float(dict(tensors["token_embeddings.weight"])[DENSE]))
            self._check(self.lib.vo_set_dense(self.handle, b"lm_head", _ptr(data), data.shape[0], data.shape[1]))

    def _check(self, status: int) -> None:
        if status:
            raise RuntimeError(self.lib.vo_last_error().decode())

    def forward(self, tokens: Sequence[int], mode: int) -> np.ndarray:
        """Appends the tokens at the current length; logits FP32 [rows, vocab]. mode 0 = FP32 reference
        executor, 1 = BF16-staged (the CUDA path's rounding points)."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty((len(ids), self.shape.vocab_size), dtype=np.float32)
        self._check(self.lib.vo_forward(self.handle, _ptr(ids), len(ids), mode, _ptr(logits)))
        return logits

    def size(self) -> int:
        return self.lib.vo_size(self.handle)

    def resize(self, length: int) -> None:
        self._check(self.lib.vo_resize(self.handle, length))

    def read_kv(self, layer: int) -> Tuple[np.ndarray, np.ndarray]:
        width = self.shape.n_kv_heads * self.shape.head_dim
        k = np.empty((self.size(), width), dtype=np.float32)
        v = np.empty_like(k)
        self._check(self.lib.vo_read_kv(self.handle, layer, _ptr(k), _ptr(v)))
        return k, v

    def __del__(self):
        try:
            self.lib.vo_destroy(self.handle)
        except Exception:
            pass


def argmax(logits: np.ndarray) -> np.ndarray:
    logits = _f32(logits)
    out = np.empty(logits.shape[0], dtype=np.uint32)
    oracle_library().vo_argmax(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out))
    return out


def top2_gap(logits: np.ndarray) -> np.ndarray:
    logits = _f32(logits)
    out = np.empty(logits.shape[0], dtype=np.float32)
    oracle_library().vo_top2_gap(_ptr(logits), logits.shape[0], logits.shape[1], _ptr(out))
    return out


def accept(inputs: Sequence[int], targets: Sequence[int]) -> int:
    a = np.ascontiguousarray(inputs, dtype=np.uint32)
    b = np.ascontiguousarray(targets, dtype=np.uint32)
    return int(oracle_library().vo_accept(_ptr(a), _ptr(b), len(a)))


# ------------------------------------------------------------------ operator-level oracle (staged arithmetic)
def op_linear(x: np.ndarray, w: np.ndarray, bias: Optional[np.ndarray]) -> np.ndarray:
    """x [rows, k], w [n, k] (FP32 arrays of BF16 values) -> round_bf16(x w^T + bias), FP64 accumulation."""
    x, w = _f32(x), _f32(w)
    out = np.empty((x.shape[0], w.shape[0]), dtype=np.float32)
    b = _f32(bias) if bias is not None else None
    oracle_library().vo_op_linear(_ptr(x), _ptr(w), _ptr(b) if b is not None else None, x.shape[0], w.shape[0],
                                  x.shape[1], _ptr(out))
    return out


def op_rms_norm(x: np.ndarray, weight: np.ndarray, eps: float) -> np.ndarray:
    x, weight = _f32(x), _f32(weight)
    out = np.empty_like(x)
    oracle_library().vo_op_rms_norm(_ptr(x), _ptr(weight), x.shape[0], x.shape[1], eps, _ptr(out))
    return out


def op_rope(x: np.ndarray, offset: int, theta: float, max_pos: int) -> np.ndarray:
    out = _f32(x).copy()
    rows, heads, d = out.shape
    oracle_library().vo_op_rope(_ptr(out), rows, heads, d, offset, theta, max_pos)
    return out


def op_rope_table(head_dim: int, theta: float, max_pos: int) -> np.ndarray:
    table = np.empty((max_pos, head_dim), dtype=np.float32)
    oracle_library().vo_op_rope_table(_ptr(table), head_dim, theta, max_pos)
    return table


def op_silu_multiply(gate: np.ndarray, up: np.ndarray) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty_like(gate)
    oracle_library().vo_op_silu_multiply(_ptr(gate), _ptr(up), gate.size, _ptr(out))
    return out


def op_add(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    oracle_library().vo_op_add(_ptr(a), _ptr(b), a.size, _ptr(out))
    return out


def op_attention(q: np.ndarray, k: np.ndarray, v: np.ndarray, offset: int, mode: int = 1) -> np.ndarray:
    """q [rows, heads, d], k/v [length, kv_heads, d] -> out [rows, heads, d]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    out = np.empty_like(q)
    oracle_library().vo_op_attention(_ptr(q), _ptr(k), _ptr(v), q.shape[0], q.shape[1], k.shape[1], q.shape[2], offset,
                                     mode, _ptr(out))
    return out


# ------------------------------------------------------------------ the unmodified reference (oracle/_ref)
def _ref_config(shape) -> _RefConfig:
    return _RefConfig(shape.vocab_size, shape.n_layers, shape.n_heads, shape.n_kv_heads, shape.hidden_size,
                      shape.head_dim, shape.intermediate_size, shape.max_position_embeddings, shape.rms_norm_eps,
                      shape.rope_theta, 1 if shape.qk_norm else 0, shape.group_size, shape.eos_token_id)


def _ref_tensors(items: List[Tuple[str, np.ndarray, bool]]):
    keep = []
    array = (_RefTensor * len(items))()
    for i, (name, data, transposed) in enumerate(items):
        data = np.ascontiguousarray(data)
        keep.append(data)
        if data.ndim == 2:
            # `transposed`: data is the physical [out, in]; the logical shape handed over is [in, out].
            shape = (data.shape[1], data.shape[0]) if transposed else data.shape
        else:
            shape = (data.shape[0], 0)
        array[i] = _RefTensor(name.encode(), data.ctypes.data, shape, data.ndim, 1 if transposed else 0)
    return array, keep


class ReferenceCpu:
    """QwenModel<float> on the CPU, driven as a verify loop: the reference's own FP32 executor. It forces
    QK-norm off and takes no AWQ weights, so only dense, qk_norm=False shapes are meaningful here."""

    def __init__(self, shape, tensors, capacity: int):
        self.lib = reference_library()
        self.shape = shape
        items = []
        for name, kinds in tensors.items():
            data = dict(kinds)[DENSE]
            values = _f32(bf16_to_float(data))
            items.append((name, values, values.ndim == 2 and name != "token_embeddings.weight"))
        if shape.tied_embeddings:
            values = _f32(bf16_to_float(dict(tensors["token_embeddings.weight"])[DENSE]))
            items.append(("lm_head", values, True))
        array, self._keep = _ref_tensors(items)
        cfg = _ref_config(shape)
        self.handle = C.c_void_p(self.lib.ref_cpu_create(C.byref(cfg), array, len(items), capacity))
        if not self.handle:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def forward(self, tokens: Sequence[int]) -> np.ndarray:
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty((len(ids), self.shape.vocab_size), dtype=np.float32)
        if self.lib.ref_cpu_forward(self.handle, _ptr(ids), len(ids), _ptr(logits)):
            raise RuntimeError(self.lib.ref_last_error().decode())
        return logits

    def greedy(self, logits: np.ndarray) -> np.ndarray:
        logits = _f32(logits)
        out = np.empty(logits.shape[0], dtype=np.uint32)
        if self.lib.ref_cpu_greedy(self.handle, _ptr(logits), logits.shape[0], _ptr(out)):
            raise RuntimeError(self.lib.ref_last_error().decode())
        return out

    def size(self) -> int:
        return self.lib.ref_cpu_size(self.handle)

    def resize(self, length: int) -> None:
        if self.lib.ref_cpu_resize(self.handle, length):
            raise RuntimeError(self.lib.ref_last_error().decode())

    def read_kv(self, layer: int) -> Tuple[np.ndarray, np.ndarray]:
        width = self.shape.n_kv_heads * self.shape.head_dim
        k = np.empty((self.size(), width), dtype=np.float32)
        v = np.empty_like(k)
        if self.lib.ref_cpu_read_kv(self.handle, layer, _ptr(k), _ptr(v)):
            raise RuntimeError(self.lib.ref_last_error().decode())
        return k, v

    def __del__(self):
        try:
            self.lib.ref_cpu_destroy(self.handle)
        except Exception:
            pass


class ReferenceCuda:
    """Qwen3Session<bf16>::prefill_eager + op::cuda::sample of the unmodified reference on the current GPU."""

    def __init__(self, shape, tensors, capacity: int):
        self.lib = reference_library()
        self.shape = shape
        dense, qweights, scales, zeros = [], [], [], []
        for name, kinds in tensors.items():
            kinds = dict(kinds)
            if QWEIGHT in kinds:
                qweights.append((name, kinds[QWEIGHT], False))
                scales.append((name, kinds[SCALES], False))
                zeros.append((name, kinds[ZEROS], False))
            else:
                data = kinds[DENSE]
                dense.append((name, data, data.ndim == 2 and name != "token_embeddings.weight"))
        if shape.tied_embeddings:
            dense.append(("lm_head", dict(tensors["token_embeddings.weight"])[DENSE], True))
        d, k1 = _ref_tensors(dense)
        q, k2 = _ref_tensors(qweights)
        s, k3 = _ref_tensors(scales)
        z, k4 = _ref_tensors(zeros)
        self._keep = (k1, k2, k3, k4)
        cfg = _ref_config(shape)
        self.handle = C.c_void_p(self.lib.ref_cuda_create(C.byref(cfg), d, len(dense), q, len(qweights), s, len(scales),
                                                          z, len(zeros), capacity))
        if not self.handle:
            raise RuntimeError(self.lib.ref_last_error().decode())

    def forward(self, tokens: Sequence[int], want_logits: bool = True) -> Tuple[Optional[np.ndarray], np.ndarray]:
        """Returns (BF16 logits as FP32 [rows, vocab] or None, greedy tokens [rows])."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        logits = np.empty((len(ids), self.shape.vocab_size), dtype=np.uint16) if want_logits else None
        greedy = np.empty(len(ids), dtype=np.uint32)
        if self.lib.ref_cuda_forward(self.handle, _ptr(ids), len(ids), _ptr(logits) if want_logits else None,
                                     _ptr(greedy)):
            raise RuntimeError(self.lib.ref_last_error().decode())
        return (bf16_to_float(logits) if want_logits else None), greedy

    def size(self) -> int:
        return self.lib.ref_cuda_size(self.handle)

    def resize(self, length: int) -> None:
        if self.lib.ref_cuda_resize(self.handle, length):
            raise RuntimeError(self.lib.ref_last_error().decode())

    def __del__(self):
        try:
            self.lib.ref_cuda_destroy(self.handle)
        except Exception:
            pass


class ReferenceOps:
    """The unmodified reference's direct CUDA operators (op::cuda::*, BF16) on DEVICE pointers of the current GPU.
    Arguments are objects with a data_ptr() (torch CUDA tensors); every call returns after a stream synchronise."""

    def __init__(self):
        self.lib = reference_library()
        if not hasattr(self.lib, "ref_op_rms_norm"):
            raise RuntimeError("oracle/_ref was built without the operator entry points; run `make -C oracle ref`")

    def _check(self, status: int) -> None:
        if status:
            raise RuntimeError(self.lib.ref_last_error().decode())

    @staticmethod
    def _p(tensor):
        return C.c_void_p(tensor.data_ptr()) if tensor is not None else None

    def rms_norm(self, x, weight, out, rows: int, features: int, eps: float) -> None:
        self._check(self.lib.ref_op_rms_norm(self._p(x), self._p(weight), self._p(out), rows, features, eps))

    def add(self, a, b, out, count: int) -> None:
        self._check(self.lib.ref_op_add(self._p(a), self._p(b), self._p(out), count))

    def silu_multiply(self, gate, up, out, count: int) -> None:
        self._check(self.lib.ref_op_silu_multiply(self._p(gate), self._p(up), self._p(out), count))

    def rope_precomputed(self, data, rows: int, heads: int, head_dim: int, table, positions: int, offset: int) -> None:
        self._check(self.lib.ref_op_rope_precomputed(self._p(data), rows, heads, head_dim, self._p(table), positions,
                                                     offset))

    def store_kv(self, source, cache, rows: int, width: int, capacity: int, offset: int) -> None:
        self._check(self.lib.ref_op_store_kv(self._p(source), self._p(cache), rows, width, capacity, offset))

    def awq_linear(self, x, rows: int, k: int, n: int, qweight, scales, padded_groups: int, zeros, group: int, bias,
                   out) -> None:
        self._check(self.lib.ref_op_awq_linear(self._p(x), rows, k, n, self._p(qweight), self._p(scales), padded_groups,
                                               self._p(zeros), group, self._p(bias), self._p(out)))

    def linear(self, x, rows: int, k: int, n: int, weight, bias, out) -> None:
        self._check(self.lib.ref_op_linear(self._p(x), rows, k, n, self._p(weight), self._p(bias), self._p(out)))

    def attention_prefill(self, q, k, v, out, rows: int, heads: int, kv_heads: int, head_dim: int, length: int,
                          offset: int) -> None:
        self._check(self.lib.ref_op_attention_prefill(self._p(q), self._p(k), self._p(v), self._p(out), rows, heads,
                                                      kv_heads, head_dim, length, offset))
