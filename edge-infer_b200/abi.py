"""ctypes declarations of the C ABI in include/edge_infer_b200.h.

Python is only the test and benchmark harness; the product is the shared library.
Loading fails loudly if the library has not been built: there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libedge_infer_b200.so"

EI_OK = 0
_STATUS_EXCEPTIONS = {
    1: ValueError,        # std::invalid_argument
    2: IndexError,        # std::out_of_range
    3: OverflowError,     # std::overflow_error
    4: RuntimeError,      # std::runtime_error
    5: AssertionError,    # std::logic_error
    6: BufferError,       # std::length_error
    7: RuntimeError,      # poisoned session
}


class PoisonedError(RuntimeError):
    """The session is unusable after a failed stream completion."""


class LogicError(AssertionError):
    """std::logic_error of the reference contract (e.g. decode before prefill)."""


class LengthError(BufferError):
    """std::length_error of the reference contract (capacity exhausted)."""


_STATUS_EXCEPTIONS[5] = LogicError
_STATUS_EXCEPTIONS[6] = LengthError
_STATUS_EXCEPTIONS[7] = PoisonedError


class View1(C.Structure):
    _fields_ = [("data", C.c_void_p), ("shape", C.c_size_t * 1), ("stride", C.c_size_t * 1)]


class View2(C.Structure):
    _fields_ = [("data", C.c_void_p), ("shape", C.c_size_t * 2), ("stride", C.c_size_t * 2)]


class View3(C.Structure):
    _fields_ = [("data", C.c_void_p), ("shape", C.c_size_t * 3), ("stride", C.c_size_t * 3)]


class Array(C.Structure):
    _fields_ = [("data", C.c_void_p), ("size", C.c_size_t)]


class Context(C.Structure):
    _fields_ = [("handle", C.c_void_p), ("stream", C.c_void_p), ("device", C.c_int32),
                ("multiprocessors", C.c_int32), ("max_threads_per_block", C.c_int32),
                ("shared_memory_limit", C.c_size_t)]


class DenseWeight(C.Structure):
    _fields_ = [("data", C.c_void_p), ("bias", C.c_void_p), ("input_features", C.c_int32),
                ("output_features", C.c_int32), ("leading_dimension", C.c_int32), ("operation", C.c_int32)]


class AwqWeight(C.Structure):
    _fields_ = [("qweight", C.c_void_p), ("scales", C.c_void_p), ("zeros", C.c_void_p), ("bias", C.c_void_p),
                ("input_features", C.c_int32), ("output_features", C.c_int32), ("group_size", C.c_int32),
                ("padded_groups", C.c_int32)]


class VerifyResult(C.Structure):
    _fields_ = [("emitted", C.c_int32), ("context", C.c_int32), ("tokens", C.c_uint32 * 16)]


class ModelConfig(C.Structure):
    _fields_ = [("vocab_size", C.c_uint64), ("n_layers", C.c_uint64), ("n_heads", C.c_uint64),
                ("n_kv_heads", C.c_uint64), ("hidden_size", C.c_uint64), ("head_dim", C.c_uint64),
                ("intermediate_size", C.c_uint64), ("max_position_embeddings", C.c_uint64),
                ("bos_token_id", C.c_uint32), ("eos_token_id", C.c_uint32), ("rms_norm_eps", C.c_float),
                ("rope_theta", C.c_float), ("quant_type", C.c_int32), ("group_size", C.c_int32),
                ("qk_norm", C.c_int32)]


class NamedTensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("data", C.c_void_p), ("shape", C.c_uint64 * 2), ("rank", C.c_int32),
                ("kind", C.c_int32)]


# name -> (restype, argtypes); every symbol the header declares.
_S = C.c_int
_P = C.c_void_p
_Z = C.c_size_t
PROTOTYPES = {
    "ei_last_error": (C.c_char_p, []),
    "ei_version": (C.c_char_p, []),
    "ei_prepare_execution_context": (_S, [_P, C.POINTER(Context)]),
    "ei_prepare_dense_bf16": (_S, [View2, View1, C.POINTER(DenseWeight)]),
    "ei_prepare_awq_bf16": (_S, [View2, View2, View2, _Z, _Z, View1, C.POINTER(AwqWeight)]),
    "ei_linear_scratch_bytes": (_Z, [_Z, _Z, _Z]),
    "ei_linear_bf16": (_S, [C.POINTER(Context), View2, C.POINTER(DenseWeight), View2, _P, _Z]),
    "ei_awq_linear_bf16": (_S, [C.POINTER(Context), View2, C.POINTER(AwqWeight), View2, _P, _Z]),
    "ei_awq_gate_up_silu_bf16": (_S, [C.POINTER(Context), View2, C.POINTER(AwqWeight), View2]),
    "ei_add_bf16": (_S, [C.POINTER(Context), Array, Array, Array]),
    "ei_silu_multiply_bf16": (_S, [C.POINTER(Context), Array, Array, Array]),
    "ei_rms_norm_bf16": (_S, [C.POINTER(Context), Array, Array, Array, _Z, _Z, C.c_float]),
    "ei_gather_bf16": (_S, [C.POINTER(Context), View1, View2, View2]),
    "ei_rope_precomputed_bf16": (_S, [C.POINTER(Context), View3, View2, _Z, _P, _P]),
    "ei_build_rope_table": (_S, [_P, _Z, _Z, C.c_float]),
    "ei_store_kv_bf16": (_S, [C.POINTER(Context), View2, View2, _Z, _P]),
    "ei_attention_scratch_bytes": (_Z, [_Z, _Z, _Z, _Z]),
    "ei_attention_prefill_bf16": (_S, [C.POINTER(Context), View3, View3, View3, View3, _Z, _P, _Z]),
    "ei_attention_verify_bf16": (_S, [C.POINTER(Context), View3, View3, View3, View3, _P, _P, _Z]),
    "ei_attention_prefill_static_bf16": (_S, [C.POINTER(Context), View3, View3, View3, View3, _Z]),
    "ei_sample_scratch_bytes": (_Z, [_Z, _Z]),
    "ei_sample_greedy_bf16": (_S, [C.POINTER(Context), View2, View1, _P, _Z]),
    "ei_verify_accept": (_S, [C.POINTER(Context), _P, _P, _Z, _P, _P, _P]),
    "ei_model_create": (_S, [C.POINTER(ModelConfig), C.POINTER(NamedTensor), _Z, C.POINTER(_P)]),
    "ei_model_destroy": (None, [_P]),
    "ei_model_config_of": (_S, [_P, C.POINTER(ModelConfig)]),
    "ei_model_weight_bytes": (_Z, [_P]),
    "ei_session_create": (_S, [_P, _Z, C.c_int, C.POINTER(_P)]),
    "ei_session_destroy": (None, [_P]),
    "ei_session_prefill": (_S, [_P, _P, _Z, C.POINTER(_P), _P]),
    "ei_session_decode": (_S, [_P, C.c_uint32, C.POINTER(_P)]),
    "ei_session_verify": (_S, [_P, _P, _Z, C.POINTER(VerifyResult), C.POINTER(_P)]),
    "ei_batch_create": (_S, [C.POINTER(_P), _Z, C.POINTER(_P)]),
    "ei_batch_destroy": (None, [_P]),
    "ei_batch_verify": (_S, [_P, _P, _Z, C.POINTER(VerifyResult)]),
    "ei_speculative_create": (_S, [_P, _P, _Z, C.POINTER(_P)]),
    "ei_speculative_destroy": (None, [_P]),
    "ei_speculative_prefill": (_S, [_P, _P, _Z, C.POINTER(C.c_uint32)]),
    "ei_speculative_enqueue": (_S, [_P, _Z]),
    "ei_speculative_drain": (_S, [_P, _P, _Z, C.POINTER(_Z), C.POINTER(VerifyResult)]),
    "ei_speculative_truncate": (_S, [_P, _Z]),
    "ei_session_verify_enqueue": (_S, [_P, _P, _Z, _Z, _Z]),
    "ei_session_drain": (_S, [_P, C.POINTER(VerifyResult), C.POINTER(C.c_uint64)]),
    "ei_session_truncate": (_S, [_P, _Z]),
    "ei_session_set_pending": (_S, [_P, C.c_uint32]),
    "ei_session_reset": (_S, [_P]),
    "ei_session_context_size": (_S, [_P, C.POINTER(_Z)]),
    "ei_session_context_capacity": (_S, [_P, C.POINTER(_Z)]),
    "ei_session_synchronize": (_S, [_P]),
    "ei_session_stream": (_P, [_P]),
    "ei_session_read_kv": (_S, [_P, _Z, _P, _P]),
    "ei_session_read_logits": (_S, [_P, _Z, _P]),
    "ei_session_launches_per_step": (_Z, [_P, _Z]),
    "ei_session_write_kv": (_S, [_P, C.c_size_t, C.c_size_t, C.c_size_t, _P, _P]),
    "ei_session_adopt_history": (_S, [_P, C.c_size_t, C.c_uint32]),
    "ei_session_inject_failure": (_S, [_P, C.c_int, C.c_int]),
    "ei_session_inject_wait_timeout": (_S, [_P, C.c_uint32]),
    "ei_session_inject_attention_wait_timeout": (_S, [_P, C.c_uint32]),
}

_lib = None


def load_library() -> C.CDLL:
    """Loads the built shared library and binds every prototype; raises if it is missing."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise ImportError(
            f"{LIB_PATH} is not built. Run `python edge-infer_b200/build.py` (or __graft_entry__.build()); "
            "there is no CPU fallback for the verify step.")
    lib = C.CDLL(str(LIB_PATH))
    for name, (restype, argtypes) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the library lacks a declared symbol
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib


def check(status: int) -> None:
    """Raises the Python counterpart of the reference's exception class for a failed call."""
    if status == EI_OK:
        return
    message = load_library().ei_last_error().decode("utf-8", "replace")
    raise _STATUS_EXCEPTIONS.get(status, RuntimeError)(message)


# ---- view helpers over torch tensors (device memory is torch's; nothing else of torch is used) ----
def view1(t) -> View1:
    if t is None:
        return View1(None, (0,), (0,))
    return View1(t.data_ptr(), (t.shape[0],), (t.stride(0),))


def view2(t) -> View2:
    return View2(t.data_ptr(), (t.shape[0], t.shape[1]), (t.stride(0), t.stride(1)))


def view3(t) -> View3:
    return View3(t.data_ptr(), tuple(t.shape), tuple(t.stride()))


def array(t) -> Array:
    return Array(t.data_ptr(), t.numel())
