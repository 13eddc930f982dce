"""Host-side mirror of the reference runtime contract over the C ABI: a prepared model shared by
sessions (Qwen3Model, runtime/include/models/qwen3_model.hpp:50-452) and the session verbs
create / prefill / decode / reset (Qwen3Session, runtime/include/qwen3.hpp:32-59), plus the verify
step itself (SpeculativeDecoder::verify_greedy, runtime/src/speculative_decoder.cpp:200-224).
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np

from . import abi

DENSE, QWEIGHT, SCALES, ZEROS = 0, 1, 2, 3


@dataclass
class Shape:
    """Decoder shape (the fields of Qwen3Config, runtime/include/models/qwen3_model.hpp:19-35)."""
    vocab_size: int
    n_layers: int
    n_heads: int
    n_kv_heads: int
    hidden_size: int
    intermediate_size: int
    head_dim: int = 128
    max_position_embeddings: int = 4096
    rms_norm_eps: float = 1e-6
    rope_theta: float = 1e6
    quant_type: int = 0
    group_size: int = 128
    qk_norm: bool = True
    qkv_bias: bool = False
    tied_embeddings: bool = False
    bos_token_id: int = 0
    eos_token_id: int = 0xFFFFFFFF

    def to_c(self) -> abi.ModelConfig:
        return abi.ModelConfig(self.vocab_size, self.n_layers, self.n_heads, self.n_kv_heads, self.hidden_size,
                               self.head_dim, self.intermediate_size, self.max_position_embeddings,
                               self.bos_token_id, self.eos_token_id, self.rms_norm_eps, self.rope_theta,
                               self.quant_type, self.group_size, 1 if self.qk_norm else 0)


def _pointer(data) -> int:
    if isinstance(data, np.ndarray):
        return data.ctypes.data
    return data.data_ptr()  # torch tensor (host or device)


def _shape(data) -> Tuple[int, ...]:
    return tuple(int(x) for x in data.shape)


class Model:
    """Prepared weights on the current device. `tensors`: name -> list of (kind, array)."""

    def __init__(self, shape: Shape, tensors: Dict[str, List[Tuple[int, object]]]):
        lib = abi.load_library()
        entries = []
        keep = []
        for name, items in tensors.items():
            for kind, data in items:
                dims = _shape(data)
                entry = abi.NamedTensor(name.encode(), _pointer(data), (dims[0], dims[1] if len(dims) > 1 else 0),
                                        len(dims), kind)
                entries.append(entry)
                keep.append(data)
        array = (abi.NamedTensor * len(entries))(*entries)
        handle = C.c_void_p()
        config = shape.to_c()
        abi.check(lib.ei_model_create(C.byref(config), array, len(entries), C.byref(handle)))
        self.shape = shape
        self._handle = handle
        self._lib = lib

    @property
    def handle(self):
        return self._handle

    def weight_bytes(self) -> int:
        return self._lib.ei_model_weight_bytes(self._handle)

    def new_session(self, capacity: int, graph: bool = False) -> "Session":
        return Session(self, capacity, graph)

    def close(self) -> None:
        if self._handle:
            self._lib.ei_model_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


@dataclass
class VerifyOutput:
    emitted: int
    context: int
    targets: List[int]          # greedy token of every row
    tokens: List[int] = field(default_factory=list)  # the emitted prefix


class Session:
    """One session: stream, workspace, device control block and managed KV cache."""

    def __init__(self, model: Model, capacity: int, graph: bool = False):
        self._lib = abi.load_library()
        self.model = model
        handle = C.c_void_p()
        abi.check(self._lib.ei_session_create(model.handle, capacity, 1 if graph else 0, C.byref(handle)))
        self._handle = handle

    # -- contract verbs ---------------------------------------------------------------------------
    def prefill(self, tokens: Sequence[int], all_logits=None) -> int:
        """Replaces the history with `tokens`; returns the device pointer of the last row's BF16 logits."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        out = C.c_void_p()
        abi.check(self._lib.ei_session_prefill(self._handle, ids.ctypes.data_as(C.c_void_p), len(ids), C.byref(out),
                                               C.c_void_p(all_logits.data_ptr()) if all_logits is not None else None))
        return out.value

    def decode(self, token: int) -> int:
        out = C.c_void_p()
        abi.check(self._lib.ei_session_decode(self._handle, int(token), C.byref(out)))
        return out.value

    def verify(self, tokens: Sequence[int]) -> VerifyOutput:
        """tokens = [pending, d1..dk]; one verify step, acceptance and KV commit on the device."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        result = abi.VerifyResult()
        logits = C.c_void_p()
        abi.check(self._lib.ei_session_verify(self._handle, ids.ctypes.data_as(C.c_void_p), len(ids), C.byref(result),
                                              C.byref(logits)))
        self.last_logits_ptr = logits.value
        targets = [int(result.tokens[i]) for i in range(len(ids))]
        return VerifyOutput(result.emitted, result.context, targets, targets[:result.emitted])

    def verify_enqueue(self, device_drafts, draft_base: int, rows: int) -> None:
        abi.check(self._lib.ei_session_verify_enqueue(self._handle, C.c_void_p(device_drafts.data_ptr()),
                                                      device_drafts.numel(), draft_base, rows))

    def drain(self) -> Tuple[VerifyOutput, int]:
        result = abi.VerifyResult()
        total = C.c_uint64()
        abi.check(self._lib.ei_session_drain(self._handle, C.byref(result), C.byref(total)))
        targets = [int(t) for t in result.tokens]
        return VerifyOutput(result.emitted, result.context, targets, targets[:result.emitted]), int(total.value)

    def truncate(self, length: int) -> None:
        abi.check(self._lib.ei_session_truncate(self._handle, length))

    def set_pending(self, token: int) -> None:
        abi.check(self._lib.ei_session_set_pending(self._handle, int(token)))

    def reset(self) -> None:
        abi.check(self._lib.ei_session_reset(self._handle))

    def context_size(self) -> int:
        out = C.c_size_t()
        abi.check(self._lib.ei_session_context_size(self._handle, C.byref(out)))
        return out.value

    def context_capacity(self) -> int:
        out = C.c_size_t()
        abi.check(self._lib.ei_session_context_capacity(self._handle, C.byref(out)))
        return out.value

    def synchronize(self) -> None:
        abi.check(self._lib.ei_session_synchronize(self._handle))

    def stream(self) -> int:
        return self._lib.ei_session_stream(self._handle) or 0

    def read_kv(self, layer: int) -> Tuple[np.ndarray, np.ndarray]:
        shape = self.model.shape
        width = shape.n_kv_heads * shape.head_dim
        n = self.context_size()
        k = np.empty((n, width), dtype=np.uint16)
        v = np.empty((n, width), dtype=np.uint16)
        abi.check(self._lib.ei_session_read_kv(self._handle, layer, k.ctypes.data_as(C.c_void_p),
                                               v.ctypes.data_as(C.c_void_p)))
        return k, v

    def read_logits(self, rows: int = 1) -> np.ndarray:
        """BF16 logits (uint16 payload) of the first `rows` rows of the session's logits buffer."""
        out = np.empty((rows, self.model.shape.vocab_size), dtype=np.uint16)
        abi.check(self._lib.ei_session_read_logits(self._handle, rows, out.ctypes.data_as(C.c_void_p)))
        return out

    def launches_per_step(self, rows: int) -> int:
        return self._lib.ei_session_launches_per_step(self._handle, rows)

    def write_kv(self, layer: int, first: int, k, v) -> None:
        """Copies K / V rows (numpy uint16 BF16 arrays or torch tensors, [rows, kv_heads*head_dim]) into the cache."""
        rows = k.shape[0]
        abi.check(self._lib.ei_session_write_kv(self._handle, layer, first, rows, C.c_void_p(_pointer(k)),
                                                C.c_void_p(_pointer(v))))

    def adopt_history(self, length: int, pending: int) -> None:
        abi.check(self._lib.ei_session_adopt_history(self._handle, length, int(pending)))

    def inject_failure(self, nth_launch: int = 0, completion: bool = False) -> None:
        abi.check(self._lib.ei_session_inject_failure(self._handle, nth_launch, 1 if completion else 0))

    def inject_wait_timeout(self, polls: int) -> None:
        """Test hook: the next weight-streaming GEMM's bounded waits run out after `polls` polls."""
        abi.check(self._lib.ei_session_inject_wait_timeout(self._handle, polls))

    def inject_attention_wait_timeout(self, polls: int) -> None:
        """Test hook: the bounded waits of the next attention launch (its K / V tile copies) run out after `polls`."""
        abi.check(self._lib.ei_session_inject_attention_wait_timeout(self._handle, polls))

    def close(self) -> None:
        if self._handle:
            self._lib.ei_session_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def bf16_to_float(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


def greedy_token(row_bits: np.ndarray) -> int:
    """Greedy token of one BF16 logit row with the reference's rules: NaN as -inf, lowest index on ties."""
    values = bf16_to_float(row_bits)
    values = np.where(np.isnan(values), -np.inf, values)
    return int(np.argmax(values))  # numpy returns the first maximum


def speculative_generate(session: Session, prompt: Sequence[int], drafts_for, max_new: int, k: int,
                         eos: Optional[int] = None) -> Tuple[List[int], List[int]]:
    """The reference's outer loop (SpeculativeDecoder::generate_with_callback,
    runtime/src/speculative_decoder.cpp:227-316) with the draft model replaced by `drafts_for(position, k)`,
    which proposes k tokens for positions position+1.. . Returns (emitted tokens, accept lengths)."""
    session.prefill(prompt)
    pending = greedy_token(session.read_logits(1)[0])
    emitted = [pending]
    accepts: List[int] = []
    capacity = session.context_capacity()
    while len(emitted) < max_new:
        room = capacity - session.context_size()
        count = min(k + 1, max_new - len(emitted), room)
        if count <= 0:
            break
        drafts = list(drafts_for(len(prompt) + len(emitted) - 1, count - 1))
        out = session.verify([pending] + drafts)
        accepts.append(out.emitted)
        tokens = out.tokens
        if eos is not None and eos in tokens:
            cut = tokens.index(eos) + 1
            session.truncate(out.context - out.emitted + cut)
            emitted.extend(tokens[:cut - 1])
            break
        emitted.extend(tokens)
        pending = tokens[-1]
    return emitted, accepts


class SessionBatch:
    """Sessions of one model verified in one forward (weights streamed once for all of them). Up to 16 stacked rows
    (sessions * rows) every session ends exactly as after its own Session.verify, bit for bit; above that - up to
    2048 stacked rows, 16 rows per session - the projections run on the tensor cores (the prompt GEMM) and the results
    agree with the single-session step within the rounding of another summation order."""

    def __init__(self, sessions: Sequence["Session"]):
        self._lib = abi.load_library()
        self.sessions = list(sessions)
        handles = (C.c_void_p * len(self.sessions))(*[s._handle for s in self.sessions])
        out = C.c_void_p()
        abi.check(self._lib.ei_batch_create(handles, len(self.sessions), C.byref(out)))
        self._handle = out

    def verify(self, tokens: Sequence[Sequence[int]]) -> List[VerifyOutput]:
        """tokens[j] = [pending, d1..dk] of session j (all of one length)."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        if ids.ndim != 2 or ids.shape[0] != len(self.sessions):
            raise ValueError("one token row per session")
        results = (abi.VerifyResult * len(self.sessions))()
        abi.check(self._lib.ei_batch_verify(self._handle, ids.ctypes.data_as(C.c_void_p), ids.shape[1], results))
        outputs = []
        for r in results:
            targets = [int(r.tokens[i]) for i in range(ids.shape[1])]
            outputs.append(VerifyOutput(r.emitted, r.context, targets, targets[:r.emitted]))
        return outputs

    def close(self) -> None:
        if self._handle:
            self._lib.ei_batch_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass



class SpeculativeDecoder:
    """A target and a draft session generating together without host round trips: mirrors the reference's
    SpeculativeDecoder (runtime/src/speculative_decoder.cpp:227-306), greedy only. A round = k + 1 draft decode
    steps chained on the device, one verify forward of [pending, d1..dk] on the target, acceptance and commit on the
    device; the host synchronises only in drain()."""

    def __init__(self, target: "Session", draft: "Session", drafts_per_round: int):
        self._lib = abi.load_library()
        self.target, self.draft, self.drafts_per_round = target, draft, int(drafts_per_round)
        out = C.c_void_p()
        abi.check(self._lib.ei_speculative_create(target._handle, draft._handle, self.drafts_per_round, C.byref(out)))
        self._handle = out

    def prefill(self, tokens: Sequence[int]) -> int:
        """Both sessions take the prompt; returns the first generated token."""
        ids = np.ascontiguousarray(tokens, dtype=np.uint32)
        first = C.c_uint32()
        abi.check(self._lib.ei_speculative_prefill(self._handle, ids.ctypes.data_as(C.c_void_p), ids.size, C.byref(first)))
        return int(first.value)

    def enqueue(self, rounds: int) -> None:
        abi.check(self._lib.ei_speculative_enqueue(self._handle, int(rounds)))

    def drain(self, limit: int = 1 << 20) -> List[int]:
        """Waits; returns every token generated since the prefill (the first token included)."""
        count = C.c_size_t()
        abi.check(self._lib.ei_speculative_drain(self._handle, None, 0, C.byref(count), None))
        room = min(int(count.value), int(limit))
        out = np.zeros(max(room, 1), dtype=np.uint32)
        abi.check(self._lib.ei_speculative_drain(self._handle, out.ctypes.data_as(C.c_void_p), room, C.byref(count), None))
        return [int(t) for t in out[:room]]

    def truncate(self, generated: int) -> None:
        abi.check(self._lib.ei_speculative_truncate(self._handle, int(generated)))

    def generate(self, tokens: Sequence[int], max_new_tokens: int, eos: Optional[int] = None,
                 rounds_per_drain: int = 8) -> List[int]:
        """Greedy generation of up to max_new_tokens tokens after the prompt, stopping after an EOS token."""
        self.prefill(tokens)
        out: List[int] = []
        while True:
            out = self.drain()
            if eos is not None and eos in out:
                out = out[:out.index(eos) + 1]
                break
            if len(out) >= max_new_tokens:
                out = out[:max_new_tokens]
                break
            self.enqueue(rounds_per_drain)
        self.truncate(len(out))
        return out

    def close(self) -> None:
        if self._handle:
            self._lib.ei_speculative_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
