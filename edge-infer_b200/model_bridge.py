"""The reference's Python binding surface for the verify path, over this library.

Mirrors `model_bridge.Model` / `model_bridge.Session` of the reference (bindings/python/model_bridge.cpp:245-275):
a prepared model built from an HF-style config and checkpoint dictionary, independent bounded sessions, and exact
greedy speculative sessions made of a target and a draft model. Generation here is greedy only - the speculative
decoder is exact greedy by construction (runtime/src/speculative_decoder.cpp:233-234) and stochastic sampling is
outside this library - so a request with top_k != 1 and a positive temperature raises ValueError before anything runs.
"""
from __future__ import annotations

from typing import Callable, Mapping, Optional, Sequence

from . import checkpoint, runtime


def _greedy_request(temperature: float, top_p: float, top_k: int) -> None:
    if not top_k >= 1 or not 0.0 < top_p <= 1.0 or temperature != temperature:
        raise ValueError("sampling policy is outside the supported parameters")
    if temperature > 0.0 and top_k != 1:
        raise ValueError("only greedy generation (top_k == 1 or temperature <= 0) is provided")


class Session:
    """One bounded generation session. `generate` starts from a complete fresh prompt; max_length counts the prompt."""

    def __init__(self, session: runtime.Session, draft: Optional[runtime.Session] = None, spec_length: int = 0):
        self._session, self._draft = session, draft
        self._decoder = runtime.SpeculativeDecoder(session, draft, spec_length) if draft is not None else None

    @property
    def capacity(self) -> int:
        return self._session.context_capacity()

    @property
    def device(self) -> str:
        return "cuda"

    @property
    def speculative(self) -> bool:
        return self._decoder is not None

    def reset(self) -> None:
        self._session.reset()
        if self._draft is not None:
            self._draft.reset()

    def generate(self, input_ids: Sequence[int], callback: Callable[[int], None], max_length: int = 100,
                 temperature: float = 1.0, top_p: float = 0.9, top_k: int = 1) -> None:
        _greedy_request(temperature, top_p, top_k)
        prompt = [int(t) for t in input_ids]
        if not prompt:
            raise ValueError("Prompt must be nonempty")
        budget = min(int(max_length), self.capacity) - len(prompt)
        if budget <= 0:
            return
        eos = self._session.model.shape.eos_token_id
        if self._decoder is not None:
            # The decoder needs room for a whole round of drafts beyond what is generated.
            room = self.capacity - len(prompt) - (self._decoder.drafts_per_round + 2)
            for token in self._decoder.generate(prompt, min(budget, max(room, 1)), eos=eos):
                callback(int(token))
            return
        self._session.prefill(prompt)
        token = runtime.greedy_token(self._session.read_logits(1)[0])
        for produced in range(budget):
            callback(int(token))
            if token == eos or produced + 1 == budget:
                break
            self._session.decode(token)
            token = runtime.greedy_token(self._session.read_logits(1)[0])


class Model:
    """Prepared immutable weights; sessions share them."""

    def __init__(self, config: Mapping, weights: Mapping, model_type: str = "qwen3_bf16", device: Optional[str] = None):
        if device not in (None, "cuda"):
            raise ValueError("this library runs on CUDA devices only")
        shape, tensors = checkpoint.admit(config, weights, model_type)
        self._model = runtime.Model(shape, tensors)

    @property
    def max_context_length(self) -> int:
        return self._model.shape.max_position_embeddings

    @property
    def device(self) -> str:
        return "cuda"

    def _capacity(self, capacity: Optional[int]) -> int:
        return min(4096, self.max_context_length) if capacity is None else int(capacity)

    def new_session(self, capacity: Optional[int] = None) -> Session:
        return Session(self._model.new_session(self._capacity(capacity), graph=True))

    def new_speculative_session(self, draft_model: "Model", capacity: Optional[int] = None,
                                spec_length: int = 4) -> Session:
        if not 1 <= int(spec_length) <= 15:
            raise ValueError("Invalid draft capacity")
        size = self._capacity(capacity)
        target = self._model.new_session(size, graph=True)
        draft = draft_model._model.new_session(min(size, draft_model.max_context_length), graph=True)
        return Session(target, draft, int(spec_length))
