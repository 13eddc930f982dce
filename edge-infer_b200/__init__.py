"""B200 (sm_100a) implementation of edge-infer's speculative-decoding verify step.

The product is the shared library built from csrc/ (C ABI in include/edge_infer_b200.h). The Python
modules here are its host-side mirror for tests and benchmarks:
  abi        - ctypes declarations, status -> exception mapping
  operators  - the direct-operator API (op::cuda names)
  runtime    - prepared Model and Session (prefill / decode / verify / reset)
  checkpoint - admission of HF-style dense / AutoAWQ-GEMV checkpoints (names, layouts, metadata)
  model_bridge - the reference's Python binding surface (Model / Session / speculative session) over the above
  sharding   - session sharding over GPUs and the reductions of the benchmark
  synthetic  - seeded synthetic models, prompts and drafts
The directory name is not an importable identifier; load it as `edge_infer_b200`
(see __graft_entry__.load_package()).
"""
from . import abi, checkpoint, model_bridge, operators, runtime, sharding, synthetic  # noqa: F401
from .runtime import Model, Session, Shape  # noqa: F401

__all__ = ["abi", "checkpoint", "model_bridge", "operators", "runtime", "sharding", "synthetic", "Model", "Session",
           "Shape"]
