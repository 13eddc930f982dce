"""Timeline of one verify step replayed from its CUDA graph: where the step's time goes between kernels.

ncu serialises kernels and hides what programmatic dependent launch overlaps; this reads the device's global timer
instead. The library is built a second time with -DEI_TIMELINE (edge-infer_b200/build.py --timeline): thread 0 of
every block of the step's kernels records when the block started, when its dependency wait returned and when it
ended. One step of the Qwen3-8B-shape AWQ session (9 rows, context about 2100) is recorded and summarised per
position in the layer, averaged over the layers:

    launched   first block start, relative to the end of the preceding kernel (negative: launched early)
    released   the last block's dependency wait returned, relative to the end of the preceding kernel
               (the hand-over latency between two kernels)
    after      from that moment to the end of the kernel's last block
    path       end of this kernel - end of the preceding one: the kernel's share of the step

    python edge-infer_b200/build.py --timeline && python edge-infer_b200/timeline.py

The recording costs a few nanoseconds per block; the recorded step is about 3 % slower than the product's.
"""
from __future__ import annotations

import ctypes
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
import __graft_entry__ as entry  # noqa: E402

UNITS = ["elementwise", "attention", "sampling", "smallm_gemm"]
NAMES = {1: "embed_norm", 2: "awq_tma (int4 GEMM)", 3: "qk_norm_rope_store", 4: "verify_attention", 5: "attention_merge",
         6: "residual_norm_vec", 7: "dense_tma (lm_head)", 8: "finalize"}
RECORD = np.dtype([("start", "u8"), ("waited", "u8"), ("end", "u8"), ("kernel", "i4"), ("block", "i4")])


def main():
    import torch

    if not torch.cuda.is_available():
        raise SystemExit("timeline needs a CUDA device")
    package = entry.load_package()
    library = Path(__file__).resolve().parent / "libedge_infer_b200_timeline.so"
    if not library.exists():
        raise SystemExit("build the recording library first: python edge-infer_b200/build.py --timeline")
    package.abi.LIB_PATH = library
    lib = package.abi.load_library()
    syn = package.synthetic
    shape = syn.qwen3_8b_awq(max_position_embeddings=4096)
    model = package.Model(shape, syn.make_device_model(shape, seed=0))
    session = model.new_session(4096, graph=True)
    session.prefill(syn.make_prompt(0, 2048, shape.vocab_size))
    rng = np.random.default_rng(0)

    def step():
        return session.verify([int(t) for t in rng.integers(0, shape.vocab_size, size=9)])

    for _ in range(4):
        step()
    torch.cuda.synchronize()
    for unit in UNITS:
        getattr(lib, "ei_timeline_" + unit)(None, None, 1)
    step()
    torch.cuda.synchronize()
    parts = []
    for unit in UNITS:
        buffer = np.zeros(1 << 16, dtype=RECORD)
        count = ctypes.c_uint(0)
        getattr(lib, "ei_timeline_" + unit)(buffer.ctypes.data_as(ctypes.c_void_p), ctypes.byref(count), 0)
        parts.append(buffer[:min(count.value, 1 << 16)])
    records = np.concatenate(parts)
    records = records[np.argsort(records["start"], kind="stable")]

    # A launch = consecutive records of one kernel in which no block appears twice.
    launches, current = [], None
    for record in records:
        kernel, block = int(record["kernel"]), int(record["block"])
        if current is None or current["kernel"] != kernel or block in current["blocks"]:
            current = {"kernel": kernel, "blocks": set(), "start": [], "waited": [], "end": []}
            launches.append(current)
        current["blocks"].add(block)
        current["start"].append(int(record["start"]))
        current["waited"].append(int(record["waited"]))
        current["end"].append(int(record["end"]))
    origin = min(launches[0]["start"])
    span = (max(max(l["end"]) for l in launches) - origin) / 1e3
    print(f"{len(records)} block records, {len(launches)} launches, step span {span:.1f} us")

    layers = int(shape.n_layers)
    per_layer = (len(launches) - 3) // layers
    rows = {}
    for index in range(1, 1 + per_layer * layers):
        launch, before = launches[index], launches[index - 1]
        previous_end = max(before["end"])
        waited = [w for w in launch["waited"] if w]
        released = max(waited) if waited else min(launch["start"])
        position = (index - 1) % per_layer
        rows.setdefault(position, []).append((
            launch["kernel"], len(launch["blocks"]), (min(launch["start"]) - previous_end) / 1e3,
            (released - previous_end) / 1e3, (max(launch["end"]) - released) / 1e3,
            (max(launch["end"]) - previous_end) / 1e3))
    print(f"{'kernel':<24}{'blocks':>7}{'launched':>10}{'released':>10}{'after':>9}{'path':>9}   (us, mean over {layers} layers)")
    total = 0.0
    for position in range(per_layer):
        data = rows[position]
        kernel, blocks = data[0][0], data[0][1]
        means = [float(np.mean([d[i] for d in data])) for i in range(2, 6)]
        total += means[3]
        print(f"{NAMES.get(kernel, str(kernel)):<24}{blocks:>7}{means[0]:>10.2f}{means[1]:>10.2f}{means[2]:>9.2f}{means[3]:>9.2f}")
    print(f"{'one layer':<24}{'':>7}{'':>10}{'':>10}{'':>9}{total:>9.2f}")
    head = launches[1 + per_layer * layers]
    print(f"after the layers: {NAMES.get(head['kernel'])} {(max(head['end']) - max(launches[per_layer * layers]['end'])) / 1e3:.1f} us, "
          f"then finalize {(max(launches[-1]['end']) - max(head['end'])) / 1e3:.1f} us; "
          f"embed_norm at the start {(max(launches[0]['end']) - origin) / 1e3:.1f} us")


if __name__ == "__main__":
    main()
