"""Writes the checkpoints of the safetensors golden test with this package's own writer: a tiny
random Qwen2 model (bfloat16 weights, biases) as one file, and the same tensors plus a float32 and
an int32 one split over two shards with an index.  Deterministic: the same bytes every time."""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def write_cases(root: str):
    import tiny
    from blackwellllm_b200.weights.random_init import write_random_model
    from blackwellllm_b200.weights.safetensors_io import TensorFiles, index_folder, write_file
    raw, kw, _ = tiny.CONFIGS["qwen"]
    single = write_random_model(os.path.join(root, "single"), raw, dtype="bfloat16", **kw)
    ents = index_folder(single)
    with TensorFiles() as files:
        tensors = {n: files.read(e) for n, e in sorted(ents.items())}
    tensors["extra.gain_f32"] = torch.linspace(-1, 1, 7, dtype=torch.float32)
    tensors["extra.table_i32"] = torch.arange(12, dtype=torch.int32).reshape(3, 4)
    names = sorted(tensors)
    half = len(names) // 2
    shards = {"model-00001-of-00002.safetensors": names[:half], "model-00002-of-00002.safetensors": names[half:]}
    out = os.path.join(root, "sharded")
    os.makedirs(out, exist_ok=True)
    weight_map = {}
    for shard, ns in shards.items():
        write_file(os.path.join(out, shard), {n: tensors[n] for n in ns})
        weight_map.update({n: shard for n in ns})
    with open(os.path.join(out, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f, indent=1)
    return single, out


if __name__ == "__main__":
    write_cases(sys.argv[1])
