"""The safetensors reader and writer against the reference project's own loader.

``tests/golden/reference_safetensors.json`` holds what fxslava/BlackwellLLM's ``SafetensorsLoader``
(src/core/safetensors.cpp, compiled on the CPU by ``tests/golden/make_safetensors_golden.sh``) found
in two checkpoints that THIS package's writer made (``tests/golden/write_safetensors_cases.py``): a
tiny random Qwen2 model in one file, and the same tensors plus a float32 and an int32 one in two
shards behind an index.  So the reference reads our files; here the same files are written again
(the writer is deterministic) and our reader must find every tensor where the reference found it.
"""
import json
import os
import sys

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
from write_safetensors_cases import write_cases  # noqa: E402

from blackwellllm_b200.weights.safetensors_io import TensorFiles, index_folder  # noqa: E402

DTYPES = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32}


def test_reader_finds_every_tensor_where_the_reference_found_it(tmp_path):
    with open(os.path.join(HERE, "golden", "reference_safetensors.json")) as f:
        golden = json.load(f)
    single, sharded = write_cases(str(tmp_path))
    for folder, key in ((single, "model.safetensors"), (sharded, "model.safetensors.index.json")):
        ents = index_folder(folder)
        ref = {e["name"]: e for e in golden[key]}
        assert sorted(ents) == sorted(ref)
        with TensorFiles() as files:
            for name, e in ents.items():
                r = ref[name]
                assert e.dtype == DTYPES[r["dtype"]] and list(e.shape) == r["shape"], name
                assert e.nbytes == r["byte_size"] and e.begin == r["file_offset"], name
                assert os.path.basename(e.path) == r["shard"], name
                t = files.read(e)
                assert t.dtype == e.dtype and tuple(t.shape) == e.shape and t.numel() * t.element_size() == e.nbytes
    kinds = {e["dtype"] for e in golden["model.safetensors.index.json"]}
    assert kinds == {"BF16", "F32", "I32"}          # the reference names the kept 32-bit kinds as we do
    with TensorFiles() as files:
        ents = index_folder(sharded)
        assert files.read(ents["extra.table_i32"]).tolist() == [[0, 1, 2, 3], [4, 5, 6, 7], [8, 9, 10, 11]]
