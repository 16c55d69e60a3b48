"""Writes tests/golden/tiny.gguf with the gguf-py package (the GGUF format's own Python implementation,
installed in this environment) and records what gguf-py's reader returns for it in
tests/golden/tiny_gguf_expected.json.  Run once, here; both outputs are committed.

    python tests/golden/make_gguf_fixture.py

The tensors are seeded synthetic Q4_K / Q6_K blocks (llm_rs_b200.synth) and small dense arrays; the
metadata covers every value type of the format, including arrays of strings and of numbers."""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import gguf  # noqa: E402
from gguf import GGMLQuantizationType as QT  # noqa: E402

from llm_rs_b200 import synth  # noqa: E402

PATH = os.path.join(HERE, "tiny.gguf")


def main():
    w = gguf.GGUFWriter(PATH, "llama")                      # writes general.architecture = "llama"
    w.add_uint8("test.u8", 200)
    w.add_int8("test.i8", -100)
    w.add_uint16("test.u16", 60000)
    w.add_int16("test.i16", -30000)
    w.add_uint32("llama.block_count", 2)
    w.add_int32("test.i32", -2000000000)
    w.add_float32("llama.attention.layer_norm_rms_epsilon", 1e-5)
    w.add_bool("test.bool", True)
    w.add_string("general.name", "tiny é中\U0001F600")
    w.add_uint64("test.u64", 2 ** 40 + 7)
    w.add_int64("test.i64", -(2 ** 40) - 7)
    w.add_float64("test.f64", 1.0 / 3.0)
    w.add_array("tokenizer.ggml.tokens", ["<s>", "</s>", "hello", "wörld", ""])
    w.add_array("tokenizer.ggml.token_type", [1, 1, 0, 0, 3])
    w.add_array("tokenizer.ggml.scores", [0.0, -1.5, 2.25, -1000.0, 1e-3])
    tensors = {
        "token_embd.weight": (QT.Q4_K, [512, 40], synth.weight(12, 512, 40, tid=901)),
        "blk.0.attn_norm.weight": (QT.F32, [512], np.linspace(0.5, 1.5, 512, dtype=np.float32)),
        "blk.0.ffn_down.weight": (QT.Q6_K, [768, 33], synth.weight(14, 768, 33, tid=902)),
        "blk.0.attn_q.weight": (QT.Q4_K, [256, 7], synth.weight(12, 256, 7, tid=903)),
        "output.weight": (QT.Q6_K, [256, 130], synth.weight(14, 256, 130, tid=904)),
        "rope_freqs.weight": (QT.F32, [32], np.arange(32, dtype=np.float32) / 7.0),
    }
    for name, (qt, shape, data) in tensors.items():
        if qt == QT.F32:
            w.add_tensor(name, data)
        else:
            # raw quantised bytes: gguf-py takes them as a uint8 array of [rows, bytes per row]
            rows = shape[1]
            w.add_tensor(name, np.ascontiguousarray(data).view(np.uint8).reshape(rows, -1), raw_dtype=qt)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()

    r = gguf.GGUFReader(PATH)
    exp = {"file_size": os.path.getsize(PATH), "data_offset": int(r.data_offset), "metadata": {}, "tensors": []}
    for key, field in r.fields.items():
        if key.startswith("GGUF."):
            continue                                          # header pseudo-fields of gguf-py's reader
        v = field.contents()
        exp["metadata"][key] = {"types": [int(t) for t in field.types], "value": v}
    for t in r.tensors:
        raw = bytes(t.data.tobytes())
        exp["tensors"].append({"name": t.name, "dtype": int(t.tensor_type), "shape": [int(d) for d in t.shape],
                               "offset": int(t.data_offset) - int(r.data_offset), "nbytes": int(t.n_bytes),
                               "sha256": hashlib.sha256(raw).hexdigest()})
    with open(os.path.join(HERE, "tiny_gguf_expected.json"), "w") as f:
        json.dump(exp, f, indent=1, ensure_ascii=True)
    print(PATH, exp["file_size"], "bytes;", len(exp["tensors"]), "tensors;", len(exp["metadata"]), "keys")


if __name__ == "__main__":
    main()
