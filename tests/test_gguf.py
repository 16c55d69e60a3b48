"""GGUF container step, no GPU: the oracle parser against the gguf-py fixture, the native parser
(llmrs_gguf_* through llm_rs_b200.gguf) against both, and the error paths of src/gguf/mod.rs:88-115."""
import hashlib
import json
import os
import struct

import numpy as np
import pytest

from oracle import gguf as OG

HERE = os.path.dirname(os.path.abspath(__file__))
TINY = os.path.join(HERE, "golden", "tiny.gguf")


@pytest.fixture(scope="module")
def expected():
    with open(os.path.join(HERE, "golden", "tiny_gguf_expected.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def G(cuda_lib):
    from llm_rs_b200 import gguf
    return gguf


def close_enough(a, b):
    if isinstance(a, float) or isinstance(b, float):
        return a == pytest.approx(b, rel=0, abs=0) or np.float32(a) == np.float32(b)
    return a == b


# ---------- the oracle, pinned by the fixture gguf-py wrote and read ----------

def test_oracle_reads_the_fixture_as_gguf_py_does(expected):
    buf = open(TINY, "rb").read()
    p = OG.parse(buf)
    assert p["version"] == 3 and p["data_offset"] == expected["data_offset"] and len(buf) == expected["file_size"]
    assert list(p["metadata"]) == list(expected["metadata"])
    for key, rec in expected["metadata"].items():
        t, et, v = p["metadata"][key]
        assert [t] + ([et] if et is not None else []) == rec["types"], key
        if isinstance(v, list):
            assert len(v) == len(rec["value"]) and all(close_enough(a, b) for a, b in zip(v, rec["value"])), key
        else:
            assert close_enough(v, rec["value"]), key
    assert len(p["tensors"]) == len(expected["tensors"])
    for t, rec in zip(p["tensors"], expected["tensors"]):
        assert {k: t[k] for k in ("name", "dtype", "shape", "offset", "nbytes")} == {k: rec[k] for k in ("name", "dtype", "shape", "offset", "nbytes")}
        assert hashlib.sha256(OG.tensor_bytes(buf, p, t["name"])).hexdigest() == rec["sha256"]


def test_oracle_writer_round_trip():
    md = [("a.u32", 4, 7, None), ("a.str", 8, "x", None), ("a.arr", 9, [1, 2, 3], 5), ("a.strs", 9, ["p", "", "q"], 8)]
    ts = [("t0", [256, 2], 12, bytes(range(256)) + bytes(32)), ("t1", [4], 0, struct.pack("<4f", 1, 2, 3, 4))]
    buf = OG.build(md, ts, version=2)
    p = OG.parse(buf)
    assert p["version"] == 2 and [m for m in p["metadata"]] == ["a.u32", "a.str", "a.arr", "a.strs"]
    assert p["metadata"]["a.arr"] == (9, 5, [1, 2, 3]) and p["metadata"]["a.strs"] == (9, 8, ["p", "", "q"])
    assert p["data_offset"] % 32 == 0 and p["tensors"][1]["offset"] == 288
    assert OG.tensor_bytes(buf, p, "t0") == ts[0][3] and OG.tensor_bytes(buf, p, "t1") == ts[1][3]


def test_storage_size_table():
    """src/tensor/mod.rs:36-93."""
    assert OG.storage_size(12, 4096 * 4096) == 4096 * 16 * 144 and OG.storage_size(14, 256) == 210
    assert OG.storage_size(0, 5) == 20 and OG.storage_size(30, 5) == 10 and OG.storage_size(8, 64) == 68
    with pytest.raises(OG.GgufFormatError):
        OG.storage_size(12, 255)


# ---------- the native parser ----------

def native_metadata_plain(g):
    return {k: OG.as_python(v) for k, v in g.metadata.items()}


def test_native_reads_the_fixture(G, expected):
    with G.GgufFile.open(TINY) as g:
        assert g.version == 3 and g.data_offset == expected["data_offset"] and g.file_size() == expected["file_size"]
        md = native_metadata_plain(g)
        assert list(md) == list(expected["metadata"])
        for key, rec in expected["metadata"].items():
            v = md[key]
            if isinstance(v, list):
                assert len(v) == len(rec["value"]) and all(close_enough(a, b) for a, b in zip(v, rec["value"])), key
            else:
                assert close_enough(v, rec["value"]), key
        assert G.arch_name(g) == "llama" and g.as_u32("llama.block_count") == 2
        assert [t.name for t in g.tensors] == [r["name"] for r in expected["tensors"]]
        for t, rec in zip(g.tensors, expected["tensors"]):
            assert (t.dtype, list(t.shape), t.offset, t.nbytes) == (rec["dtype"], rec["shape"], rec["offset"], rec["nbytes"])
            tv = g.tensor_view(t.name)
            assert tv.name == t.name and list(tv.shape) == rec["shape"] and int(tv.dtype) == rec["dtype"]
            assert hashlib.sha256(tv.data.tobytes()).hexdigest() == rec["sha256"]
        with pytest.raises(G.GgufError) as e:
            g.tensor_view("blk.9.nope")
        assert e.value.code == -9 and "tensor not found: blk.9.nope" in str(e.value)


def write(tmp_path, name, buf):
    p = tmp_path / name
    p.write_bytes(buf)
    return str(p)


def test_native_equals_oracle_on_built_files(G, tmp_path):
    rng = np.random.default_rng(5)
    raw = lambda n: rng.integers(0, 256, n, dtype=np.uint8).tobytes()
    md = [("general.architecture", 8, "llama", None), ("k.u8", 0, 255, None), ("k.i8", 1, -128, None),
          ("k.u16", 2, 65535, None), ("k.i16", 3, -32768, None), ("k.u32", 4, 2 ** 32 - 1, None), ("k.i32", 5, -2 ** 31, None),
          ("k.f32", 6, 1.5, None), ("k.bool", 7, 0, None), ("k.u64", 10, 2 ** 64 - 1, None), ("k.i64", 11, -2 ** 63, None),
          ("k.f64", 12, -2.5e300, None), ("k.empty", 9, [], 4), ("k.bools", 9, [1, 0, 1], 7), ("k.i64s", 9, [-1, 2 ** 40], 11),
          ("k.f64s", 9, [0.5, -0.25], 12), ("k.u8s", 9, list(range(7)), 0), ("dup", 4, 1, None), ("dup", 4, 2, None),
          ("k.estr", 8, "", None)]
    ts = [("a", [256, 3], 12, raw(3 * 144)), ("b", [512, 2, 1, 1], 14, raw(4 * 210)), ("c", [5], 30, raw(10)),
          ("d", [64, 2], 8, raw(4 * 34)), ("e", [3, 2], 26, raw(24)), ("a", [4], 0, raw(16))]
    for version in (2, 3):
        buf = OG.build(md, ts, version=version)
        p = OG.parse(buf)
        with G.GgufFile(write(tmp_path, f"v{version}.gguf", buf)) as g:
            assert g.version == version and g.data_offset == p["data_offset"]
            want = {k: v[2] for k, v in p["metadata"].items()}
            got = native_metadata_plain(g)
            assert list(got) == list(want)          # 'dup' appears once, at its first position, with the later value
            for k in want:
                assert got[k] == want[k], k
            assert got["dup"] == 2 and g.as_u32("dup") == 2
            assert g.as_u32("k.u64") == 2 ** 32 - 1 and g.as_u32("k.i64") == 0 and g.as_u32("k.i32") == 2 ** 31
            assert g.as_u32("k.u8") is None and g.as_u32("k.f32") is None and g.as_u32("missing") is None
            assert [(t.name, t.dtype, list(t.shape), t.offset, t.nbytes) for t in g.tensors] == \
                   [(t["name"], t["dtype"], t["shape"], t["offset"], t["nbytes"]) for t in p["tensors"]]
            for name in ("a", "b", "c", "d", "e"):    # "a" twice: the first entry is the one found
                assert g.tensor_view(name).data.tobytes() == OG.tensor_bytes(buf, p, name)


def test_directory_longer_than_the_first_read(G, tmp_path):
    """A token list of several megabytes: the native reader fetches the directory in growing prefixes."""
    toks = [f"tok{i:07d}" * 3 for i in range(120000)]                # ~4.7 MB of strings
    md = [("tokenizer.ggml.tokens", 9, toks, 8), ("after", 4, 77, None)]
    ts = [("w", [256, 4], 12, bytes([i % 251 for i in range(4 * 144)]))]
    buf = OG.build(md, ts)
    with G.GgufFile(write(tmp_path, "big_dir.gguf", buf)) as g:
        assert g.metadata["tokenizer.ggml.tokens"] == toks and g.metadata["after"] == 77
        assert g.data_offset == OG.parse(buf)["data_offset"] > 4 << 20
        assert g.tensor_view("w").data.tobytes() == ts[0][3]


@pytest.mark.parametrize("case,code,text", [
    ("magic", -8, "invalid GGUF magic: 0x46554748"), ("version1", -8, "unsupported GGUF version: 1"),
    ("version4", -8, "unsupported GGUF version: 4"), ("dtype", -8, "unknown dtype: 4"), ("dtype31", -8, "unknown dtype: 31"),
    ("mtype", -8, "unknown metadata type: 13"), ("atype", -8, "unknown metadata type: 9"), ("utf8", -8, "invalid UTF-8 in string"),
    ("truncated", -8, "file ends inside the GGUF directory"), ("outside", -8, "lies outside the file"),
    ("blocks", -8, "not divisible by block size 256"), ("missing", -7, "IO error"), ("empty", -8, "file ends inside"),
    ("biglen", -8, "file ends inside the GGUF directory"), ("bigcount", -8, "file ends inside the GGUF directory"),
])
def test_native_errors(G, tmp_path, case, code, text):
    good = OG.build([("k", 8, "v", None)], [("t", [256], 12, bytes(144))])
    head = struct.pack("<IIQQ", OG.GGUF_MAGIC, 3, 0, 1) + struct.pack("<Q", 1) + b"k"
    tinfo = lambda shape, dt, off: struct.pack("<IIQQ", OG.GGUF_MAGIC, 3, 1, 0) + struct.pack("<Q", 1) + b"t" + \
        struct.pack("<I", len(shape)) + b"".join(struct.pack("<Q", d) for d in shape) + struct.pack("<IQ", dt, off)
    bufs = {
        "magic": struct.pack("<I", OG.GGUF_MAGIC + 1) + good[4:],
        "version1": good[:4] + struct.pack("<I", 1) + good[8:], "version4": good[:4] + struct.pack("<I", 4) + good[8:],
        "dtype": tinfo([256], 4, 0) + bytes(256), "dtype31": tinfo([256], 31, 0) + bytes(256),
        "mtype": head + struct.pack("<I", 13) + bytes(64), "atype": head + struct.pack("<IIQ", 9, 9, 1) + bytes(64),
        "utf8": head + struct.pack("<IQ", 8, 2) + b"\xff\xfe" + bytes(32),
        "truncated": good[:40], "outside": tinfo([256], 12, 0) + bytes(100), "blocks": tinfo([255], 12, 0) + bytes(256),
        "empty": b"",
        # lengths that reach beyond the file, in a file longer than the first prefix read: an error at once,
        # not a reason to read the rest of the file
        "biglen": head + struct.pack("<IQ", 8, 1 << 40) + bytes(3 << 20),
        "bigcount": head + struct.pack("<IIQ", 9, 4, 1 << 61) + bytes(3 << 20),
    }
    path = str(tmp_path / "nope.gguf") if case == "missing" else write(tmp_path, case + ".gguf", bufs[case])
    with pytest.raises(G.GgufError) as e:
        G.GgufFile(path)
    assert e.value.code == code and text in str(e.value), str(e.value)
    if case in bufs and case not in ("outside", "blocks"):           # the oracle refuses the same files
        with pytest.raises(OG.GgufFormatError):
            OG.parse(bufs[case])
