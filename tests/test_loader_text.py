"""The safetensors reader against the installed `safetensors` package's own view of the same file and
the error cases of the reference's reader (crates/loader/src/safetensors.rs tests, lib.rs:474-492), the
prompt sidecar parser against the reference's unit-test vectors (crates/embed/src/stella.rs:573-640),
the tokenizer facade and the text-level limits with a small tokenizer built here. No GPU."""
import json
import os
import struct

import numpy as np
import pytest

from logismos_b200.embed import EncodeOpts, InputTooLong, UnsupportedDim, UnsupportedPrompt
from logismos_b200.loader import LoaderError, Reader
from logismos_b200.text import (Prompt, StellaTextModel, Tokenizer, apply_prompt, check_token_limit, extract_json_string_field,
                                load_prompts)


def save(path, tensors, metadata=None):
    from safetensors.numpy import save_file
    save_file(tensors, str(path), metadata=metadata)


def test_reader_matches_the_safetensors_package(tmp_path):
    rng = np.random.default_rng(0)
    t = {"a": np.array([[1, 2], [3, 4]], np.float32), "b": np.array([10, 20], np.float32),   # the reference's tiny fixture
         "model.layers.0.w": rng.standard_normal((3, 5, 7)).astype(np.float32), "h": rng.standard_normal(9).astype(np.float16),
         "i": rng.integers(-9, 9, (4, 2)).astype(np.int32), "u": rng.integers(0, 255, 11).astype(np.uint8),
         "s": rng.integers(-9, 9, 6).astype(np.int8), "e": np.zeros((0, 4), np.float32)}
    p = tmp_path / "x.safetensors"
    save(p, t, metadata={"format": "pt", "note": "a \"quoted\" \\ value"})
    r = Reader(p)
    from safetensors import safe_open
    with safe_open(str(p), "np") as f:
        assert sorted(r.names()) == sorted(f.keys()) and len(r) == len(t)
        for n in f.keys():
            v = r.get(n)
            ref = f.get_tensor(n)
            assert v.shape == ref.shape and v.array.dtype == ref.dtype and np.array_equal(v.array, ref), n
    assert r.get("a").dtype == "F32" and r.get("h").dtype == "F16" and r.get("i").dtype == "I32"
    # archive ordering is by on-disk offset, and the data region starts after the 8-byte length + header
    raw = open(p, "rb").read()
    hlen = struct.unpack("<Q", raw[:8])[0]
    hdr = json.loads(raw[8:8 + hlen])
    by_off = sorted((k for k in hdr if k != "__metadata__"), key=lambda k: (hdr[k]["data_offsets"][0], k))
    assert r.names() == by_off and r.data_region_start() == 8 + hlen
    with pytest.raises(LoaderError, match="tensor not found"):
        r.get("missing")
    r.close()


def write_raw(path, header: dict, data: bytes):
    h = json.dumps(header).encode()
    open(path, "wb").write(struct.pack("<Q", len(h)) + h + data)


def test_reader_rejects_what_the_format_forbids(tmp_path):
    p = str(tmp_path / "bad.safetensors")
    ok = {"a": {"dtype": "F32", "shape": [2], "data_offsets": [0, 8]}}
    write_raw(p, ok, b"\0" * 8)
    assert Reader(p).get("a").shape == (2,)
    cases = {
        "range does not match": ({"a": {"dtype": "F32", "shape": [3], "data_offsets": [0, 8]}}, b"\0" * 8),
        "hole or overlaps": ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [4, 8]}}, b"\0" * 8),
        "does not end at the end": ({"a": {"dtype": "F32", "shape": [1], "data_offsets": [0, 4]}}, b"\0" * 8),
        "outside the file": ({"a": {"dtype": "F32", "shape": [4], "data_offsets": [0, 16]}}, b"\0" * 8),
        "unmapped safetensors dtype": ({"a": {"dtype": "I64", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8),
        "unknown dtype": ({"a": {"dtype": "Q9", "shape": [1], "data_offsets": [0, 8]}}, b"\0" * 8),
        "lacks dtype": ({"a": {"shape": [2], "data_offsets": [0, 8]}}, b"\0" * 8),
    }
    for msg, (hdr, data) in cases.items():
        write_raw(p, hdr, data)
        with pytest.raises(LoaderError, match=msg):
            Reader(p)
    open(p, "wb").write(b"\x10\0\0")
    with pytest.raises(LoaderError, match="shorter than"):
        Reader(p)
    open(p, "wb").write(struct.pack("<Q", 1 << 40) + b"{}")
    with pytest.raises(LoaderError, match="header length"):
        Reader(p)
    open(p, "wb").write(struct.pack("<Q", 4) + b"[1] ")
    with pytest.raises(LoaderError, match="not a JSON object"):
        Reader(p)
    with pytest.raises(LoaderError):
        Reader(str(tmp_path / "absent.safetensors"))


def test_get_detects_a_file_that_changed_under_the_mapping(tmp_path):  # crates/loader/src/lib.rs:474-492
    p = tmp_path / "t.safetensors"
    save(p, {"a": np.arange(64, dtype=np.float32), "b": np.arange(8, dtype=np.float32)})
    r = Reader(p)
    assert r.get("a").shape == (64,)
    with open(p, "r+b") as f:
        f.truncate(os.path.getsize(p) + 16)   # the length no longer matches what was mapped
    with pytest.raises(LoaderError, match="changed after it was opened"):
        r.get("b")
    r.close()


def test_prompt_sidecar_parser_reference_vectors(tmp_path):  # crates/embed/src/stella.rs:573-640
    assert extract_json_string_field(r'{"name": "line1\nline2\ttab\rcr\"quote\\backslash"}', "name") == 'line1\nline2\ttab\rcr"quote\\backslash'
    assert extract_json_string_field('{"name": "caf\\u00e9"}', "name") == "cafu00e9"   # \u is not decoded
    assert extract_json_string_field('{"other": "value"}', "name") is None
    assert extract_json_string_field('{"name": "unterminated', "name") is None
    assert load_prompts(tmp_path) == {}   # an absent sidecar is not an error
    (tmp_path / "config_sentence_transformers.json").write_text(
        json.dumps({"prompts": {"s2p_query": "Instruct: retrieve passages.\nQuery: ", "s2s_query": "Instruct: similar.\nQuery: "}}))
    pr = load_prompts(tmp_path)
    assert pr == {"s2p_query": "Instruct: retrieve passages.\nQuery: ", "s2s_query": "Instruct: similar.\nQuery: "}
    os.mkdir(tmp_path / "d"); os.mkdir(tmp_path / "d" / "config_sentence_transformers.json")
    with pytest.raises(Exception):   # a directory in the file's place is an I/O fault, not "absent"
        load_prompts(tmp_path / "d")
    assert apply_prompt(pr, None, "x") == "x"
    assert apply_prompt(pr, Prompt.s2s_query(), "x") == "Instruct: similar.\nQuery: x"
    assert apply_prompt({}, Prompt.s2p_query(), "x") == "x"           # role without a string: unprefixed
    assert apply_prompt(pr, Prompt.custom("Q: "), "x") == "Q: x"
    with pytest.raises(UnsupportedPrompt):
        apply_prompt(pr, Prompt("future_role"), "x")
    check_token_limit(512, 512)
    with pytest.raises(InputTooLong, match="got 513, limit 512"):
        check_token_limit(513, 512)


def make_tokenizer(path, vocab_words):
    """A small word-level tokenizer.json with an EOS appended by the post-processor (the real checkpoint's
    tokenizer also appends its EOS id)."""
    from tokenizers import Tokenizer as HfTok
    from tokenizers.models import WordLevel
    from tokenizers.pre_tokenizers import Whitespace
    from tokenizers.processors import TemplateProcessing
    vocab = {w: i for i, w in enumerate(["<unk>", "<eos>"] + vocab_words)}
    t = HfTok(WordLevel(vocab, unk_token="<unk>"))
    t.add_special_tokens(["<unk>", "<eos>"])
    t.pre_tokenizer = Whitespace()
    t.post_processor = TemplateProcessing(single="$A <eos>", special_tokens=[("<eos>", 1)])
    t.save(str(path))


class FakeIdModel:
    """Stands for the GPU model below the text layer: records the ragged batch it was given."""

    def __init__(self):
        self.calls = []

    def default_dim(self):
        return 128

    def supported_dims(self):
        return [64, 128]

    def max_tokens(self):
        return 6

    def encode_ids_batch(self, ids, cu, opts):
        self.calls.append((ids.tolist(), cu.tolist(), opts.dim))
        return np.zeros((len(cu) - 1, opts.dim or 128), np.float32)


def test_text_front_end_tokenises_prefixes_and_limits(tmp_path):
    words = ["hello", "world", "query", ":", "a", "b", "c", "d", "e"]
    make_tokenizer(tmp_path / "tokenizer.json", words)
    tok = Tokenizer.from_file(tmp_path / "tokenizer.json")
    assert tok.encode("hello world", True) == [2, 3, 1] and tok.encode("hello world", False) == [2, 3]
    assert tok.decode([2, 3, 1], True) == "hello world" and tok.vocab_size() == 11
    with pytest.raises(Exception):
        Tokenizer.from_file(tmp_path / "absent.json")
    m = FakeIdModel()
    tm = StellaTextModel(m, tok, {"s2p_query": "query : "})
    tm.encode_batch(["hello", "a b c"], EncodeOpts(prompt=Prompt.s2p_query()))
    assert m.calls[-1] == ([4, 5, 2, 1, 4, 5, 6, 7, 8, 1], [0, 4, 10], None)   # prefix + text + EOS, one ragged batch
    tm.encode("hello world", EncodeOpts(dim=64))
    assert m.calls[-1] == ([2, 3, 1], [0, 3], 64)
    n = len(m.calls)
    with pytest.raises(UnsupportedDim):        # the dim is checked before tokenising
        tm.encode("hello", EncodeOpts(dim=999))
    with pytest.raises(InputTooLong, match="got 7, limit 6"):   # never truncated
        tm.encode_batch(["hello", "a b c d e a"])
    with pytest.raises(InputTooLong):
        tm.encode("a b c", EncodeOpts(max_tokens=3))
    assert len(m.calls) == n                   # nothing reached the device
    tm.encode("a b c d e a b", EncodeOpts(max_tokens=8))   # the caller may raise the limit
    assert m.calls[-1][1] == [0, 8]
