"""The text front end of the embedding model: tokenizer facade, prompt application and the
``max_tokens`` rule, i.e. ``EmbeddingModel::encode(&str)`` / ``encode_batch(&[&str])`` above the
id-level GPU model.

Mirrors, in the reference:
  tokenize::Tokenizer                    crates/tokenize/src/lib.rs:41-98 (a facade over the HuggingFace
                                         `tokenizers` library; the same library is used here through its
                                         Python binding)
  Prompt, EncodeOpts                     crates/core/src/lib.rs:40-69
  StellaModel::encode / encode_batch     crates/embed/src/stella.rs:264-325 (dim check first, prompt,
                                         tokenise with special tokens, over-long input is an error and
                                         never truncated, all-ones mask)
  apply_prompt, check_token_limit        crates/embed/src/stella.rs:341-378
  load_prompts, extract_json_string_field  crates/embed/src/stella.rs:525-567
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np

from .embed import EncodeOpts, InputTooLong, IoError, StellaModel, TokenizeError, UnsupportedDim, UnsupportedPrompt


@dataclass(frozen=True)
class Prompt:
    """core::Prompt (crates/core/src/lib.rs:46-53): ``Prompt.s2s_query()``, ``Prompt.s2p_query()``,
    ``Prompt.custom(prefix)``."""
    kind: str
    text: str = ""

    @staticmethod
    def s2s_query() -> "Prompt":
        return Prompt("s2s_query")

    @staticmethod
    def s2p_query() -> "Prompt":
        return Prompt("s2p_query")

    @staticmethod
    def custom(prefix: str) -> "Prompt":
        return Prompt("custom", prefix)


class Tokenizer:
    """tokenize::Tokenizer (crates/tokenize/src/lib.rs:41-98)."""

    def __init__(self, inner):
        self._inner = inner

    @classmethod
    def from_file(cls, path: str) -> "Tokenizer":
        try:
            import tokenizers
            return cls(tokenizers.Tokenizer.from_file(str(path)))
        except Exception as e:  # Error::Upstream
            raise TokenizeError(str(e)) from e

    def encode(self, text: str, add_special_tokens: bool = True) -> List[int]:
        try:
            return list(self._inner.encode(text, add_special_tokens=add_special_tokens).ids)
        except Exception as e:
            raise TokenizeError(str(e)) from e

    def decode(self, ids: Sequence[int], skip_special_tokens: bool = True) -> str:
        try:
            return self._inner.decode([int(i) for i in ids], skip_special_tokens=skip_special_tokens)
        except Exception as e:
            raise TokenizeError(str(e)) from e

    def vocab_size(self) -> int:
        return int(self._inner.get_vocab_size(with_added_tokens=True))

    def vocab_size_base(self) -> int:
        return int(self._inner.get_vocab_size(with_added_tokens=False))


def extract_json_string_field(text: str, key: str) -> Optional[str]:
    """Finds ``"<key>": "<value>"`` in JSON text and returns the value with the escapes \\n \\t \\r \\" \\\\
    decoded; any other escaped character stands for itself, so ``\\uXXXX`` is NOT decoded (the
    reference's stated behaviour, crates/embed/src/stella.rs:541-567 and its tests :573-600)."""
    needle = '"%s"' % key
    k = text.find(needle)
    if k < 0:
        return None
    after = text[k + len(needle):]
    colon = after.find(":")
    if colon < 0:
        return None
    rest = after[colon + 1:]
    q = rest.find('"')
    if q < 0:
        return None
    out, it = [], iter(rest[q + 1:])
    for c in it:
        if c == '"':
            return "".join(out)
        if c == "\\":
            n = next(it, None)
            if n is None:
                return None
            out.append({"n": "\n", "t": "\t", "r": "\r", '"': '"', "\\": "\\"}.get(n, n))
        else:
            out.append(c)
    return None


def load_prompts(root: str) -> Dict[str, str]:
    """crates/embed/src/stella.rs:525-539: the roles ``s2s_query`` / ``s2p_query`` of
    ``config_sentence_transformers.json``; an absent file is an empty map, any other I/O fault is an
    error."""
    path = os.path.join(str(root), "config_sentence_transformers.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            text = f.read()
    except FileNotFoundError:
        return {}
    except OSError as e:
        raise IoError(str(e)) from e
    out = {}
    for key in ("s2s_query", "s2p_query"):
        v = extract_json_string_field(text, key)
        if v is not None:
            out[key] = v
    return out


def apply_prompt(prompts: Dict[str, str], prompt: Optional[Prompt], text: str) -> str:
    """crates/embed/src/stella.rs:341-357."""
    if prompt is None:
        return text
    if not isinstance(prompt, Prompt):
        raise UnsupportedPrompt("unsupported prompt")
    if prompt.kind in ("s2s_query", "s2p_query"):
        p = prompts.get(prompt.kind)
        return text if p is None else p + text
    if prompt.kind == "custom":
        return prompt.text + text
    raise UnsupportedPrompt("unsupported prompt")


def check_token_limit(token_count: int, max_tokens: int):
    """crates/embed/src/stella.rs:365-378: an error, never truncation."""
    if token_count > max_tokens:
        raise InputTooLong(f"input exceeds max_tokens: got {token_count}, limit {max_tokens}")


class StellaTextModel:
    """``embed::StellaModel`` as ``core::EmbeddingModel`` (crates/core/src/lib.rs:139-163): text in,
    unit-norm fp32 vectors out. ``model`` is the id-level GPU model; a batch is tokenised on the host
    and runs as ONE ragged batch on the device (the reference fans sentences out over CPU workers)."""

    def __init__(self, model: StellaModel, tokenizer: Tokenizer, prompts: Optional[Dict[str, str]] = None):
        self.model, self.tokenizer, self.prompts = model, tokenizer, dict(prompts or {})

    @classmethod
    def load(cls, root: str, dims: Sequence[int] = (1024,), **kw) -> "StellaTextModel":
        """StellaModel::load (crates/embed/src/stella.rs:138-201): weights, tokenizer.json, dense heads and
        the optional prompt sidecar of one checkpoint directory."""
        model = StellaModel.load(root, dims, **kw)
        return cls(model, Tokenizer.from_file(os.path.join(str(root), "tokenizer.json")), load_prompts(root))

    def default_dim(self) -> int:
        return self.model.default_dim()

    def supported_dims(self) -> List[int]:
        return self.model.supported_dims()

    def max_tokens(self) -> int:
        return self.model.max_tokens()

    def _ids(self, text: str, opts: EncodeOpts) -> List[int]:
        dim = opts.dim if opts.dim is not None else self.default_dim()
        if dim not in self.supported_dims():  # checked before anything else (stella.rs:301-304)
            raise UnsupportedDim(f"unsupported dim {dim}")
        max_tokens = opts.max_tokens if opts.max_tokens is not None else self.max_tokens()
        ids = self.tokenizer.encode(apply_prompt(self.prompts, opts.prompt, text), True)
        check_token_limit(len(ids), max_tokens)
        return ids

    def encode(self, text: str, opts: EncodeOpts = EncodeOpts()) -> np.ndarray:
        return self.encode_batch([text], opts)[0]

    def encode_batch(self, texts: Sequence[str], opts: EncodeOpts = EncodeOpts()) -> np.ndarray:
        """Fails on the first text (in order) that cannot be encoded, as the reference's fail-fast
        collect does; nothing runs on the device in that case."""
        runs = [self._ids(t, opts) for t in texts]
        cu = np.zeros(len(runs) + 1, np.int32)
        cu[1:] = np.cumsum([len(r) for r in runs])
        ids = np.asarray([i for r in runs for i in r], np.uint32)
        id_opts = EncodeOpts(dim=opts.dim, max_tokens=max(opts.max_tokens or 0, self.max_tokens()))
        return self.model.encode_ids_batch(ids, cu, id_opts)
