"""Pure text -> token transformations: NFC normalisation, tokenisation, document -> shard hashing
(nmoe/data/transforms.py).  Tokenizers: any tiktoken encoding that is available offline, or the
built-in ``bytes`` tokenizer (UTF-8 bytes, vocab 257, EOS 256) which needs no vocabulary file."""
from __future__ import annotations

import hashlib
import unicodedata
from functools import lru_cache
from typing import List, Tuple

DEFAULT_TOKENIZER = "o200k_harmony"
DEFAULT_VOCAB_SIZE = 201088
DEFAULT_EOS_TOKEN_ID = 199999


def normalize_text(text: str) -> str:
  """Idempotent: NFC + strip."""
  return unicodedata.normalize("NFC", text).strip() if text else ""


class ByteTokenizer:
  name, n_vocab, eos = "bytes", 257, 256

  def encode_ordinary(self, text: str) -> List[int]:
    return list(text.encode("utf-8"))

  def decode(self, ids) -> str:
    return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


@lru_cache(maxsize=8)
def get_tokenizer(name: str):
  if name == "bytes":
    return ByteTokenizer()
  import tiktoken
  return tiktoken.get_encoding(name)


def tokenizer_info(name: str) -> Tuple[int, int]:
  """(vocab_size, eos_token_id)."""
  if name == "bytes":
    return ByteTokenizer.n_vocab, ByteTokenizer.eos
  if name == DEFAULT_TOKENIZER:
    return DEFAULT_VOCAB_SIZE, DEFAULT_EOS_TOKEN_ID
  enc = get_tokenizer(name)
  return enc.n_vocab, getattr(enc, "eot_token", enc.n_vocab - 1)


def tokenize(text: str, tokenizer_name: str = DEFAULT_TOKENIZER) -> List[int]:
  return get_tokenizer(tokenizer_name).encode_ordinary(text) if text else []


def get_shard_id(doc_id: str, num_shards: int) -> int:
  """md5(doc_id) -> shard index, stable across runs and machines."""
  return int(hashlib.md5(doc_id.encode("utf-8")).hexdigest()[:16], 16) % num_shards


def make_file_name(dataset: str, version: str, shard_idx: int, extension: str = "npy") -> str:
  return f"{dataset}-{version}-shard-{shard_idx:06d}.{extension}"
