"""The Stack v2: from the table of file ids to a text corpus.

The dataset ships *ids*, not code: one row per file (or per repository with a ``files`` list) with the Software
Heritage blob id, the declared encoding, path, repository, language, size, star / fork counts and licence fields.  The
bytes live in the ``softwareheritage`` bucket as ``content/{blob_id}``, gzip-compressed.  Materialising is therefore

  1. select    the ``top_n`` most popular files of this worker's slice of the table
               (score = log1p(stars) + 0.5 * log1p(forks)), after dropping vendored / generated files, lock files,
               binaries and dependency directories, files outside [min_bytes, max_bytes], and at most
               ``max_files_per_repo`` per repository (its best ones);
  2. fetch     the blobs with a few threads through a *blob store* (the bucket via the aws CLI or boto3, or a local
               mirror directory), gunzip, sniff out binaries, decode with the declared encoding;
  3. write     ``part_NNNNN.jsonl.zst`` (gzip when ``zstandard`` is missing) under ``{output_root}/worker_{i:04d}/``,
               rotating by rows and bytes, plus a ``summary.json``.

Reference: nmoe/data/stack_v2_materialize.py:1-534 (same selection rule, same row fields, same output layout).
"""
from __future__ import annotations

import gzip
import heapq
import json
import math
import subprocess
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

BUCKET = "softwareheritage"

_SKIP_DIRS = frozenset({"node_modules", "vendor", "third_party", "third-party", "dist", "build", "target", "pods", "carthage", ".git",
                        "bower_components", "__pycache__"})
_SKIP_FILES = frozenset({"package-lock.json", "yarn.lock", "pnpm-lock.yaml", "cargo.lock", "go.sum", "poetry.lock", "composer.lock",
                         "gemfile.lock"})
_SKIP_EXT = frozenset({".png", ".jpg", ".jpeg", ".gif", ".bmp", ".ico", ".pdf", ".zip", ".tar", ".gz", ".bz2", ".xz", ".7z", ".mp4",
                       ".mp3", ".wav", ".class", ".jar", ".so", ".dll", ".exe", ".dylib", ".o", ".a", ".pyc", ".ttf", ".otf", ".woff",
                       ".woff2", ".bin"})


def skip_path(path: str) -> bool:
  """Dependency and build directories, lock files, binary formats: text a model should not spend tokens on."""
  parts = path.lower().replace("\\", "/").split("/")
  if any(p in _SKIP_DIRS for p in parts[:-1]):
    return True
  base = parts[-1]
  dot = base.rfind(".")
  return base in _SKIP_FILES or (dot >= 0 and base[dot:] in _SKIP_EXT) or base.endswith(".min.js")


@dataclass(frozen=True)
class FileRef:
  blob_id: str
  path: str = ""
  repo_name: str = ""
  language: str = ""
  src_encoding: str = ""
  length_bytes: int = 0
  star_events_count: int = 0
  fork_events_count: int = 0
  is_vendor: bool = False
  is_generated: bool = False
  license_type: str = ""
  detected_licenses: Tuple[str, ...] = ()
  snapshot_id: str = ""
  revision_id: str = ""
  branch_name: str = ""

  @property
  def score(self) -> float:
    return math.log1p(max(0, self.star_events_count)) + 0.5 * math.log1p(max(0, self.fork_events_count))

  @classmethod
  def from_row(cls, r: Dict[str, Any]) -> Optional["FileRef"]:
    if not r.get("blob_id"):
      return None
    def i(k):
      try:
        return int(r.get(k) or 0)
      except (TypeError, ValueError):
        return 0
    s = lambda k: "" if r.get(k) is None else str(r.get(k))
    lic = r.get("detected_licenses")
    return cls(s("blob_id"), s("path"), s("repo_name"), s("language") or s("gha_language"), s("src_encoding"), i("length_bytes"),
               i("star_events_count"), i("fork_events_count"), bool(r.get("is_vendor")), bool(r.get("is_generated")), s("license_type"),
               tuple(str(x) for x in lic) if isinstance(lic, (list, tuple)) else (), s("snapshot_id"), s("revision_id"), s("branch_name"))


# ---------------------------------------------------------------------------------------------- table
def table_files(input_root) -> List[Path]:
  """The id table's files: ``{root}/data/**/*.parquet`` (the layout a Hugging Face download leaves), else any
  ``*.parquet`` / ``*.jsonl`` under the root."""
  root = Path(input_root)
  base = root / "data" if (root / "data").is_dir() else root
  files = sorted(base.rglob("*.parquet")) or sorted(base.rglob("*.jsonl"))
  if not files:
    raise FileNotFoundError(f"no .parquet or .jsonl id tables under {base}")
  return files


def iter_table(paths: Sequence[Path]) -> Iterator[Dict[str, Any]]:
  """Rows of the id table, one per file: a repository-level row with a ``files`` list is spread over its files."""
  from .hydra_labels import iter_rows
  for p in paths:
    for row in iter_rows(Path(p), 2048):
      files = row.get("files")
      if isinstance(files, list):
        top = {k: v for k, v in row.items() if k != "files"}
        for f in files:
          if isinstance(f, dict):
            yield {**top, **f}
      else:
        yield row


def select_top(rows: Iterable[Dict[str, Any]], top_n: int, *, min_bytes: int = 256, max_bytes: int = 256_000,
               exclude_vendor: bool = True, exclude_generated: bool = True, max_files_per_repo: int = 200,
               languages: Optional[Sequence[str]] = None, stats: Optional[dict] = None) -> List[FileRef]:
  """The ``top_n`` best-scored files that pass the filters, with at most ``max_files_per_repo`` per repository -- the
  repository's *best* files, whatever order the table lists them in.  Best first; ties by blob id, so the result does
  not depend on the order of the table either.

  Memory stays near ``top_n``: every repository keeps a small heap of its best files, and when the candidates pile up
  past ``4 * top_n`` they are cut back to the best ``top_n``.  The cut is exact, because a file outside the best
  ``top_n`` can only be overtaken further: a file is evicted from its repository's heap only by a better file of the
  same repository, which takes its place above."""
  langs = {l.lower() for l in languages} if languages else None
  st = stats if stats is not None else {}
  st.update({"scanned": 0, "filtered": 0})
  per_repo: Dict[str, List[Tuple[float, str, int, FileRef]]] = {}
  in_play = set()                 # blob ids among the candidates: the same content under another path or fork counts once
  count = seq = 0

  def prune() -> None:
    nonlocal count
    keep = heapq.nlargest(top_n, (c for h in per_repo.values() for c in h), key=lambda c: (c[0], c[1]))
    per_repo.clear()
    in_play.clear()
    for c in keep:
      per_repo.setdefault(c[3].repo_name, []).append(c)
      in_play.add(c[1])
    for h in per_repo.values():
      heapq.heapify(h)
    count = len(keep)

  for r in rows:
    st["scanned"] += 1
    ref = FileRef.from_row(r)
    if (ref is None or (ref.path and skip_path(ref.path)) or (exclude_vendor and ref.is_vendor) or (exclude_generated and ref.is_generated)
        or not min_bytes <= ref.length_bytes <= max_bytes or (langs is not None and ref.language.lower() not in langs)):
      st["filtered"] += 1
      continue
    if ref.blob_id in in_play:
      st["duplicates"] = st.get("duplicates", 0) + 1
      continue
    seq += 1
    cand = (ref.score, ref.blob_id, seq, ref)      # seq: entries never compare as far as the FileRef
    h = per_repo.setdefault(ref.repo_name, [])
    if max_files_per_repo > 0 and ref.repo_name and len(h) >= max_files_per_repo:
      if (cand[0], cand[1]) > (h[0][0], h[0][1]):
        in_play.discard(heapq.heapreplace(h, cand)[1])
        in_play.add(ref.blob_id)
    else:
      heapq.heappush(h, cand)
      in_play.add(ref.blob_id)
      count += 1
      if count > 4 * max(1, top_n):
        prune()
  best = heapq.nlargest(top_n, (c for h in per_repo.values() for c in h), key=lambda c: (c[0], c[1]))
  st["selected"] = len(best)
  return [c[3] for c in best]


# ---------------------------------------------------------------------------------------------- blobs
def looks_binary(buf: bytes) -> bool:
  if not buf or b"\x00" in buf[:65536]:
    return True
  head = buf[:4096]
  return sum(1 for b in head if b >= 32 or 9 <= b <= 13) / len(head) < 0.6


def decode_text(raw: bytes, declared: str = "") -> Optional[str]:
  """Text of a blob, or None for binaries: the declared encoding first, then UTF-8, then Latin-1 (which never fails
  and is what most undeclared legacy sources are).  Two- and four-byte encodings are full of zero bytes, so for those
  (declared, or given away by a byte-order mark) the sniff looks at the decoded characters instead of the bytes."""
  enc = (declared or "").strip()
  wide = enc.lower().replace("_", "-").startswith(("utf-16", "utf-32", "ucs-2", "ucs-4")) or raw[:2] in (b"\xff\xfe", b"\xfe\xff")
  if wide:
    try:
      text = raw.decode(enc if enc.lower().replace("_", "-").startswith(("utf-", "ucs-")) else "utf-16")
    except (UnicodeDecodeError, LookupError):
      return None
    head = text[:4096]
    return text if head and sum(1 for c in head if c.isprintable() or c in "\t\n\r") / len(head) >= 0.6 else None
  if looks_binary(raw):
    return None
  for name in ([enc] if enc else []) + ["utf-8", "latin-1"]:
    try:
      return raw.decode(name)
    except (UnicodeDecodeError, LookupError):
      continue
  return None


def _gunzip(raw: bytes) -> bytes:
  return gzip.decompress(raw) if raw[:2] == b"\x1f\x8b" else raw


class DirBlobs:
  """A local mirror: ``{root}/{id}``, ``{root}/{id[:2]}/{id}``, each optionally ``.gz``."""

  def __init__(self, root):
    self.root = Path(root)

  def get(self, blob_id: str) -> Optional[bytes]:
    for cand in (self.root / blob_id, self.root / blob_id[:2] / blob_id, self.root / f"{blob_id}.gz", self.root / blob_id[:2] / f"{blob_id}.gz"):
      if cand.is_file():
        return _gunzip(cand.read_bytes())
    return None


class S3Blobs:
  """``s3://softwareheritage/content/{id}`` through boto3 when it is installed, else the aws command-line client.
  Credentials come from the environment, as both tools expect."""

  def __init__(self, bucket: str = BUCKET, run: Callable = subprocess.run, client: Any = None):
    self.bucket, self.run, self.client = bucket, run, client
    if client is None:
      try:
        import boto3  # type: ignore
        self.client = boto3.client("s3")
      except Exception:
        self.client = None

  def get(self, blob_id: str) -> Optional[bytes]:
    try:
      if self.client is not None:
        return _gunzip(self.client.get_object(Bucket=self.bucket, Key=f"content/{blob_id}")["Body"].read())
      r = self.run(["aws", "s3", "cp", f"s3://{self.bucket}/content/{blob_id}", "-", "--only-show-errors"], capture_output=True)
      return _gunzip(r.stdout) if r.returncode == 0 and r.stdout else None
    except Exception:                    # one unreadable blob must not end a run over millions
      return None


# ---------------------------------------------------------------------------------------------- output
class RotatingJsonl:
  """``part_00000.jsonl.zst``, ``part_00001...``: a new part after ``max_rows`` rows or ``max_bytes`` uncompressed
  bytes.  gzip (``.jsonl.gz``) when the zstandard package is not installed."""

  def __init__(self, out_dir, max_rows: int = 50_000, max_bytes: int = 256 << 20, compression: str = "auto"):
    self.dir, self.max_rows, self.max_bytes = Path(out_dir), max_rows, max_bytes
    self.dir.mkdir(parents=True, exist_ok=True)
    if compression == "auto":
      try:
        import zstandard  # type: ignore  # noqa: F401
        compression = "zst"
      except ImportError:
        compression = "gz"
    self.compression = compression
    self.parts: List[str] = []
    self.rows = self.bytes = self._part_rows = self._part_bytes = 0
    self._fh = self._raw = None

  def _open(self) -> None:
    path = self.dir / f"part_{len(self.parts):05d}.jsonl.{self.compression}"
    self.parts.append(path.name)
    if self.compression == "zst":
      import zstandard  # type: ignore
      self._raw = open(path, "wb")
      self._fh = zstandard.ZstdCompressor(level=3).stream_writer(self._raw)
    elif self.compression == "gz":
      self._raw, self._fh = None, gzip.open(path, "wb", compresslevel=5)
    else:
      self._raw, self._fh = None, open(path, "wb")
    self._part_rows = self._part_bytes = 0

  def write(self, obj: Dict[str, Any]) -> None:
    line = (json.dumps(obj, ensure_ascii=False) + "\n").encode("utf-8")
    if self._fh is None or self._part_rows >= self.max_rows or (self._part_rows and self._part_bytes + len(line) > self.max_bytes):
      self.close()
      self._open()
    self._fh.write(line)
    self._part_rows += 1
    self._part_bytes += len(line)
    self.rows += 1
    self.bytes += len(line)

  def close(self) -> None:
    if self._fh is not None:
      self._fh.close()
      if self._raw is not None:
        self._raw.close()
      self._fh = self._raw = None


def materialize(refs: Sequence[FileRef], blobs, writer: RotatingJsonl, *, threads: int = 16, max_bytes: int = 256_000,
                print_fn: Callable = print, log_every: int = 10_000) -> Dict[str, int]:
  """Fetch, decode and write the selected files, in selection order.  Returns counts: written, missing (no blob),
  binary (sniffed out or undecodable), oversize (the table's size field was wrong)."""
  st = {"written": 0, "missing": 0, "binary": 0, "oversize": 0}
  t0 = time.time()
  with ThreadPoolExecutor(max_workers=max(1, threads)) as pool:
    for i, (ref, raw) in enumerate(zip(refs, pool.map(lambda r: blobs.get(r.blob_id), refs))):
      if raw is None:
        st["missing"] += 1
      elif len(raw) > max_bytes:
        st["oversize"] += 1
      else:
        text = decode_text(raw, ref.src_encoding)
        if text is None:
          st["binary"] += 1
        else:
          meta = {k: v for k, v in asdict(ref).items() if k not in ("blob_id", "src_encoding")}
          meta["detected_licenses"] = list(ref.detected_licenses)
          writer.write({"id": ref.blob_id, "text": text, **meta, "score": round(ref.score, 4)})
          st["written"] += 1
      if log_every and (i + 1) % log_every == 0:
        print_fn(f"[stack_v2] {i + 1:,}/{len(refs):,} fetched, {st['written']:,} written, {(i + 1) / max(1e-9, time.time() - t0):.0f} files/s")
  writer.close()
  return st


def run(input_root, output_root, *, worker_index: int, num_workers: int, top_n: int, blobs, min_bytes: int = 256,
        max_bytes: int = 256_000, exclude_vendor: bool = True, exclude_generated: bool = True, max_files_per_repo: int = 200,
        languages: Optional[Sequence[str]] = None, threads: int = 16, print_fn: Callable = print) -> Dict[str, Any]:
  """One worker's share: table files ``i % num_workers == worker_index`` -> selection -> ``worker_{i:04d}/part_*``."""
  if not 0 <= worker_index < num_workers:
    raise ValueError(f"worker index {worker_index} outside [0, {num_workers})")
  mine = [p for i, p in enumerate(table_files(input_root)) if i % num_workers == worker_index]
  sel: Dict[str, int] = {}
  refs = select_top(iter_table(mine), top_n, min_bytes=min_bytes, max_bytes=max_bytes, exclude_vendor=exclude_vendor,
                    exclude_generated=exclude_generated, max_files_per_repo=max_files_per_repo, languages=languages, stats=sel)
  print_fn(f"[stack_v2] worker {worker_index}/{num_workers}: {len(mine)} table file(s), scanned {sel['scanned']:,}, selected {len(refs):,}")
  out = Path(output_root) / f"worker_{worker_index:04d}"
  w = RotatingJsonl(out)
  st = materialize(refs, blobs, w, threads=threads, max_bytes=max_bytes, print_fn=print_fn)
  summary = {"worker_index": worker_index, "num_workers": num_workers, "table_files": [p.name for p in mine], **sel, **st,
             "parts": w.parts, "uncompressed_bytes": w.bytes}
  (out / "summary.json").write_text(json.dumps(summary, indent=1))
  return summary
