"""Fetching arXiv's bulk source archives and reading papers out of them.

arXiv publishes its sources as monthly tar files in a requester-pays S3 bucket, listed by an XML manifest
(``src/arXiv_src_manifest.xml``: one ``<file>`` per tar with ``filename``, ``size``, ``md5sum``, ``yymm``, ``seq_num``,
``num_items``).  A bulk tar holds one member per paper, ``<yymm>/<id>.gz`` (a gzipped TeX file or a gzipped tar of the
paper's files) or ``<yymm>/<id>.pdf`` (no source).

This module is transport-agnostic: a *fetcher* turns a manifest key into bytes on disk.
  * ``S3CliFetcher``  the ``aws s3 cp --request-payer requester`` route (needs the aws CLI and credentials),
  * ``HttpFetcher``   any HTTP(S) mirror, with ``Range`` resume and retries,
  * ``FileFetcher``   a directory that already holds the tars (an NFS copy, a test fixture).
``download`` walks a selection of the manifest with a small thread pool, skips what is already complete (size and md5),
verifies checksums, and keeps going past a failed tar when asked to.  ``iter_bulk_tar`` then yields one
``{"id", "files"}`` per paper, which ``nmoe_b200.data.arxiv.main_tex`` / ``latex_to_text`` turn into text.
Reference: nmoe/data/arxiv/download.py:33-290 (manifest, S3 tars, cost estimate), nmoe/data/arxiv/sources.py:43-376.
"""
from __future__ import annotations

import gzip
import hashlib
import io
import shutil
import subprocess
import tarfile
import time
import xml.etree.ElementTree as ET
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass
from pathlib import Path
from typing import Callable, Dict, Iterator, List, Optional

BUCKET = "arxiv"
REGION = "us-east-1"
USD_PER_GB = 0.09          # S3 data transfer out, paid by the requester


@dataclass(frozen=True)
class TarEntry:
  key: str                 # e.g. src/arXiv_src_2301_004.tar
  size: int
  md5: str
  yymm: str
  seq: int
  items: int

  @property
  def name(self) -> str:
    return self.key.rsplit("/", 1)[-1]

  def sort_key(self):
    # yymm is two-digit year + month: 91..99 are the 1990s
    yy = int(self.yymm[:2]) if self.yymm[:2].isdigit() else 0
    return (1900 + yy if yy >= 91 else 2000 + yy, self.yymm[2:], self.seq)


def parse_manifest(path) -> List[TarEntry]:
  out = []
  for f in ET.parse(str(path)).getroot().iter("file"):
    get = lambda tag, default="": (f.findtext(tag) or default).strip()
    if not get("filename"):
      continue
    out.append(TarEntry(get("filename"), int(get("size", "0") or 0), get("md5sum"), get("yymm"), int(get("seq_num", "0") or 0),
                        int(get("num_items", "0") or 0)))
  return sorted(out, key=TarEntry.sort_key)


def select(entries: List[TarEntry], start: Optional[str] = None, end: Optional[str] = None,
           max_bytes: Optional[int] = None, max_files: Optional[int] = None) -> List[TarEntry]:
  """Entries whose month lies in [start, end] (``yymm`` strings, compared chronologically), cut by a byte / file budget."""
  def chrono(yymm: str):
    return TarEntry("", 0, "", yymm, 0, 0).sort_key()[:2]
  out, total = [], 0
  for e in entries:
    if start and chrono(e.yymm) < chrono(start):
      continue
    if end and chrono(e.yymm) > chrono(end):
      continue
    if max_bytes is not None and total + e.size > max_bytes:
      break
    if max_files is not None and len(out) >= max_files:
      break
    out.append(e)
    total += e.size
  return out


def estimate_cost(entries: List[TarEntry]) -> Dict[str, float]:
  gb = sum(e.size for e in entries) / 1e9
  return {"files": len(entries), "gigabytes": round(gb, 2), "papers": sum(e.items for e in entries),
          "usd_requester_pays": round(gb * USD_PER_GB, 2)}


def md5_of(path: Path, chunk: int = 1 << 22) -> str:
  h = hashlib.md5()
  with open(path, "rb") as f:
    for b in iter(lambda: f.read(chunk), b""):
      h.update(b)
  return h.hexdigest()


# ------------------------------------------------------------------ fetchers
class FetchError(RuntimeError):
  pass


class FileFetcher:
  """The tars already exist under ``root`` (by key, or flat by file name)."""

  def __init__(self, root):
    self.root = Path(root)

  def fetch(self, key: str, dest: Path) -> None:
    for cand in (self.root / key, self.root / key.rsplit("/", 1)[-1]):
      if cand.is_file():
        shutil.copyfile(cand, dest)
        return
    raise FetchError(f"{key} not found under {self.root}")


class HttpFetcher:
  """GET ``{base_url}/{key}``; a partial ``dest`` is continued with a Range request when the server allows it."""

  def __init__(self, base_url: str, retries: int = 4, backoff_s: float = 1.0, timeout_s: float = 60.0,
               headers: Optional[Dict[str, str]] = None, sleep: Callable[[float], None] = time.sleep):
    self.base, self.retries, self.backoff, self.timeout, self.headers, self.sleep = \
        base_url.rstrip("/"), retries, backoff_s, timeout_s, dict(headers or {}), sleep

  def fetch(self, key: str, dest: Path) -> None:
    import http.client
    import urllib.error
    import urllib.request
    url = f"{self.base}/{key}"
    last: Optional[Exception] = None
    for attempt in range(self.retries + 1):
      have = dest.stat().st_size if dest.exists() else 0
      req = urllib.request.Request(url, headers={**self.headers, **({"Range": f"bytes={have}-"} if have else {})})
      try:
        with urllib.request.urlopen(req, timeout=self.timeout) as r:
          resumed = have > 0 and r.status == 206
          want = r.headers.get("Content-Length")
          with open(dest, "ab" if resumed else "wb") as f:
            before = f.tell()
            shutil.copyfileobj(r, f, 1 << 20)
            got = f.tell() - before
        # a body shorter than announced reads as a clean end of stream: check the count
        if want is None or got >= int(want):
          return
        last = IOError(f"body cut after {got} of {want} bytes")
      except urllib.error.HTTPError as e:
        if e.code == 416 and have:          # nothing left to send: the file was already complete
          return
        if e.code in (403, 404):
          raise FetchError(f"{url}: HTTP {e.code}") from e
        last = e
      except (urllib.error.URLError, http.client.HTTPException, OSError, TimeoutError) as e:
        last = e      # a connection cut in mid-body leaves the bytes received so far in dest; the next attempt continues
      self.sleep(self.backoff * (2 ** attempt))
    raise FetchError(f"{url}: gave up after {self.retries + 1} attempts: {last}")


class S3CliFetcher:
  """``aws s3 cp s3://arxiv/<key> <dest> --request-payer requester``: the caller's AWS account pays for the transfer."""

  def __init__(self, profile: Optional[str] = None, bucket: str = BUCKET, region: str = REGION,
               run: Callable = subprocess.run):
    self.profile, self.bucket, self.region, self.run = profile, bucket, region, run

  def command(self, key: str, dest: Path) -> List[str]:
    cmd = ["aws", "s3", "cp", f"s3://{self.bucket}/{key}", str(dest), "--request-payer", "requester", "--region", self.region,
           "--only-show-errors"]
    return cmd + (["--profile", self.profile] if self.profile else [])

  def fetch(self, key: str, dest: Path) -> None:
    try:
      r = self.run(self.command(key, dest), capture_output=True, text=True)
    except FileNotFoundError as e:
      raise FetchError("the aws command-line client is not installed") from e
    if r.returncode != 0:
      raise FetchError(f"aws s3 cp {key}: {(r.stderr or '').strip()[:300]}")


def make_fetcher(kind: str, *, base_url: Optional[str] = None, root: Optional[str] = None, profile: Optional[str] = None):
  if kind == "s3":
    return S3CliFetcher(profile)
  if kind == "http":
    if not base_url:
      raise ValueError("--fetch http needs --base-url")
    return HttpFetcher(base_url)
  if kind == "file":
    if not root:
      raise ValueError("--fetch file needs --root")
    return FileFetcher(root)
  raise ValueError(f"unknown fetcher {kind!r} (s3 | http | file)")


# ------------------------------------------------------------------ download loop
@dataclass
class DownloadReport:
  fetched: List[str]
  skipped: List[str]
  failed: Dict[str, str]

  @property
  def ok(self) -> bool:
    return not self.failed


def _complete(path: Path, e: TarEntry, verify: bool) -> bool:
  if not path.is_file() or (e.size and path.stat().st_size != e.size):
    return False
  return not (verify and e.md5) or md5_of(path) == e.md5


def download(entries: List[TarEntry], out_dir, fetcher, *, workers: int = 4, verify: bool = True,
             keep_going: bool = False, print_fn: Callable = print) -> DownloadReport:
  """Fetch every entry into ``out_dir/<file name>``.  A file that is already complete is skipped; a fetched file whose
  size or md5 disagrees with the manifest is deleted and counted as failed (a truncated tar must not look finished)."""
  out_dir = Path(out_dir)
  out_dir.mkdir(parents=True, exist_ok=True)
  rep = DownloadReport([], [], {})

  def one(e: TarEntry):
    dest = out_dir / e.name
    if _complete(dest, e, verify):
      return e, "skipped", ""
    part = dest.with_suffix(dest.suffix + ".part")
    try:
      fetcher.fetch(e.key, part)
      if not _complete(part, e, verify):
        got = part.stat().st_size if part.exists() else 0
        part.unlink(missing_ok=True)
        return e, "failed", f"size/md5 mismatch (got {got} bytes, manifest says {e.size})"
      part.replace(dest)
      return e, "fetched", ""
    except FetchError as err:
      return e, "failed", str(err)

  with ThreadPoolExecutor(max_workers=max(1, workers)) as pool:
    for e, what, why in pool.map(one, entries):
      if what == "failed":
        rep.failed[e.name] = why
        print_fn(f"[arxiv] FAILED {e.name}: {why}")
        if not keep_going:
          break
      else:
        (rep.fetched if what == "fetched" else rep.skipped).append(e.name)
        print_fn(f"[arxiv] {what} {e.name} ({e.size / 1e6:.1f} MB, {e.items} papers)")
  return rep


# ------------------------------------------------------------------ reading a bulk tar
def _paper_files(arxiv_id: str, blob: bytes, max_member: int = 8 << 20) -> Dict[str, bytes]:
  """Files of one paper from its ``.gz`` member: a gzipped tar of the submission, or a single gzipped TeX file."""
  try:
    raw = gzip.decompress(blob)
  except OSError:
    return {}
  try:
    with tarfile.open(fileobj=io.BytesIO(raw), mode="r:") as tf:
      return {m.name: tf.extractfile(m).read() for m in tf.getmembers() if m.isfile() and m.size < max_member}
  except tarfile.TarError:
    return {f"{arxiv_id}.tex": raw}


def iter_bulk_tar(tar_path) -> Iterator[dict]:
  """One ``{"id", "files"}`` per paper that has sources (PDF-only members are skipped)."""
  with tarfile.open(str(tar_path), mode="r:*") as tf:
    for m in tf:
      if not m.isfile() or not m.name.endswith(".gz"):
        continue
      arxiv_id = m.name.rsplit("/", 1)[-1][:-3]
      files = _paper_files(arxiv_id, tf.extractfile(m).read())
      if files:
        yield {"id": arxiv_id, "files": files}


def iter_bulk_text(tar_dir, min_chars: int = 500) -> Iterator[dict]:
  """``{"id", "text"}`` for every paper of every bulk tar under ``tar_dir`` whose main TeX file converts to text."""
  from .arxiv import latex_to_text, main_tex
  for tar_path in sorted(Path(tar_dir).glob("*.tar")):
    for paper in iter_bulk_tar(tar_path):
      tex = main_tex(paper["files"])
      if tex is None:
        continue
      text = latex_to_text(tex)
      if len(text) >= min_chars:
        yield {"id": paper["id"], "text": text, "source_tar": tar_path.name}
