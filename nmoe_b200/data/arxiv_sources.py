"""arXiv as document sources for shard building: LaTeX from the bulk tars, ar5iv HTML, or both formats of a paper.

  ``ArxivTarSource``     monthly bulk tars (see ``arxiv_download``) -> one ``arxiv:{id}:latex`` document per paper with
                         sources: main TeX file found, ``\\input`` / ``\\include`` inlined, LaTeX -> text.
  ``Ar5ivSource``        the ar5iv HTML5 + MathML conversions, laid out ``{tier}/{yymm}/{id}.html`` under the quality
                         tiers ``no_problem`` / ``warning`` / ``error`` -> one ``arxiv:{id}:html`` document per page,
                         math kept as TeX.
  ``ArxivPairedSource``  LaTeX documents, each followed by the HTML rendering of the same paper when there is one (both
                         marked ``has_paired_format``): the two texts say the same thing in two notations.

All three take ``worker_index`` / ``num_workers`` and split *files* (tars, pages) between workers, so indexed jobs
never open each other's inputs; ``stats`` counts what was read, kept and dropped.  ``create_source`` knows them as
``arxiv_tars``, ``ar5iv`` and ``arxiv_paired``.  Reference: nmoe/data/arxiv/sources.py:43-714.
"""
from __future__ import annotations

import re
from pathlib import Path
from typing import Dict, Iterator, List, Optional, Sequence

from .sources import DataSource, Document

TIERS = ("no_problem", "warning", "error")
MAX_TEXT_CHARS = 2_000_000          # a "paper" longer than this is a conversion accident (a thesis dump, a data file)
_VERSION = re.compile(r"v\d+$")


def paper_id_of(path: Path) -> str:
  """``2301.01234v2.html`` -> ``2301.01234``; old-style ``hep-th9901001.html`` stays as it is."""
  return _VERSION.sub("", path.stem)


class ArxivTarSource(DataSource):
  def __init__(self, tar_dir, *, worker_index: int = 0, num_workers: int = 1, max_docs: Optional[int] = None, min_chars: int = 500):
    self.dir, self.idx, self.n, self.max_docs, self.min_chars = Path(tar_dir), worker_index, max(1, num_workers), max_docs, min_chars
    self.name = "arxiv_latex"
    self.stats = {"tars": 0, "papers": 0, "kept": 0, "no_main_tex": 0, "too_short": 0, "too_long": 0, "bad_tars": 0}

  def tars(self) -> List[Path]:
    return [p for i, p in enumerate(sorted(self.dir.glob("*.tar"))) if i % self.n == self.idx]

  def shard(self, index: int, count: int) -> "ArxivTarSource":
    # compose with the split this source already has: worker (i of n) of worker (idx of self.n)
    return ArxivTarSource(self.dir, worker_index=self.idx + self.n * index, num_workers=self.n * count, max_docs=self.max_docs,
                          min_chars=self.min_chars)

  def __iter__(self) -> Iterator[Document]:
    import tarfile
    from .arxiv import latex_to_text, main_tex
    from .arxiv_download import iter_bulk_tar
    kept = 0
    for tar in self.tars():
      self.stats["tars"] += 1
      try:
        for paper in iter_bulk_tar(tar):
          self.stats["papers"] += 1
          tex = main_tex(paper["files"])
          if tex is None:
            self.stats["no_main_tex"] += 1
            continue
          text = latex_to_text(tex)
          if len(text) < self.min_chars or len(text) > MAX_TEXT_CHARS:
            self.stats["too_short" if len(text) < self.min_chars else "too_long"] += 1
            continue
          self.stats["kept"] += 1
          kept += 1
          yield Document(f"arxiv:{paper['id']}:latex", text, {"arxiv_id": paper["id"], "format": "latex", "source_tar": tar.name})
          if self.max_docs and kept >= self.max_docs:
            return
      except (tarfile.TarError, OSError, EOFError):
        self.stats["bad_tars"] += 1        # a truncated download: the papers read so far stand, the next tar goes on


def html_document(path: Path, min_chars: int = 100) -> Optional[Document]:
  """One ar5iv page as a document, or None when it is unreadable, empty or absurdly long."""
  from .arxiv_html import extract_html_metadata, html_to_text
  try:
    html = path.read_text(encoding="utf-8", errors="ignore")
    text = html_to_text(html, preserve_math=True)
  except Exception:                        # a page the converter cannot digest is dropped, not fatal
    return None
  if len(text.strip()) < min_chars or len(text) > MAX_TEXT_CHARS:
    return None
  try:
    m = extract_html_metadata(html)
  except Exception:
    m = None
  pid = paper_id_of(path)
  meta = {"arxiv_id": pid, "format": "html", "tier": path.parts[-3] if len(path.parts) >= 3 else None}
  if m is not None:
    meta.update({"title": m.title, "authors": m.authors, "abstract": m.abstract, "categories": m.categories})
  return Document(f"arxiv:{pid}:html", text, meta)


def html_pages(html_dir: Path, tiers: Sequence[str]) -> List[Path]:
  """Pages of the chosen tiers, best tier first, each tier in path order."""
  out: List[Path] = []
  for t in tiers:
    if t not in TIERS:
      raise ValueError(f"unknown ar5iv quality tier {t!r}; one of {TIERS}")
    d = Path(html_dir) / t
    if d.is_dir():
      out += sorted(d.rglob("*.html"))
  return out


class Ar5ivSource(DataSource):
  def __init__(self, html_dir, *, quality_levels: Sequence[str] = ("no_problem", "warning"), worker_index: int = 0,
               num_workers: int = 1, max_docs: Optional[int] = None):
    self.dir, self.tiers, self.idx, self.n, self.max_docs = Path(html_dir), tuple(quality_levels), worker_index, max(1, num_workers), max_docs
    self.name = "arxiv_ar5iv_html"
    self.stats = {"pages": 0, "kept": 0, "dropped": 0}

  def shard(self, index: int, count: int) -> "Ar5ivSource":
    return Ar5ivSource(self.dir, quality_levels=self.tiers, worker_index=self.idx + self.n * index, num_workers=self.n * count,
                       max_docs=self.max_docs)

  def estimate_size(self) -> Optional[int]:
    return len(html_pages(self.dir, self.tiers)) // self.n

  def __iter__(self) -> Iterator[Document]:
    for i, page in enumerate(html_pages(self.dir, self.tiers)):
      if i % self.n != self.idx:
        continue
      self.stats["pages"] += 1
      doc = html_document(page)
      if doc is None:
        self.stats["dropped"] += 1
        continue
      self.stats["kept"] += 1
      yield doc
      if self.max_docs and self.stats["kept"] >= self.max_docs:
        return


class ArxivPairedSource(DataSource):
  def __init__(self, tar_dir, html_dir, *, emit_both_formats: bool = True, quality_levels: Sequence[str] = ("no_problem", "warning"),
               worker_index: int = 0, num_workers: int = 1, max_docs: Optional[int] = None):
    self.tar_dir, self.html_dir, self.both, self.tiers = Path(tar_dir), Path(html_dir), emit_both_formats, tuple(quality_levels)
    self.idx, self.n, self.max_docs = worker_index, max(1, num_workers), max_docs
    self.name = "arxiv_paired"
    self.stats = {"latex_only": 0, "both_formats": 0, "total_docs": 0}

  def shard(self, index: int, count: int) -> "ArxivPairedSource":
    return ArxivPairedSource(self.tar_dir, self.html_dir, emit_both_formats=self.both, quality_levels=self.tiers,
                             worker_index=self.idx + self.n * index, num_workers=self.n * count, max_docs=self.max_docs)

  def html_index(self) -> Dict[str, Path]:
    """Paper id -> its page; when several tiers hold the paper the best tier wins (``html_pages`` lists it first)."""
    index: Dict[str, Path] = {}
    for p in html_pages(self.html_dir, self.tiers):
      index.setdefault(paper_id_of(p), p)
    return index

  def __iter__(self) -> Iterator[Document]:
    pages = self.html_index() if self.both else {}
    seen = set()
    n = 0
    for doc in ArxivTarSource(self.tar_dir, worker_index=self.idx, num_workers=self.n):
      pid = doc.metadata["arxiv_id"]
      if pid in seen:                      # a paper replaced within the month appears in two tars: first copy stands
        continue
      seen.add(pid)
      twin = html_document(pages[pid]) if pid in pages else None
      if twin is not None:
        doc.metadata["has_paired_format"] = twin.metadata["has_paired_format"] = True
        self.stats["both_formats"] += 1
      else:
        self.stats["latex_only"] += 1
      for d in (doc, twin):
        if d is not None:
          yield d
          n += 1
          self.stats["total_docs"] = n
          if self.max_docs and n >= self.max_docs:
            return
