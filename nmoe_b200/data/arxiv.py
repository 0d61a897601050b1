"""arXiv sources and Stack-v2 blobs -> JSONL documents for the shard builder.

``arxiv-prep`` walks a directory of downloaded arXiv source archives (``<id>.tar.gz`` / ``<id>.gz`` /
plain ``.tex``), picks the main TeX file of each paper (the one with ``\\documentclass``; ``\\input`` /
``\\include`` are inlined), strips markup with ``latex_to_text`` and writes ``{"id", "text"}`` rows.
``stack-v2-materialize`` joins a Stack-v2 id table (JSONL rows with ``blob_id``, ``src_encoding``,
``language``, ``path``) with blob files that are already on disk (``<root>/<blob_id>`` or
``<root>/<blob_id[:2]>/<blob_id>``, optionally gzip-compressed) and writes the decoded file contents.

Fetching the archives / blobs themselves needs network access and S3 credentials (requester-pays
buckets) and is left to ``arxiv-download`` / an external sync; everything here works offline.

Reference counterparts: nmoe/data/arxiv/* and nmoe/data/stack_v2_materialize.py.
"""
from __future__ import annotations

import gzip
import io
import json
import re
import tarfile
from pathlib import Path
from typing import Dict, Iterator, Optional, Tuple

_COMMENT = re.compile(r"(?<!\\)%.*")
_ENV_DROP = re.compile(r"\\begin\{(figure|table|tikzpicture|thebibliography|lstlisting|verbatim)\*?\}.*?\\end\{\1\*?\}", re.S)
_MATH_ENV = re.compile(r"\\begin\{(equation|align|gather|multline|eqnarray|displaymath)\*?\}(.*?)\\end\{\1\*?\}", re.S)
_SECTION = re.compile(r"\\(part|chapter|section|subsection|subsubsection|paragraph)\*?\{([^{}]*)\}")
_KEEP_ARG = re.compile(r"\\(textbf|textit|emph|texttt|textrm|textsc|underline|mbox|text|title|author|caption)\{([^{}]*)\}")
_DROP_CMD_ARG = re.compile(r"\\(label|ref|eqref|cite[tp]?|citep|citet|bibliography|bibliographystyle|usepackage|documentclass|"
                           r"input|include|includegraphics|vspace|hspace|pagestyle|thispagestyle|newcommand|renewcommand|def)"
                           r"(\[[^\]]*\])*(\{[^{}]*\})*")
_CMD = re.compile(r"\\[a-zA-Z@]+\*?(\[[^\]]*\])?")
_INPUT = re.compile(r"\\(?:input|include)\{([^{}]+)\}")


def latex_to_text(src: str) -> str:
  """Readable text from LaTeX: comments, floats and the bibliography go away, section titles become
  lines of their own, inline / display math is kept verbatim between dollar signs, other commands are
  dropped while the text of the common formatting commands is kept."""
  s = _COMMENT.sub("", src)
  m = re.search(r"\\begin\{document\}", s)
  if m:
    s = s[m.end():]
  s = s.split("\\end{document}")[0]
  s = _ENV_DROP.sub(" ", s)
  s = _MATH_ENV.sub(lambda m: " $$" + " ".join(m.group(2).split()) + "$$ ", s)
  s = re.sub(r"\\begin\{abstract\}", "\nAbstract\n", s)
  s = _SECTION.sub(lambda m: "\n\n" + m.group(2).strip() + "\n", s)
  for _ in range(3):                                   # nested formatting commands
    s = _KEEP_ARG.sub(lambda m: m.group(2), s)
  s = _DROP_CMD_ARG.sub(" ", s)
  s = re.sub(r"\\(begin|end)\{[^{}]*\}", " ", s)
  s = s.replace("\\\\", "\n").replace("~", " ").replace("\\&", "&").replace("\\%", "%").replace("\\_", "_").replace("\\$", "$")
  # protect math before stripping the remaining commands
  parts = re.split(r"(\$\$.*?\$\$|\$[^$]*\$)", s, flags=re.S)
  for i in range(0, len(parts), 2):
    parts[i] = _CMD.sub(" ", parts[i]).replace("{", "").replace("}", "")
  s = "".join(parts)
  s = re.sub(r"[ \t]+", " ", s)
  s = re.sub(r" *\n *", "\n", s)
  return re.sub(r"\n{3,}", "\n\n", s).strip()


def _read_member(files: Dict[str, bytes], name: str) -> Optional[str]:
  for cand in (name, name + ".tex"):
    for key in (cand, "./" + cand):
      if key in files:
        return files[key].decode("utf-8", errors="replace")
  return None


def _inline_inputs(text: str, files: Dict[str, bytes], depth: int = 0) -> str:
  if depth > 4:
    return text

  def sub(m):
    inner = _read_member(files, m.group(1).strip())
    return _inline_inputs(inner, files, depth + 1) if inner is not None else " "

  return _INPUT.sub(sub, text)


def main_tex(files: Dict[str, bytes]) -> Optional[str]:
  """The paper's main TeX source with its inputs inlined; None when there is no ``\\documentclass``."""
  best: Tuple[int, Optional[str]] = (-1, None)
  for name, data in files.items():
    if not name.lower().endswith(".tex"):
      continue
    t = data.decode("utf-8", errors="replace")
    if "\\documentclass" in t and len(t) > best[0]:
      best = (len(t), t)
  return _inline_inputs(best[1], files) if best[1] is not None else None


def read_archive(path: Path) -> Dict[str, bytes]:
  """name -> bytes for a .tar.gz / .tar / .gz (single file) / .tex source."""
  raw = path.read_bytes()
  if path.suffix == ".tex":
    return {path.name: raw}
  try:
    with tarfile.open(fileobj=io.BytesIO(raw), mode="r:*") as tf:
      return {m.name: tf.extractfile(m).read() for m in tf.getmembers() if m.isfile() and m.size < (8 << 20)}
  except tarfile.TarError:
    pass
  try:
    return {path.stem + ".tex": gzip.decompress(raw)}
  except OSError:
    return {}


def iter_arxiv(directory: str, min_chars: int = 500) -> Iterator[dict]:
  for p in sorted(Path(directory).rglob("*")):
    if not p.is_file() or p.suffix not in (".gz", ".tar", ".tgz", ".tex"):
      continue
    tex = main_tex(read_archive(p))
    if tex is None:
      continue
    text = latex_to_text(tex)
    if len(text) >= min_chars:
      yield {"id": p.name.split(".tar")[0].removesuffix(".gz").removesuffix(".tex"), "text": text}


def find_blob(root: Path, blob_id: str) -> Optional[Path]:
  for cand in (root / blob_id, root / blob_id[:2] / blob_id, root / f"{blob_id}.gz", root / blob_id[:2] / f"{blob_id}.gz"):
    if cand.exists():
      return cand
  return None


def iter_stack_v2(table_jsonl: str, blob_root: str, languages: Optional[set] = None, max_bytes: int = 1 << 20) -> Iterator[dict]:
  root = Path(blob_root)
  with open(table_jsonl, "r", encoding="utf-8") as f:
    for line in f:
      if not line.strip():
        continue
      row = json.loads(line)
      if languages and row.get("language") not in languages:
        continue
      p = find_blob(root, row["blob_id"])
      if p is None:
        continue
      raw = p.read_bytes()
      if p.suffix == ".gz":
        raw = gzip.decompress(raw)
      if len(raw) > max_bytes:
        continue
      try:
        text = raw.decode(row.get("src_encoding") or "utf-8")
      except (UnicodeDecodeError, LookupError):
        continue
      yield {"id": row["blob_id"], "text": text, "language": row.get("language"), "path": row.get("path")}


def write_jsonl(rows: Iterator[dict], out_path: str) -> int:
  n = 0
  with open(out_path, "w", encoding="utf-8") as f:
    for r in rows:
      f.write(json.dumps(r, ensure_ascii=False) + "\n")
      n += 1
  return n
