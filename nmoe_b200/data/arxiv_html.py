"""ar5iv / LaTeXML HTML -> plain text with the mathematics kept as LaTeX, plus metadata from the page and from
arXiv API (Atom) responses.  Everything works on local files or strings; only ``MetadataClient.fetch`` touches the
network.  Reference counterparts: nmoe/data/arxiv/html.py (html_to_text, mathml_to_latex, extract_html_metadata) and
nmoe/data/arxiv/metadata.py (ArxivMetadata, the API client).

The HTML is parsed with the standard library into a small element tree (no lxml on this image), then walked:

* the document title (``h1.ltx_title_document``), the abstract (``div.ltx_abstract``) and every ``section`` of
  ``article.ltx_document`` are emitted in order, headings on lines of their own;
* ``<math>`` elements become ``$...$`` (``display="block"``: ``$$...$$``): the ``alttext`` attribute when LaTeXML left
  the original TeX there, otherwise a structural MathML -> LaTeX conversion (fractions, scripts, roots, under/over,
  fenced rows, tables -> matrix rows, Greek letters and operators from a code-point table);
* navigation, bibliography, footnote marks, scripts and styles are dropped.
"""
from __future__ import annotations

import json
import re
import time
import xml.etree.ElementTree as ET
from dataclasses import asdict, dataclass, field
from html.parser import HTMLParser
from typing import Dict, Iterable, Iterator, List, Optional

# ------------------------------------------------------------------------------------------------ a light DOM
_VOID = {"area", "base", "br", "col", "embed", "hr", "img", "input", "link", "meta", "source", "track", "wbr"}


class Node:
  __slots__ = ("tag", "attrs", "children", "parent")

  def __init__(self, tag: str, attrs: Dict[str, str], parent: Optional["Node"]):
    self.tag, self.attrs, self.children, self.parent = tag, attrs, [], parent

  def classes(self) -> List[str]:
    return (self.attrs.get("class") or "").split()

  def iter(self) -> Iterator["Node"]:
    yield self
    for c in self.children:
      if isinstance(c, Node):
        yield from c.iter()

  def find(self, tag: str, cls: Optional[str] = None) -> Optional["Node"]:
    for n in self.iter():
      if n.tag == tag and (cls is None or cls in n.classes()):
        return n
    return None

  def find_all(self, tag: str, cls: Optional[str] = None) -> List["Node"]:
    return [n for n in self.iter() if n.tag == tag and (cls is None or cls in n.classes())]


class _Builder(HTMLParser):
  def __init__(self):
    super().__init__(convert_charrefs=True)
    self.root = Node("#root", {}, None)
    self.cur = self.root

  def handle_starttag(self, tag, attrs):
    n = Node(tag, {k: (v or "") for k, v in attrs}, self.cur)
    self.cur.children.append(n)
    if tag not in _VOID:
      self.cur = n

  def handle_startendtag(self, tag, attrs):
    self.cur.children.append(Node(tag, {k: (v or "") for k, v in attrs}, self.cur))

  def handle_endtag(self, tag):
    n = self.cur
    while n is not None and n.tag != tag:
      n = n.parent
    if n is not None and n.parent is not None:
      self.cur = n.parent

  def handle_data(self, data):
    self.cur.children.append(data)


def parse_html(html: str) -> Node:
  b = _Builder()
  b.feed(html)
  b.close()
  return b.root


# ------------------------------------------------------------------------------------------------ MathML -> LaTeX
_SYMBOLS = {
  "α": r"\alpha", "β": r"\beta", "γ": r"\gamma", "δ": r"\delta", "ε": r"\epsilon", "ϵ": r"\epsilon", "ζ": r"\zeta",
  "η": r"\eta", "θ": r"\theta", "ι": r"\iota", "κ": r"\kappa", "λ": r"\lambda", "μ": r"\mu", "ν": r"\nu", "ξ": r"\xi",
  "π": r"\pi", "ρ": r"\rho", "σ": r"\sigma", "τ": r"\tau", "υ": r"\upsilon", "φ": r"\phi", "ϕ": r"\phi", "χ": r"\chi",
  "ψ": r"\psi", "ω": r"\omega", "Γ": r"\Gamma", "Δ": r"\Delta", "Θ": r"\Theta", "Λ": r"\Lambda", "Ξ": r"\Xi",
  "Π": r"\Pi", "Σ": r"\Sigma", "Φ": r"\Phi", "Ψ": r"\Psi", "Ω": r"\Omega",
  "∑": r"\sum", "∏": r"\prod", "∫": r"\int", "∬": r"\iint", "∮": r"\oint", "∞": r"\infty", "∂": r"\partial",
  "∇": r"\nabla", "×": r"\times", "÷": r"\div", "±": r"\pm", "∓": r"\mp", "≤": r"\leq", "≥": r"\geq", "≠": r"\neq",
  "≈": r"\approx", "≡": r"\equiv", "∝": r"\propto", "∼": r"\sim", "≪": r"\ll", "≫": r"\gg", "∈": r"\in",
  "∉": r"\notin", "⊂": r"\subset", "⊃": r"\supset", "⊆": r"\subseteq", "⊇": r"\supseteq", "∪": r"\cup", "∩": r"\cap",
  "∅": r"\emptyset", "∀": r"\forall", "∃": r"\exists", "¬": r"\neg", "∧": r"\land", "∨": r"\lor", "⇒": r"\Rightarrow",
  "⇐": r"\Leftarrow", "⇔": r"\Leftrightarrow", "→": r"\rightarrow", "←": r"\leftarrow", "↔": r"\leftrightarrow",
  "↦": r"\mapsto", "⋅": r"\cdot", "·": r"\cdot", "…": r"\ldots", "⋯": r"\cdots", "⋮": r"\vdots", "⋱": r"\ddots",
  "⟨": r"\langle", "⟩": r"\rangle", "⌊": r"\lfloor", "⌋": r"\rfloor", "⌈": r"\lceil", "⌉": r"\rceil", "∘": r"\circ",
  "⊗": r"\otimes", "⊕": r"\oplus", "†": r"\dagger", "ℝ": r"\mathbb{R}", "ℂ": r"\mathbb{C}", "ℕ": r"\mathbb{N}",
  "ℤ": r"\mathbb{Z}", "ℚ": r"\mathbb{Q}", "ℓ": r"\ell", "ℏ": r"\hbar", "′": "'", "−": "-", "∗": "*",
  "⁢": "", "⁡": "", "⁣": "", "​": "",          # invisible times / function application / separators
}
_ACCENTS = {"^": r"\hat", "ˆ": r"\hat", "~": r"\tilde", "˜": r"\tilde", "¯": r"\bar", "‾": r"\bar", "→": r"\vec",
            "˙": r"\dot", "¨": r"\ddot", "ˇ": r"\check"}


def _sym(text: str) -> str:
  return "".join(_SYMBOLS.get(ch, ch) for ch in text)


def _text_of(n) -> str:
  if isinstance(n, str):
    return n
  return "".join(_text_of(c) for c in n.children)


def _group(s: str) -> str:
  s = s.strip()
  return s if len(s) == 1 or re.fullmatch(r"\\[A-Za-z]+|[0-9.]+", s) else "{" + s + "}"


def mathml_to_latex(n) -> str:
  """Structural conversion of a MathML (presentation) subtree."""
  if isinstance(n, str):
    return _sym(n.strip())
  t = n.tag.split(":")[-1]
  kids = [c for c in n.children if isinstance(c, Node)]
  conv = [mathml_to_latex(c) for c in kids]
  if t in ("mi", "mn", "mo", "mtext", "ms"):
    s = _sym(_text_of(n).strip())
    if t == "mtext":
      return r"\text{" + s + "}" if s else ""
    if t == "mi" and n.attrs.get("mathvariant") == "bold":
      return r"\mathbf{" + s + "}"
    if t == "mi" and len(s) > 1 and s.isalpha():
      return "\\" + s if s in ("sin", "cos", "tan", "log", "ln", "exp", "max", "min", "lim", "sup", "inf", "det", "arg") \
          else r"\mathrm{" + s + "}"
    if t == "mo" and s.startswith("\\") and s[1:].isalpha():
      return s + " "
    return s
  if t in ("math", "mrow", "mstyle", "mpadded", "mphantom", "semantics", "menclose"):
    if t == "semantics" and kids:
      return conv[0]                                  # presentation child first, annotations ignored
    return "".join(conv)
  if t in ("annotation", "annotation-xml", "none", "mprescripts"):
    return ""
  if t == "mfrac" and len(conv) == 2:
    return r"\frac{" + conv[0] + "}{" + conv[1] + "}"
  if t == "msqrt":
    return r"\sqrt{" + "".join(conv) + "}"
  if t == "mroot" and len(conv) == 2:
    return r"\sqrt[" + conv[1] + "]{" + conv[0] + "}"
  if t == "msup" and len(conv) == 2:
    return _group(conv[0]) + "^" + _group(conv[1])
  if t == "msub" and len(conv) == 2:
    return _group(conv[0]) + "_" + _group(conv[1])
  if t == "msubsup" and len(conv) == 3:
    return _group(conv[0]) + "_" + _group(conv[1]) + "^" + _group(conv[2])
  if t == "mover" and len(conv) == 2:
    acc = _text_of(kids[1]).strip()
    if acc in _ACCENTS:
      return _ACCENTS[acc] + "{" + conv[0] + "}"
    return r"\overset{" + conv[1] + "}{" + conv[0] + "}"
  if t == "munder" and len(conv) == 2:
    return (conv[0].strip() + "_" + _group(conv[1])) if conv[0].strip() in (r"\sum", r"\prod", r"\lim", r"\max", r"\min", r"\int") \
        else r"\underset{" + conv[1] + "}{" + conv[0] + "}"
  if t == "munderover" and len(conv) == 3:
    return conv[0].strip() + "_" + _group(conv[1]) + "^" + _group(conv[2])
  if t == "mfenced":
    op, cl = n.attrs.get("open", "("), n.attrs.get("close", ")")
    return r"\left" + _sym(op or ".") + ",".join(conv) + r"\right" + _sym(cl or ".")
  if t == "mtable":
    rows = [mathml_to_latex(r) for r in kids]
    return r"\begin{matrix}" + r" \\ ".join(rows) + r"\end{matrix}"
  if t in ("mtr", "mlabeledtr"):
    return " & ".join(conv)
  if t == "mtd":
    return "".join(conv)
  if t == "mspace":
    return " "
  return "".join(conv)


def math_to_tex(n: Node, prefer_alttext: bool = True) -> str:
  alt = (n.attrs.get("alttext") or "").strip()
  body = alt if (prefer_alttext and alt) else mathml_to_latex(n)
  body = " ".join(body.split())
  if not body:
    return ""
  return f"$${body}$$" if n.attrs.get("display") == "block" else f"${body}$"


# ------------------------------------------------------------------------------------------------ HTML -> text
_DROP_TAGS = {"script", "style", "nav", "header", "footer", "noscript", "svg", "figure", "button"}
_DROP_CLASSES = {"ltx_bibliography", "ltx_note_mark", "ltx_tag_note", "ltx_role_footnote", "ltx_page_footer",
                 "ltx_page_header", "ltx_TOC", "ltx_dates", "ltx_authors", "ltx_pagination", "ar5iv-footer"}
_BLOCK_TAGS = {"p", "div", "section", "li", "tr", "h1", "h2", "h3", "h4", "h5", "h6", "blockquote", "br", "table", "ul", "ol", "dd", "dt"}
_HEADINGS = {"h1", "h2", "h3", "h4", "h5", "h6"}


def _emit(n, out: List[str], preserve_math: bool) -> None:
  if isinstance(n, str):
    out.append(n)
    return
  if n.tag in _DROP_TAGS or (set(n.classes()) & _DROP_CLASSES):
    return
  if n.tag == "math":
    out.append(" " + (math_to_tex(n) if preserve_math else _text_of(n)) + " ")
    return
  if n.tag == "cite":                       # citation marks add nothing to the text
    return
  block = n.tag in _BLOCK_TAGS
  if block:
    out.append("\n\n" if n.tag in _HEADINGS or n.tag in ("p", "section", "li") else "\n")
  for c in n.children:
    _emit(c, out, preserve_math)
  if block:
    out.append("\n\n" if n.tag in _HEADINGS else "\n")


def _normalise(text: str) -> str:
  text = text.replace("\xa0", " ")
  text = re.sub(r"[ \t]+", " ", text)
  text = re.sub(r"\$ ([.,;:!?)\]])", r"$\1", text)        # the padding around a formula must not detach punctuation
  text = re.sub(r"([(\[]) \$", r"\1$", text)
  text = re.sub(r" *\n *", "\n", text)
  text = re.sub(r"\n{3,}", "\n\n", text)
  return text.strip()


def element_text(n: Node, preserve_math: bool = True) -> str:
  out: List[str] = []
  _emit(n, out, preserve_math)
  return _normalise("".join(out))


def html_to_text(html: str, *, preserve_math: bool = True, include_abstract: bool = True, include_title: bool = True) -> str:
  root = parse_html(html)
  parts: List[str] = []
  article = root.find("article", "ltx_document") or root.find("article")
  scope = article or root
  if include_title:
    t = scope.find("h1", "ltx_title_document") or root.find("h1")
    if t is not None:
      parts.append(element_text(t, preserve_math))
  abstract = scope.find("div", "ltx_abstract")
  if include_abstract and abstract is not None:
    parts.append(re.sub(r"^Abstract\.?\s*", "", element_text(abstract, preserve_math)))
  if article is not None:
    top = [s for s in article.find_all("section") if not any(p.tag == "section" for p in _ancestors(s, article))]
    for s in top:
      if set(s.classes()) & _DROP_CLASSES:
        continue
      txt = element_text(s, preserve_math)
      if txt:
        parts.append(txt)
  if len(parts) <= (1 if include_title else 0):
    body = root.find("body") or root
    skip = {id(abstract)} if (abstract is not None and not include_abstract) else set()
    out: List[str] = []
    for c in body.children:
      if not (isinstance(c, Node) and id(c) in skip):
        _emit(c, out, preserve_math)
    parts = [_normalise("".join(out))]
  return _normalise("\n\n".join(p for p in parts if p))


def _ancestors(n: Node, stop: Node) -> Iterator[Node]:
  p = n.parent
  while p is not None and p is not stop:
    yield p
    p = p.parent


# ------------------------------------------------------------------------------------------------ metadata
@dataclass
class PaperMetadata:
  arxiv_id: Optional[str] = None
  title: Optional[str] = None
  authors: List[str] = field(default_factory=list)
  abstract: Optional[str] = None
  categories: List[str] = field(default_factory=list)
  primary_category: Optional[str] = None
  submitted: Optional[str] = None          # ISO 8601
  updated: Optional[str] = None
  doi: Optional[str] = None
  journal_ref: Optional[str] = None
  comment: Optional[str] = None
  license: Optional[str] = None

  def to_json(self) -> str:
    return json.dumps(asdict(self), ensure_ascii=False)


_ID_RE = re.compile(r"(\d{4}\.\d{4,5}|[a-z\-]+(?:\.[A-Z]{2})?/\d{7})(v\d+)?")


def extract_html_metadata(html: str) -> PaperMetadata:
  """Title, authors, abstract and arXiv id as the ar5iv page states them."""
  root = parse_html(html)
  m = PaperMetadata()
  t = root.find("h1", "ltx_title_document")
  if t is not None:
    m.title = element_text(t, preserve_math=True)
  m.authors = [a for a in (element_text(p, False).split("\n")[0].strip(" ,") for p in root.find_all("span", "ltx_personname")) if a]
  ab = root.find("div", "ltx_abstract")
  if ab is not None:
    m.abstract = re.sub(r"^Abstract\.?\s*", "", element_text(ab, preserve_math=True))
  for n in root.iter():
    if n.tag in ("meta", "link", "a"):
      for key in ("content", "href"):
        hit = _ID_RE.search(n.attrs.get(key, "")) if "arxiv" in n.attrs.get(key, "").lower() else None
        if hit:
          m.arxiv_id = hit.group(1)
          return m
  return m


_ATOM = {"a": "http://www.w3.org/2005/Atom", "x": "http://arxiv.org/schemas/atom"}


def parse_atom_feed(xml_text: str) -> Dict[str, PaperMetadata]:
  """arXiv API response (``http://export.arxiv.org/api/query?id_list=...``) -> {arxiv id without version: metadata}."""
  out: Dict[str, PaperMetadata] = {}
  feed = ET.fromstring(xml_text)
  for e in feed.findall("a:entry", _ATOM):
    raw = (e.findtext("a:id", default="", namespaces=_ATOM) or "").rsplit("/abs/", 1)[-1]
    hit = _ID_RE.search(raw)
    if not hit:
      continue
    pm = PaperMetadata(arxiv_id=hit.group(1))
    squeeze = lambda s: " ".join(s.split()) if s else None
    pm.title = squeeze(e.findtext("a:title", namespaces=_ATOM))
    pm.abstract = squeeze(e.findtext("a:summary", namespaces=_ATOM))
    pm.authors = [squeeze(a.findtext("a:name", namespaces=_ATOM)) for a in e.findall("a:author", _ATOM)]
    pm.categories = [c.attrib.get("term", "") for c in e.findall("a:category", _ATOM)]
    pc = e.find("x:primary_category", _ATOM)
    pm.primary_category = pc.attrib.get("term") if pc is not None else (pm.categories[0] if pm.categories else None)
    pm.submitted, pm.updated = e.findtext("a:published", namespaces=_ATOM), e.findtext("a:updated", namespaces=_ATOM)
    pm.doi, pm.journal_ref = e.findtext("x:doi", namespaces=_ATOM), squeeze(e.findtext("x:journal_ref", namespaces=_ATOM))
    pm.comment = squeeze(e.findtext("x:comment", namespaces=_ATOM))
    for l in e.findall("a:link", _ATOM):
      if l.attrib.get("title") == "license" or "license" in l.attrib.get("rel", ""):
        pm.license = l.attrib.get("href")
    out[pm.arxiv_id] = pm
  return out


def load_metadata_snapshot(path: str, categories: Optional[Iterable[str]] = None) -> Iterator[PaperMetadata]:
  """Rows of the public metadata snapshot (JSON lines with id / title / authors / categories / abstract / versions),
  optionally restricted to papers with at least one of ``categories`` (prefix match: "cs." keeps every cs.* paper)."""
  want = tuple(categories) if categories else None
  with open(path, "r", encoding="utf-8") as f:
    for line in f:
      line = line.strip()
      if not line:
        continue
      r = json.loads(line)
      cats = (r.get("categories") or "").split() if isinstance(r.get("categories"), str) else list(r.get("categories") or [])
      if want and not any(c.startswith(w) for c in cats for w in want):
        continue
      authors = r.get("authors_parsed")
      names = [" ".join(x for x in (a[1], a[0]) if x).strip() for a in authors] if authors else \
          [a.strip() for a in re.split(r",| and ", r.get("authors") or "") if a.strip()]
      vers = r.get("versions") or []
      yield PaperMetadata(arxiv_id=r.get("id"), title=" ".join((r.get("title") or "").split()) or None, authors=names,
                          abstract=" ".join((r.get("abstract") or "").split()) or None, categories=cats,
                          primary_category=cats[0] if cats else None,
                          submitted=vers[0].get("created") if vers else None,
                          updated=vers[-1].get("created") if vers else r.get("update_date"), doi=r.get("doi"),
                          journal_ref=r.get("journal-ref"), comment=r.get("comments"), license=r.get("license"))


class MetadataClient:
  """arXiv API client with the service's rate limit (one request per ``delay`` seconds, up to 100 ids each).
  ``fetch`` / ``get`` / ``search`` need network access; ``parse`` works on a saved response.  ``opener(url) -> str`` can
  replace the HTTP call (tests, a caching proxy)."""

  API = "http://export.arxiv.org/api/query"

  def __init__(self, delay: float = 3.0, opener=None, sleep=time.sleep):
    self.delay, self._last, self._sleep = delay, 0.0, sleep
    self._open = opener or self._http

  parse = staticmethod(parse_atom_feed)

  @staticmethod
  def _http(url: str) -> str:
    from urllib.request import urlopen
    with urlopen(url, timeout=60) as r:
      return r.read().decode("utf-8")

  def _request(self, query: str) -> str:
    wait = self.delay - (time.time() - self._last)
    if wait > 0:
      self._sleep(wait)
    self._last = time.time()
    return self._open(f"{self.API}?{query}")

  def fetch(self, arxiv_ids: List[str], batch_size: int = 100) -> Dict[str, PaperMetadata]:
    from urllib.parse import quote
    out: Dict[str, PaperMetadata] = {}
    for i in range(0, len(arxiv_ids), batch_size):
      batch = arxiv_ids[i:i + batch_size]
      out.update(parse_atom_feed(self._request(f"id_list={quote(','.join(batch))}&max_results={len(batch)}")))
    return out

  def get(self, arxiv_id: str) -> Optional[PaperMetadata]:
    return self.fetch([arxiv_id]).get(_ID_RE.sub(lambda m: m.group(1), arxiv_id))

  def search(self, category: str, start_date: Optional[str] = None, end_date: Optional[str] = None, max_results: int = 1000,
             page: int = 200) -> List[PaperMetadata]:
    """Papers of a category (``cs.LG``), newest first, optionally submitted within [start_date, end_date]
    (``YYYYMMDD``).  The service pages its answers; this walks the pages until ``max_results`` papers or an empty page
    (nmoe/data/arxiv/metadata.py:232-291 lists ids the same way)."""
    from urllib.parse import quote
    q = f"cat:{category}"
    if start_date or end_date:
      q += f" AND submittedDate:[{start_date or '*'} TO {end_date or '*'}]"
    out: List[PaperMetadata] = []
    seen = set()
    while len(out) < max_results:
      n = min(page, max_results - len(out))
      got = parse_atom_feed(self._request(f"search_query={quote(q)}&start={len(seen)}&max_results={n}&sortBy=submittedDate&sortOrder=descending"))
      fresh = [m for k, m in got.items() if k not in seen]
      if not fresh:
        break
      seen.update(got)
      out += fresh
    return out[:max_results]

  def list_ids(self, category: str, start_date: Optional[str] = None, end_date: Optional[str] = None, max_results: int = 1000) -> List[str]:
    return [m.arxiv_id for m in self.search(category, start_date, end_date, max_results) if m.arxiv_id]
