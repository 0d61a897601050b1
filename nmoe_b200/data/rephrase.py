"""Knowledge rephrasing: style-diverse rewrites of documents, chunk by chunk, with a fidelity filter.

Long documents are split into overlapping token windows; every (document, version, chunk) becomes
one request to the continuous-batching engine, so a large job keeps the batch full regardless of
document lengths.  Versions cycle through the style prompts.  ``compute_fidelity`` compares a
rewrite with its source (length ratio, content-word recall, number / entity carry-over) and
``filter_by_fidelity`` drops rewrites that lost or invented too much.

Reference counterpart: nmoe/data/rephrase.py:30-388.
"""
from __future__ import annotations

import re
from dataclasses import dataclass
from typing import Dict, Iterable, List, Optional, Sequence

import torch

from .score import ChatFormat, Tokenizer

STYLE_PROMPTS: Dict[str, str] = {
  "formal": "Rewrite this text in formal academic style while preserving all factual information and key concepts.",
  "casual": "Rephrase this content in clear, conversational language while keeping all important facts and ideas.",
  "technical": "Rewrite this using precise technical terminology while maintaining complete accuracy and detail.",
  "simplified": "Rephrase this in simpler, more accessible language for a general audience, preserving all essential information.",
}
DEFAULT_INSTRUCTION = "Rewrite this text in different words while preserving all information."


def format_prompt(tok: Tokenizer, text: str, instruction: str = DEFAULT_INSTRUCTION, fmt: Optional[ChatFormat] = None) -> List[int]:
  fmt = fmt or ChatFormat()
  return tok.encode(fmt.render([("system", "Reasoning: low"), ("developer", instruction), ("user", text)]))


def chunk_text(text: str, tok: Tokenizer, chunk_size: int = 2048, overlap: int = 256) -> List[str]:
  """Token windows of ``chunk_size`` that overlap by ``overlap`` tokens, decoded back to text."""
  ids = tok.encode(text)
  if len(ids) <= chunk_size:
    return [text]
  overlap = min(overlap, chunk_size // 2)      # an overlap of a window or more would never advance
  step = max(1, chunk_size - overlap)
  out = []
  for s in range(0, len(ids), step):
    out.append(tok.decode(ids[s:s + chunk_size]))
    if s + chunk_size >= len(ids):
      break
  return out


def sample_top_p(logits: torch.Tensor, temperature: float = 0.8, top_p: float = 0.9,
                 generator: Optional[torch.Generator] = None) -> int:
  """Nucleus sampling of one row of logits."""
  if temperature <= 0:
    return int(logits.argmax())
  p = torch.softmax(logits.float() / temperature, dim=-1)
  sp, si = torch.sort(p, descending=True)
  keep = (sp.cumsum(0) - sp) < top_p
  sp = sp * keep
  return int(si[torch.multinomial(sp / sp.sum(), 1, generator=generator)])


@dataclass
class Rewrite:
  doc: int
  version: int
  style: str
  text: str


def rephrase_batch(engine, tok: Tokenizer, texts: Sequence[str], *, num_versions: int = 1, chunk_size: int = 2048,
                   overlap: int = 256, use_style_diversity: bool = True, max_new_factor: float = 1.3,
                   temperature: float = 0.8, top_p: float = 0.9, stop_tokens: Iterable[int] = (),
                   fmt: Optional[ChatFormat] = None, seed: int = 0) -> List[Rewrite]:
  """``num_versions`` rewrites of every text (chunks are rewritten independently and joined)."""
  styles = list(STYLE_PROMPTS) if use_style_diversity else ["default"]
  stop = set(int(t) for t in stop_tokens)
  gen = torch.Generator(device="cpu").manual_seed(seed)
  # A chunk, its instructions and its rewrite (up to max_new_factor times the chunk) share the engine's context: the
  # largest chunk that leaves the rewrite its full budget.  Asking for more would cut rewrites short without a word.
  overhead = max(len(format_prompt(tok, "", STYLE_PROMPTS.get(st, DEFAULT_INSTRUCTION), fmt)) for st in styles[:max(1, num_versions)])
  fit = int((engine.max_seq_len - overhead - 18) / (1.0 + max_new_factor))
  if fit < 16:
    raise ValueError(f"a context of {engine.max_seq_len} tokens leaves no room to rewrite anything: the instructions alone take "
                     f"{overhead} tokens with this tokenizer; raise the context length")
  if chunk_size > fit:
    chunk_size, overlap = fit, min(overlap, fit // 8)
  rephrase_batch.last_info = {"chunk_size": chunk_size, "overlap": min(overlap, chunk_size // 2), "dropped_chunks": 0}
  jobs = []                                   # (doc, version, chunk index, style)
  sid_of = {}
  for d, text in enumerate(texts):
    chunks = chunk_text(text, tok, chunk_size, overlap)
    for v in range(num_versions):
      style = styles[v % len(styles)]
      instr = STYLE_PROMPTS.get(style, DEFAULT_INSTRUCTION)
      for c, ch in enumerate(chunks):
        prompt = format_prompt(tok, ch, instr, fmt)
        budget = int(len(tok.encode(ch)) * max_new_factor) + 16
        room = engine.max_seq_len - len(prompt) - 1
        if room <= 0:                         # cannot happen after the fit above unless a tokenizer is wildly non-additive
          rephrase_batch.last_info["dropped_chunks"] += 1
          continue
        sid = engine.add(prompt, max(1, min(budget, room)))
        sid_of[sid] = (d, v, c, style)
        jobs.append(sid)
  while not engine.idle:
    res = engine.step()
    if res is None:
      break
    logits, ids = res
    rows = logits.float().cpu()
    for row, sid in zip(rows, ids):
      t = sample_top_p(row, temperature, top_p, gen)
      engine.update(sid, t, finished=t in stop)
  parts: Dict[tuple, Dict[int, str]] = {}
  style_of: Dict[tuple, str] = {}
  for sid in jobs:
    d, v, c, style = sid_of[sid]
    s = engine.finished[sid]
    parts.setdefault((d, v), {})[c] = tok.decode(s.tokens[s.prompt_len:]).strip()
    style_of[(d, v)] = style
  return [Rewrite(d, v, style_of[(d, v)], "\n".join(p for _, p in sorted(cs.items()))) for (d, v), cs in sorted(parts.items())]


_WORD = re.compile(r"[A-Za-z][A-Za-z\-']{3,}")
_NUM = re.compile(r"\d+(?:[.,]\d+)*")
_STOP = frozenset("this that with from have will would could should their there which about into than then them they were been being also such only other some more most very what when where while your these those".split())


def compute_fidelity(source: str, rewrite: str) -> Dict[str, float]:
  """Cheap lexical checks: length ratio, recall of the source's content words and numbers, and the
  share of the rewrite's numbers that are new (a proxy for invented facts)."""
  sw = {w.lower() for w in _WORD.findall(source)} - _STOP
  rw = {w.lower() for w in _WORD.findall(rewrite)} - _STOP
  sn, rn = set(_NUM.findall(source)), set(_NUM.findall(rewrite))
  return {
    "length_ratio": len(rewrite) / max(1, len(source)),
    "word_recall": len(sw & rw) / max(1, len(sw)),
    "number_recall": len(sn & rn) / len(sn) if sn else 1.0,
    "novel_numbers": len(rn - sn) / len(rn) if rn else 0.0,
  }


@torch.inference_mode()
def embed_texts(model, tok: Tokenizer, texts: Sequence[str], *, layer: Optional[int] = None, max_ctx: int = 4096,
                batch_size: int = 16) -> torch.Tensor:
  """Unit-norm mean-pooled hidden states of the grading backbone at ``layer`` (default: its probe layer), [N, H] on
  the CPU.  Texts are padded into batches and the padding is masked out of the mean."""
  from ..serve.model import pool_hidden
  from .hydra import pad_batch
  layer = layer if layer is not None else model.cfg.probe_layer
  dev = next(model.parameters()).device
  out = []
  for i in range(0, len(texts), batch_size):
    docs = [(tok.encode(t)[:max_ctx] or [0]) for t in texts[i:i + batch_size]]
    ids, pos, mask = pad_batch(docs, max_ctx, dev)
    _, taps = model(ids, pos, up_to_layer=layer, return_hidden_states=True, no_logits=True)
    out.append(torch.nn.functional.normalize(pool_hidden(taps[layer], mask), dim=-1).cpu())
  return torch.cat(out) if out else torch.zeros(0, model.cfg.hidden_size)


def semantic_fidelity(model, tok: Tokenizer, sources: Sequence[str], rewrites: Sequence[Rewrite], **kw) -> List[float]:
  """Cosine similarity, clamped to [0, 1], between each rewrite and its source in the backbone's embedding space
  (nmoe/data/rephrase.py:296-361).  Each distinct source is embedded once however many versions it has."""
  used = sorted({r.doc for r in rewrites})
  src = dict(zip(used, embed_texts(model, tok, [sources[d] for d in used], **kw)))
  rew = embed_texts(model, tok, [r.text for r in rewrites], **kw)
  return [float((src[r.doc] * rew[i]).sum().clamp(0.0, 1.0)) for i, r in enumerate(rewrites)]


def filter_by_fidelity(sources: Sequence[str], rewrites: Sequence[Rewrite], *, min_length_ratio: float = 0.5,
                       max_length_ratio: float = 2.0, min_word_recall: float = 0.3, min_number_recall: float = 0.8,
                       max_novel_numbers: float = 0.2, semantic: Optional[Sequence[float]] = None,
                       min_semantic: float = 0.85) -> List[Rewrite]:
  """Rewrites that pass the lexical bounds and, when ``semantic`` scores (one per rewrite, from ``semantic_fidelity``)
  are given, reach ``min_semantic``."""
  if semantic is not None and len(semantic) != len(rewrites):
    raise ValueError("one semantic score per rewrite is needed")
  keep = []
  for i, r in enumerate(rewrites):
    f = compute_fidelity(sources[r.doc], r.text)
    if (min_length_ratio <= f["length_ratio"] <= max_length_ratio and f["word_recall"] >= min_word_recall
        and f["number_recall"] >= min_number_recall and f["novel_numbers"] <= max_novel_numbers
        and (semantic is None or semantic[i] >= min_semantic)):
      keep.append(r)
  return keep
