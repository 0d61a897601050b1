"""``python -m nmoe_b200.data.cli <command>`` (nmoe/data/cli.py:1421-1643).

prep | prep-mixture | verify | info | regenerate-index | dedup | cluster | inspect | merge-manifests | flow
hydra-grade | hydra-oracle-label | hydra-train | hydra-calibrate | rephrase   (grading model: --checkpoint)
arxiv-download fetches the bulk source tars (aws CLI, an HTTP mirror or a directory); arxiv-prep converts them."""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Optional

from .errors import PipelineError


def _prep_task(a) -> int:
  """``prep --task ID``: build a registered corpus from its raw recipe with the registry's preparation steps."""
  from .registry import Registry
  reg = Registry.load(a.registry)
  if a.corpus_root:
    reg.root = Path(a.corpus_root)
  t = reg.task(a.task)
  grader, tau = None, 0.0
  wants = t.prep.get("hydra_filter") or t.prep.get("hydra_audit")
  if wants and not a.no_hydra:
    if not (a.checkpoint and a.heads_dir):
      print(f"task {a.task!r} is filtered by the quality grader: pass --checkpoint and --heads-dir, or --no-hydra", file=sys.stderr)
      return 2
    grader, tau = _mixture_grader(a, {})
  m = reg.build(a.task, a.split, grader=grader, tau_keep=tau, no_hydra=a.no_hydra or grader is None, max_documents=a.max_documents,
                tokenizer=a.tokenizer if a.tokenizer != "o200k_harmony" else None, num_shards=a.num_shards if a.num_shards != 8 else None)
  print(f"wrote {m.num_shards} shards, {m.total_documents:,} documents, {m.total_tokens:,} tokens for task {a.task}")
  return 0


def cmd_tasks(a) -> int:
  """Which registered corpora are ready to train on (shards found) and which can be built (raw material found)."""
  from .registry import Registry
  reg = Registry.load(a.registry)
  if a.corpus_root:
    reg.root = Path(a.corpus_root)
  rows = reg.status()
  if a.json:
    print(json.dumps({"root": str(reg.root), "contract": reg.contract, "tasks": rows}, indent=1))
    return 0
  print(f"corpus root {reg.root}  contract {reg.contract.get('tokenizer')} / vocab {reg.contract.get('vocab_size')} / eos {reg.contract.get('eos_token_id')}")
  for r in rows:
    state = "ready" if r["ready"] else ("buildable" if r["buildable"] else "missing")
    tok = f"{r['tokens'] / 1e9:.2f} B tokens" if r["tokens"] else ""
    raw = "" if r["raw_files"] is None else f"{r['raw_files']} raw file(s)"
    print(f"  {r['task']:<22} {r['domain']:<8} {state:<10} {r['shards']:>6} shard(s) {tok:<16} {r['raw_kind'] or '-':<12} {raw}")
  return 0


def cmd_prep(a) -> int:
  from .prep import ParallelPrepPipeline, PrepConfig, PrepPipeline
  from .sources import create_source
  if a.task:
    return _prep_task(a)
  if not (a.output and a.name):
    raise SystemExit("prep needs --output and --name (or --task ID to build a registered corpus)")
  if a.source in ("arxiv_tars", "ar5iv", "arxiv_paired"):
    # --input is the directory of bulk tars (of ar5iv pages for `ar5iv`); --html-dir the ar5iv tree for the paired form
    kw = {"arxiv_tars": {"tar_dir": a.input}, "ar5iv": {"html_dir": a.input},
          "arxiv_paired": {"tar_dir": a.input, "html_dir": a.html_dir}}[a.source]
    if a.source == "arxiv_paired" and not a.html_dir:
      raise SystemExit("--source arxiv_paired needs --html-dir")
  else:
    kw = {"paths": a.input} if a.source in ("jsonl", "jsonl_zst", "text", "arrow", "parquet") else \
        {"dataset": a.dataset, "subset": a.subset, "split": a.split}
    if a.source not in ("text",):
      kw["text_field"] = a.text_field
  cfg = PrepConfig(output_dir=a.output, dataset=a.name, version=a.version, tokenizer=a.tokenizer, num_shards=a.num_shards,
                   max_documents=a.max_documents, max_tokens=a.max_tokens)
  audited = None
  def make_source():
    return create_source(a.source, **kw)
  if a.hydra_filter or a.hydra_audit_dir:
    # grading runs in this process (one model on one GPU): worker processes and the stage graph are for ungraded input
    if a.workers > 1 or a.runner != "process":
      raise SystemExit("--hydra-filter / --hydra-audit-dir grade in the main process: use --workers 1 --runner process")
    from .sources import AuditedSource, FilteredSource, ScoringSource
    score, tau_keep = _mixture_grader(a, {})
    if a.hydra_audit_dir:
      audited = AuditedSource(ScoringSource(make_source(), score, a.hydra_batch_size), a.hydra_audit_dir,
                              tau_keep if a.hydra_filter else None)
      src = audited
    else:
      src = FilteredSource(make_source(), tau_keep, score_fn=score, batch_size=a.hydra_batch_size)
    m = PrepPipeline(src, cfg).run()
  elif a.runner != "process":
    from .prep import run_beam_pipeline
    m = run_beam_pipeline(make_source(), cfg, runner=a.runner)
  elif a.workers > 1:
    m = ParallelPrepPipeline(make_source, cfg, a.workers).run()
  else:
    m = PrepPipeline(make_source(), cfg).run()
  print(f"wrote {m.num_shards} shards, {m.total_documents:,} documents, {m.total_tokens:,} tokens -> {a.output}")
  if audited is not None:
    print(f"graded {audited.seen:,} documents, kept {audited.kept:,}; scores of all of them -> {a.hydra_audit_dir}/scores.jsonl")
  return 0


def _parse_count(v) -> Optional[int]:
  """'100M' / '1.5B' / '20000' -> int."""
  if v is None:
    return None
  m = {"k": 1e3, "m": 1e6, "b": 1e9, "t": 1e12}
  v = str(v).strip().lower()
  return int(float(v[:-1]) * m[v[-1]]) if v and v[-1] in m else int(float(v))


def _mixture_grader(a, mix: dict):
  """The quality filter of ``prep-mixture --hydra-filter``: flags first, then the mixture file's [hydra] table."""
  from . import hydra as H
  h = mix.get("hydra", {})
  ckpt = a.checkpoint or h.get("checkpoint")
  heads = a.heads_dir or h.get("heads_dir")
  calib_dir = a.calibration or h.get("calibration") or heads
  if not ckpt or not heads:
    raise SystemExit("--hydra-filter needs a grading checkpoint and a heads directory (flags, or [hydra] in the mixture file)")
  a.checkpoint = ckpt
  model, dev = _grading_model(a)
  probe, judge = H.load_heads(heads, model.cfg.hidden_size, dev)
  calib = H.Calibration.load(calib_dir)
  score = H.make_flow_grader(model, probe, judge, calib, _tokenizer(a.tokenizer), max_ctx=a.hydra_max_ctx, batch_size=a.hydra_batch_size)
  return score, calib.tau_keep


def cmd_prep_mixture(a) -> int:
  """Build the sources of a mixture/flow under {output_root}/{stage}/{source}/{split}.

  Several workers (``--worker-index i --num-workers n``) split the list of (stage, source) pairs round-robin, so an
  indexed batch job prepares a large mixture in parallel without coordination.  ``--limit`` bounds the documents read
  per source and prints a SHA-256 over the ids of the documents that were kept, which two runs with the same
  ``--seed`` must reproduce.  Reference: nmoe/data/cli.py:1483-1511 (prep-mixture flags)."""
  import hashlib
  from ..config import load_toml
  from .mixture import resolve_plan
  from .prep import PrepConfig, PrepPipeline
  from .sources import FilteredSource, create_source
  mixture = a.mixture or a.config
  if not mixture:
    raise SystemExit("prep-mixture needs --mixture (or --config) <mixture.toml>")
  mix = load_toml(mixture)
  flow = a.flow
  if flow is None:
    flows = sorted(load_toml(a.flow_profiles).get("flow", {}))
    if len(flows) != 1:
      raise SystemExit(f"--flow is required: {a.flow_profiles} defines {flows}")
    flow = flows[0]
  plan = resolve_plan(mixture_toml=Path(mixture), flow_profiles_toml=Path(a.flow_profiles),
                      flow_section=f"flow.{flow}", seq_len=a.seq_len, active_params_b=a.active_params_b)
  root = Path(a.output or a.output_root or Path(a.data_root) / "flows" / flow)
  jobs = [(st, sp) for st in plan.stages if a.stage in (None, st.stage_id) for sp in st.sources]
  jobs = [j for i, j in enumerate(jobs) if i % max(1, a.num_workers) == a.worker_index]
  grader = None
  if a.hydra_filter and not a.dry_run:
    grader = _mixture_grader(a, mix)
  print(f"plan {plan.plan_id} hash {plan.plan_hash[:12]} seed {a.seed}: worker {a.worker_index}/{a.num_workers} takes "
        f"{len(jobs)} source(s) -> {root}")
  failed = 0
  for st, sp in jobs:
    for split in [x.strip() for x in a.splits.split(",") if x.strip()]:
      out = root / st.stage_id / sp.id / split
      need = _parse_count(a.max_tokens) or sp.quota_sequences * (a.seq_len + 1)
      if a.dry_run:
        where = f"hf:{sp.hf.dataset}" + (f"/{sp.hf.subset}" if sp.hf.subset else "") if sp.hf is not None else \
                (str(Path(a.local_root) / sp.id) if a.local_root else "(no source)")
        print(f"would build {st.stage_id}/{sp.id}/{split}: {need:,} tokens from {where} -> {out}")
        continue
      if (out / "manifest.json").exists() and not a.force:
        print(f"skip {st.stage_id}/{sp.id}/{split}: {out}/manifest.json exists (--force rebuilds)")
        continue
      try:
        if sp.hf is not None:
          hf_split = sp.hf.split if split == "train" else (sp.hf.valid_split or split)
          src = create_source("hf", dataset=sp.hf.dataset, subset=sp.hf.subset, split=hf_split,
                              text_field=sp.hf.text_field, data_files=sp.hf.data_files)
        elif a.local_root:
          src = create_source("jsonl", paths=str(Path(a.local_root) / sp.id))
        else:
          print(f"skip {sp.id}: no hf_dataset in the mixture and no --local-root", file=sys.stderr)
          continue
        digest = hashlib.sha256(f"seed={a.seed}".encode())
        src = _Limited(src, a.limit, digest)
        if grader is not None:
          src = FilteredSource(src, grader[1], grader[0], a.hydra_batch_size)
        m = PrepPipeline(src, PrepConfig(str(out), sp.id, tokenizer=a.tokenizer, num_shards=a.num_shards, max_tokens=need,
                                         source_info={"plan_hash": plan.plan_hash, "seed": a.seed, "stage": st.stage_id})).run()
        kept = f", kept {src.kept}/{src.seen} after the quality filter" if grader is not None else ""
        print(f"{st.stage_id}/{sp.id}/{split}: {m.total_tokens:,} tokens (quota {need:,}){kept}; sample ids sha256 {digest.hexdigest()[:16]}")
      except Exception as e:  # noqa: BLE001 - one bad source must not lose a night's work when asked to go on
        if not a.continue_on_error:
          raise
        failed += 1
        print(f"FAILED {st.stage_id}/{sp.id}/{split}: {type(e).__name__}: {e}", file=sys.stderr)
  return 1 if failed else 0


class _Limited:
  """First ``limit`` documents of a source (all when None); folds every document id into ``digest``."""

  def __init__(self, base, limit: Optional[int], digest):
    self.base, self.limit, self.digest = base, limit, digest
    self.name = getattr(base, "name", "source")

  def __iter__(self):
    for i, d in enumerate(self.base):
      if self.limit is not None and i >= self.limit:
        return
      self.digest.update(str(d.doc_id).encode())
      yield d


def cmd_verify(a) -> int:
  from .sinks import verify_manifest
  m = verify_manifest(Path(a.path), check_checksums=not a.fast)
  print(f"OK: {m.num_shards} shards, {m.total_tokens:,} tokens")
  return 0


def cmd_info(a) -> int:
  from .inspect import dataset_summary
  print(json.dumps(dataset_summary(Path(a.path)), indent=1))
  return 0


def cmd_regenerate_index(a) -> int:
  from .index import regenerate_index_from_shard
  for p in sorted(Path(a.path).glob("*.npy")) if Path(a.path).is_dir() else [Path(a.path)]:
    print(regenerate_index_from_shard(p, a.eos_token_id))
  return 0


def cmd_dedup(a) -> int:
  from .dedup import dedup_exact, dedup_within_docs, stream_near_dedup
  from .sources import create_source
  src = create_source("jsonl", paths=a.input, text_field=a.text_field)
  if a.within:      # repeats inside a document go first, so that pages differing only in boilerplate can match
    src = dedup_within_docs(src, a.within)
  docs = dedup_exact(src)
  if a.near:
    docs = stream_near_dedup(docs, threshold=a.threshold)
  n = 0
  with open(a.output, "w", encoding="utf-8") as f:
    for d in docs:
      f.write(json.dumps({"id": d.doc_id, a.text_field: d.text, **d.metadata}) + "\n")
      n += 1
  print(f"kept {n:,} documents -> {a.output}")
  return 0


def cmd_cluster(a) -> int:
  import numpy as np
  from .diversity import cluster_embeddings, coverage_metrics
  x = np.load(a.embeddings)
  _, assign = cluster_embeddings(x, a.k)
  print(json.dumps(coverage_metrics(assign, a.k), indent=1))
  if a.output:
    np.save(a.output, assign)
  return 0


def cmd_inspect(a) -> int:
  from . import inspect as I
  if a.doc is not None:
    print(json.dumps(I.document(Path(a.shard), a.doc, a.tokenizer), indent=1))
  elif a.start is not None:
    print(json.dumps(I.shard_window(Path(a.shard), a.start, a.length, a.tokenizer), indent=1))
  else:
    print(json.dumps(I.shard_stats(Path(a.shard)), indent=1))
  return 0


def cmd_merge_manifests(a) -> int:
  from .sinks import load_manifest, merge_manifests, write_manifest_file
  m = merge_manifests([load_manifest(Path(p)) for p in a.parts])
  write_manifest_file(Path(a.output), m)
  print(f"merged {len(a.parts)} manifests: {m.num_shards} shards, {m.total_tokens:,} tokens")
  return 0


def _flow_profile(a) -> int:
  """``flow --config flow_profiles.toml --profile NAME``: a ``[profiles.NAME]`` table names a mixture file, a flow and
  the arguments of one ``prep-mixture`` call (nmoe/data/cli.py:1212-1266); this runs that call for this worker."""
  from ..config import load_toml
  cfg_path = Path(a.config or "configs/flow_profiles.toml")
  if not cfg_path.exists():
    print(f"flow profiles file not found: {cfg_path}", file=sys.stderr)
    return 1
  profiles = load_toml(cfg_path).get("profiles") or {}
  prof = profiles.get(a.profile)
  if not isinstance(prof, dict):
    print(f"unknown profile {a.profile!r}; {cfg_path} has: {', '.join(sorted(profiles)) or 'none'}", file=sys.stderr)
    return 1
  if not prof.get("mixture"):
    print(f"[profiles.{a.profile}] names no mixture file", file=sys.stderr)
    return 1
  argv = ["prep-mixture", "--config", str(prof["mixture"]), "--flow-profiles", str(cfg_path)]
  for key, flag in (("flow", "--flow"), ("stage", "--stage"), ("splits", "--splits"), ("seed", "--seed"), ("limit", "--limit"),
                    ("output_root", "--output-root"), ("tokenizer", "--tokenizer"), ("num_shards", "--num-shards"),
                    ("data_root", "--data-root"), ("max_tokens", "--max-tokens")):
    if prof.get(key) not in (None, ""):
      argv += [flag, str(prof[key])]
  for key, flag in (("dry_run", "--dry-run"), ("force", "--force"), ("hydra_filter", "--hydra-filter"), ("continue_on_error", "--continue-on-error")):
    if prof.get(key) or getattr(a, key, False):
      argv.append(flag)
  for key, flag in (("data_root", "--data-root"), ("output_root", "--output-root")):      # the command line wins over the table
    if getattr(a, key, None):
      argv += [flag, str(getattr(a, key))]
  argv += ["--num-workers", str(a.num_workers), "--worker-index", str(a.worker_index)]
  return main(argv)


def cmd_flow(a) -> int:
  """Run a data flow; its grading / rephrasing stages load the grading model named in the spec
  (``grade.checkpoint`` + ``grade.heads``, ``rephrase.checkpoint``)."""
  from .flow import load_spec, run_flow
  if a.profile or a.config:
    return _flow_profile(a)
  if not a.spec:
    print("flow needs a specification file, or --config FLOW_PROFILES --profile NAME", file=sys.stderr)
    return 2
  spec = load_spec(Path(a.spec))
  grader = rephraser = None
  model = None
  tok = None
  if spec.grade.get("enabled") or spec.rephrase.get("enabled"):
    import argparse as _ap
    ck = spec.grade.get("checkpoint") or spec.rephrase.get("checkpoint")
    if not ck:
      print("the flow enables grading / rephrasing but names no checkpoint", file=sys.stderr)
      return 2
    model, dev = _grading_model(_ap.Namespace(checkpoint=ck))
    tok = _tokenizer(spec.prep.get("tokenizer", "o200k_harmony"))
  if spec.grade.get("enabled"):
    from . import hydra as H
    probe, judge = H.load_heads(spec.grade["heads"], model.cfg.hidden_size, dev)
    calib = H.Calibration.load(spec.grade.get("calibration", spec.grade["heads"]))
    grader = H.make_flow_grader(model, probe, judge, calib, tok, max_ctx=int(spec.grade.get("max_ctx", 4096)),
                                batch_size=int(spec.grade.get("batch_size", 32)))
  if spec.rephrase.get("enabled"):
    from ..serve import Engine
    from .rephrase import rephrase_batch
    eng = Engine(model, max_seq_len=int(spec.rephrase.get("max_ctx", 4096)), max_batch=int(spec.rephrase.get("batch_size", 32)))
    rp = spec.rephrase
    n_ver = int(rp.get("num_versions", 1))
    def rephraser(texts):
      out = rephrase_batch(eng, tok, texts, num_versions=n_ver, chunk_size=int(rp.get("chunk_size", 2048)),
                           use_style_diversity=bool(rp.get("style_diversity", True)), temperature=float(rp.get("temperature", 0.8)),
                           top_p=float(rp.get("top_p", 0.9)), stop_tokens=[getattr(tok, "eot", -1)], seed=int(rp.get("seed", 0)))
      if rp.get("filter", True):          # drop rewrites that lost the source's content (lexical bounds, then embeddings)
        from .rephrase import filter_by_fidelity, semantic_fidelity
        thr = rp.get("semantic_threshold")
        sem = semantic_fidelity(model, tok, texts, out, max_ctx=int(rp.get("max_ctx", 4096))) if thr is not None and out else None
        out = filter_by_fidelity(texts, out, semantic=sem, min_semantic=float(thr or 0.0))
      by_doc = {}
      for r in out:
        by_doc.setdefault(r.doc, []).append(r.text)
      return [by_doc.get(i, [t] if n_ver == 1 else []) for i, t in enumerate(texts)]
  if a.staged or spec.prep.get("staged"):
    from .staged import run_flow_staged      # every stage on disk; an interrupted run continues
    run_flow_staged(spec, grader=grader, rephraser=rephraser)
  else:
    run_flow(spec, grader=grader, rephraser=rephraser)
  return 0


def _read_jsonl(path: str, text_field: str, limit=None):
  rows = []
  with open(path, "r", encoding="utf-8") as f:
    for line in f:
      if line.strip():
        j = json.loads(line)
        if text_field in j:
          rows.append(j)
          if limit and len(rows) >= limit:
            break
  return rows


def _tokenizer(name: str):
  """tiktoken encoding when available, else the byte-level tokenizer (tests, offline boxes)."""
  from .score import ByteTokenizer
  if name == "bytes":
    return ByteTokenizer()
  try:
    import tiktoken  # type: ignore
    return tiktoken.get_encoding(name)
  except Exception:
    print(f"tokenizer {name!r} is not available here; using UTF-8 bytes", file=sys.stderr)
    return ByteTokenizer()


def _grading_model(a):
  import torch
  from ..serve.checkpoint import load_model
  dev = "cuda" if torch.cuda.is_available() else "cpu"
  return load_model(a.checkpoint, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32), dev


def _grading_inputs(a, tok):
  """(ids, token lists) of the documents to grade: a JSONL of texts (``--input``), or a list of shard references
  (``--input-docids`` with ``--data-root``) whose tokens are read from the shards without going through text.
  With ``--resume``, ids already present in the output file are left out."""
  done = set()
  if getattr(a, "resume", False) and os.path.exists(a.output):
    for line in open(a.output, encoding="utf-8"):
      try:
        done.add(str(json.loads(line).get("doc_id")))
      except json.JSONDecodeError:      # a line cut by a crash: its document is graded again
        pass
  if getattr(a, "input_docids", None):
    if not a.data_root:
      raise SystemExit("--input-docids needs --data-root")
    from .docid import SpanReader, read_refs
    reader = SpanReader(a.data_root)
    refs = list(read_refs(a.input_docids, skip=done))[:a.max_documents]
    return [str(r) for r in refs], [reader.tokens(r, a.max_ctx) for r in refs], len(done)
  if not a.input:
    raise SystemExit("one of --input / --input-docids is required")
  rows = _read_jsonl(a.input, a.text_field, a.max_documents)
  ids = [str(r.get("doc_id", r.get("id", i))) for i, r in enumerate(rows)]
  keep = [i for i, d in enumerate(ids) if d not in done]
  return [ids[i] for i in keep], [tok.encode(rows[i][a.text_field])[:a.max_ctx] for i in keep], len(done)


def cmd_hydra_grade(a) -> int:
  """Documents in -> JSONL out with q_probe / rubric scores / decision per document (probe early exit, judge)."""
  from . import hydra as H
  if not a.output:
    raise SystemExit("hydra-grade needs --output")
  model, dev = _grading_model(a)
  probe, judge = H.load_heads(a.heads, model.cfg.hidden_size, dev)
  calib = H.Calibration.load(a.calibration or a.heads)
  ids, docs, n_done = _grading_inputs(a, _tokenizer(a.tokenizer))
  probe_only = judged = 0
  with open(a.output, "a" if n_done else "w", encoding="utf-8") as f:
    # graded in slabs so that a long run leaves its finished part on disk for --resume
    for i0 in range(0, len(docs), a.flush_every):
      out = H.grade(model, probe, judge, docs[i0:i0 + a.flush_every], ids[i0:i0 + a.flush_every], calib,
                    batch_size=a.batch_size, max_ctx=a.max_ctx, early_exit=not a.no_early_exit)
      for r in out:
        f.write(json.dumps(r) + "\n")
      f.flush()
      probe_only += H.grade.last_stats["probe_only"]
      judged += H.grade.last_stats["judged"]
  print(f"graded {len(docs)} documents ({n_done} already done): {probe_only} dropped at the probe, {judged} judged -> {a.output}")
  return 0


def cmd_docids(a) -> int:
  """List the documents of a prepared dataset as shard references (optionally a hash-sampled fraction of them)."""
  from .docid import enumerate_refs, sample_refs, write_refs
  refs = enumerate_refs(a.data_root, a.source, a.subdir, a.min_tokens)
  if a.fraction < 1.0:
    refs = sample_refs(refs, a.fraction, a.seed)
  if a.limit:
    import itertools
    refs = itertools.islice(refs, a.limit)
  n = write_refs(a.output, refs)
  print(f"{n} document references -> {a.output}")
  return 0


def cmd_hydra_oracle_label(a) -> int:
  """Ask the grading model itself for rubric scores (JSON answers) through the batching engine.  Input is a JSONL of
  texts, or a list of shard references whose tokens are decoded back to text; ``--resume`` skips ids already in the
  output.  Rows carry ``doc_id`` so that ``hydra-train --oracle-labels`` can join them with the shards again."""
  from ..serve import Engine
  from .score import grade_prompts
  if not a.output:
    raise SystemExit("hydra-oracle-label needs --output")
  model, _ = _grading_model(a)
  tok = _tokenizer(a.tokenizer)
  ids, docs, n_done = _grading_inputs(a, tok)
  texts = [tok.decode(d) for d in docs]
  eng = Engine(model, max_seq_len=a.max_ctx, max_batch=a.batch_size)
  parsed = 0
  with open(a.output, "a" if n_done else "w", encoding="utf-8") as f:
    for i0 in range(0, len(texts), a.flush_every):
      res = grade_prompts(eng, tok, texts[i0:i0 + a.flush_every], max_new=a.max_new, max_ctx=a.max_ctx,
                          stop_tokens=[getattr(tok, "eot", -1)])
      for did, g in zip(ids[i0:i0 + a.flush_every], res):
        f.write(json.dumps({"doc_id": did, "id": did, "ok": g["scores"] is not None, **g}) + "\n")
        parsed += int(g["scores"] is not None)
      f.flush()
  print(f"labelled {len(texts)} documents ({parsed} parsed, {n_done} already done) -> {a.output}")
  return 0


def cmd_hydra_calibrate(a) -> int:
  """Rubric weights and keep / drop thresholds.  ``--labels`` alone fits them to oracle labels at a target keep rate;
  ``--judged`` with ``--oracle`` fits them to the judge head's own predictions against the oracle's keep decision."""
  import torch
  from . import hydra as H
  if a.labels:
    rows = [json.loads(l) for l in open(a.labels, encoding="utf-8") if l.strip()]
    try:
      cal, n = H.calibrate_from_labels(rows, a.target_keep)
    except ValueError as e:
      print(str(e), file=sys.stderr)
      return 1
    p = cal.save(a.output)
    print(json.dumps({"weights": cal.weights, "tau_drop": cal.tau_drop, "tau_keep": cal.tau_keep, "count": n, "path": str(p)}, indent=1))
    return 0
  if not (a.judged and a.oracle):
    print("hydra-calibrate needs --labels, or --judged with --oracle", file=sys.stderr)
    return 2
  judged = {str(j["doc_id"]): j for j in map(json.loads, open(a.judged, encoding="utf-8")) if j.get("scores")}
  oracle = {str(j.get("doc_id", j.get("id"))): j for j in map(json.loads, open(a.oracle, encoding="utf-8")) if j.get("aggregated") is not None}
  keys = sorted(set(judged) & set(oracle))
  if not keys:
    print("no overlapping documents between --judged and --oracle", file=sys.stderr)
    return 2
  pred = torch.tensor([[judged[k]["scores"][d] for d in H.RUBRIC] for k in keys])
  keep = torch.tensor([oracle[k]["aggregated"] >= a.oracle_keep for k in keys])
  cal = H.calibrate(pred, keep, keep_precision=a.keep_precision)
  p = cal.save(a.output)
  print(f"{len(keys)} documents: tau_drop={cal.tau_drop:.3f} tau_keep={cal.tau_keep:.3f} -> {p}")
  return 0


def cmd_hydra_train(a) -> int:
  """One training phase (A / B / C) of the probe and judge heads over frozen backbone features."""
  import itertools
  import torch
  from . import hydra as H
  from ..serve.model import pool_hidden
  model, dev = _grading_model(a)
  cfg = model.cfg
  tok = _tokenizer(a.tokenizer)
  rows = _read_jsonl(a.input, a.text_field, a.max_documents) if a.input else []
  if not rows and not (a.labels or a.oracle_labels):
    raise SystemExit("hydra-train needs --input, or --labels / --oracle-labels")
  if a.oracle_labels and not a.data_root:
    raise SystemExit("--oracle-labels needs --data-root")
  try:
    probe, judge = H.load_heads(a.heads, cfg.hidden_size, dev)
  except FileNotFoundError:
    probe, judge = H.ProbeHead(cfg.hidden_size).to(dev), H.JudgeHead(cfg.hidden_size).to(dev)

  def features(batch):
    ids, pos, mask = H.pad_batch(batch["docs"], a.max_ctx, dev)
    with torch.no_grad():
      _, taps = model(ids, pos, up_to_layer=cfg.judge_layer, return_hidden_states=True, no_logits=True)
    return pool_hidden(taps[cfg.probe_layer], mask), taps[cfg.judge_layer].float(), mask

  def batches():
    g = torch.Generator().manual_seed(0)
    for _ in itertools.count():
      idx = torch.randperm(len(rows), generator=g)[:a.batch_size].tolist()
      b = {"docs": [tok.encode(rows[i][a.text_field])[:a.max_ctx] for i in idx]}
      nan = float("nan")
      b["targets"] = {k: torch.tensor([float(rows[i].get(k, nan)) for i in idx], device=dev)
                      for k, (w, kind) in H.PROBE_TASKS.items() if kind == "reg"}
      b["rubric"] = torch.tensor([[float((rows[i].get("scores") or {}).get(d, nan)) for d in H.RUBRIC] for i in idx], device=dev)
      yield b

  def label_batches():
    """Batches from label tables / oracle labels over shards instead of one flat JSONL."""
    from . import hydra_labels as L
    tables = [L.TableLabels(spec.split(":", 2)[2], L.FIELD_MAPS[spec.split(":", 2)[0]], spec.split(":", 2)[1], a.max_ctx)
              for spec in (a.labels or [])]          # each: <field map>:<domain>:<path or glob>
    if a.phase == "A":
      return L.probe_batches(L.mix(tables, seed=a.seed), a.batch_size, tok.encode, a.max_ctx, dev)
    graded = [t for t in tables if t.fields.grade]
    pairs = L.GradedPairs(L.mix(graded, seed=a.seed), seed=a.seed) if graded and a.phase == "B" else None      # only phase B ranks
    if a.oracle_labels:
      oracle = L.OracleLabels(a.oracle_labels, a.data_root, a.max_ctx)
    else:
      oracle = L.mix(tables, seed=a.seed + 1)        # phase C needs documents only
    return L.judge_batches(oracle, a.batch_size, tok.encode, a.max_ctx, pairs, a.pairs_per_batch if pairs else 0, dev)

  use_labels = bool(a.labels or a.oracle_labels)
  losses = H.train_heads(H.PhaseConfig(a.phase, steps=a.steps, lr=a.lr), probe, judge, label_batches() if use_labels else batches(), features,
                         log=lambda s, l: print(f"phase {a.phase} step {s} loss {l:.4f}"))
  H.save_heads(a.heads, probe, judge)
  print(f"phase {a.phase}: loss {losses[0]:.4f} -> {losses[-1]:.4f}; heads saved to {a.heads}")
  return 0


def cmd_rephrase(a) -> int:
  from ..serve import Engine
  from .rephrase import filter_by_fidelity, rephrase_batch
  model, _ = _grading_model(a)
  tok = _tokenizer(a.tokenizer)
  rows = _read_jsonl(a.input, a.text_field, a.max_documents)
  texts = [r[a.text_field] for r in rows]
  eng = Engine(model, max_seq_len=a.max_ctx, max_batch=a.batch_size)
  rew = rephrase_batch(eng, tok, texts, num_versions=a.num_versions, chunk_size=a.chunk_size, stop_tokens=[getattr(tok, "eot", -1)])
  sem = None
  if a.semantic_threshold is not None and not a.no_filter:      # embedding-space agreement with the source, same backbone
    from .rephrase import semantic_fidelity
    sem = semantic_fidelity(model, tok, texts, rew, max_ctx=a.max_ctx, batch_size=a.batch_size)
  kept = rew if a.no_filter else filter_by_fidelity(texts, rew, semantic=sem, min_semantic=a.semantic_threshold or 0.0)
  with open(a.output, "w", encoding="utf-8") as f:
    for r in kept:
      f.write(json.dumps({"id": rows[r.doc].get("id", r.doc), "version": r.version, "style": r.style, "text": r.text}) + "\n")
  info = rephrase_batch.last_info
  note = f" (chunks of {info['chunk_size']} tokens to fit the context)" if info["chunk_size"] < a.chunk_size else ""
  print(f"{len(rew)} rewrites, {len(kept)} kept -> {a.output}{note}")
  return 0


def cmd_arxiv_download(a) -> int:
  """Fetch arXiv bulk source tars listed in the manifest: a month range and / or a byte budget, through the AWS
  command-line client (requester pays), an HTTP mirror, or a directory.  ``--dry-run`` prints the selection and what the
  S3 transfer would cost."""
  from . import arxiv_download as AD
  fetcher = None if a.dry_run else AD.make_fetcher(a.fetch, base_url=a.base_url, root=a.root, profile=a.aws_profile)
  manifest = Path(a.manifest) if a.manifest else Path(a.output) / "arXiv_src_manifest.xml"
  if not manifest.exists():
    if fetcher is None:
      print(f"no manifest at {manifest}: fetch it first (run without --dry-run) or pass --manifest", file=sys.stderr)
      return 2
    manifest.parent.mkdir(parents=True, exist_ok=True)
    fetcher.fetch("src/arXiv_src_manifest.xml", manifest)
  picked = AD.select(AD.parse_manifest(manifest), a.start, a.end, _parse_count(a.max_bytes), a.max_files)
  print(json.dumps(AD.estimate_cost(picked)))
  if a.dry_run:
    for e in picked:
      print(f"{e.key}\t{e.size}\t{e.items}")
    return 0
  rep = AD.download(picked, a.output, fetcher, workers=a.workers, verify=not a.no_verify, keep_going=a.keep_going)
  print(f"fetched {len(rep.fetched)}, already complete {len(rep.skipped)}, failed {len(rep.failed)} -> {a.output}")
  return 0 if rep.ok else 1


def cmd_arxiv_prep(a) -> int:
  """Papers -> JSONL of plain text.  ``--input`` holds per-paper archives, or (with ``--bulk``) arXiv's monthly tars."""
  from .arxiv import iter_arxiv, write_jsonl
  if a.bulk:
    from .arxiv_download import iter_bulk_text
    n = write_jsonl(iter_bulk_text(a.input, a.min_chars), a.output)
  else:
    n = write_jsonl(iter_arxiv(a.input, a.min_chars), a.output)
  print(f"{n} papers -> {a.output}")
  return 0


def cmd_stack_v2(a) -> int:
  """The Stack v2 ids -> text.  Two forms: ``--input-root`` (the id table as downloaded, parquet) with ``--output-root``,
  ``--top-n`` and worker indices: popularity selection, blobs from the Software Heritage bucket (``--s3``) or a mirror
  directory (``--blobs``), rotating compressed JSONL parts; or ``--table`` (JSONL) with ``--blobs`` and ``--output``:
  every listed file that is present, into one JSONL."""
  if a.input_root:
    from . import stack_v2 as S
    if not a.output_root or a.top_n is None:
      raise SystemExit("--input-root needs --output-root and --top-n")
    if not (a.blobs or a.s3):
      raise SystemExit("name the blob store: --blobs DIR (a mirror) or --s3 (the Software Heritage bucket)")
    blobs = S.DirBlobs(a.blobs) if a.blobs else S.S3Blobs()
    truth = lambda v: str(v).strip().lower() in ("1", "true", "t", "yes", "y")
    summ = S.run(a.input_root, a.output_root, worker_index=a.worker_index, num_workers=a.num_workers, top_n=a.top_n, blobs=blobs,
                 min_bytes=a.min_bytes, max_bytes=a.max_bytes or 256_000, exclude_vendor=truth(a.exclude_vendor),
                 exclude_generated=truth(a.exclude_generated), max_files_per_repo=a.max_files_per_repo,
                 languages=a.languages.split(",") if a.languages else None, threads=a.threads)
    print(json.dumps({k: summ[k] for k in ("scanned", "selected", "written", "missing", "binary", "oversize")}))
    return 0
  if not (a.table and a.blobs and a.output):
    raise SystemExit("stack-v2-materialize needs --input-root ..., or --table with --blobs and --output")
  from .arxiv import iter_stack_v2, write_jsonl
  langs = set(a.languages.split(",")) if a.languages else None
  n = write_jsonl(iter_stack_v2(a.table, a.blobs, langs, a.max_bytes or (1 << 20)), a.output)
  print(f"{n} files -> {a.output}")
  return 0


def build_parser() -> argparse.ArgumentParser:
  ap = argparse.ArgumentParser(prog="nmoe_b200.data.cli")
  sub = ap.add_subparsers(dest="command", required=True)
  p = sub.add_parser("prep"); p.set_defaults(fn=cmd_prep)
  p.add_argument("--source", default="jsonl", help="jsonl | jsonl_zst | text | arrow | parquet | hf | hffs | arxiv_tars | ar5iv | arxiv_paired")
  p.add_argument("--html-dir", help="ar5iv tree ({tier}/{yymm}/{id}.html) for --source arxiv_paired")
  p.add_argument("--input"); p.add_argument("--dataset"); p.add_argument("--subset")
  p.add_argument("--split", default="train"); p.add_argument("--text-field", default="text"); p.add_argument("--output")
  p.add_argument("--task", help="build this corpus of the task registry instead of an ad-hoc source"); p.add_argument("--registry", default="configs/tasks.toml")
  p.add_argument("--corpus-root", help="override [corpus] root of the registry"); p.add_argument("--no-hydra", action="store_true")
  p.add_argument("--name"); p.add_argument("--version", default="v1"); p.add_argument("--tokenizer", default="o200k_harmony")
  p.add_argument("--num-shards", type=int, default=8); p.add_argument("--workers", type=int, default=1)
  p.add_argument("--max-documents", type=int); p.add_argument("--max-tokens", type=int)
  p.add_argument("--runner", default="process", choices=["process", "beam", "local", "auto"],
                 help="process: worker processes on this host; beam / local / auto: the stage graph on Apache Beam or the built-in runner")
  p.add_argument("--hydra-filter", action="store_true", help="keep only documents the quality grader scores at or above its keep threshold")
  p.add_argument("--hydra-audit-dir", help="write the score of every document, kept or not, to this directory")
  p.add_argument("--checkpoint"); p.add_argument("--heads-dir"); p.add_argument("--calibration")
  p.add_argument("--hydra-batch-size", type=int, default=32); p.add_argument("--hydra-max-ctx", type=int, default=4096)
  p = sub.add_parser("prep-mixture"); p.set_defaults(fn=cmd_prep_mixture)
  p.add_argument("--mixture"); p.add_argument("--config", help="same as --mixture")
  p.add_argument("--flow-profiles", default="configs/flow_profiles.toml"); p.add_argument("--flow")
  p.add_argument("--data-root", default="/data"); p.add_argument("--seq-len", type=int, default=4096); p.add_argument("--local-root")
  p.add_argument("--active-params-b", type=float); p.add_argument("--tokenizer", default="o200k_harmony"); p.add_argument("--num-shards", type=int, default=8)
  p.add_argument("--output"); p.add_argument("--output-root", help="same as --output; default {data-root}/flows/{flow}")
  p.add_argument("--stage", choices=["pretrain", "mid", "long"]); p.add_argument("--splits", default="train")
  p.add_argument("--seed", type=int, default=0); p.add_argument("--limit", type=int); p.add_argument("--max-tokens")
  p.add_argument("--force", action="store_true"); p.add_argument("--dry-run", action="store_true"); p.add_argument("--continue-on-error", action="store_true")
  p.add_argument("--worker-index", type=int, default=0); p.add_argument("--num-workers", type=int, default=1)
  p.add_argument("--hydra-filter", action="store_true"); p.add_argument("--checkpoint"); p.add_argument("--heads-dir"); p.add_argument("--calibration")
  p.add_argument("--hydra-batch-size", type=int, default=32); p.add_argument("--hydra-max-ctx", type=int, default=4096)
  p = sub.add_parser("tasks"); p.set_defaults(fn=cmd_tasks); p.add_argument("--registry", default="configs/tasks.toml")
  p.add_argument("--corpus-root"); p.add_argument("--json", action="store_true")
  p = sub.add_parser("verify"); p.set_defaults(fn=cmd_verify); p.add_argument("path"); p.add_argument("--fast", action="store_true")
  p = sub.add_parser("info"); p.set_defaults(fn=cmd_info); p.add_argument("path")
  p = sub.add_parser("regenerate-index"); p.set_defaults(fn=cmd_regenerate_index); p.add_argument("path"); p.add_argument("--eos-token-id", type=int, default=199999)
  p = sub.add_parser("dedup"); p.set_defaults(fn=cmd_dedup); p.add_argument("--input", required=True); p.add_argument("--output", required=True)
  p.add_argument("--text-field", default="text"); p.add_argument("--near", action="store_true"); p.add_argument("--threshold", type=float, default=0.8)
  p.add_argument("--within", choices=["lines", "paragraphs"], help="also drop repeated lines / paragraphs inside each document")
  p = sub.add_parser("cluster"); p.set_defaults(fn=cmd_cluster); p.add_argument("--embeddings", required=True); p.add_argument("--k", type=int, default=64); p.add_argument("--output")
  p = sub.add_parser("inspect"); p.set_defaults(fn=cmd_inspect); p.add_argument("shard"); p.add_argument("--doc", type=int)
  p.add_argument("--start", type=int); p.add_argument("--length", type=int, default=64); p.add_argument("--tokenizer")
  p = sub.add_parser("merge-manifests"); p.set_defaults(fn=cmd_merge_manifests); p.add_argument("parts", nargs="+"); p.add_argument("--output", required=True)
  p = sub.add_parser("flow"); p.set_defaults(fn=cmd_flow); p.add_argument("spec", nargs="?"); p.add_argument("--staged", action="store_true")
  p.add_argument("--config", help="flow profiles TOML with [profiles.NAME] tables"); p.add_argument("--profile")
  p.add_argument("--num-workers", type=int, default=1); p.add_argument("--worker-index", type=int, default=0)
  p.add_argument("--data-root"); p.add_argument("--output-root"); p.add_argument("--dry-run", action="store_true"); p.add_argument("--force", action="store_true")
  def model_args(p, heads=False, optional_io=False):
    p.add_argument("--checkpoint", required=True); p.add_argument("--input", required=not (heads or optional_io)); p.add_argument("--output", required=not (heads or optional_io))
    p.add_argument("--text-field", default="text"); p.add_argument("--tokenizer", default="o200k_harmony")
    p.add_argument("--max-ctx", type=int, default=4096); p.add_argument("--batch-size", type=int, default=32)
    p.add_argument("--max-documents", type=int)
    if heads:
      p.add_argument("--heads", required=True)
  p = sub.add_parser("hydra-grade"); p.set_defaults(fn=cmd_hydra_grade); model_args(p, heads=True)
  p.add_argument("--calibration"); p.add_argument("--no-early-exit", action="store_true")
  p.add_argument("--input-docids", help="JSONL of {doc_id: shard reference}; tokens are read from the shards"); p.add_argument("--data-root")
  p.add_argument("--resume", action="store_true"); p.add_argument("--flush-every", type=int, default=4096)
  p = sub.add_parser("docids"); p.set_defaults(fn=cmd_docids)
  p.add_argument("--data-root", required=True); p.add_argument("--source", required=True); p.add_argument("--output", required=True)
  p.add_argument("--subdir", default=""); p.add_argument("--min-tokens", type=int, default=0); p.add_argument("--fraction", type=float, default=1.0)
  p.add_argument("--seed", type=int, default=0); p.add_argument("--limit", type=int)
  p = sub.add_parser("hydra-oracle-label"); p.set_defaults(fn=cmd_hydra_oracle_label); model_args(p, optional_io=True); p.add_argument("--max-new", type=int, default=256)
  p.add_argument("--input-docids"); p.add_argument("--data-root"); p.add_argument("--resume", action="store_true"); p.add_argument("--flush-every", type=int, default=1024)
  p = sub.add_parser("hydra-train"); p.set_defaults(fn=cmd_hydra_train); model_args(p, heads=True)
  p.add_argument("--phase", choices=["A", "B", "C"], required=True); p.add_argument("--steps", type=int, default=1000); p.add_argument("--lr", type=float, default=1e-3)
  p.add_argument("--labels", action="append", help="<eai|fineweb_edu>:<web|code|science|math>:<parquet/JSONL path or glob>; repeatable")
  p.add_argument("--oracle-labels", help="JSONL of {doc_id: shard reference, scores}"); p.add_argument("--data-root")
  p.add_argument("--pairs-per-batch", type=int, default=8); p.add_argument("--seed", type=int, default=0)
  p = sub.add_parser("hydra-calibrate"); p.set_defaults(fn=cmd_hydra_calibrate)
  p.add_argument("--judged"); p.add_argument("--oracle"); p.add_argument("--output", required=True)
  p.add_argument("--labels", help="oracle labels JSONL: calibrate from these alone"); p.add_argument("--target-keep", type=float, default=0.5)
  p.add_argument("--oracle-keep", type=float, default=0.6); p.add_argument("--keep-precision", type=float, default=0.9)
  p = sub.add_parser("rephrase"); p.set_defaults(fn=cmd_rephrase); model_args(p)
  p.add_argument("--num-versions", type=int, default=1); p.add_argument("--chunk-size", type=int, default=2048); p.add_argument("--no-filter", action="store_true")
  p.add_argument("--semantic-threshold", type=float, help="also require this cosine similarity to the source in the backbone's embedding space (0.85 is a usual bar)")
  p = sub.add_parser("arxiv-download"); p.set_defaults(fn=cmd_arxiv_download)
  p.add_argument("--output", required=True); p.add_argument("--manifest"); p.add_argument("--fetch", default="s3", choices=["s3", "http", "file"])
  p.add_argument("--base-url"); p.add_argument("--root"); p.add_argument("--aws-profile"); p.add_argument("--start"); p.add_argument("--end")
  p.add_argument("--max-bytes"); p.add_argument("--max-files", type=int); p.add_argument("--workers", type=int, default=4)
  p.add_argument("--no-verify", action="store_true"); p.add_argument("--keep-going", action="store_true"); p.add_argument("--dry-run", action="store_true")
  p = sub.add_parser("arxiv-prep"); p.set_defaults(fn=cmd_arxiv_prep)
  p.add_argument("--input", required=True); p.add_argument("--output", required=True); p.add_argument("--min-chars", type=int, default=500)
  p.add_argument("--bulk", action="store_true", help="--input holds arXiv's monthly bulk tars")
  p = sub.add_parser("stack-v2-materialize"); p.set_defaults(fn=cmd_stack_v2)
  p.add_argument("--table"); p.add_argument("--blobs"); p.add_argument("--output")
  p.add_argument("--languages"); p.add_argument("--max-bytes", type=int, help="default 256000 with --input-root, 1 MiB with --table")
  p.add_argument("--input-root", help="the id table: {root}/data/**/*.parquet"); p.add_argument("--output-root")
  p.add_argument("--worker-index", type=int, default=0); p.add_argument("--num-workers", type=int, default=1)
  p.add_argument("--top-n", type=int, help="files to keep from this worker's slice of the table, most popular first")
  p.add_argument("--min-bytes", type=int, default=256); p.add_argument("--exclude-vendor", default="true"); p.add_argument("--exclude-generated", default="true")
  p.add_argument("--max-files-per-repo", type=int, default=200); p.add_argument("--s3", action="store_true"); p.add_argument("--threads", type=int, default=16)
  return ap


def main(argv=None) -> int:
  a = build_parser().parse_args(argv)
  try:
    return a.fn(a)
  except PipelineError as e:
    e.exit()
  except (FileNotFoundError, NotADirectoryError, IsADirectoryError, PermissionError) as e:
    if os.environ.get("NMOE_DEBUG"):
      raise
    # a mistyped path is the commonest failure of a command line: one line, not a traceback (NMOE_DEBUG=1 for the latter)
    print(f"{a.command}: {e.strerror or e}: {e.filename or ''}".rstrip(": "), file=sys.stderr)
    return 2


if __name__ == "__main__":
  sys.exit(main())
