"""``python -m nmoe_b200.data.cli <command>`` (nmoe/data/cli.py:1421-1643).

prep | prep-mixture | verify | info | regenerate-index | dedup | cluster | inspect | merge-manifests | flow
Corpus-curation commands that need a grading model (hydra-*, rephrase) and the download-only commands
(arxiv-download, arxiv-prep) are registered too and explain what they need when it is missing."""
from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

from .errors import PipelineError


def cmd_prep(a) -> int:
  from .prep import ParallelPrepPipeline, PrepConfig, PrepPipeline
  from .sources import create_source
  kw = {"paths": a.input} if a.source in ("jsonl", "jsonl_zst", "text", "arrow", "parquet") else \
      {"dataset": a.dataset, "subset": a.subset, "split": a.split}
  if a.source not in ("text",):
    kw["text_field"] = a.text_field
  cfg = PrepConfig(output_dir=a.output, dataset=a.name, version=a.version, tokenizer=a.tokenizer, num_shards=a.num_shards,
                   max_documents=a.max_documents, max_tokens=a.max_tokens)
  if a.workers > 1:
    m = ParallelPrepPipeline(lambda: create_source(a.source, **kw), cfg, a.workers).run()
  else:
    m = PrepPipeline(create_source(a.source, **kw), cfg).run()
  print(f"wrote {m.num_shards} shards, {m.total_documents:,} documents, {m.total_tokens:,} tokens -> {a.output}")
  return 0


def cmd_prep_mixture(a) -> int:
  """Build every source of a mixture/flow under {data_root}/flows/{flow}/{stage}/{source}/train."""
  from .mixture import resolve_plan
  from .prep import PrepConfig, PrepPipeline
  from .sources import create_source
  plan = resolve_plan(mixture_toml=Path(a.mixture), flow_profiles_toml=Path(a.flow_profiles),
                      flow_section=f"flow.{a.flow}", seq_len=a.seq_len, active_params_b=a.active_params_b)
  for st in plan.stages:
    for sp in st.sources:
      out = Path(a.data_root) / "flows" / a.flow / st.stage_id / sp.id / "train"
      if sp.hf is not None:
        src = create_source("hf", dataset=sp.hf.dataset, subset=sp.hf.subset, split=sp.hf.split,
                            text_field=sp.hf.text_field, data_files=sp.hf.data_files)
      elif a.local_root:
        src = create_source("jsonl", paths=str(Path(a.local_root) / sp.id))
      else:
        print(f"skip {sp.id}: no hf_dataset in the mixture and no --local-root", file=sys.stderr)
        continue
      need = sp.quota_sequences * (a.seq_len + 1)
      m = PrepPipeline(src, PrepConfig(str(out), sp.id, tokenizer=a.tokenizer, num_shards=a.num_shards, max_tokens=need)).run()
      print(f"{st.stage_id}/{sp.id}: {m.total_tokens:,} tokens (quota {need:,})")
  return 0


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
  from .dedup import dedup_exact, stream_near_dedup
  from .sources import create_source
  src = create_source("jsonl", paths=a.input, text_field=a.text_field)
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


def cmd_flow(a) -> int:
  from .flow import load_spec, run_flow
  run_flow(load_spec(Path(a.spec)))
  return 0


def cmd_needs_model(a) -> int:
  print(f"'{a.command}' runs the HYDRA grading / rephrasing stack, which needs gpt-oss checkpoint files "
        f"(--checkpoint) that are not part of this repository; see nmoe_b200/data/hydra.py", file=sys.stderr)
  return 2


def cmd_needs_network(a) -> int:
  print(f"'{a.command}' downloads from S3 / arXiv and needs network access and boto3", file=sys.stderr)
  return 2


def build_parser() -> argparse.ArgumentParser:
  ap = argparse.ArgumentParser(prog="nmoe_b200.data.cli")
  sub = ap.add_subparsers(dest="command", required=True)
  p = sub.add_parser("prep"); p.set_defaults(fn=cmd_prep)
  p.add_argument("--source", default="jsonl"); p.add_argument("--input"); p.add_argument("--dataset"); p.add_argument("--subset")
  p.add_argument("--split", default="train"); p.add_argument("--text-field", default="text"); p.add_argument("--output", required=True)
  p.add_argument("--name", required=True); p.add_argument("--version", default="v1"); p.add_argument("--tokenizer", default="o200k_harmony")
  p.add_argument("--num-shards", type=int, default=8); p.add_argument("--workers", type=int, default=1)
  p.add_argument("--max-documents", type=int); p.add_argument("--max-tokens", type=int)
  p = sub.add_parser("prep-mixture"); p.set_defaults(fn=cmd_prep_mixture)
  p.add_argument("--mixture", required=True); p.add_argument("--flow-profiles", required=True); p.add_argument("--flow", required=True)
  p.add_argument("--data-root", default="/data"); p.add_argument("--seq-len", type=int, default=4096); p.add_argument("--local-root")
  p.add_argument("--active-params-b", type=float); p.add_argument("--tokenizer", default="o200k_harmony"); p.add_argument("--num-shards", type=int, default=8)
  p = sub.add_parser("verify"); p.set_defaults(fn=cmd_verify); p.add_argument("path"); p.add_argument("--fast", action="store_true")
  p = sub.add_parser("info"); p.set_defaults(fn=cmd_info); p.add_argument("path")
  p = sub.add_parser("regenerate-index"); p.set_defaults(fn=cmd_regenerate_index); p.add_argument("path"); p.add_argument("--eos-token-id", type=int, default=199999)
  p = sub.add_parser("dedup"); p.set_defaults(fn=cmd_dedup); p.add_argument("--input", required=True); p.add_argument("--output", required=True)
  p.add_argument("--text-field", default="text"); p.add_argument("--near", action="store_true"); p.add_argument("--threshold", type=float, default=0.8)
  p = sub.add_parser("cluster"); p.set_defaults(fn=cmd_cluster); p.add_argument("--embeddings", required=True); p.add_argument("--k", type=int, default=64); p.add_argument("--output")
  p = sub.add_parser("inspect"); p.set_defaults(fn=cmd_inspect); p.add_argument("shard"); p.add_argument("--doc", type=int)
  p.add_argument("--start", type=int); p.add_argument("--length", type=int, default=64); p.add_argument("--tokenizer")
  p = sub.add_parser("merge-manifests"); p.set_defaults(fn=cmd_merge_manifests); p.add_argument("parts", nargs="+"); p.add_argument("--output", required=True)
  p = sub.add_parser("flow"); p.set_defaults(fn=cmd_flow); p.add_argument("spec")
  for name in ("rephrase", "hydra-oracle-label", "hydra-calibrate", "hydra-grade", "hydra-train"):
    p = sub.add_parser(name); p.set_defaults(fn=cmd_needs_model); p.add_argument("rest", nargs="*")
  for name in ("arxiv-download", "arxiv-prep"):
    p = sub.add_parser(name); p.set_defaults(fn=cmd_needs_network); p.add_argument("rest", nargs="*")
  return ap


def main(argv=None) -> int:
  a = build_parser().parse_args(argv)
  try:
    return a.fn(a)
  except PipelineError as e:
    e.exit()


if __name__ == "__main__":
  sys.exit(main())
