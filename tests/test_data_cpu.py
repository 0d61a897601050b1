"""Shard building, index, manifest verification, dedup, flow -- CPU only, `bytes` tokenizer."""
import json

import numpy as np
import torch
import pytest

from nmoe_b200.data import cli, dedup, diversity, flow as flow_mod, index, inspect as insp, sinks
from nmoe_b200.data.errors import ShardChecksumError, SourceNotFoundError
from nmoe_b200.data.sources import Document, JSONLSource


def _write_jsonl(path, n=50):
  with open(path, "w") as f:
    for i in range(n):
      f.write(json.dumps({"id": f"d{i}", "text": f"document number {i} " + "lorem ipsum " * (i % 7 + 1)}) + "\n")


def test_prep_verify_inspect_roundtrip(tmp_path):
  _write_jsonl(tmp_path / "a.jsonl")
  out = tmp_path / "shards"
  assert cli.main(["prep", "--source", "jsonl", "--input", str(tmp_path / "a.jsonl"), "--output", str(out), "--name", "toy",
                   "--tokenizer", "bytes", "--num-shards", "3"]) == 0
  m = sinks.verify_manifest(out)
  assert m.total_documents == 50 and m.num_shards == 3 and m.eos_token_id == 256
  s0 = out / m.shards[0].path
  rd = index.IndexReader(index.index_path_for_shard(s0))
  toks = np.load(s0)
  for s, e in rd.iter_documents():
    assert toks[e - 1] == 256 and (toks[s:e - 1] < 256).all()
  doc = insp.document(s0, 0, "bytes")
  assert doc["text"].startswith("document number")
  # deterministic placement + index regeneration gives the same boundaries
  before = rd.to_array()
  index.index_path_for_shard(s0).unlink()
  index.regenerate_index_from_shard(s0, 256)
  assert (index.IndexReader(index.index_path_for_shard(s0)).to_array() == before).all()
  # corruption is detected
  arr = np.load(s0); arr[0] ^= 1; np.save(s0, arr)
  with pytest.raises(ShardChecksumError):
    sinks.verify_manifest(out)


def test_parallel_prep_matches_serial(tmp_path):
  from nmoe_b200.data.prep import ParallelPrepPipeline, PrepConfig, PrepPipeline
  _write_jsonl(tmp_path / "a.jsonl", 80)
  mk = lambda: JSONLSource(str(tmp_path / "a.jsonl"))
  a = PrepPipeline(mk(), PrepConfig(str(tmp_path / "s"), "toy", tokenizer="bytes", num_shards=4, log_every=0)).run()
  b = ParallelPrepPipeline(mk, PrepConfig(str(tmp_path / "p"), "toy", tokenizer="bytes", num_shards=4, log_every=0), workers=2).run()
  assert [s.checksum for s in a.shards] == [s.checksum for s in b.shards]


def test_sources_errors_and_sharding(tmp_path):
  with pytest.raises(SourceNotFoundError):
    JSONLSource(str(tmp_path / "missing"))
  _write_jsonl(tmp_path / "a.jsonl", 10)
  src = JSONLSource(str(tmp_path / "a.jsonl"))
  ids = [d.doc_id for d in src]
  parts = [[d.doc_id for d in src.shard(i, 3)] for i in range(3)]
  assert sorted(sum(parts, [])) == sorted(ids) and parts[0] == ids[0::3]


def test_dedup_exact_and_near():
  docs = [Document("a", "the quick brown fox jumps over the lazy dog " * 5),
          Document("b", "The quick brown fox jumps over the lazy dog " * 5),
          Document("c", "the quick brown fox jumps over the lazy dog " * 5 + "again"),
          Document("d", "completely different content about tensor cores and memory bandwidth " * 4)]
  assert [d.doc_id for d in dedup.dedup_exact(docs)] == ["a", "c", "d"]
  kept = [d.doc_id for d in dedup.stream_near_dedup(docs, threshold=0.7, num_perm=32, bands=8)]
  assert kept == ["a", "d"]


def test_dedup_inside_a_document(tmp_path):
  page = "Home | About | Contact\nFirst paragraph of the article.\n}\nHome  |  about | contact\n\nSecond one.\n}\nFirst paragraph of the article."
  assert dedup.dedup_within(page, "lines") == "Home | About | Contact\nFirst paragraph of the article.\n}\n\nSecond one.\n}"
  paras = "Subscribe to our newsletter today!\n\nReal content here, long enough.\n \nSubscribe to our  newsletter today!\n\nshort\n\nshort"
  assert dedup.dedup_within(paras, "paragraphs") == "Subscribe to our newsletter today!\n\nReal content here, long enough.\n\nshort\n\nshort"
  with pytest.raises(ValueError):
    dedup.dedup_within(page, "words")
  # through the command: two pages that differ only in a repeated banner become exact duplicates
  from nmoe_b200.data.cli import main
  banner = "Accept all cookies to continue"
  rows = [{"id": "p1", "text": f"{banner}\nThe body of the page, identical.\n{banner}"},
          {"id": "p2", "text": f"{banner}\nThe body of the page, identical."},
          {"id": "p3", "text": "Another page entirely."}]
  (tmp_path / "in.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
  assert main(["dedup", "--input", str(tmp_path / "in.jsonl"), "--output", str(tmp_path / "plain.jsonl")]) == 0
  assert main(["dedup", "--input", str(tmp_path / "in.jsonl"), "--output", str(tmp_path / "within.jsonl"), "--within", "lines"]) == 0
  assert len(open(tmp_path / "plain.jsonl").readlines()) == 3
  assert [json.loads(l)["id"] for l in open(tmp_path / "within.jsonl")] == ["p1", "p3"]


def test_cluster_coverage():
  rng = np.random.default_rng(0)
  x = np.concatenate([rng.normal(c, 0.1, size=(100, 8)) for c in (-3, 0, 3)])
  _, assign = diversity.cluster_embeddings(x, 3)
  m = diversity.coverage_metrics(assign, 3)
  assert m["empty_clusters"] == 0 and m["max_share"] < 0.5


def test_flow_env_overrides_and_guard(tmp_path):
  _write_jsonl(tmp_path / "raw.jsonl", 30)
  spec_path = tmp_path / "flow.toml"
  spec_path.write_text(f'[source]\nkind = "jsonl"\npaths = "{tmp_path / "raw.jsonl"}"\n[prep]\noutput_dir = "{tmp_path / "out"}"\n'
                       'dataset = "f"\ntokenizer = "bytes"\nnum_shards = 2\n[grade]\nenabled = true\nthreshold = 0.5\n')
  spec = flow_mod.load_spec(spec_path, env={"NMOE_DATAFLOW__GRADE__THRESHOLD": "0.9"})
  assert spec.grade["threshold"] == 0.9
  m = flow_mod.run_flow(spec, grader=lambda texts: [1.0 if "1" in t else 0.0 for t in texts], print_fn=lambda *a: None)
  assert 0 < m.total_documents < 30
  other = flow_mod.load_spec(spec_path, env={})
  with pytest.raises(RuntimeError, match="different flow"):
    flow_mod.run_flow(other, grader=lambda t: [1.0] * len(t), print_fn=lambda *a: None)


def test_arxiv_prep_and_stack_v2_materialize(tmp_path):
  import gzip, io, json, tarfile
  from nmoe_b200.data.arxiv import latex_to_text
  from nmoe_b200.data.cli import main
  tex = r"""\documentclass{article}
\usepackage{amsmath} % comment to drop
\begin{document}
\title{On \emph{Widgets}}
\begin{abstract} We study widgets. \end{abstract}
\section{Introduction}
Widgets \cite{foo} satisfy $a^2 + b^2 = c^2$ and more~\ref{x}.
\input{body}
\begin{figure} \includegraphics{fig.png} \caption{gone} \end{figure}
\begin{equation} E = mc^2 \label{e} \end{equation}
\begin{thebibliography}{9} \bibitem{foo} Foo. \end{thebibliography}
\end{document}"""
  body = r"\subsection{Details} The \textbf{main} result holds for 100\% of cases."
  src = tmp_path / "src"; src.mkdir()
  buf = io.BytesIO()
  with tarfile.open(fileobj=buf, mode="w:gz") as tf:
    for name, data in (("main.tex", tex), ("body.tex", body)):
      ti = tarfile.TarInfo(name); b = data.encode(); ti.size = len(b); tf.addfile(ti, io.BytesIO(b))
  (src / "2401.00001.tar.gz").write_bytes(buf.getvalue())
  out = tmp_path / "arxiv.jsonl"
  assert main(["arxiv-prep", "--input", str(src), "--output", str(out), "--min-chars", "10"]) == 0
  row = json.loads(out.read_text().splitlines()[0])
  t = row["text"]
  assert row["id"] == "2401.00001" and "Introduction" in t and "Details" in t and "main result holds for 100% of cases" in t
  assert "$a^2 + b^2 = c^2$" in t and "$$E = mc^2$$" in t.replace(" $$", "$$").replace("$$ ", "$$")
  assert "gone" not in t and "Foo." not in t and "\\" not in t.replace("$a^2", "").split("$$")[0] and "comment" not in t
  assert latex_to_text(r"\begin{document}x \textit{\textbf{y}} z\end{document}") == "x y z"
  blobs = tmp_path / "blobs"; (blobs / "ab").mkdir(parents=True)
  (blobs / "ab" / "abcd1234.gz").write_bytes(gzip.compress("def f():\n  return 1\n".encode()))
  (blobs / "ffee").write_bytes("fn main() {}".encode("utf-16"))
  table = tmp_path / "ids.jsonl"
  table.write_text("\n".join(json.dumps(r) for r in (
    {"blob_id": "abcd1234", "src_encoding": "utf-8", "language": "Python", "path": "a.py"},
    {"blob_id": "ffee", "src_encoding": "utf-16", "language": "Rust", "path": "m.rs"},
    {"blob_id": "missing", "src_encoding": "utf-8", "language": "Python", "path": "x.py"})))
  out2 = tmp_path / "code.jsonl"
  assert main(["stack-v2-materialize", "--table", str(table), "--blobs", str(blobs), "--output", str(out2), "--languages", "Python,Rust"]) == 0
  rows = [json.loads(l) for l in out2.read_text().splitlines()]
  assert [r["id"] for r in rows] == ["abcd1234", "ffee"] and rows[0]["text"].startswith("def f()") and rows[1]["text"] == "fn main() {}"


def test_ar5iv_html_to_text_and_mathml():
  from nmoe_b200.data.arxiv_html import (extract_html_metadata, html_to_text, load_metadata_snapshot, mathml_to_latex,
                                          parse_atom_feed, parse_html)
  html = """<html><head><link rel="canonical" href="https://arxiv.org/abs/2301.12345v2"></head><body>
  <nav>menu</nav><article class="ltx_document">
  <h1 class="ltx_title ltx_title_document">Sparse Things</h1>
  <div class="ltx_authors"><span class="ltx_personname">Ada L.</span><span class="ltx_personname">Bob K.</span></div>
  <div class="ltx_abstract"><h6>Abstract</h6><p>We study <math alttext="x^{2}"><msup><mi>x</mi><mn>2</mn></msup></math>.</p></div>
  <section class="ltx_section"><h2>1 Intro</h2><p>Energy is
   <math display="block"><mrow><mi>E</mi><mo>=</mo><mfrac><mn>1</mn><mn>2</mn></mfrac><mi>m</mi><msup><mi>v</mi><mn>2</mn></msup>
   <mo>+</mo><munderover><mo>&#x2211;</mo><mrow><mi>i</mi><mo>=</mo><mn>1</mn></mrow><mi>n</mi></munderover><msub><mi>&#x3b1;</mi><mi>i</mi></msub></mrow></math>
   as shown<cite>[3]</cite>.</p>
   <section class="ltx_subsection"><h3>1.1 Detail</h3><p>Nested text.</p></section></section>
  <section class="ltx_bibliography"><h2>References</h2><p>[3] Someone.</p></section>
  </article><footer>foot</footer></body></html>"""
  text = html_to_text(html)
  assert text.startswith("Sparse Things")
  assert "We study $x^{2}$." in text and "Abstract" not in text.split("\n")[2]
  assert r"$$E=\frac{1}{2}mv^2+\sum_{i=1}^n\alpha_i$$" in text
  assert "1 Intro" in text and "1.1 Detail" in text and text.count("Nested text.") == 1
  assert "References" not in text and "menu" not in text and "foot" not in text and "[3]" not in text
  assert "Abstract" not in html_to_text(html, include_abstract=False).replace("Sparse", "")
  meta = extract_html_metadata(html)
  assert meta.title == "Sparse Things" and meta.authors == ["Ada L.", "Bob K."] and meta.arxiv_id == "2301.12345"
  root = parse_html("<math><msqrt><mi>x</mi></msqrt><mo>&#x2264;</mo><mover><mi>y</mi><mo>^</mo></mover>"
                    "<mfenced open='[' close=']'><mi>a</mi><mi>b</mi></mfenced></math>")
  assert mathml_to_latex(root.find("math")) == r"\sqrt{x}\leq \hat{y}\left[a,b\right]"
  atom = """<feed xmlns="http://www.w3.org/2005/Atom" xmlns:arxiv="http://arxiv.org/schemas/atom">
  <entry><id>http://arxiv.org/abs/2301.12345v2</id><title>Sparse
   Things</title><summary> An abstract. </summary><author><name>Ada L.</name></author>
   <published>2023-01-30T00:00:00Z</published><updated>2023-02-01T00:00:00Z</updated>
   <arxiv:primary_category term="cs.LG"/><category term="cs.LG"/><category term="stat.ML"/>
   <arxiv:doi>10.1/x</arxiv:doi></entry></feed>"""
  m = parse_atom_feed(atom)["2301.12345"]
  assert (m.title, m.primary_category, m.categories, m.doi, m.authors) == ("Sparse Things", "cs.LG", ["cs.LG", "stat.ML"], "10.1/x", ["Ada L."])


def test_metadata_snapshot_filter(tmp_path):
  from nmoe_b200.data.arxiv_html import load_metadata_snapshot
  p = tmp_path / "snap.jsonl"
  rows = [{"id": "2301.1", "title": "A\n b", "authors_parsed": [["Lovelace", "Ada", ""]], "categories": "cs.LG stat.ML",
           "abstract": " x ", "versions": [{"created": "Mon"}, {"created": "Tue"}]},
          {"id": "2301.2", "title": "B", "authors": "C. D. and E. F.", "categories": "math.AG", "abstract": "y"}]
  p.write_text("\n".join(json.dumps(r) for r in rows))
  got = list(load_metadata_snapshot(str(p), categories=["cs."]))
  assert [g.arxiv_id for g in got] == ["2301.1"] and got[0].title == "A b" and got[0].authors == ["Ada Lovelace"]
  assert got[0].submitted == "Mon" and got[0].updated == "Tue"
  assert [g.authors for g in load_metadata_snapshot(str(p), categories=["math"])] == [["C. D.", "E. F."]]


def test_prep_mixture_profiles_workers_limit(tmp_path, capsys):
  """A mixture file that names its own stage tables ([profiles]) resolves against the shared flow profiles; two
  workers split the sources; --limit bounds the documents and the sample-id digest repeats for the same seed."""
  from nmoe_b200.data.cli import main
  from nmoe_b200.data.mixture import resolve_plan
  mix = tmp_path / "mix.toml"
  mix.write_text('[profiles]\npretrain_profile = "mine"\n[mixtures.mine]\ntotal_tokens_b = 0.001\n'
                 'sources = [{id = "a", tokens_b = 3.0}, {id = "b", tokens_b = 1.0}]\n')
  flows = tmp_path / "flows.toml"
  flows.write_text('[flow.dev]\nmode = "dev"\nstages = ["pretrain", "mid"]\ntokens_b = 0.00002\n'
                   '[flow.dev.mixture]\npretrain = "pretrain_main"\nmid = "mid_quality"\n')
  plan = resolve_plan(mixture_toml=mix, flow_profiles_toml=flows, flow_section="flow.dev", seq_len=64)
  assert [s.stage_id for s in plan.stages] == ["pretrain"] and [sp.id for sp in plan.stages[0].sources] == ["a", "b"]
  q = [sp.quota_sequences for sp in plan.stages[0].sources]
  assert q[0] == 3 * q[1] or abs(q[0] - 3 * q[1]) <= 3
  for name in ("a", "b"):
    d = tmp_path / "raw" / name
    d.mkdir(parents=True)
    (d / "x.jsonl").write_text("".join(json.dumps({"id": f"{name}{i}", "text": f"{name} document number {i} " * 8}) + "\n" for i in range(40)))
  common = ["prep-mixture", "--config", str(mix), "--flow-profiles", str(flows), "--seq-len", "64", "--tokenizer", "bytes",
            "--num-shards", "2", "--local-root", str(tmp_path / "raw"), "--seed", "7", "--limit", "10"]
  outs = []
  for w in (0, 1):
    assert main(common + ["--output", str(tmp_path / "out"), "--worker-index", str(w), "--num-workers", "2"]) == 0
    outs.append(capsys.readouterr().out)
  assert "pretrain/a/train" in outs[0] and "pretrain/b/train" not in outs[0] and "pretrain/b/train" in outs[1]
  assert (tmp_path / "out/pretrain/a/train/manifest.json").exists() and (tmp_path / "out/pretrain/b/train/manifest.json").exists()
  # same seed, same documents -> same digest; an existing manifest is left alone without --force
  assert main(common + ["--output", str(tmp_path / "out2"), "--stage", "pretrain"]) == 0
  again = capsys.readouterr().out
  dig = lambda text, key: [l.split("sha256 ")[1] for l in text.splitlines() if key in l and "sha256" in l][0]
  assert dig(again, "pretrain/a/train") == dig(outs[0], "pretrain/a/train")
  assert main(common + ["--output", str(tmp_path / "out2")]) == 0
  assert "manifest.json exists" in capsys.readouterr().out
  assert main(common + ["--output", str(tmp_path / "out3"), "--dry-run"]) == 0
  assert "would build pretrain/a/train" in capsys.readouterr().out and not (tmp_path / "out3").exists()


def test_flow_writes_every_rephrased_version(tmp_path):
  """keep_original + a rephraser that answers a list per document: the shards hold the original and every version."""
  raw = tmp_path / "raw.jsonl"
  raw.write_text("".join(json.dumps({"id": f"d{i}", "text": f"text {i} " * 6}) + "\n" for i in range(5)))
  spec = tmp_path / "flow.toml"
  spec.write_text(f'[source]\nkind = "jsonl"\npaths = "{raw}"\n[prep]\noutput_dir = "{tmp_path / "out"}"\ndataset = "f"\n'
                  'tokenizer = "bytes"\nnum_shards = 1\n[rephrase]\nenabled = true\nkeep_original = true\nnum_versions = 3\n')
  s = flow_mod.load_spec(spec, env={})
  m = flow_mod.run_flow(s, rephraser=lambda texts: [[t.upper(), t + "again", ""] for t in texts], env={}, print_fn=lambda *_: None)
  assert m.total_documents == 5 * 3                # original + two non-empty versions
  k2 = flow_mod.load_spec("configs/dataflow/dataprep_k2.toml", env={})
  assert k2.rephrase["num_versions"] == 10 and k2.grade["enabled"] and k2.source["kind"] == "hf"


def test_flow_profile_presets_expand_to_prep_mixture(tmp_path, capsys):
  """`flow --config flow_profiles.toml --profile NAME` runs the prep-mixture call its [profiles.NAME] table describes."""
  from nmoe_b200.data.cli import main
  base = ["flow", "--config", "configs/flow_profiles.toml", "--dry-run", "--data-root", str(tmp_path)]
  assert main([*base, "--profile", "hydra_fixture"]) == 0
  out = capsys.readouterr().out
  assert "plan hydra_fixture:dev" in out and "seed 123" in out and str(tmp_path / "flows" / "hydra_fixture") in out
  assert main([*base, "--profile", "mini", "--num-workers", "2", "--worker-index", "1"]) == 0
  assert "worker 1/2" in capsys.readouterr().out
  assert main([*base, "--profile", "nope"]) == 1 and "hydra_fixture, mini" in capsys.readouterr().err
  assert main(["flow"]) == 2


def test_staged_flow_keeps_stage_files_and_continues_after_an_interruption(tmp_path):
  """Each stage writes its own file; a run cut in the grading or rephrasing stage computes only what is missing when
  it is started again, and ends with the same shards as the streaming flow."""
  from nmoe_b200.data.staged import StagedFlow, run_flow_staged
  raw = tmp_path / "raw.jsonl"
  raw.write_text("".join(json.dumps({"id": f"d{i}", "text": f"text {i} " * 6, "lang": "en"}) + "\n" for i in range(20)))
  def spec_for(out):
    sp = tmp_path / f"{out}.toml"
    sp.write_text(f'[source]\nkind = "jsonl"\npaths = "{raw}"\n[prep]\noutput_dir = "{tmp_path / out}"\ndataset = "f"\n'
                  'tokenizer = "bytes"\nnum_shards = 2\n[grade]\nenabled = true\nthreshold = 0.5\nbatch_size = 4\n'
                  '[rephrase]\nenabled = true\nkeep_original = true\nbatch_size = 3\n')
    return flow_mod.load_spec(sp, env={})
  score_of = lambda t: float(int(t.split()[1]) % 2)          # odd documents are kept
  calls = {"grade": 0, "re": 0}
  class Cut(Exception):
    pass
  def grader(texts, fail_after=None):
    if fail_after is not None and calls["grade"] >= fail_after:
      raise Cut()
    calls["grade"] += len(texts)
    return [score_of(t) for t in texts]
  def rephraser(texts, fail_after=None):
    if fail_after is not None and calls["re"] >= fail_after:
      raise Cut()
    calls["re"] += len(texts)
    return [[t.upper(), ""] for t in texts]
  quiet = dict(env={}, print_fn=lambda *_: None)
  s = spec_for("staged")
  with pytest.raises(Cut):
    run_flow_staged(s, grader=lambda t: grader(t, fail_after=8), rephraser=rephraser, **quiet)
  st = tmp_path / "staged" / "stages"
  assert calls["grade"] == 8 and len((st / "scores.jsonl").read_text().splitlines()) == 8
  with open(st / "scores.jsonl", "a") as f:
    f.write('{"id": "d8", "sco')                             # the write the crash cut short
  with pytest.raises(Cut):
    run_flow_staged(s, grader=grader, rephraser=lambda t: rephraser(t, fail_after=3), **quiet)
  assert calls["grade"] == 20                                # 12 more, not 20 more
  assert json.loads((st / "state.json").read_text())["done"] == {"raw": 20, "scores": 20, "kept": 10}
  m = run_flow_staged(s, grader=lambda t: 1 / 0, rephraser=rephraser, **quiet)      # grading is not run again
  assert calls["re"] == 10 and m.total_documents == 20       # 10 kept originals + 10 rephrased versions
  rows = [json.loads(l) for l in open(st / "rephrased.jsonl")]
  assert len(rows) == 20 and sum(1 for r in rows if r.get("rephrased")) == 10 and all(r["lang"] == "en" for r in rows)
  assert {r["id"] for r in rows if r.get("rephrased")} == {f"d{i}#v0" for i in range(1, 20, 2)}
  assert all(r["score"] == 1.0 for r in map(json.loads, open(st / "kept.jsonl")))
  again = StagedFlow(s, grader=None, rephraser=None, **quiet)                          # everything is done: no model needed
  assert all(again.done(x) for x in ("raw", "scores", "kept", "rephrased", "shards"))
  assert again.run().total_tokens == m.total_tokens
  # same tokens as the streaming flow
  calls.update(grade=0, re=0)
  m2 = flow_mod.run_flow(spec_for("stream"), grader=grader, rephraser=rephraser, **quiet)
  assert (m2.total_documents, m2.total_tokens) == (m.total_documents, m.total_tokens)
  sinks.verify_manifest(tmp_path / "staged")
  # a different specification in the same directory is refused
  sp = tmp_path / "staged.toml"
  sp.write_text(sp.read_text().replace("threshold = 0.5", "threshold = 0.7"))
  with pytest.raises(RuntimeError, match="different flow specification"):
    StagedFlow(flow_mod.load_spec(sp, env={}), **quiet)


def test_stage_graph_runner_builds_the_same_shards_as_the_serial_pipeline(tmp_path):
  """The Beam-shaped stage graph (tokenise -> group by shard -> write), run by the built-in runner, must produce a
  dataset that verifies and holds the same tokens per shard as the serial pipeline."""
  from nmoe_b200.data.prep import PrepConfig, PrepPipeline, run_beam_pipeline
  _write_jsonl(tmp_path / "raw.jsonl", 60)
  mk = lambda: JSONLSource(str(tmp_path / "raw.jsonl"))
  a = PrepPipeline(mk(), PrepConfig(str(tmp_path / "s"), "toy", tokenizer="bytes", num_shards=4, log_every=0)).run()
  b = run_beam_pipeline(mk(), PrepConfig(str(tmp_path / "b"), "toy", tokenizer="bytes", num_shards=4, log_every=0), runner="local")
  assert (a.total_tokens, a.total_documents, a.num_shards) == (b.total_tokens, b.total_documents, b.num_shards)
  sinks.verify_manifest(tmp_path / "b")
  for sa, sb in zip(sorted((tmp_path / "s").rglob("*.npy")), sorted((tmp_path / "b").rglob("*.npy"))):
    ta, tb = np.load(sa), np.load(sb)
    assert ta.size == tb.size and sorted(ta.tolist()) == sorted(tb.tolist())
  with pytest.raises(RuntimeError, match="apache_beam"):
    run_beam_pipeline(mk(), PrepConfig(str(tmp_path / "c"), "toy", tokenizer="bytes", num_shards=2), runner="beam")


def _bulk_tar(path, papers):
  """An arXiv-style monthly tar: <yymm>/<id>.gz members (gzipped tar of the submission, or a gzipped TeX file)."""
  import gzip, io, tarfile
  with tarfile.open(path, "w") as tf:
    for pid, files in papers.items():
      if isinstance(files, dict):
        inner = io.BytesIO()
        with tarfile.open(fileobj=inner, mode="w") as it:
          for name, text in files.items():
            b = text.encode()
            ti = tarfile.TarInfo(name); ti.size = len(b)
            it.addfile(ti, io.BytesIO(b))
        blob = gzip.compress(inner.getvalue())
        name = f"2301/{pid}.gz"
      elif files is None:
        blob, name = b"%PDF-1.4", f"2301/{pid}.pdf"
      else:
        blob, name = gzip.compress(files.encode()), f"2301/{pid}.gz"
      ti = tarfile.TarInfo(name); ti.size = len(blob)
      tf.addfile(ti, io.BytesIO(blob))


def test_arxiv_bulk_download_over_http_resumes_verifies_and_converts(tmp_path):
  """Manifest -> selection -> fetch from a local HTTP server (127.0.0.1) with resume of a partial file, md5 check that
  rejects a corrupted tar, skip of complete files; then papers come out of the bulk tar as text."""
  import functools, http.server, threading
  from nmoe_b200.data import arxiv_download as AD
  body = "Deep networks generalise. " * 40
  doc = "\\documentclass{article}\\begin{document}\\section{Intro}" + body + "\\input{sec}\\end{document}"
  srv_root = tmp_path / "srv" / "src"
  srv_root.mkdir(parents=True)
  _bulk_tar(srv_root / "arXiv_src_2301_001.tar", {"2301.00001": {"main.tex": doc, "sec.tex": "Second part. " * 30},
                                                  "2301.00002": doc.replace("\\input{sec}", ""), "2301.00003": None})
  _bulk_tar(srv_root / "arXiv_src_2302_001.tar", {"2302.00001": doc.replace("\\input{sec}", "")})
  _bulk_tar(srv_root / "arXiv_src_9912_001.tar", {"9912.00001": doc.replace("\\input{sec}", "")})
  ents = []
  for f, yymm in (("arXiv_src_2302_001.tar", "2302"), ("arXiv_src_9912_001.tar", "9912"), ("arXiv_src_2301_001.tar", "2301")):
    p = srv_root / f
    ents.append(f"<file><filename>src/{f}</filename><md5sum>{AD.md5_of(p)}</md5sum><num_items>3</num_items>"
                f"<seq_num>1</seq_num><size>{p.stat().st_size}</size><yymm>{yymm}</yymm></file>")
  manifest = tmp_path / "manifest.xml"
  manifest.write_text("<arXivSRC>" + "".join(ents) + "</arXivSRC>")
  entries = AD.parse_manifest(manifest)
  assert [e.yymm for e in entries] == ["9912", "2301", "2302"]           # chronological: 1999 before 2023
  assert [e.yymm for e in AD.select(entries, start="2301")] == ["2301", "2302"]
  assert [e.yymm for e in AD.select(entries, end="2301", max_files=1)] == ["9912"]
  assert AD.estimate_cost(entries)["files"] == 3

  handler = functools.partial(http.server.SimpleHTTPRequestHandler, directory=str(tmp_path / "srv"))
  class Quiet(http.server.ThreadingHTTPServer):
    pass
  handler.log_message = lambda *a, **k: None
  httpd = Quiet(("127.0.0.1", 0), handler)
  th = threading.Thread(target=httpd.serve_forever, daemon=True)
  th.start()
  try:
    out = tmp_path / "dl"
    fetcher = AD.HttpFetcher(f"http://127.0.0.1:{httpd.server_address[1]}", retries=1, backoff_s=0.01)
    picked = AD.select(entries, start="2301")
    rep = AD.download(picked, out, fetcher, workers=2, print_fn=lambda *_: None)
    assert rep.ok and sorted(rep.fetched) == ["arXiv_src_2301_001.tar", "arXiv_src_2302_001.tar"]
    rep2 = AD.download(picked, out, fetcher, print_fn=lambda *_: None)
    assert rep2.fetched == [] and len(rep2.skipped) == 2                 # complete files are left alone
    # a corrupted local copy is re-fetched; a manifest with a wrong checksum is reported and leaves no file behind
    (out / "arXiv_src_2302_001.tar").write_bytes(b"garbage")
    rep3 = AD.download(picked, out, fetcher, print_fn=lambda *_: None)
    assert rep3.fetched == ["arXiv_src_2302_001.tar"]
    bad = [AD.TarEntry(picked[0].key, picked[0].size, "0" * 32, picked[0].yymm, 1, 3)]
    rep4 = AD.download(bad, tmp_path / "dl2", fetcher, print_fn=lambda *_: None)
    assert not rep4.ok and not list((tmp_path / "dl2").glob("*.tar*"))
    missing = [AD.TarEntry("src/nope.tar", 1, "", "2303", 1, 0)]
    assert "HTTP 404" in AD.download(missing, tmp_path / "dl3", fetcher, print_fn=lambda *_: None).failed["nope.tar"]
    # the command-line face, through a directory fetcher
    assert cli.main(["arxiv-download", "--output", str(tmp_path / "dl4"), "--manifest", str(manifest), "--fetch", "file",
                     "--root", str(tmp_path / "srv"), "--start", "2301", "--end", "2301"]) == 0
    assert [p.name for p in (tmp_path / "dl4").glob("*.tar")] == ["arXiv_src_2301_001.tar"]
  finally:
    httpd.shutdown()
  papers = list(AD.iter_bulk_tar(out / "arXiv_src_2301_001.tar"))
  assert [p["id"] for p in papers] == ["2301.00001", "2301.00002"]      # the PDF-only member has no sources
  assert set(papers[0]["files"]) == {"main.tex", "sec.tex"}
  assert cli.main(["arxiv-prep", "--bulk", "--input", str(out), "--output", str(tmp_path / "papers.jsonl"), "--min-chars", "100"]) == 0
  rows = [json.loads(l) for l in (tmp_path / "papers.jsonl").read_text().splitlines()]
  assert [r["id"] for r in rows] == ["2301.00001", "2301.00002", "2302.00001"]
  assert "Second part." in rows[0]["text"] and "documentclass" not in rows[0]["text"]
  # the S3 route builds the requester-pays command and reports the client's error text
  calls = []
  class R:
    returncode, stderr = 1, "fatal error: Unable to locate credentials"
  s3 = AD.S3CliFetcher(profile="lab", run=lambda cmd, **kw: (calls.append(cmd), R())[1])
  with pytest.raises(AD.FetchError, match="credentials"):
    s3.fetch("src/arXiv_src_2301_001.tar", tmp_path / "x.tar")
  assert calls[0][:4] == ["aws", "s3", "cp", "s3://arxiv/src/arXiv_src_2301_001.tar"] and "requester" in calls[0] and "lab" in calls[0]


def test_http_fetcher_continues_a_transfer_that_was_cut(tmp_path):
  """First response: full Content-Length but only half the body, then the connection drops.  The retry must ask for
  the rest with a Range header and append it."""
  import http.server, threading
  from nmoe_b200.data.arxiv_download import HttpFetcher
  payload = bytes(range(256)) * 400
  seen = []

  class H(http.server.BaseHTTPRequestHandler):
    def log_message(self, *a):
      pass
    def do_GET(self):
      rng = self.headers.get("Range")
      seen.append(rng)
      if rng is None:
        self.send_response(200)
        self.send_header("Content-Length", str(len(payload)))
        self.end_headers()
        self.wfile.write(payload[:len(payload) // 2])
        self.wfile.flush()
        self.connection.close()
        return
      start = int(rng.split("=")[1].rstrip("-"))
      self.send_response(206)
      self.send_header("Content-Length", str(len(payload) - start))
      self.send_header("Content-Range", f"bytes {start}-{len(payload) - 1}/{len(payload)}")
      self.end_headers()
      self.wfile.write(payload[start:])

  httpd = http.server.ThreadingHTTPServer(("127.0.0.1", 0), H)
  threading.Thread(target=httpd.serve_forever, daemon=True).start()
  try:
    dest = tmp_path / "f.bin"
    HttpFetcher(f"http://127.0.0.1:{httpd.server_address[1]}", retries=2, backoff_s=0.01).fetch("x/f.bin", dest)
  finally:
    httpd.shutdown()
  assert dest.read_bytes() == payload
  assert seen[0] is None and seen[1] == f"bytes={len(payload) // 2}-"


def _ar5iv_page(pid, body):
  return (f'<html><head><link rel="canonical" href="https://arxiv.org/abs/{pid}"></head><body><article class="ltx_document">'
          f'<h1 class="ltx_title ltx_title_document">Paper {pid}</h1><div class="ltx_authors"><span class="ltx_personname">A. Uthor</span></div>'
          f'<section class="ltx_section"><h2>1 Intro</h2><p>{body} <math alttext="x^{{2}}"><msup><mi>x</mi><mn>2</mn></msup></math></p></section>'
          f'</article></body></html>')


def test_arxiv_sources_latex_html_and_paired(tmp_path):
  """Bulk tars and ar5iv pages as document sources: worker splits over files, quality tiers, pairing of the two formats
  of one paper, and the whole thing through `create_source` into shards."""
  from nmoe_b200.data import arxiv_sources as A
  from nmoe_b200.data.prep import PrepConfig, PrepPipeline
  from nmoe_b200.data.sources import create_source
  body = "Deep networks generalise well. " * 30
  doc = "\\documentclass{article}\\begin{document}\\section{Intro}" + body + "\\end{document}"
  tars = tmp_path / "tars"
  tars.mkdir()
  _bulk_tar(tars / "arXiv_src_2301_001.tar", {"2301.00001": {"main.tex": doc}, "2301.00002": doc, "2301.00009": None,
                                              "2301.00004": "\\documentclass{article}\\begin{document}tiny\\end{document}"})
  _bulk_tar(tars / "arXiv_src_2301_002.tar", {"2301.00003": doc, "2301.00001": doc})          # 00001 again: replaced in-month
  (tars / "arXiv_src_2301_003.tar").write_bytes(b"this is not a tar file")
  html = tmp_path / "ar5iv"
  for tier, pid in (("no_problem", "2301.00001v2"), ("warning", "2301.00001"), ("warning", "2301.00003"), ("error", "2301.00002"),
                    ("no_problem", "2301.07777")):
    d = html / tier / "2301"
    d.mkdir(parents=True, exist_ok=True)
    (d / f"{pid}.html").write_text(_ar5iv_page(pid, f"Rendered from {tier}. " + "Content sentence. " * 12))
  (html / "no_problem" / "2301" / "2301.08888.html").write_text("<html><body><p>short</p></body></html>")

  latex = A.ArxivTarSource(tars)
  docs = list(latex)
  assert [d.doc_id for d in docs] == ["arxiv:2301.00001:latex", "arxiv:2301.00002:latex", "arxiv:2301.00003:latex", "arxiv:2301.00001:latex"]
  assert latex.stats["too_short"] == 1 and latex.stats["bad_tars"] == 1 and latex.stats["tars"] == 3 and "Deep networks" in docs[0].text
  w0, w1 = list(A.ArxivTarSource(tars, worker_index=0, num_workers=2)), list(A.ArxivTarSource(tars, worker_index=1, num_workers=2))
  assert len(w0) == 2 and len(w1) == 2 and {d.metadata["source_tar"] for d in w1} == {"arXiv_src_2301_002.tar"}
  assert [d.doc_id for d in latex.shard(1, 2)] == [d.doc_id for d in w1]
  assert len(list(A.ArxivTarSource(tars, max_docs=2))) == 2

  pages = A.Ar5ivSource(html)
  got = list(pages)
  assert [d.doc_id for d in got] == ["arxiv:2301.00001:html", "arxiv:2301.07777:html", "arxiv:2301.00001:html", "arxiv:2301.00003:html"]
  assert got[0].metadata["tier"] == "no_problem" and got[0].metadata["title"].startswith("Paper") and "$x^{2}$" in got[0].text
  assert pages.stats == {"pages": 5, "kept": 4, "dropped": 1} and pages.estimate_size() == 5
  assert len(list(A.Ar5ivSource(html, quality_levels=["error"]))) == 1
  with pytest.raises(ValueError):
    list(A.Ar5ivSource(html, quality_levels=["perfect"]))
  assert sorted(d.doc_id for s in (pages.shard(0, 2), pages.shard(1, 2)) for d in s) == sorted(d.doc_id for d in got)

  paired = A.ArxivPairedSource(tars, html)
  ids = [d.doc_id for d in paired]
  assert ids == ["arxiv:2301.00001:latex", "arxiv:2301.00001:html", "arxiv:2301.00002:latex", "arxiv:2301.00003:latex", "arxiv:2301.00003:html"]
  assert paired.stats == {"latex_only": 1, "both_formats": 2, "total_docs": 5}
  first = list(paired)
  assert first[0].metadata["has_paired_format"] and first[1].metadata["has_paired_format"] and "has_paired_format" not in first[2].metadata
  assert "Rendered from no_problem" in first[1].text                      # the better tier's page wins
  assert [d.doc_id for d in A.ArxivPairedSource(tars, html, emit_both_formats=False)] == [i for i in ids if i.endswith("latex")]

  src = create_source("arxiv_paired", tar_dir=str(tars), html_dir=str(html))
  m = PrepPipeline(src, PrepConfig(str(tmp_path / "out"), "arxiv", tokenizer="bytes", num_shards=2, log_every=0)).run()
  assert m.total_documents == 5
  sinks.verify_manifest(tmp_path / "out")
  from nmoe_b200.data.cli import main
  assert main(["prep", "--source", "arxiv_paired", "--input", str(tars), "--html-dir", str(html), "--output", str(tmp_path / "cli"),
               "--name", "arxiv", "--tokenizer", "bytes", "--num-shards", "2"]) == 0
  assert sinks.load_manifest(tmp_path / "cli").total_tokens == m.total_tokens
  assert main(["prep", "--source", "ar5iv", "--input", str(html), "--output", str(tmp_path / "cli2"), "--name", "a5", "--tokenizer", "bytes",
               "--num-shards", "1"]) == 0
  assert sinks.load_manifest(tmp_path / "cli2").total_documents == 4


def test_arxiv_metadata_client_pages_rate_limits_and_strips_versions():
  from urllib.parse import parse_qs, urlparse
  from nmoe_b200.data.arxiv_html import MetadataClient
  entry = lambda i: (f"<entry><id>http://arxiv.org/abs/2301.{i:05d}v1</id><title>Paper {i}</title><summary>S</summary>"
                     f"<author><name>A</name></author><category term='cs.LG'/><published>2023-01-{1 + i % 28:02d}T00:00:00Z</published></entry>")
  feed = lambda es: "<feed xmlns='http://www.w3.org/2005/Atom'>" + "".join(es) + "</feed>"
  calls, naps = [], []
  def opener(url):
    q = parse_qs(urlparse(url).query)
    calls.append(q)
    if "id_list" in q:
      return feed(entry(int(x.split(".")[1][:5])) for x in q["id_list"][0].split(","))
    start, n = int(q["start"][0]), int(q["max_results"][0])
    return feed(entry(i) for i in range(start, min(start + n, 450)))            # the category holds 450 papers
  c = MetadataClient(delay=3.0, opener=opener, sleep=naps.append)
  got = c.search("cs.LG", "20230101", "20230131", max_results=1000, page=200)
  assert len(got) == 450 and got[0].arxiv_id == "2301.00000" and got[-1].title == "Paper 449"
  assert [int(q["start"][0]) for q in calls] == [0, 200, 400, 450] and "submittedDate:[20230101 TO 20230131]" in calls[0]["search_query"][0]
  assert len(naps) == 3 and all(0 < t <= 3.0 for t in naps)                   # every request after the first waits its turn
  assert len(c.search("cs.LG", max_results=250)) == 250 and c.list_ids("cs.LG", max_results=3) == ["2301.00000", "2301.00001", "2301.00002"]
  calls.clear()
  many = c.fetch([f"2301.{i:05d}" for i in range(230)])
  assert len(many) == 230 and [len(q["id_list"][0].split(",")) for q in calls] == [100, 100, 30]
  assert c.get("2301.00007v3").title == "Paper 7" and c.get("2301.00007").arxiv_id == "2301.00007"


def test_stack_v2_selection_fetch_and_rotating_output(tmp_path):
  """Id table (parquet, file-level and repository-level rows) -> popularity selection with per-repository caps and
  path / vendor / size filters -> blobs from a mirror -> rotating compressed parts."""
  import gzip as gz
  import random
  import pyarrow as pa
  import pyarrow.parquet as pq
  from nmoe_b200.data import stack_v2 as S
  from nmoe_b200.data.cli import main
  assert S.skip_path("src/node_modules/x/index.js") and S.skip_path("Cargo.lock") and S.skip_path("a/b/logo.PNG") and S.skip_path("lib/jquery.min.js")
  assert not S.skip_path("src/build_utils.py") and not S.skip_path("vendor.py") and not S.skip_path("docs/dist.md")
  assert S.decode_text(b"\x00\x01\x02binary") is None and S.decode_text("caf\xe9".encode("latin-1"), "") == "caf\xe9"
  assert S.decode_text("héllo".encode("utf-16"), "utf-16") == "héllo" and S.looks_binary(bytes(range(1, 9)) * 100)

  rnd = random.Random(0)
  rows = []
  for i in range(300):
    repo = f"org/repo{i % 12}"
    rows.append({"blob_id": f"b{i:04d}", "src_encoding": "utf-8", "path": f"src/f{i}.py", "repo_name": repo, "language": "Python",
                 "is_vendor": i % 50 == 0, "is_generated": i % 60 == 1, "length_bytes": 300 + i, "star_events_count": rnd.randint(0, 5000),
                 "fork_events_count": rnd.randint(0, 500), "detected_licenses": ["MIT"], "license_type": "permissive"})
  rows[5]["path"] = "node_modules/dep/index.js"
  rows[6]["length_bytes"] = 10
  rows[7]["length_bytes"] = 10 ** 7
  brute = [S.FileRef.from_row(r) for r in rows]
  ok = [f for f in brute if not (f.is_vendor or f.is_generated or S.skip_path(f.path) or not 256 <= f.length_bytes <= 256_000)]
  def expected(top_n, cap):
    by_repo = {}
    for f in sorted(ok, key=lambda f: (f.score, f.blob_id), reverse=True):
      if len(by_repo.setdefault(f.repo_name, [])) < cap:
        by_repo[f.repo_name].append(f)
    return sorted((f for v in by_repo.values() for f in v), key=lambda f: (f.score, f.blob_id), reverse=True)[:top_n]
  for top_n, cap in ((40, 5), (10, 200), (500, 3), (7, 1)):
    st = {}
    got = S.select_top(rows, top_n, max_files_per_repo=cap, stats=st)
    assert [f.blob_id for f in got] == [f.blob_id for f in expected(top_n, cap)], (top_n, cap)
    shuffled = rows[:]
    rnd.shuffle(shuffled)
    assert [f.blob_id for f in S.select_top(shuffled, top_n, max_files_per_repo=cap)] == [f.blob_id for f in got]      # order-independent
    assert st["scanned"] == 300 and st["selected"] == len(got)
  assert S.select_top(rows, 5, languages=["rust"]) == []
  forks = [dict(rows[20], repo_name=f"fork{k}/repo") for k in range(5)]          # the same blob in five forks: once
  st = {}
  assert len({f.blob_id for f in S.select_top(rows + forks, 300, stats=st)}) == len(S.select_top(rows + forks, 300)) and st["duplicates"] == 5

  # on disk: one file-level parquet and one repository-level parquet with a `files` list; a blob mirror
  root = tmp_path / "stack" / "data" / "Python"
  root.mkdir(parents=True)
  pq.write_table(pa.Table.from_pylist(rows[:150]), str(root / "part0.parquet"))
  grouped = {}
  for r in rows[150:]:
    grouped.setdefault(r["repo_name"], []).append({k: v for k, v in r.items() if k != "repo_name"})
  pq.write_table(pa.Table.from_pylist([{"repo_name": k, "files": v} for k, v in grouped.items()]), str(root / "part1.parquet"))
  assert sum(1 for _ in S.iter_table(S.table_files(tmp_path / "stack"))) == 300
  mirror = tmp_path / "mirror"
  mirror.mkdir()
  want = expected(30, 4)
  for k, f in enumerate(want):
    body = f"# {f.path}\nprint({k})\n".encode()
    if k == 3:
      body = b"\x00\x00\x00 not text"
    if k == 4:
      continue                                                   # missing from the mirror
    (mirror / f"{f.blob_id}.gz").write_bytes(gz.compress(body)) if k % 2 else (mirror / f.blob_id).write_bytes(body)
  out = tmp_path / "out"
  assert main(["stack-v2-materialize", "--input-root", str(tmp_path / "stack"), "--output-root", str(out), "--top-n", "30",
               "--max-files-per-repo", "4", "--blobs", str(mirror), "--threads", "4"]) == 0
  summ = json.loads((out / "worker_0000" / "summary.json").read_text())
  assert (summ["selected"], summ["written"], summ["missing"], summ["binary"]) == (30, 28, 1, 1) and len(summ["parts"]) == 1
  part = out / "worker_0000" / summ["parts"][0]
  if part.suffix == ".zst":
    import zstandard
    text = zstandard.ZstdDecompressor().stream_reader(open(part, "rb")).read().decode()
  else:
    text = gz.open(part, "rt").read()
  got = [json.loads(l) for l in text.splitlines()]
  assert [g["id"] for g in got] == [f.blob_id for k, f in enumerate(want) if k not in (3, 4)]
  assert got[0]["text"].startswith("# src/") and got[0]["repo_name"].startswith("org/") and got[0]["detected_licenses"] == ["MIT"] and got[0]["score"] > 0
  # two workers split the table files; rotation by rows
  w = S.RotatingJsonl(tmp_path / "rot", max_rows=3, compression="none")
  for i in range(8):
    w.write({"i": i})
  w.close()
  assert w.parts == ["part_00000.jsonl.none", "part_00001.jsonl.none", "part_00002.jsonl.none"] and w.rows == 8
  s1 = S.run(tmp_path / "stack", tmp_path / "two", worker_index=1, num_workers=2, top_n=5, blobs=S.DirBlobs(mirror), print_fn=lambda *_: None)
  assert s1["table_files"] == ["part1.parquet"] and s1["scanned"] == 150
  # the bucket through the command-line client
  calls = []
  def fake_run(cmd, capture_output=True):
    calls.append(cmd)
    import types
    return types.SimpleNamespace(returncode=0 if "b0001" in cmd[3] else 1, stdout=gz.compress(b"x = 1\n") if "b0001" in cmd[3] else b"")
  s3 = S.S3Blobs(run=fake_run, client=None)
  s3.client = None
  assert s3.get("b0001") == b"x = 1\n" and s3.get("nope") is None and calls[0][:4] == ["aws", "s3", "cp", "s3://softwareheritage/content/b0001"]


def test_loader_preflight_modes(tmp_path, monkeypatch):
  from nmoe_b200.data.loader import preflight
  from nmoe_b200.data.mixture import single_source_plan
  shard = tmp_path / "s.npy"
  np.save(shard, np.arange(1000, dtype=np.uint32))
  said = []
  ok = single_source_plan([str(shard)], 16, 800)
  short = single_source_plan([str(shard)], 16, 100_000)
  preflight(ok, 16, said.append, mode="strict")
  assert said == []
  preflight(short, 16, said.append)
  assert len(said) == 1 and "will wrap" in said[0]
  with pytest.raises(RuntimeError, match="preflight failed.*data_path"):
    preflight(short, 16, said.append, mode="strict")
  preflight(short, 16, said.append, mode="off")
  assert len(said) == 1
  monkeypatch.setenv("NMOE_PREFLIGHT", "strict")
  with pytest.raises(RuntimeError):
    preflight(short, 16, said.append)
  with pytest.raises(ValueError):
    preflight(short, 16, said.append, mode="loud")
  with pytest.raises(RuntimeError, match="no .npy shards"):
    preflight(single_source_plan([], 16, 10), 16, said.append, mode="off")


def test_task_registry_status_build_and_contract(tmp_path, capsys):
  """configs/tasks.toml made executable: status of tasks, a build through the registry's preparation steps (hygiene,
  exact dedup on text and on tokens), the contract check, the command-line forms."""
  from nmoe_b200.data.cli import main
  from nmoe_b200.data.registry import ContractViolation, Registry, TaskNotBuildable
  shipped = Registry.load("configs/tasks.toml")
  assert len(shipped.tasks) >= 14 and shipped.contract["eos_token_id"] == 199999 and shipped.task("stack_v2").prep["exact_dedup_text"]
  assert shipped.task("arxiv").prep["hydra_filter"] is False and shipped.task("dclm").prep["hydra_filter"] is True
  assert shipped.task("fineweb_edu").shard_dir() == "fineweb_edu/train"
  raw = tmp_path / "raw"
  raw.mkdir()
  rows = [{"id": f"d{i}", "text": f"Document number {i} has enough characters to be kept by hygiene."} for i in range(20)]
  rows += [{"id": "dup", "text": rows[3]["text"].upper()}, {"id": "tiny", "text": "too short"},
           {"id": "ctl", "text": "Control \x00characters\x07 are removed from this otherwise fine document."}]
  (raw / "a.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
  reg_file = tmp_path / "tasks.toml"
  reg_file.write_text(f'''
[corpus]
root = "{tmp_path / "corpus"}"
[corpus.contract]
tokenizer = "bytes"
vocab_size = 257
eos_token_id = 256
dtype = "uint32"
[corpus.prep_defaults]
hygiene = true
exact_dedup_text = true
hydra_filter = false
exact_dedup_tokens = true
num_shards = 2
[tasks.toy]
domain = "web"
[tasks.toy.shards]
train = "toy/train/**/*.npy"
[tasks.toy.raw]
kind = "jsonl"
glob = "{raw}/*.jsonl"
text_field = "text"
id_field = "id"
[tasks.graded]
[tasks.graded.shards]
train = "graded/train/*.npy"
[tasks.graded.raw]
kind = "jsonl"
glob = "{raw}/*.jsonl"
[tasks.graded.prep]
hydra_filter = true
[tasks.no_recipe]
[tasks.no_recipe.shards]
train = "nr/train/*.npy"
''')
  reg = Registry.load(reg_file)
  st = {r["task"]: r for r in reg.status()}
  assert st["toy"]["buildable"] and not st["toy"]["ready"] and st["toy"]["raw_files"] == 1 and not st["no_recipe"]["buildable"]
  m = reg.build("toy", tokenizer="bytes", print_fn=lambda *_: None)
  assert m.total_documents == 21                       # 23 rows - the tiny one - the duplicate (case-folded)
  reg.check_contract(m)
  st = {r["task"]: r for r in reg.status()}
  assert st["toy"]["ready"] and st["toy"]["shards"] == 2 and st["toy"]["tokens"] == m.total_tokens
  shard_text = b"".join(bytes(int(t) for t in np.load(p) if t < 256) for p in reg.shard_files("toy")).decode()
  assert "Control characters are removed" in shard_text and "too short" not in shard_text
  m.eos_token_id = 1
  with pytest.raises(ContractViolation, match="eos_token_id"):
    reg.check_contract(m)
  with pytest.raises(TaskNotBuildable):
    reg.build("no_recipe", tokenizer="bytes")
  with pytest.raises(TaskNotBuildable, match="grading model"):
    reg.build("graded", tokenizer="bytes")
  kept = reg.build("graded", tokenizer="bytes", grader=lambda texts: [float("9" in t) for t in texts], tau_keep=0.5, print_fn=lambda *_: None)
  assert kept.total_documents == 2                     # documents 9 and 19
  with pytest.raises(ValueError, match="unknown preparation keys"):
    Registry({"corpus": {"root": "/x"}, "tasks": {"t": {"prep": {"dedupe": True}}}})
  # command line
  assert main(["tasks", "--registry", str(reg_file)]) == 0
  out = capsys.readouterr().out
  assert "toy" in out and "ready" in out and "no_recipe" in out and "missing" in out
  assert main(["tasks", "--registry", str(reg_file), "--json"]) == 0
  assert {t["task"] for t in json.loads(capsys.readouterr().out)["tasks"]} == {"toy", "graded", "no_recipe"}
  assert main(["prep", "--task", "toy", "--registry", str(reg_file), "--corpus-root", str(tmp_path / "c2"), "--tokenizer", "bytes",
               "--output", "unused", "--name", "unused"]) == 0
  assert sinks.load_manifest(tmp_path / "c2" / "toy" / "train").total_documents == 21
  assert main(["prep", "--task", "graded", "--registry", str(reg_file), "--tokenizer", "bytes"]) == 2      # needs a grader or --no-hydra
  assert main(["prep", "--task", "graded", "--registry", str(reg_file), "--corpus-root", str(tmp_path / "c3"), "--tokenizer", "bytes", "--no-hydra"]) == 0


def test_inspection_and_maintenance_commands_on_a_small_dataset(tmp_path, capsys):
  """verify / info / inspect / regenerate-index / merge-manifests / cluster through the command line."""
  from nmoe_b200.data.cli import main
  _write_jsonl(tmp_path / "raw.jsonl", 30)
  common = ["prep", "--source", "jsonl", "--input", str(tmp_path / "raw.jsonl"), "--name", "toy", "--tokenizer", "bytes", "--num-shards", "2"]
  assert main([*common, "--output", str(tmp_path / "a")]) == 0
  capsys.readouterr()
  assert main(["verify", str(tmp_path / "a")]) == 0 and "OK: 2 shards" in capsys.readouterr().out
  assert main(["verify", str(tmp_path / "a"), "--fast"]) == 0
  capsys.readouterr()
  assert main(["info", str(tmp_path / "a")]) == 0
  info = json.loads(capsys.readouterr().out)
  assert info["dataset"] == "toy" and info["num_shards"] == 2 and info["total_documents"] == 30
  shard = sorted((tmp_path / "a").glob("*.npy"))[0]
  assert main(["inspect", str(shard)]) == 0
  stats = json.loads(capsys.readouterr().out)
  assert stats["documents"] > 0 and stats["tokens"] > 0
  assert main(["inspect", str(shard), "--doc", "0", "--tokenizer", "bytes"]) == 0
  doc = json.loads(capsys.readouterr().out)
  assert doc["doc"] == 0 and doc["ids"][-1] == 256 and isinstance(doc.get("text"), str)
  assert main(["inspect", str(shard), "--start", "2", "--length", "5"]) == 0
  assert len(json.loads(capsys.readouterr().out)["ids"]) == 5
  # a lost index comes back from the end-of-document tokens
  idx = shard.with_suffix(".idx")
  before = idx.read_bytes()
  idx.unlink()
  assert main(["regenerate-index", str(shard), "--eos-token-id", "256"]) == 0 and idx.read_bytes() == before
  capsys.readouterr()
  def verify_fails(*flags):
    with pytest.raises(SystemExit):
      main(["verify", str(tmp_path / "a"), *flags])
    return capsys.readouterr().err
  idx.write_bytes(b"garbage")                                                          # unreadable
  assert "E-INDEX-MISSING" in (err := verify_fails()) and "unreadable" in err
  idx.write_bytes(before[:32] + before[48:] + before[32:48])                           # first document moved to the end
  assert "do not tile" in verify_fails("--fast")
  idx.write_bytes(before[:-16])                                                        # header still promises the last document
  assert "E-INDEX-MISSING" in verify_fails("--fast")
  idx.write_bytes(before)
  assert main(["verify", str(tmp_path / "a")]) == 0
  # two workers' outputs merged into one manifest
  assert main([*common, "--output", str(tmp_path / "b"), "--max-documents", "10"]) == 0
  capsys.readouterr()
  assert main(["merge-manifests", str(tmp_path / "a"), str(tmp_path / "b"), "--output", str(tmp_path / "merged.json")]) == 0
  merged = json.loads((tmp_path / "merged.json").read_text())
  assert merged["total_documents"] == 40 and merged["num_shards"] == 4 and "merged 2 manifests" in capsys.readouterr().out
  # clustering of embeddings
  rng = np.random.default_rng(0)
  np.save(tmp_path / "emb.npy", np.concatenate([rng.normal(c, 0.1, size=(40, 8)) for c in (-2, 2)]).astype(np.float32))
  assert main(["cluster", "--embeddings", str(tmp_path / "emb.npy"), "--k", "2", "--output", str(tmp_path / "assign.npy")]) == 0
  cov = json.loads(capsys.readouterr().out)
  assert cov["empty_clusters"] == 0 and sorted(np.bincount(np.load(tmp_path / "assign.npy")).tolist()) == [40, 40]


def test_text_parquet_and_arrow_sources(tmp_path):
  import pyarrow as pa
  import pyarrow.parquet as pq
  from nmoe_b200.data.cli import main
  from nmoe_b200.data.errors import SourceNotFoundError
  from nmoe_b200.data.sources import create_source
  rows = [{"id": f"r{i}", "text": f"row {i} " * 5, "extra": i} for i in range(7)] + [{"id": "empty", "text": "", "extra": -1}]
  tbl = pa.Table.from_pylist(rows)
  pq.write_table(tbl, str(tmp_path / "a.parquet"))
  with pa.ipc.new_file(str(tmp_path / "b.arrow"), tbl.schema) as w:
    w.write_table(tbl)
  with pa.ipc.new_stream(str(tmp_path / "c.arrow"), tbl.schema) as w:                  # the streaming variant of the format
    w.write_table(tbl)
  for pat in ("a.parquet", "b.arrow", "c.arrow"):
    docs = list(create_source("arrow", paths=str(tmp_path / pat)))
    assert [d.doc_id for d in docs] == [f"r{i}" for i in range(7)] and docs[2].text == "row 2 " * 5, pat
  noid = list(create_source("parquet", paths=str(tmp_path / "a.parquet"), id_field=None))
  assert noid[0].doc_id == "a.parquet:0" and noid[6].doc_id == "a.parquet:6"
  (tmp_path / "notes.txt").write_text("first block\nstill first\n\nsecond block\n\n\n")
  (tmp_path / "readme.md").write_text("a markdown file")
  whole = list(create_source("text", paths=str(tmp_path)))
  assert sorted(d.doc_id for d in whole) == ["notes.txt", "readme.md"]
  parts = list(create_source("text", paths=str(tmp_path / "notes.txt"), split_on="\n\n"))
  assert [d.text.strip() for d in parts] == ["first block\nstill first", "second block"]
  with pytest.raises(SourceNotFoundError):
    create_source("arrow", paths=str(tmp_path / "none"))
  with pytest.raises(SourceNotFoundError, match="unknown source kind"):
    create_source("csv", paths=str(tmp_path))
  assert main(["prep", "--source", "parquet", "--input", str(tmp_path / "a.parquet"), "--output", str(tmp_path / "out"), "--name", "p",
               "--tokenizer", "bytes", "--num-shards", "1"]) == 0
  assert sinks.load_manifest(tmp_path / "out").total_documents == 7
  assert main(["prep", "--source", "text", "--input", str(tmp_path / "notes.txt"), "--output", str(tmp_path / "out2"), "--name", "t",
               "--tokenizer", "bytes", "--num-shards", "1"]) == 0
  assert sinks.load_manifest(tmp_path / "out2").total_documents == 1


def test_journey_prepare_a_mixture_train_on_it_and_resume_exactly(tmp_path, monkeypatch, capsys):
  """raw JSONL of two sources -> `prep-mixture` -> `train()` with flow_mode on the prepared shards -> a run cut at step 3
  and restarted ends where the uninterrupted run ends (loader cursors of both sources are part of the checkpoint)."""
  import nmoe_b200.metrics as M
  from nmoe_b200.config import Config
  from nmoe_b200.data.cli import main
  from nmoe_b200.train import train
  mix = tmp_path / "mix.toml"
  mix.write_text('[profiles]\npretrain_profile = "mine"\n[mixtures.mine]\ntotal_tokens_b = 0.001\n'
                 'sources = [{id = "a", tokens_b = 3.0}, {id = "b", tokens_b = 1.0}]\n')
  flows = tmp_path / "flows.toml"
  flows.write_text('[flow.dev]\nmode = "dev"\nstages = ["pretrain"]\ntokens_b = 0.00002\n[flow.dev.mixture]\npretrain = "pretrain_main"\n')
  for name in ("a", "b"):
    d = tmp_path / "raw" / name
    d.mkdir(parents=True)
    (d / "x.jsonl").write_text("".join(json.dumps({"id": f"{name}{i}", "text": f"{name} document number {i} says hello. " * 12}) + "\n" for i in range(60)))
  assert main(["prep-mixture", "--config", str(mix), "--flow-profiles", str(flows), "--flow", "dev", "--seq-len", "32", "--tokenizer", "bytes",
               "--num-shards", "2", "--local-root", str(tmp_path / "raw"), "--data-root", str(tmp_path / "data")]) == 0
  capsys.readouterr()
  assert (tmp_path / "data" / "flows" / "dev" / "pretrain" / "a" / "train" / "manifest.json").exists()
  def cfg_for(tag, **kw):
    base = dict(vocab_size=257, eos_token_id=256, tokenizer="bytes", dim=64, n_layers=2, n_heads=2, inter_dim=128, moe_inter_dim=32,
                n_routed_experts=4, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=32, kv_lora_rank=16,
                qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, batch_size=4, seq_len=32, max_position_embeddings=64,
                warmup_steps=2, steps=6, log_every=1, checkpoint_every=100, activation_checkpoint="none", data_path=None,
                data_root=str(tmp_path / "data"), mixture_toml=str(mix), flow_profiles_toml=str(flows), flow_mode="dev",
                checkpoint_dir=str(tmp_path / tag / "ck"), metrics_dir=str(tmp_path / tag / "m"), experiments_db=str(tmp_path / tag / "e.db"))
    base.update(kw)
    return Config(**base)
  monkeypatch.setenv("NMOE_RUN", "whole")
  whole = train(cfg_for("whole"))
  assert whole["steps_completed"] == 6 and "streaming" not in capsys.readouterr().out
  # the same run, stopped after step 3 by a signal and started again
  import os, signal
  real_log = M.log_training_step
  def log_and_signal(metrics, s, *a, **kw):
    if s == 3:
      os.kill(os.getpid(), signal.SIGUSR1)
    return real_log(metrics, s, *a, **kw)
  monkeypatch.setattr(M, "log_training_step", log_and_signal)
  monkeypatch.setenv("NMOE_RUN", "cut")
  assert train(cfg_for("cut"))["steps_completed"] == 3
  monkeypatch.setattr(M, "log_training_step", real_log)
  rest = train(cfg_for("cut"))
  assert rest["steps_completed"] == 6 and rest["final_loss"] == whole["final_loss"]
  # a different mixture plan under the same checkpoint directory is refused
  mix.write_text(mix.read_text().replace("tokens_b = 3.0", "tokens_b = 2.0"))
  with pytest.raises(RuntimeError, match="plan"):
    train(cfg_for("cut", steps=6))


def test_mixture_sources_resolve_through_the_corpus_registry(tmp_path, monkeypatch):
  """A corpus built once with `prep --task` feeds a flow whose directory holds nothing for that source; a source that is
  nowhere makes training refuse to start with the list of what is missing."""
  from nmoe_b200.config import Config
  from nmoe_b200.data.cli import main
  from nmoe_b200.data.loader import build_loader
  raw = tmp_path / "raw"
  raw.mkdir()
  (raw / "a.jsonl").write_text("".join(json.dumps({"id": f"d{i}", "text": f"registered corpus document {i} with some length. " * 6}) + "\n" for i in range(50)))
  reg = tmp_path / "tasks.toml"
  reg.write_text(f'[corpus]\nroot = "{tmp_path / "corpus"}"\n[corpus.contract]\ntokenizer = "bytes"\nvocab_size = 257\neos_token_id = 256\ndtype = "uint32"\n'
                 f'[corpus.prep_defaults]\nhygiene = true\nnum_shards = 2\n[tasks.web_a]\n[tasks.web_a.shards]\ntrain = "web_a/train/**/*.npy"\n'
                 f'[tasks.web_a.raw]\nkind = "jsonl"\nglob = "{raw}/*.jsonl"\n')
  assert main(["prep", "--task", "web_a", "--registry", str(reg), "--tokenizer", "bytes"]) == 0
  mix = tmp_path / "mix.toml"
  mix.write_text('[profiles]\npretrain_profile = "mine"\n[mixtures.mine]\ntotal_tokens_b = 0.001\nsources = [{id = "web_a", tokens_b = 1.0}]\n')
  flows = tmp_path / "flows.toml"
  flows.write_text('[flow.dev]\nmode = "dev"\nstages = ["pretrain"]\ntokens_b = 0.00001\n[flow.dev.mixture]\npretrain = "pretrain_main"\n')
  kw = dict(vocab_size=257, eos_token_id=256, tokenizer="bytes", dim=8, n_layers=1, n_heads=1, batch_size=2, seq_len=16, steps=3, data_path=None,
            data_root=str(tmp_path / "data"), mixture_toml=str(mix), flow_profiles_toml=str(flows), flow_mode="dev")
  said = []
  loader, plan = build_loader(Config(**kw, tasks_toml=str(reg)), 0, 1, print_fn=said.append)
  assert len(plan.stages[0].sources[0].paths) == 2 and str(tmp_path / "corpus") in plan.stages[0].sources[0].paths[0]
  x, y = loader.next()
  assert x.shape == (2, 16) and torch.equal(x[:, 1:], y[:, :-1])
  with pytest.raises(RuntimeError, match="not ready.*pretrain/web_a"):
    build_loader(Config(**kw), 0, 1, print_fn=said.append)                      # no registry: nothing under the flow directory
  mix.write_text(mix.read_text().replace('id = "web_a"', 'id = "web_b"'))
  with pytest.raises(RuntimeError, match="pretrain/web_b.*tasks of"):
    build_loader(Config(**kw, tasks_toml=str(reg)), 0, 1, print_fn=said.append)


def test_flow_command_streaming_and_staged_give_the_same_dataset(tmp_path, capsys, monkeypatch):
  from nmoe_b200.data.cli import main
  raw = tmp_path / "raw.jsonl"
  raw.write_text("".join(json.dumps({"id": f"d{i}", "text": f"flow document {i} " * 6}) + "\n" for i in range(25)))
  def spec(out):
    p = tmp_path / f"{out}.toml"
    p.write_text(f'[source]\nkind = "jsonl"\npaths = "{raw}"\n[prep]\noutput_dir = "{tmp_path / out}"\ndataset = "f"\ntokenizer = "bytes"\nnum_shards = 2\n')
    return str(p)
  assert main(["flow", spec("s1")]) == 0 and main(["flow", spec("s2"), "--staged"]) == 0
  a, b = sinks.load_manifest(tmp_path / "s1"), sinks.load_manifest(tmp_path / "s2")
  assert (a.total_documents, a.total_tokens) == (b.total_documents, b.total_tokens) == (25, a.total_tokens)
  assert (tmp_path / "s2" / "stages" / "raw.jsonl").exists() and json.loads((tmp_path / "s2" / "stages" / "state.json").read_text())["done"]["shards"] == 25
  # two indexed workers through the environment, as a batch job sets it
  monkeypatch.setenv("NMOE_FLOW_WORKERS", "2")
  for i in (0, 1):
    monkeypatch.setenv("JOB_COMPLETION_INDEX", str(i))
    assert main(["flow", spec("s3"), "--staged"]) == 0
  parts = [sinks.load_manifest(tmp_path / "s3" / f"worker_{i:04d}") for i in (0, 1)]
  assert sum(p.total_documents for p in parts) == 25 and all(p.total_documents > 0 for p in parts)
  # a specification that asks for grading without naming a model is refused before any work
  p = tmp_path / "g.toml"
  p.write_text(open(spec("s4")).read() + "[grade]\nenabled = true\n")
  assert main(["flow", str(p)]) == 2 and "names no checkpoint" in capsys.readouterr().err


def test_prep_command_with_worker_processes_matches_the_serial_run(tmp_path):
  from nmoe_b200.data.cli import main
  _write_jsonl(tmp_path / "raw.jsonl", 80)
  common = ["prep", "--source", "jsonl", "--input", str(tmp_path / "raw.jsonl"), "--name", "toy", "--tokenizer", "bytes", "--num-shards", "4"]
  assert main([*common, "--output", str(tmp_path / "serial")]) == 0
  assert main([*common, "--output", str(tmp_path / "par"), "--workers", "2"]) == 0
  a, b = sinks.load_manifest(tmp_path / "serial"), sinks.load_manifest(tmp_path / "par")
  assert (a.total_documents, a.total_tokens) == (b.total_documents, b.total_tokens)
  assert [s.num_tokens for s in a.shards] == [s.num_tokens for s in b.shards]          # the same documents land in the same shards
  sinks.verify_manifest(tmp_path / "par")
  with pytest.raises(SystemExit, match="main process"):
    main([*common, "--output", str(tmp_path / "x"), "--workers", "2", "--hydra-filter", "--checkpoint", "c", "--heads-dir", "h"])


def test_a_mistyped_path_is_one_line_not_a_traceback(tmp_path, capsys, monkeypatch):
  from nmoe_b200.data.cli import main
  assert main(["info", str(tmp_path / "nowhere")]) == 2
  err = capsys.readouterr().err
  assert err.startswith("info: ") and "nowhere" in err and "Traceback" not in err
  assert main(["verify", str(tmp_path)]) == 2 and "manifest.json" in capsys.readouterr().err
  monkeypatch.setenv("NMOE_DEBUG", "1")
  with pytest.raises(FileNotFoundError):
    main(["info", str(tmp_path / "nowhere")])
