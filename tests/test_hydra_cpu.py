"""Curation stack on CPU with a tiny backbone: heads, three training phases, calibration, grading with
early exit (resumed from the probe layer), JSON score parsing, chunked rephrasing, fidelity filter."""
import itertools

import pytest

import torch

from nmoe_b200.data import hydra as H
from nmoe_b200.data import rephrase as RP
from nmoe_b200.data import score as SC
from nmoe_b200.serve import Engine, ServeConfig, Transformer
from nmoe_b200.serve.model import pool_hidden


def backbone():
  torch.manual_seed(0)
  cfg = ServeConfig(num_hidden_layers=3, num_experts=4, experts_per_token=2, vocab_size=300, hidden_size=32,
                    intermediate_size=32, head_dim=8, num_attention_heads=4, num_key_value_heads=2, sliding_window=8,
                    initial_context_length=64, rope_scaling_factor=1.0, probe_layer=2, judge_layer=3)
  m = Transformer(cfg, dtype=torch.float32)
  m.init_weights(std=0.3)
  return m


def test_heads_train_calibrate_and_grade_with_early_exit():
  m = backbone()
  cfg = m.cfg
  torch.manual_seed(1)
  docs = [torch.randint(0, 256, (int(n),)).tolist() for n in torch.randint(6, 20, (48,))]
  # synthetic "quality": documents dominated by low byte values are good
  quality = torch.tensor([sum(1 for t in d if t < 128) / len(d) for d in docs])
  probe, judge = H.ProbeHead(cfg.hidden_size), H.JudgeHead(cfg.hidden_size, mid_dim=32, n_heads=4)

  def features(batch):
    ids, pos, mask = H.pad_batch(batch["docs"], 64, "cpu")
    with torch.no_grad():
      _, taps = m(ids, pos, return_hidden_states=True, no_logits=True)
    return pool_hidden(taps[cfg.probe_layer], mask), taps[cfg.judge_layer], mask

  def batches(with_pairs):
    for i in itertools.count():
      idx = torch.randperm(len(docs))[:16]
      q = quality[idx]
      b = {"docs": [docs[j] for j in idx], "targets": {"gate": q, "domain": (q > 0.5).long()},
           "rubric": (q * 4).unsqueeze(-1).expand(-1, 5).clone()}
      if with_pairs:
        order = torch.argsort(q, descending=True)
        b["pairs"] = torch.stack((order[:4], order[-4:]), dim=1)
      yield b

  la = H.train_heads(H.PhaseConfig("A", steps=60, lr=1e-2), probe, judge, batches(False), features)
  lb = H.train_heads(H.PhaseConfig("B", steps=60, lr=3e-3), probe, judge, batches(True), features)
  lc = H.train_heads(H.PhaseConfig("C", steps=30, lr=1e-2), probe, judge, batches(False), features)
  assert sum(la[-5:]) < sum(la[:5]) and sum(lb[-5:]) < sum(lb[:5]) and all(map(lambda v: v == v, lc))
  # calibration on the judge's predictions
  ids, pos, mask = H.pad_batch(docs, 64, "cpu")
  with torch.no_grad():
    _, taps = m(ids, pos, return_hidden_states=True, no_logits=True)
    pred = judge(taps[cfg.judge_layer], mask)
  cal = H.calibrate(pred, quality > 0.5, keep_precision=0.7)
  assert 0.0 <= cal.tau_drop <= cal.tau_keep and abs(sum(cal.weights.values()) - 1.0) < 1e-4
  # grading: early exit rows never reach the judge; resumed rows equal a full pass
  cal2 = H.Calibration(cal.weights, tau_drop=float(quality.median()), tau_keep=0.9)
  rows = H.grade(m, probe, judge, docs, [f"d{i}" for i in range(len(docs))], cal2, batch_size=16, max_ctx=64)
  assert [r["doc_id"] for r in rows] == [f"d{i}" for i in range(len(docs))]
  early = [r for r in rows if r["early_exit"]]
  late = [r for r in rows if not r["early_exit"]]
  assert early and late and all(r["decision"] == "drop" and r["scores"] is None for r in early)
  assert H.grade.last_stats["judged"] == len(late)
  rows_full = H.grade(m, probe, judge, docs, [f"d{i}" for i in range(len(docs))], cal2, batch_size=16, max_ctx=64,
                      early_exit=False)
  by_id = {r["doc_id"]: r for r in rows_full}
  for r in late:
    assert abs(r["aggregated"] - by_id[r["doc_id"]]["aggregated"]) < 1e-4
  # heads round-trip
  import tempfile
  with tempfile.TemporaryDirectory() as d:
    H.save_heads(d, probe, judge); cal.save(d)
    p2, j2 = H.load_heads(d, cfg.hidden_size)
    assert torch.equal(p2.proj.weight, probe.proj.weight) and H.Calibration.load(d).tau_keep == cal.tau_keep


def test_score_parsing_prompt_trim_and_aggregates():
  tok = SC.ByteTokenizer()
  assert SC.parse_scores('noise {"helpfulness": 3, "correctness": 4, "coherence": 2, "complexity": 1, "density": 0} tail') == {
    "helpfulness": 3.0, "correctness": 4.0, "coherence": 2.0, "complexity": 1.0, "density": 0.0}
  assert SC.parse_scores('{"helpfulness": 9, "correctness": 4, "coherence": 2, "complexity": 1, "density": 0}') is None
  assert SC.parse_scores("no json here") is None
  assert abs(SC.compute_aggregated({k: 2 for k in SC.RUBRIC}) - 0.5) < 1e-9
  assert abs(SC.compute_aggregated_code({k: 4 for k in SC.CODE_RUBRIC}) - 1.0) < 1e-9
  ids = SC.right_trim(tok, "x" * 5000, max_ctx=1024, max_new=128)
  assert len(ids) <= 1024 - 128
  assert tok.decode(SC.build_prompt(tok, "hello")).endswith("<|start|>assistant<|message|>")


def test_rephrase_pipeline_and_fidelity_filter():
  m = backbone()
  tok = SC.ByteTokenizer()
  eng = Engine(m, max_seq_len=420, max_batch=8, block_size=8)
  texts = ["The reactor reached 450 degrees in 12 minutes. " * 3, "Short note about 7 cats."]
  rew = RP.rephrase_batch(eng, tok, texts, num_versions=2, chunk_size=96, overlap=16, max_new_factor=0.2, stop_tokens=[tok.eot])
  assert len(rew) == 4 and {r.style for r in rew} == {"formal", "casual"} and eng.idle
  chunks = RP.chunk_text(texts[0], tok, 96, 16)
  assert len(chunks) > 1 and chunks[0][-16:] == chunks[1][:16]
  good = RP.Rewrite(0, 0, "formal", "In 12 minutes the reactor attained 450 degrees.")
  bad = RP.Rewrite(0, 1, "casual", "The reactor melted in 99 minutes at 3000 degrees, killing 4.")
  kept = RP.filter_by_fidelity(["The reactor reached 450 degrees in 12 minutes."], [good, bad])
  assert kept == [good]
  # embedding-space agreement with the source: identical text scores 1, batches and padding do not change a score
  src = ["The reactor reached 450 degrees in 12 minutes.", "Cats sleep most of the day, often in sunny places near windows."]
  same = [RP.Rewrite(0, 0, "formal", src[0]), RP.Rewrite(1, 0, "formal", src[1]), RP.Rewrite(0, 1, "casual", "zzzz qqqq 0000 !!!!")]
  sem = RP.semantic_fidelity(m, tok, src, same, max_ctx=64, batch_size=2)
  assert abs(sem[0] - 1.0) < 1e-5 and abs(sem[1] - 1.0) < 1e-5 and sem[2] < sem[0] and all(0.0 <= v <= 1.0 for v in sem)
  one_by_one = RP.semantic_fidelity(m, tok, src, same, max_ctx=64, batch_size=1)
  assert all(abs(a - b) < 1e-5 for a, b in zip(sem, one_by_one))
  e = RP.embed_texts(m, tok, src, max_ctx=64)
  assert e.shape == (2, m.cfg.hidden_size) and torch.allclose(e.norm(dim=-1), torch.ones(2), atol=1e-5)
  lex_ok = [RP.Rewrite(0, 0, "formal", src[0]), RP.Rewrite(0, 1, "casual", src[0] + " Indeed.")]
  assert RP.filter_by_fidelity(src, lex_ok, semantic=[0.99, 0.5], min_semantic=0.85) == lex_ok[:1]
  import pytest
  with pytest.raises(ValueError):
    RP.filter_by_fidelity(src, lex_ok, semantic=[0.9])


def test_cli_train_grade_roundtrip(tmp_path):
  import json
  from nmoe_b200.data.cli import main
  from nmoe_b200.serve.checkpoint import dequant_mxfp4, load_model, save_model
  m = backbone()
  ck = tmp_path / "ckpt"
  save_model(m, str(ck))
  m2 = load_model(str(ck), device="cpu", dtype=torch.float32)
  assert torch.equal(m2.unembed, m.unembed)
  data = tmp_path / "docs.jsonl"
  with open(data, "w") as f:
    for i in range(24):
      f.write(json.dumps({"id": f"d{i}", "text": ("good clean prose " if i % 2 else "@@## 9911 ") * 3, "gate": float(i % 2)}) + "\n")
  heads = tmp_path / "heads"
  common = ["--checkpoint", str(ck), "--input", str(data), "--tokenizer", "bytes", "--max-ctx", "64", "--batch-size", "8"]
  assert main(["hydra-train", *common, "--output", str(tmp_path / "unused"), "--heads", str(heads), "--phase", "A", "--steps", "30", "--lr", "0.01"]) == 0
  from nmoe_b200.data import hydra as H
  H.Calibration(tau_drop=0.5, tau_keep=0.9).save(str(heads))
  out = tmp_path / "graded.jsonl"
  assert main(["hydra-grade", *common, "--output", str(out), "--heads", str(heads)]) == 0
  rows = [json.loads(l) for l in open(out)]
  assert len(rows) == 24 and {r["decision"] for r in rows} <= {"keep", "band", "drop"}
  # MXFP4 expansion used by the published checkpoint layout
  blocks = torch.tensor([[[0x21, 0xF7] + [0] * 14]], dtype=torch.uint8)      # codes 1,2,7,15 -> 0.5, 1, 6, -6
  w = dequant_mxfp4(blocks, torch.tensor([[128]], dtype=torch.uint8), torch.float32)
  assert w[0, :4].tolist() == [1.0, 2.0, 12.0, -12.0]


def test_flow_with_grading_stage_filters_documents(tmp_path):
  """A data flow whose grading stage loads the grading model, heads and calibration named in its spec."""
  import json
  from nmoe_b200.data import hydra as H
  from nmoe_b200.data.cli import main
  from nmoe_b200.serve.checkpoint import save_model
  m = backbone()
  ck, heads = tmp_path / "ckpt", tmp_path / "heads"
  save_model(m, str(ck))
  torch.manual_seed(3)
  probe, judge = H.ProbeHead(m.cfg.hidden_size), H.JudgeHead(m.cfg.hidden_size, mid_dim=32, n_heads=4)
  H.save_heads(str(heads), probe, judge)
  raw = tmp_path / "raw"; raw.mkdir()
  with open(raw / "docs.jsonl", "w") as f:
    for i in range(20):
      f.write(json.dumps({"id": f"d{i}", "text": f"document number {i} " * 4}) + "\n")
  # pick thresholds from the judge's own scores so that some documents pass and some do not
  from nmoe_b200.data.score import ByteTokenizer
  tok = ByteTokenizer()
  texts = [json.loads(l)["text"] for l in open(raw / "docs.jsonl")]
  scores = H.make_flow_grader(m, None, judge, H.Calibration(), tok, max_ctx=64)(texts)
  thr = sorted(scores)[len(scores) // 2]
  H.Calibration(tau_drop=0.0, tau_keep=1.0).save(str(heads))
  out = tmp_path / "out"
  spec = tmp_path / "flow.toml"
  spec.write_text(f"""
[source]
kind = "jsonl"
paths = "{raw / 'docs.jsonl'}"
[grade]
enabled = true
threshold = {thr}
batch_size = 8
max_ctx = 64
checkpoint = "{ck}"
heads = "{heads}"
[prep]
output_dir = "{out}"
dataset = "web"
tokenizer = "bytes"
num_shards = 1
""")
  assert main(["flow", str(spec)]) == 0
  man = json.loads((out / "manifest.json").read_text())
  kept = man["total_documents"] if "total_documents" in man else man["documents"]
  assert 0 < kept < 20


# ---------------------------------------------------------------------------------------------- shard references
def _tiny_dataset(root, n_docs=40, seed=0):
  """Two shards with index files under root/web/v1; returns the documents' token lists in reference order."""
  import numpy as np
  from nmoe_b200.data.sinks import ShardWriter
  rng = np.random.default_rng(seed)
  d = root / "web" / "v1"
  d.mkdir(parents=True)
  docs = []
  for sh in range(2):
    w = ShardWriter(d, "web", "v1", sh, eos_token_id=255)
    for _ in range(n_docs // 2):
      t = rng.integers(1, 250, size=int(rng.integers(5, 60))).tolist()
      w.add_document(t)
      docs.append(t)
    w.finalize()
  return docs


def test_shard_reference_roundtrip_reader_and_sampling(tmp_path):
  import pytest
  from nmoe_b200.data import docid as D
  r = D.SpanRef.make("common_crawl", "/cc\\v1/shard_000001.npy", 12, 40)
  assert str(r) == "common_crawl//cc/v1/shard_000001.npy#s=12:e=40" and len(r) == 28
  assert D.SpanRef.parse(str(r)) == r and D.is_ref(str(r)) and not D.is_ref("row:17")
  for bad in ("nosource.npy#s=1:e=2", "a//b.npy", "a//b.npy#s=5", "a//b.npy#s=x:e=3"):
    with pytest.raises(ValueError):
      D.SpanRef.parse(bad)
  with pytest.raises(ValueError):
    D.SpanRef("a", "b.npy", 9, 3)
  with pytest.raises(ValueError):
    D.SpanRef.parse("a//../../etc/x.npy#s=0:e=1").path(tmp_path)      # must not leave the data root

  docs = _tiny_dataset(tmp_path)
  refs = list(D.enumerate_refs(tmp_path, "web"))
  assert len(refs) == len(docs) and all(x.rel_path.startswith("web/v1/") for x in refs)
  reader = D.SpanReader(tmp_path, max_open=1)
  for ref, t in zip(refs, docs):
    assert reader.tokens(ref) == t + [255]                     # the span includes the end-of-document token
    assert reader.tokens(str(ref), drop_eos=255) == t
  assert reader.tokens(refs[0], max_tokens=3) == docs[0][:3]
  with pytest.raises(ValueError):
    reader.tokens(D.SpanRef("web", refs[0].rel_path, 0, 10 ** 9))
  assert len(list(D.enumerate_refs(tmp_path, "web", min_tokens=30))) < len(refs)

  half = set(map(str, D.sample_refs(refs, 0.5, seed=3)))
  assert 5 < len(half) < 35
  assert half == set(map(str, D.sample_refs(reversed(refs), 0.5, seed=3)))       # order-independent
  assert half <= set(map(str, D.sample_refs(refs, 0.8, seed=3)))                 # growing the fraction only adds
  assert half != set(map(str, D.sample_refs(refs, 0.5, seed=4)))
  p = tmp_path / "refs.jsonl"
  assert D.write_refs(p, refs) == len(refs)
  assert list(D.read_refs(p, skip=[str(refs[0])])) == refs[1:]


def _write_parquet(path, rows):
  import pyarrow as pa
  import pyarrow.parquet as pq
  pq.write_table(pa.Table.from_pylist(rows), str(path))


def test_label_tables_oracle_labels_and_pair_sampler(tmp_path):
  import json
  import random
  from nmoe_b200.data import docid as D
  from nmoe_b200.data import hydra_labels as L
  # a table with nested quality signals and taxonomy codes
  eai = tmp_path / "eai.parquet"
  _write_parquet(eai, [
    {"text": "alpha " * 50, "quality_signals": {"fasttext": {"dclm": 0.7, "fineweb_edu_approx": 0.2, "eai_web_code": 0.0,
                                                              "eai_general_math": 0.1, "english": 0.99}},
     "eai_taxonomy": {"extraction_artifacts": {"primary": {"code": 3}}, "missing_content": {"primary": {"code": 1}}}},
    {"text": "", "quality_signals": {"fasttext": {"dclm": 0.1, "fineweb_edu_approx": 0.1, "eai_web_code": 0.1,
                                                   "eai_general_math": 0.1, "english": 0.5}},
     "eai_taxonomy": {"extraction_artifacts": {"primary": {"code": 0}}, "missing_content": {"primary": {"code": 0}}}},
    {"text": "beta", "quality_signals": {"fasttext": {"dclm": None, "fineweb_edu_approx": 0.4, "eai_web_code": 0.9,
                                                       "eai_general_math": 0.0, "english": 0.8}},
     "eai_taxonomy": {"extraction_artifacts": {"primary": {"code": 99}}, "missing_content": {"primary": {"code": None}}}},
  ])
  got = list(L.TableLabels(eai, L.EAI_FIELDS, "code", max_ctx=16))
  assert len(got) == 2 and got[0].domain == "code"                            # the empty text is skipped
  assert len(got[0].text) == 64                                               # 16 tokens x 4 characters
  assert got[0].signals["fasttext_dclm"] == 0.7 and got[0].classes == {"extraction_artifacts": 3, "missing_content": 1}
  assert "fasttext_dclm" not in got[1].signals and got[1].classes == {}       # null and out-of-range stay unset
  t = L.probe_targets(got)
  assert torch.isnan(t["fasttext_dclm"][1]) and t["extraction_artifacts"].tolist() == [3, -1] and t["domain"].tolist() == [1, 1]

  # graded rows (JSON lines work like parquet), filtered by the language score
  rnd = random.Random(0)
  fw = tmp_path / "fw.jsonl"
  with open(fw, "w") as f:
    for i in range(600):
      f.write(json.dumps({"text": f"doc {i}", "language_score": 0.95 if i % 10 else 0.3, "int_score": rnd.choice([0, 1, 2, 3, 4, 5]),
                          "token_count": rnd.choice([100, 300, 700, 1500, 3000])}) + "\n")
  src = L.TableLabels(str(tmp_path / "fw.*"), L.FINEWEB_EDU_FIELDS)
  rows = list(src)
  assert len(rows) == 540 and all(r.signals["lang_score"] >= 0.9 for r in rows)
  assert [L.length_bucket(n) for n in (None, 0, 255, 256, 1024, 2047, 2048, 10 ** 6)] == [2, 0, 0, 1, 3, 3, 4, 4]
  ps = L.GradedPairs(src, seed=1)
  pairs = ps.next_pairs(50)
  assert len(pairs) == 50 and ps.relaxed == 0
  for hi, lo in pairs:
    assert hi.grade - lo.grade >= 2 and L.length_bucket(hi.n_tokens) == L.length_bucket(lo.n_tokens)
  assert {L.length_bucket(hi.n_tokens) for hi, _ in pairs} == {0, 1, 2, 3, 4}
  assert [(a.text, b.text) for a, b in L.GradedPairs(src, seed=1).next_pairs(50)] == [(a.text, b.text) for a, b in pairs]
  # only adjacent grades available: relaxed pairs are issued, but held to the allowed share
  near = [L.Labelled(text=f"n{i}", grade=2 + i % 2, n_tokens=100) for i in range(40)]
  ps2 = L.GradedPairs(near, max_relaxed_frac=1.0, seed=0)
  assert all(hi.grade - lo.grade == 1 for hi, lo in ps2.next_pairs(10)) and ps2.relaxed == 10
  import pytest
  with pytest.raises(RuntimeError):
    L.GradedPairs([L.Labelled(text="x", grade=3, n_tokens=10)] * 4, seed=0).next_pairs(1)
  # reservoir: a cell holds at most cell_cap documents and later arrivals do get in
  ps3 = L.GradedPairs([], cell_cap=8, seed=0)
  for i in range(400):
    ps3.add(L.Labelled(text=str(i), grade=1, n_tokens=10))
  kept = [int(s.text) for s in ps3.cells[0][1]]
  assert len(kept) == 8 and max(kept) >= 8 and ps3.arrived[0][1] == 400

  # oracle labels over shard references
  docs = _tiny_dataset(tmp_path / "data")
  refs = list(D.enumerate_refs(tmp_path / "data", "web"))
  lab = tmp_path / "oracle.jsonl"
  with open(lab, "w") as f:
    for i, r in enumerate(refs[:10]):
      f.write(json.dumps({"doc_id": str(r), "ok": True, "scores": {d: (i + k) % 5 for k, d in enumerate(L.RUBRIC)}}) + "\n")
    f.write(json.dumps({"doc_id": str(refs[10]), "scores": {"helpfulness": 3}}) + "\n")          # incomplete
    f.write(json.dumps({"doc_id": "web//web/v1/missing.npy#s=0:e=4", "scores": {d: 1 for d in L.RUBRIC}}) + "\n")
    f.write(json.dumps({"doc_id": str(refs[11]), "ok": False, "scores": {d: 1 for d in L.RUBRIC}}) + "\n")
  orc = L.OracleLabels(lab, tmp_path / "data", max_ctx=32, eos_token_id=255)
  labelled = list(orc)
  assert len(labelled) == 10 and orc.skipped == 3
  assert labelled[0].tokens == docs[0][:32] and labelled[3].rubric == (3.0, 4.0, 0.0, 1.0, 2.0)

  # batches in the shape train_heads reads
  enc = lambda s: list(s.encode())
  b = next(L.probe_batches(L.mix([L.TableLabels(eai, L.EAI_FIELDS, "web")]), 4, enc, 16))
  assert len(b["docs"]) == 4 and "gate" not in b["targets"] and b["targets"]["lang_score"].shape == (4,)
  jb = next(L.judge_batches(orc, 6, enc, 32, pairs=ps, pairs_per_batch=3))
  assert len(jb["docs"]) == 12 and jb["rubric"].shape == (12, 5) and jb["pairs"].tolist() == [[6, 7], [8, 9], [10, 11]]
  assert torch.isfinite(jb["rubric"][:6]).all() and torch.isnan(jb["rubric"][6:]).all()


def test_cli_docids_grade_from_shards_with_resume_and_train_from_labels(tmp_path):
  import json
  from nmoe_b200.data.cli import main
  from nmoe_b200.data import docid as D
  from nmoe_b200.serve.checkpoint import save_model
  m = backbone()
  ck = tmp_path / "ckpt"
  save_model(m, str(ck))
  root = tmp_path / "data"
  _tiny_dataset(root)
  refs_file = tmp_path / "refs.jsonl"
  assert main(["docids", "--data-root", str(root), "--source", "web", "--output", str(refs_file)]) == 0
  refs = list(D.read_refs(refs_file))
  assert len(refs) == 40
  heads = tmp_path / "heads"
  H.save_heads(str(heads), H.ProbeHead(32), H.JudgeHead(32))
  H.Calibration(tau_drop=-1.0, tau_keep=2.0).save(str(heads))
  out = tmp_path / "graded.jsonl"
  base = ["--checkpoint", str(ck), "--tokenizer", "bytes", "--max-ctx", "64", "--batch-size", "8", "--heads", str(heads)]
  grade = ["hydra-grade", *base, "--input-docids", str(refs_file), "--data-root", str(root), "--output", str(out)]
  assert main([*grade, "--max-documents", "15"]) == 0
  first = [json.loads(l) for l in open(out)]
  assert [r["doc_id"] for r in first] == [str(r) for r in refs[:15]]
  with open(out, "a") as f:
    f.write('{"doc_id": "web//cut')                    # a line cut by a crash
  out.write_text(out.read_text().rsplit("\n", 1)[0] + "\n")      # (dropped again: the file must stay line-parseable)
  assert main([*grade, "--resume"]) == 0
  rows = [json.loads(l) for l in open(out)]
  assert [r["doc_id"] for r in rows] == [str(r) for r in refs] and rows[:15] == first

  # training from label tables and oracle labels over the same shards
  fw = tmp_path / "fw.jsonl"
  with open(fw, "w") as f:
    for i in range(120):
      f.write(json.dumps({"text": "word " * (5 + i % 7), "language_score": 0.97, "int_score": i % 6, "token_count": 100 + i}) + "\n")
  lab = tmp_path / "oracle.jsonl"
  with open(lab, "w") as f:
    for i, r in enumerate(refs):
      f.write(json.dumps({"doc_id": str(r), "scores": {d: i % 5 for d in H.RUBRIC}}) + "\n")
  train = ["hydra-train", *base, "--steps", "6", "--lr", "0.01", "--labels", f"fineweb_edu:web:{fw}"]
  assert main([*train, "--phase", "A"]) == 0
  assert main([*train, "--phase", "B", "--oracle-labels", str(lab), "--data-root", str(root), "--pairs-per-batch", "2"]) == 0
  assert main([*train, "--phase", "C"]) == 0


def test_prep_with_quality_filter_and_audit_trail(tmp_path):
  """`prep --hydra-filter --hydra-audit-dir`: shards hold only kept documents, the audit file scores every document."""
  import json
  from nmoe_b200.data.cli import main
  from nmoe_b200.data.sinks import load_manifest
  from nmoe_b200.serve.checkpoint import save_model
  save_model(backbone(), str(tmp_path / "ckpt"))
  heads = tmp_path / "heads"
  H.save_heads(str(heads), H.ProbeHead(32), H.JudgeHead(32))
  raw = tmp_path / "raw.jsonl"
  raw.write_text("".join(json.dumps({"id": f"d{i}", "text": f"document number {i} " * (2 + i % 5)}) + "\n" for i in range(30)))
  base = ["prep", "--source", "jsonl", "--input", str(raw), "--name", "q", "--tokenizer", "bytes", "--num-shards", "2",
          "--checkpoint", str(tmp_path / "ckpt"), "--heads-dir", str(heads), "--hydra-batch-size", "8", "--hydra-max-ctx", "64"]
  # audit only: everything is kept, every score is on file
  H.Calibration(tau_drop=-1.0, tau_keep=0.5).save(str(heads))
  assert main([*base, "--output", str(tmp_path / "all"), "--hydra-audit-dir", str(tmp_path / "audit_all")]) == 0
  rows = [json.loads(l) for l in open(tmp_path / "audit_all" / "scores.jsonl")]
  assert len(rows) == 30 and all(r["kept"] for r in rows) and load_manifest(tmp_path / "all").total_documents == 30
  scores = sorted(r["score"] for r in rows)
  # filter at the median score: about half survives, and the audit trail says which
  H.Calibration(tau_drop=-1.0, tau_keep=scores[15]).save(str(heads))
  assert main([*base, "--output", str(tmp_path / "kept"), "--hydra-filter", "--hydra-audit-dir", str(tmp_path / "audit")]) == 0
  rows = [json.loads(l) for l in open(tmp_path / "audit" / "scores.jsonl")]
  kept = [r for r in rows if r["kept"]]
  assert len(rows) == 30 and 0 < len(kept) < 30 and all(r["score"] >= scores[15] for r in kept)
  assert load_manifest(tmp_path / "kept").total_documents == len(kept)
  assert json.loads((tmp_path / "audit" / "summary.json").read_text()) == {"seen": 30, "kept": len(kept), "threshold": scores[15]}
  # filter without an audit directory gives the same shards
  assert main([*base, "--output", str(tmp_path / "kept2"), "--hydra-filter"]) == 0
  assert load_manifest(tmp_path / "kept2").total_tokens == load_manifest(tmp_path / "kept").total_tokens


def test_calibration_from_labels_alone_and_oracle_labelling_over_shards(tmp_path):
  import json
  import random
  from nmoe_b200.data.cli import main
  from nmoe_b200.data import docid as D
  from nmoe_b200.serve.checkpoint import save_model
  rnd = random.Random(0)
  rows = []
  for i in range(400):
    sc = {d: rnd.randint(0, 4) for d in H.RUBRIC}
    # the oracle's overall score only looks at two of the five dimensions
    rows.append({"doc_id": f"d{i}", "scores": sc, "aggregated": 0.75 * sc["correctness"] / 4 + 0.25 * sc["density"] / 4})
  rows.append({"doc_id": "bad", "scores": None})
  cal, n = H.calibrate_from_labels(rows, target_keep=0.3)
  assert n == 400 and abs(cal.weights["correctness"] - 0.75) < 0.02 and abs(cal.weights["density"] - 0.25) < 0.02
  assert cal.weights["helpfulness"] < 0.02 and abs(sum(cal.weights.values()) - 1.0) < 1e-9 and cal.tau_drop <= cal.tau_keep
  agg = [H.aggregate_scores(r["scores"], cal.weights) for r in rows[:400]]
  assert abs(sum(a >= cal.tau_keep for a in agg) / 400 - 0.3) < 0.06 and abs(sum(a <= cal.tau_drop for a in agg) / 400 - 0.3) < 0.06
  no_agg = [{"scores": r["scores"]} for r in rows[:400]]                      # without "aggregated": the plain mean
  cal2, _ = H.calibrate_from_labels(no_agg, 0.5)
  assert all(abs(w - 0.2) < 0.02 for w in cal2.weights.values()) and cal2.tau_drop == cal2.tau_keep
  lab = tmp_path / "labels.jsonl"
  lab.write_text("".join(json.dumps(r) + "\n" for r in rows))
  assert main(["hydra-calibrate", "--labels", str(lab), "--target-keep", "0.3", "--output", str(tmp_path / "cal")]) == 0
  loaded = H.Calibration.load(str(tmp_path / "cal"))
  assert abs(loaded.tau_keep - cal.tau_keep) < 1e-9 and abs(loaded.weights["correctness"] - cal.weights["correctness"]) < 1e-9
  assert main(["hydra-calibrate", "--output", str(tmp_path / "cal")]) == 2

  # oracle labelling from shard references, continued after a first partial run
  save_model(backbone(), str(tmp_path / "ckpt"))
  _tiny_dataset(tmp_path / "data", n_docs=12)
  refs_file = tmp_path / "refs.jsonl"
  D.write_refs(refs_file, D.enumerate_refs(tmp_path / "data", "web"))
  out = tmp_path / "oracle.jsonl"
  cmd = ["hydra-oracle-label", "--checkpoint", str(tmp_path / "ckpt"), "--tokenizer", "bytes", "--max-ctx", "64", "--batch-size", "4",
         "--max-new", "4", "--input-docids", str(refs_file), "--data-root", str(tmp_path / "data"), "--output", str(out)]
  assert main([*cmd, "--max-documents", "5"]) == 0
  assert main([*cmd, "--resume"]) == 0
  got = [json.loads(l) for l in open(out)]
  assert [g["doc_id"] for g in got] == [str(r) for r in D.read_refs(refs_file)] and all("ok" in g and "raw" in g for g in got)


def test_rephrase_command_with_and_without_filters(tmp_path):
  import json
  from nmoe_b200.data.cli import main
  from nmoe_b200.serve.checkpoint import save_model
  save_model(backbone(), str(tmp_path / "ckpt"))
  docs = tmp_path / "docs.jsonl"
  docs.write_text("".join(json.dumps({"id": f"d{i}", "text": f"The reactor reached {400 + i} degrees in {10 + i} minutes. " * 2}) + "\n" for i in range(3)))
  base = ["rephrase", "--checkpoint", str(tmp_path / "ckpt"), "--input", str(docs), "--tokenizer", "bytes", "--max-ctx", "1200", "--batch-size", "4",
          "--num-versions", "2", "--chunk-size", "2048"]
  assert main([*base, "--output", str(tmp_path / "raw.jsonl"), "--no-filter"]) == 0
  rows = [json.loads(l) for l in open(tmp_path / "raw.jsonl")]
  assert len(rows) == 6 and {r["id"] for r in rows} == {"d0", "d1", "d2"} and {r["version"] for r in rows} == {0, 1} and all("style" in r for r in rows)
  import pytest
  with pytest.raises(ValueError, match="leaves no room"):
    main([*base[:base.index("--max-ctx")], "--max-ctx", "200", *base[base.index("--max-ctx") + 2:], "--output", str(tmp_path / "x.jsonl")])
  # a random backbone writes noise: the lexical bounds drop all of it, with or without the embedding check
  assert main([*base, "--output", str(tmp_path / "lex.jsonl")]) == 0 and open(tmp_path / "lex.jsonl").read() == ""
  assert main([*base, "--output", str(tmp_path / "sem.jsonl"), "--semantic-threshold", "0.85"]) == 0 and open(tmp_path / "sem.jsonl").read() == ""


def test_calibrate_command_from_judged_rows_against_oracle_labels(tmp_path, capsys):
  """`hydra-calibrate --judged --oracle`: the judge's own predictions joined with oracle labels by document id
  (`doc_id` or `id` on the oracle side), thresholds that separate the oracle's keeps."""
  import json
  import random
  from nmoe_b200.data.cli import main
  rnd = random.Random(1)
  judged, oracle = [], []
  for i in range(200):
    good = i % 2 == 0
    sc = {d: min(4.0, max(0.0, (3.2 if good else 1.0) + rnd.uniform(-0.6, 0.6))) for d in H.RUBRIC}
    judged.append({"doc_id": f"d{i}", "scores": sc})
    oracle.append({("doc_id" if i % 3 else "id"): f"d{i}", "aggregated": 0.8 if good else 0.2, "scores": sc})
  judged.append({"doc_id": "early", "scores": None})                         # dropped at the probe: no rubric scores
  (tmp_path / "judged.jsonl").write_text("".join(json.dumps(r) + "\n" for r in judged))
  (tmp_path / "oracle.jsonl").write_text("".join(json.dumps(r) + "\n" for r in oracle))
  assert main(["hydra-calibrate", "--judged", str(tmp_path / "judged.jsonl"), "--oracle", str(tmp_path / "oracle.jsonl"),
               "--output", str(tmp_path / "cal"), "--oracle-keep", "0.6", "--keep-precision", "0.95"]) == 0
  assert "200 documents" in capsys.readouterr().out
  cal = H.Calibration.load(str(tmp_path / "cal"))
  agg = lambda r: H.aggregate_scores(r["scores"], cal.weights)
  keeps = [agg(r) >= cal.tau_keep for r in judged[:200]]
  assert sum(k and i % 2 == 0 for i, k in enumerate(keeps)) >= 90 and sum(k and i % 2 == 1 for i, k in enumerate(keeps)) <= 5
  assert cal.tau_drop <= cal.tau_keep
  (tmp_path / "other.jsonl").write_text(json.dumps({"doc_id": "zzz", "aggregated": 0.5}) + "\n")
  assert main(["hydra-calibrate", "--judged", str(tmp_path / "judged.jsonl"), "--oracle", str(tmp_path / "other.jsonl"), "--output", str(tmp_path / "c2")]) == 2


def test_hydra_train_command_phases_b_and_c_from_a_flat_jsonl(tmp_path, capsys):
  import json
  from nmoe_b200.data.cli import main
  from nmoe_b200.serve.checkpoint import save_model
  save_model(backbone(), str(tmp_path / "ckpt"))
  data = tmp_path / "docs.jsonl"
  with open(data, "w") as f:
    for i in range(16):
      row = {"id": f"d{i}", "text": ("clear and useful prose " if i % 2 else "zz## 00 ") * 4}
      if i < 12:
        row["scores"] = {d: float(3 if i % 2 else 1) for d in H.RUBRIC}
      f.write(json.dumps(row) + "\n")
  heads = tmp_path / "heads"
  common = ["hydra-train", "--checkpoint", str(tmp_path / "ckpt"), "--input", str(data), "--tokenizer", "bytes", "--max-ctx", "64",
            "--batch-size", "8", "--heads", str(heads), "--steps", "40", "--lr", "0.002"]
  assert main([*common, "--phase", "B"]) == 0
  out = capsys.readouterr().out
  first, last = [float(x) for x in out.strip().splitlines()[-1].split("loss ")[1].split(";")[0].split(" -> ")]
  assert last < first                                                        # the judge learns the two levels
  assert main([*common, "--phase", "C"]) == 0 and (heads / "hydra_probe.pt").exists() or any(heads.iterdir())
  with pytest.raises(SystemExit):
    main(["hydra-train", "--checkpoint", str(tmp_path / "ckpt"), "--heads", str(heads), "--phase", "A", "--tokenizer", "bytes"])


def test_grading_a_jsonl_resumes_by_document_id(tmp_path):
  import json
  from nmoe_b200.data.cli import main
  from nmoe_b200.serve.checkpoint import save_model
  save_model(backbone(), str(tmp_path / "ckpt"))
  heads = tmp_path / "heads"
  H.save_heads(str(heads), H.ProbeHead(32), H.JudgeHead(32))
  H.Calibration(tau_drop=-1.0, tau_keep=2.0).save(str(heads))
  data = tmp_path / "docs.jsonl"
  data.write_text("".join(json.dumps({"id": f"d{i}", "text": f"some text for document {i}"}) + "\n" for i in range(9)))
  cmd = ["hydra-grade", "--checkpoint", str(tmp_path / "ckpt"), "--input", str(data), "--tokenizer", "bytes", "--max-ctx", "64",
         "--batch-size", "4", "--heads", str(heads), "--output", str(tmp_path / "g.jsonl"), "--flush-every", "4"]
  assert main([*cmd, "--max-documents", "5"]) == 0
  first = [json.loads(l) for l in open(tmp_path / "g.jsonl")]
  assert [r["doc_id"] for r in first] == [f"d{i}" for i in range(5)]
  assert main([*cmd, "--resume"]) == 0
  rows = [json.loads(l) for l in open(tmp_path / "g.jsonl")]
  assert [r["doc_id"] for r in rows] == [f"d{i}" for i in range(9)] and rows[:5] == first
  assert main(cmd) == 0 and len(open(tmp_path / "g.jsonl").readlines()) == 9          # without --resume: from scratch
  one = main([*cmd[:cmd.index("--output")], "--output", str(tmp_path / "h.jsonl"), "--no-early-exit"])
  assert one == 0 and all(not json.loads(l)["early_exit"] for l in open(tmp_path / "h.jsonl"))
