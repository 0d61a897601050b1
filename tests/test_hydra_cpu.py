"""Curation stack on CPU with a tiny backbone: heads, three training phases, calibration, grading with
early exit (resumed from the probe layer), JSON score parsing, chunked rephrasing, fidelity filter."""
import itertools

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
