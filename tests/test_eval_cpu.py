"""Evaluation stack on CPU with a toy model, the `bytes` tokenizer and local JSONL tasks."""
import json

import torch

from nmoe_b200.config import Config
from nmoe_b200.eval import choices, execution, run_gen
from nmoe_b200.eval.tasks import gpqa, gsm8k, humaneval
from nmoe_b200.train import Trainer


def _cfg(**kw):
  base = dict(vocab_size=257, eos_token_id=256, tokenizer="bytes", dim=64, n_layers=2, n_heads=2, inter_dim=128,
              moe_inter_dim=32, n_routed_experts=4, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1,
              q_lora_rank=32, kv_lora_rank=16, qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, batch_size=2,
              seq_len=64, max_position_embeddings=512, activation_checkpoint="none")
  base.update(kw)
  return Config(**base)


def test_chunked_lse_and_argmax_match_dense():
  torch.manual_seed(0)
  h, w = torch.randn(7, 32), torch.randn(1000, 32)
  dense = torch.logsumexp((h @ w.t()) * 0.125, -1)
  assert torch.allclose(choices.logsumexp_vocab_chunked(h, w, logit_scale=0.125, chunk=64), dense, atol=1e-5)
  assert torch.equal(run_gen.argmax_vocab_chunked(h, w, chunk=64), (h @ w.t()).argmax(-1))
  v, i = run_gen.topk_vocab_chunked(h, w, 5, chunk=64)
  assert torch.equal(i, ((h @ w.t()) * 0.125).topk(5, -1).indices)


def test_choice_eval_runs_and_option_scores_are_loglikelihoods(tmp_path):
  torch.manual_seed(1)
  cfg = _cfg()
  tr = Trainer(cfg)
  task_file = tmp_path / "t.jsonl"
  with open(task_file, "w") as f:
    for i in range(6):
      f.write(json.dumps({"question": f"what is {i}?", "choices": ["yes", "no", "maybe"], "answer": i % 3}) + "\n")
  toml = tmp_path / "tasks.toml"
  toml.write_text(f'[tasks.toy]\nkind = "choices"\nsource = "jsonl:{task_file}"\n[groups]\ncore = ["toy"]\n')
  res = choices.run_eval(tr.model, cfg, rank=0, world=1, max_examples=6, tasks_file=str(toml))
  assert res["toy"]["n"] == 6 and 0.0 <= res["toy"]["acc"] <= 1.0
  # score of an option == sum of per-token log-softmax from full logits
  from nmoe_b200.data.transforms import get_tokenizer
  from nmoe_b200.eval.adapters import Choice
  enc = get_tokenizer("bytes")
  ex = Choice("Question: hi\nAnswer:", ["yes", "no"], 0)
  tr.model.eval()
  s = choices.score_options(tr.model, enc, ex, pad_to=64, pad_id=256)
  p = enc.encode_ordinary(ex.prompt); o = enc.encode_ordinary(" yes")
  toks = torch.tensor([(p + o) + [256] * (64 - len(p + o))])
  with torch.no_grad():
    lp = torch.log_softmax(tr.model(toks)[0].float(), -1)
  want = sum(lp[len(p) - 1 + j, o[j]].item() for j in range(len(o)))
  assert abs(s[0] - want) < 1e-3


def test_lockstep_generation_runs_fixed_number_of_forwards():
  torch.manual_seed(2)
  tr = Trainer(_cfg())
  tr.model.eval()
  calls = {"n": 0}
  orig = tr.model.hidden
  def counted(t):
    calls["n"] += 1
    return orig(t)
  tr.model.hidden = counted
  out = run_gen.generate_lockstep(tr.model, [72, 105], max_new=5, eos_id=256, steps_global=8)
  assert calls["n"] == 8 and len(out) <= 5
  calls["n"] = 0
  assert run_gen.generate_lockstep(tr.model, [72], max_new=5, eos_id=256, steps_global=8, active=False) == []
  assert calls["n"] == 8


def test_task_scorers_and_sandbox():
  assert gsm8k.is_correct("so the total is 1,234.", "#### 1234")
  assert not gsm8k.is_correct("no number", "#### 5")
  assert gpqa.is_correct(" B", "B") and gpqa.extract_answer("the answer is c") == "C"
  assert humaneval.truncate("    return 1\n\ndef other():\n  pass") == "    return 1\n"
  ok = execution.humaneval_check("def add(a, b):\n", "    return a + b\n", "def check(f):\n    assert f(1, 2) == 3\n", "add")
  bad = execution.humaneval_check("def add(a, b):\n", "    return a - b\n", "def check(f):\n    assert f(1, 2) == 3\n", "add")
  assert ok and not bad
  assert execution.run_python("while True: pass", timeout_s=1.0) == (False, "timeout")


def test_sandbox_kills_processes_the_program_left_behind(tmp_path):
  """A generated program that forks a sleeper and returns (or times out) must not leave the sleeper running."""
  import os
  import time
  from nmoe_b200.eval.execution import run_python
  marker = tmp_path / "pid"
  prog = f"""
import os, time, sys
pid = os.fork()
if pid == 0:
    os.close(1); os.close(2)          # detach from the pipes so that the parent's exit ends the run
    time.sleep(60)
    os._exit(0)
open({str(marker)!r}, "w").write(str(pid))
sys.exit(0)
"""
  ok, _ = run_python(prog, timeout_s=5.0)
  assert ok
  pid = int(marker.read_text())
  deadline = time.time() + 3
  alive = True
  while time.time() < deadline:
    try:
      os.kill(pid, 0)
      # a zombie still answers kill(0): look at its state
      state = open(f"/proc/{pid}/stat").read().split()[2]
      alive = state not in ("Z", "X")
    except (ProcessLookupError, FileNotFoundError):
      alive = False
    if not alive:
      break
    time.sleep(0.1)
  assert not alive, "forked child survived the sandbox"
  # and a program that hangs is cut off with its children
  ok, out = run_python("import os, time\nos.fork()\ntime.sleep(60)\n", timeout_s=1.0)
  assert not ok and out == "timeout"


def test_core_suite_row_formats_fewshot_and_span_scoring(tmp_path):
  """Every task of configs/eval/tasks_core.toml parses rows of its dataset's layout; few-shot rows become a prefix;
  the span scorer is SQuAD's exact match / F1 over the accepted answers."""
  import json, tomllib
  from nmoe_b200.eval import adapters as A
  from nmoe_b200.eval.choices import load_tasks
  from nmoe_b200.eval.tasks import span
  tasks = tomllib.load(open("configs/eval/tasks_core.toml", "rb"))
  assert set(load_tasks("configs/eval/tasks_core.toml", "core")) == set(tasks["groups"]["core"])
  assert A.parse_hf_source("hf:allenai/ai2_arc:ARC-Easy:test", {}) == ("allenai/ai2_arc", "ARC-Easy", "test")
  assert A.parse_hf_source("hf:google/boolq:validation", {}) == ("google/boolq", None, "validation")
  rows = {
    "arc_easy": {"question": "2+2?", "choices": {"text": ["3", "4", "5"], "label": ["1", "2", "3"]}, "answerKey": "2"},
    "hellaswag": {"ctx": "A man is", "endings": ["x", "y", "z", "w"], "label": "3"},
    "mmlu": {"question": "q", "choices": ["a", "b", "c", "d"], "answer": 2},
    "openbookqa": {"question_stem": "stem", "choices": {"text": ["a", "b"], "label": ["A", "B"]}, "answerKey": "B"},
    "winogrande": {"sentence": "The cup fell because _ was wet.", "option1": "the cup", "option2": "the table", "answer": "2"},
    "boolq": {"passage": "p", "question": "is it", "answer": True},
    "copa": {"premise": "It rained.", "choice1": "The road got wet.", "choice2": "The sun rose.", "question": "effect", "label": 0},
  }
  want = {"arc_easy": 1, "hellaswag": 3, "mmlu": 2, "openbookqa": 1, "winogrande": 1, "boolq": 1, "copa": 0}
  for name, row in rows.items():
    f = tmp_path / f"{name}.jsonl"
    f.write_text("".join(json.dumps(row) + "\n" for _ in range(8)))
    t = dict(tasks["tasks"][name], source=f"jsonl:{f}")
    ex = list(A.iter_choices(t, max_examples=2))
    assert len(ex) == 2 and ex[0].answer_idx == want[name], name
    if name == "mmlu":
      assert ex[0].prompt.count("Question: q") == 6          # five solved shots + the question
    if name == "winogrande":
      assert ex[0].prompt == "The cup fell because" and ex[0].options[1] == "the table was wet."
    if name == "copa":
      assert ex[0].prompt == "It rained therefore" and ex[0].options[0] == "the road got wet."
  f = tmp_path / "squad.jsonl"
  f.write_text("".join(json.dumps({"context": "Paris is in France.", "question": "Where is Paris?",
                                   "answers": {"text": ["France", "in France"]}}) + "\n" for _ in range(4)))
  sp = list(A.iter_span(dict(tasks["tasks"]["squad"], source=f"jsonl:{f}"), max_examples=5))
  assert len(sp) == 2 and sp[0].meta["answers"] == ["France", "in France"] and sp[0].prompt.count("Answer:") == 3
  assert span.is_correct(" The France.\nQuestion: next", "France", sp[0].meta)
  assert not span.is_correct("Germany", "France", sp[0].meta)
  assert abs(span.best_f1("in the country France", ["France", "in France"]) - 0.8) < 1e-6


def _task_file(tmp_path, n=40):
  """A task file with a multiple-choice group, its generation group, and JSONL sources for both."""
  mc = tmp_path / "mc.jsonl"
  mc.write_text("".join(json.dumps({"question": f"q{i}?", "choices": ["a", "b", "c", "d"], "answer": i % 4}) + "\n" for i in range(n)))
  sp = tmp_path / "span.jsonl"
  sp.write_text("".join(json.dumps({"context": f"the value is v{i}.", "question": "what is the value?", "answers": {"text": [f"v{i}"]}}) + "\n"
                        for i in range(n)))
  tf = tmp_path / "tasks.toml"
  tf.write_text(f'[groups]\ncore = ["mc_a", "mc_b"]\ncore_gen = ["qa"]\n'
                f'[tasks.mc_a]\nkind = "choices"\nsource = "jsonl:{mc}"\n[tasks.mc_b]\nkind = "choices"\nsource = "jsonl:{mc}"\n'
                f'[tasks.qa]\nkind = "gen"\nscorer = "span"\nformat = "squad"\nsource = "jsonl:{sp}"\nmax_new = 4\n'
                f'[tasks.offline]\nkind = "choices"\nsource = "hf:some/dataset:test"\n')
  return tf


def test_runner_task_selection_budget_and_snapshot_roundtrip(tmp_path, monkeypatch):
  from nmoe_b200.eval import runner
  from nmoe_b200.eval.hooks import save_eval_snapshot
  from nmoe_b200.metrics import MetricsWriter
  tf = _task_file(tmp_path, n=6)
  assert list(runner.select_tasks(str(tf), "core")) == ["mc_a", "mc_b", "qa"]
  assert list(runner.select_tasks(str(tf), "qa")) == ["qa"] and list(runner.select_tasks(str(tf), "chat:mc_b|nope|qa")) == ["mc_b", "qa"]
  assert runner.select_tasks(str(tf), "unknown") == {} and len(runner.select_tasks(str(tf), "all")) == 4
  cfg = _cfg(metrics_dir=str(tmp_path / "m"), checkpoint_dir=str(tmp_path / "ck"), eval_tasks_file=str(tf), eval_tasks="core")
  torch.manual_seed(0)
  tr = Trainer(cfg)
  res = runner.run_snapshot_eval(tr.model, cfg, run_id="r", step=7, max_examples=4, print_fn=lambda *_: None)
  assert set(res) == {"mc_a", "mc_b", "qa"} and res["qa"]["n"] == 4 and "f1" in res["qa"] and "centered_acc" in res["mc_a"]
  w = MetricsWriter("r", cfg.metrics_dir, 0)
  assert w.query("eval/CORE")[0][0] == 7 and w.query("eval/task/mc_a/centered") and w.query("eval/task/qa/acc") and w.query("eval/qa/f1")
  w.close()
  # no time left: the first task still runs, the rest is reported as skipped
  res = runner.run_snapshot_eval(tr.model, cfg, run_id="r", step=8, max_examples=2, max_time_s=0.0, print_fn=lambda *_: None)
  assert list(res) == ["mc_a"] and runner.run_snapshot_eval.last_summary["skipped"] == ["mc_b", "qa"]
  # a snapshot carries its configuration, so the runner can rebuild the model from the directory alone
  snap = save_eval_snapshot(tr.model, cfg, "r", 9)
  runner.main(["--snapshot", str(snap), "--run", "r", "--step", "9", "--tasks", "mc_a", "--tasks-file", str(tf), "--max-examples", "3"])
  summ = json.loads((snap / "summary.json").read_text())
  assert summ["step"] == 9 and not summ["simulated"] and [t["task"] for t in summ["tasks"]] == ["mc_a"] and summ["tasks"][0]["n"] == 3
  direct = runner.run_snapshot_eval(tr.model, cfg, run_id="r2", step=9, which="mc_a", max_examples=3, print_fn=lambda *_: None)
  assert summ["results"]["mc_a"] == direct["mc_a"]                   # same weights, same answer


def test_simulated_model_hits_its_target_accuracies_through_the_real_plumbing(tmp_path):
  from nmoe_b200.eval import runner
  from nmoe_b200.eval.simulate import SimConfig, SimulatedModel, simulate_suite
  from nmoe_b200.metrics import MetricsWriter
  tf = _task_file(tmp_path, n=400)
  tasks = runner.select_tasks(str(tf), "all")
  res = simulate_suite(tasks, SimConfig(acc_choices=0.7, acc_span=0.4, seed=1), max_examples=400)
  assert abs(res["mc_a"]["acc"] - 0.7) < 0.06 and abs(res["qa"]["acc"] - 0.4) < 0.07 and res["qa"]["f1"] >= res["qa"]["acc"]
  assert abs(res["mc_a"]["centered_acc"] - (res["mc_a"]["acc"] - 0.25) / 0.75) < 1e-9
  assert res["offline"]["n"] == 400 and abs(res["offline"]["acc"] - 0.7) < 0.06          # unreadable source: synthetic examples
  assert simulate_suite(tasks, SimConfig(acc_choices=0.7, acc_span=0.4, seed=1), 400) == res  # deterministic
  assert simulate_suite(tasks, SimConfig(acc_choices=0.7, acc_span=0.4, seed=2), 400) != res
  m = SimulatedModel(SimConfig(acc_unittest=0.25, acc_judge=0.9))
  assert abs(sum(m.passes_tests(f"p{i}") for i in range(2000)) / 2000 - 0.25) < 0.03
  assert abs(sum(m.judged_keep(f"p{i}") for i in range(2000)) / 2000 - 0.9) < 0.03
  # through the command: no model file needed, summary and metric rows written
  cfg = _cfg(metrics_dir=str(tmp_path / "m"), eval_tasks_file=str(tf), eval_tasks="core")
  snap = tmp_path / "snap"
  snap.mkdir()
  import dataclasses
  (snap / "config.json").write_text(json.dumps({k: v for k, v in dataclasses.asdict(cfg).items() if not k.startswith("_")}, default=str))
  runner.main(["--snapshot", str(snap), "--run", "sim", "--step", "3", "--simulate", "--sim-acc-choices", "0.9", "--max-examples", "300"])
  summ = json.loads((snap / "summary.json").read_text())
  assert summ["simulated"] and abs(summ["CORE"] - (0.9 - 0.25) / 0.75) < 0.08 and {t["task"] for t in summ["tasks"]} == {"mc_a", "mc_b", "qa"}
  w = MetricsWriter("sim", cfg.metrics_dir, 0)
  assert abs(w.query("eval/CORE")[0][1] - summ["CORE"]) < 1e-12
  w.close()


def test_ticket_mode_end_to_end_with_competing_consumers(tmp_path, monkeypatch):
  """eval_mode = "k8s_job": training writes snapshot + ticket; the consumer claims it by rename, runs the runner in a
  child process, records the summary, removes the snapshot; a second consumer cannot take the same ticket; a broken
  ticket fails without stopping the queue; a stale claim is taken over."""
  import os
  import time
  from nmoe_b200.eval import tickets
  from nmoe_b200.eval.hooks import maybe_schedule_eval
  tf = _task_file(tmp_path, n=4)
  cfg = _cfg(metrics_dir=str(tmp_path / "m"), checkpoint_dir=str(tmp_path / "ck"), eval_tasks_file=str(tf), eval_tasks="core",
             eval_enabled=True, eval_every=5, eval_mode="k8s_job", eval_budget_max_examples=3)
  torch.manual_seed(0)
  tr = Trainer(cfg)
  monkeypatch.setenv("RANK", "0")
  assert maybe_schedule_eval(4, cfg, tr.model, "runT", lambda *_: None) is None           # not an evaluation step
  ticket = maybe_schedule_eval(5, cfg, tr.model, "runT", lambda *_: None)
  qdir = tmp_path / "m" / "eval_tickets"
  assert ticket.parent == qdir and tickets.pending(qdir) == [ticket]
  snap = json.loads(ticket.read_text())["snapshot"]
  assert os.path.exists(os.path.join(snap, "model.pt")) and os.path.exists(os.path.join(snap, "config.json"))
  (qdir / "broken_0000001.json").write_text("{not json")
  os.utime(qdir / "broken_0000001.json", (1, 1))                                       # oldest: tried first
  # another consumer got there first: the rename source is gone
  stolen = tickets.claim(ticket, "other-1")
  assert stolen.name == "runT_0000005.json.claimed.other-1" and tickets.claim(ticket, "me-2") is None
  assert tickets.pending(qdir, stale_s=3600) == [qdir / "broken_0000001.json"]
  counts = tickets.serve(qdir, once=True, stale_s=3600, print_fn=lambda *_: None)
  assert counts == {"done": 0, "failed": 1} and (qdir / "broken_0000001.json.failed").exists()
  # ... and died: after the stale time its claim is up for grabs
  os.utime(stolen, (time.time() - 7200, time.time() - 7200))
  counts = tickets.serve(qdir, once=True, stale_s=3600, extra=["--max-examples", "3"], print_fn=lambda *_: None)
  assert counts == {"done": 1, "failed": 0}
  done = json.loads((qdir / "runT_0000005.json.done").read_text())
  assert done["summary"]["step"] == 5 and {t["task"] for t in done["summary"]["tasks"]} == {"mc_a", "mc_b", "qa"}
  assert not os.path.exists(snap) and tickets.pending(qdir) == []
  from nmoe_b200.metrics import MetricsWriter
  w = MetricsWriter("runT", cfg.metrics_dir, 0)
  assert w.query("eval/CORE")[0][0] == 5                                               # the child process recorded the results
  w.close()
  assert tickets.runner_command({"snapshot": "S", "run": "R", "step": 3, "tasks": "core"}, ["--simulate"])[3:] == \
      ["--snapshot", "S", "--run", "R", "--step", "3", "--tasks", "core", "--simulate"]


def test_task_files_expand_environment_placeholders(tmp_path, monkeypatch):
  """The shipped task files point at local copies of the sets through ${NMOE_EVAL_DATA:-/data/eval}."""
  from nmoe_b200.eval import runner
  monkeypatch.setenv("NMOE_EVAL_DATA", str(tmp_path))
  assert choices.load_tasks("configs/eval/tasks.toml", "core")["piqa"]["source"] == f"jsonl:{tmp_path}/piqa_validation.jsonl"
  assert runner.select_tasks("configs/eval/tasks.toml", "gsm8k")["gsm8k"]["source"] == f"jsonl:{tmp_path}/gsm8k_test.jsonl"
  monkeypatch.delenv("NMOE_EVAL_DATA")
  assert runner.select_tasks("configs/eval/tasks.toml", "piqa")["piqa"]["source"] == "jsonl:/data/eval/piqa_validation.jsonl"
  assert list(runner.select_tasks("configs/eval/tasks.toml", "chat")) == ["arc_easy", "arc_challenge", "mmlu", "gsm8k", "humaneval"]


def test_reserved_gpu_mode_spawns_a_runner_that_finishes(tmp_path, monkeypatch):
  """eval_mode = "reserved_gpu": rank 0 saves a snapshot and starts the runner as a child process; the child rebuilds the
  model from the snapshot alone and leaves its summary and metric rows (on this machine it runs on the CPU)."""
  from nmoe_b200.eval.hooks import maybe_schedule_eval
  from nmoe_b200.metrics import MetricsWriter
  tf = _task_file(tmp_path, n=4)
  cfg = _cfg(metrics_dir=str(tmp_path / "m"), checkpoint_dir=str(tmp_path / "ck"), eval_tasks_file=str(tf), eval_tasks="mc_a",
             eval_enabled=True, eval_every=2, eval_mode="reserved_gpu", eval_reserved_gpu_id=0, eval_budget_max_examples=3)
  torch.manual_seed(0)
  tr = Trainer(cfg)
  monkeypatch.setenv("RANK", "1")
  assert maybe_schedule_eval(2, cfg, tr.model, "runR", lambda *_: None) is None          # only rank 0 schedules
  monkeypatch.setenv("RANK", "0")
  said = []
  p = maybe_schedule_eval(2, cfg, tr.model, "runR", said.append)
  assert p.wait(timeout=120) == 0 and "runner pid" in said[0]
  snap = tmp_path / "ck" / "eval_snapshots" / "runR_step0000002"
  summ = json.loads((snap / "summary.json").read_text())
  assert summ["step"] == 2 and [t["task"] for t in summ["tasks"]] == ["mc_a"] and summ["tasks"][0]["n"] == 3
  w = MetricsWriter("runR", cfg.metrics_dir, 0)
  assert w.query("eval/task/mc_a/acc")[0][0] == 2
  w.close()


def test_checkpoint_evaluation_commands_choices_and_generation(tmp_path, monkeypatch, capsys):
  """`python -m nmoe_b200.eval.choices CONFIG` and `... eval.run_gen CONFIG`: load the latest checkpoint of a trained
  configuration and score it, from a TOML file as a user would."""
  from nmoe_b200.train import train
  tf = _task_file(tmp_path, n=4)
  toml = tmp_path / "cfg.toml"
  keys = dict(vocab_size=257, eos_token_id=256, tokenizer="bytes", dim=64, n_layers=2, n_heads=2, inter_dim=128, moe_inter_dim=32,
              n_routed_experts=4, n_activated_experts=2, n_shared_experts=1, n_dense_layers=1, q_lora_rank=32, kv_lora_rank=16,
              qk_nope_head_dim=16, qk_rope_head_dim=8, v_head_dim=16, batch_size=2, seq_len=64, max_position_embeddings=512,
              activation_checkpoint="none", steps=2, checkpoint_every=2, log_every=1, data_path="synthetic",
              checkpoint_dir=str(tmp_path / "ck"), metrics_dir=str(tmp_path / "m"), experiments_db=str(tmp_path / "e.db"),
              eval_tasks_file=str(tf), eval_tasks="core")
  toml.write_text("".join(f"{k} = {json.dumps(v)}\n" for k, v in keys.items()))
  from nmoe_b200.config import from_toml
  monkeypatch.setenv("NMOE_RUN", "evalcmd")
  train(from_toml(toml, [], env={}))
  capsys.readouterr()
  choices.main([str(toml), "--max-examples", "3"])
  out = capsys.readouterr().out
  assert "mean_centered=" in out and "mc_a:acc=" in out and "mc_b:acc=" in out and "n=3" in out
  choices.main([str(toml), "--max-examples", "2", "--group", "mc_b", "--tasks-file", str(tf)])
  run_gen.main([str(toml), "--tasks-file", str(tf), "--max-examples", "2", "--max-new", "3"])
  assert "qa: acc=" in capsys.readouterr().out


def test_choice_task_selection_by_group_name_or_whole_file(tmp_path):
  import pytest
  tf = _task_file(tmp_path, n=2)
  assert list(choices.load_tasks(str(tf), "core")) == ["mc_a", "mc_b"] and list(choices.load_tasks(str(tf), "mc_b")) == ["mc_b"]
  assert list(choices.load_tasks(str(tf), "")) == ["mc_a", "mc_b", "offline"]           # everything that is multiple choice
  with pytest.raises(KeyError, match="no group or task named 'nope'"):
    choices.load_tasks(str(tf), "nope")
  flat = tmp_path / "flat.toml"
  flat.write_text('[tasks.only]\nkind = "choices"\nsource = "jsonl:/nowhere.jsonl"\n')
  assert list(choices.load_tasks(str(flat), "core")) == ["only"]                         # no groups: the file is the group


def test_training_with_inline_evaluation_records_both_tag_families(tmp_path, monkeypatch):
  from nmoe_b200.metrics import MetricsWriter
  from nmoe_b200.train import train
  tf = _task_file(tmp_path, n=4)
  monkeypatch.setenv("NMOE_RUN", "inl")
  cfg = _cfg(steps=4, log_every=2, checkpoint_every=100, data_path="synthetic", checkpoint_dir=str(tmp_path / "ck"),
             metrics_dir=str(tmp_path / "m"), experiments_db=str(tmp_path / "e.db"), eval_tasks_file=str(tf), eval_tasks="core",
             eval_enabled=True, eval_every=2, eval_mode="inline", eval_budget_max_examples=2)
  train(cfg)
  w = MetricsWriter("inl", cfg.metrics_dir, 0)
  assert [s for s, _ in w.query("eval_choices/mc_a/acc")] == [2, 4]                 # the training loop's own evaluation
  assert [s for s, _ in w.query("eval/CORE")] == [2, 4] and w.query("eval/task/qa/acc")     # the snapshot runner, inline
  w.close()
