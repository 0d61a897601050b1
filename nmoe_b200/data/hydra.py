"""HYDRA: model-based corpus grading with an early exit.

A frozen grading backbone (``nmoe_b200.serve.Transformer``) is tapped twice:

  probe   a bank of linear heads on the mean-pooled hidden state after ``probe_layer`` blocks:
          a quality gate plus cheap auxiliary targets (domain, classifier-score regressions,
          extraction-artifact / missing-content classes).  Documents whose gate falls below
          ``tau_drop`` are dropped right there.
  judge   a small encoder on the full hidden sequence after ``judge_layer`` blocks: a learned query
          token attends over the projected sequence and a linear head reads five rubric scores
          (0..4).  Their weighted mean decides keep / band / drop.

The survivors of the probe are *resumed* from the probe layer (``from_layer`` / ``hidden_in``), so the
first ``probe_layer`` blocks run once per document.

Training is three phases over frozen features: (A) probe on weak labels, (B) judge on oracle
labels plus a pairwise ranking term, (C) probe gate distilled from the judge.  Calibration picks
``tau_drop`` / ``tau_keep`` on oracle-labelled data.

Reference counterparts: heads and phases nmoe/data/train.py:92-670, grading nmoe/data/hydra.py:382-507,
calibration nmoe/data/hydra.py:207-287.
"""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from pathlib import Path
from typing import Callable, Dict, Iterable, Iterator, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

RUBRIC = ("helpfulness", "correctness", "coherence", "complexity", "density")

# name -> (width, kind); kind: "reg" (masked MSE on finite targets) or "cls" (masked CE on targets >= 0)
PROBE_TASKS: Dict[str, Tuple[int, str]] = {
  "gate": (1, "reg"), "domain": (4, "cls"), "fasttext_dclm": (1, "reg"), "fasttext_edu": (1, "reg"),
  "fasttext_code": (1, "reg"), "fasttext_math": (1, "reg"), "lang_score": (1, "reg"),
  "extraction_artifacts": (8, "cls"), "missing_content": (8, "cls"),
}


class ProbeHead(nn.Module):
  """All probe tasks as one linear map (a single GEMM) whose output columns are named slices."""

  def __init__(self, hidden_dim: int, tasks: Optional[Dict[str, Tuple[int, str]]] = None):
    super().__init__()
    self.tasks = dict(tasks or PROBE_TASKS)
    self.slices: Dict[str, slice] = {}
    o = 0
    for name, (w, _) in self.tasks.items():
      self.slices[name] = slice(o, o + w)
      o += w
    self.proj = nn.Linear(hidden_dim, o)

  def forward(self, pooled: torch.Tensor) -> Dict[str, torch.Tensor]:
    y = self.proj(pooled.to(self.proj.weight.dtype))
    return {n: (y[:, s].squeeze(-1) if self.tasks[n][0] == 1 else y[:, s]) for n, s in self.slices.items()}

  def loss(self, out: Dict[str, torch.Tensor], target: Dict[str, torch.Tensor],
           weights: Optional[Dict[str, float]] = None) -> torch.Tensor:
    total = out["gate"].new_zeros(())
    for name, (_, kind) in self.tasks.items():
      if name not in target:
        continue
      w = (weights or {}).get(name, 1.0)
      t = target[name]
      if kind == "reg":
        m = torch.isfinite(t)
        if m.any():
          total = total + w * F.mse_loss(out[name][m].float(), t[m].float())
      else:
        m = t >= 0
        if m.any():
          total = total + w * F.cross_entropy(out[name][m].float(), t[m])
    return total


class JudgeHead(nn.Module):
  """query token + projector + one pre-norm encoder block + rubric head -> [B, 5] scores in 0..4."""

  def __init__(self, hidden_dim: int, mid_dim: int = 512, n_heads: int = 8):
    super().__init__()
    self.in_norm = nn.LayerNorm(hidden_dim)
    self.q_token = nn.Parameter(torch.randn(hidden_dim) * 0.02)
    self.proj = nn.Linear(hidden_dim, mid_dim)
    self.n_heads = n_heads
    self.norm1, self.norm2 = nn.LayerNorm(mid_dim), nn.LayerNorm(mid_dim)
    self.qkv = nn.Linear(mid_dim, 3 * mid_dim)
    self.attn_out = nn.Linear(mid_dim, mid_dim)
    self.ff1, self.ff2 = nn.Linear(mid_dim, 4 * mid_dim), nn.Linear(4 * mid_dim, mid_dim)
    self.rubric = nn.Linear(mid_dim, len(RUBRIC))

  def forward(self, h_seq: torch.Tensor, mask: Optional[torch.Tensor] = None) -> torch.Tensor:
    """h_seq [B,S,H] (any float dtype; NaN/inf are squashed), mask [B,S] True = real token."""
    B, S, H = h_seq.shape
    h = torch.nan_to_num(h_seq.float(), nan=0.0, posinf=1e4, neginf=-1e4)
    h = self.in_norm(h)
    z = self.proj(torch.cat((self.q_token.expand(B, 1, H), h), dim=1))          # [B, 1+S, M]
    # only the query row is read out, so attention is computed for that row alone
    y = self.norm1(z)
    q, k, v = self.qkv(y).chunk(3, dim=-1)
    M = q.size(-1)
    hd = M // self.n_heads
    q0 = q[:, :1].reshape(B, 1, self.n_heads, hd).transpose(1, 2)
    kk = k.reshape(B, 1 + S, self.n_heads, hd).transpose(1, 2)
    vv = v.reshape(B, 1 + S, self.n_heads, hd).transpose(1, 2)
    am = None
    if mask is not None:
      am = torch.cat((mask.new_ones(B, 1), mask), dim=1).view(B, 1, 1, 1 + S)
    a = F.scaled_dot_product_attention(q0, kk, vv, attn_mask=am).transpose(1, 2).reshape(B, M)
    x = z[:, 0] + self.attn_out(a)
    x = x + self.ff2(F.gelu(self.ff1(self.norm2(x))))
    return self.rubric(x)

  @staticmethod
  def aggregate(rubric: torch.Tensor, weights: Optional[Sequence[float]] = None) -> torch.Tensor:
    r = (rubric.float() / 4.0).clamp(0.0, 1.0)
    if weights is None:
      return r.mean(-1)
    w = torch.as_tensor(weights, dtype=r.dtype, device=r.device)
    return (r * w).sum(-1) / w.sum().clamp(min=1e-12)


# ---------------------------------------------------------------------------------------------- calibration
@dataclass
class Calibration:
  weights: Dict[str, float] = field(default_factory=lambda: {k: 1.0 for k in RUBRIC})
  tau_drop: float = 0.30
  tau_keep: float = 0.55

  def weight_vector(self) -> List[float]:
    return [float(self.weights.get(k, 0.0)) for k in RUBRIC]

  def save(self, directory: str) -> Path:
    p = Path(directory)
    p.mkdir(parents=True, exist_ok=True)
    (p / "calibration_summary.json").write_text(json.dumps(asdict(self), indent=1))
    return p / "calibration_summary.json"

  @staticmethod
  def load(directory: str) -> "Calibration":
    j = json.loads((Path(directory) / "calibration_summary.json").read_text())
    return Calibration(j.get("weights") or {k: 1.0 for k in RUBRIC}, float(j.get("tau_drop", 0.3)), float(j.get("tau_keep", 0.55)))


def aggregate_scores(scores: Dict[str, float], weights: Optional[Dict[str, float]] = None) -> float:
  w = weights or {k: 1.0 for k in RUBRIC}
  num = sum(min(max(float(scores[k]) / 4.0, 0.0), 1.0) * float(w.get(k, 0.0)) for k in RUBRIC if k in scores)
  den = sum(float(w.get(k, 0.0)) for k in RUBRIC if k in scores)
  return num / den if den > 0 else 0.0


def calibrate_from_labels(rows: Sequence[dict], target_keep: float = 0.5) -> Tuple[Calibration, int]:
  """Calibration from oracle labels alone (nmoe/data/hydra.py:207-251): rubric weights are the non-negative
  least-squares fit of the five scores (each / 4) to the row's ``aggregated`` value (their mean when it has none),
  normalised to sum to one; ``tau_keep`` is the score quantile above which ``target_keep`` of the labelled documents
  lie, ``tau_drop`` the one below which ``target_keep`` of them lie, swapped if needed so that drop <= keep.  Returns the
  calibration and the number of rows used."""
  if not 0.0 < target_keep < 1.0:
    raise ValueError("target_keep must lie strictly between 0 and 1")
  xs, ys = [], []
  for r in rows:
    sc = r.get("scores")
    if not sc:
      continue
    x = [min(max(float(sc.get(k, 0.0)) / 4.0, 0.0), 1.0) for k in RUBRIC]
    xs.append(x)
    ys.append(float(r["aggregated"]) if r.get("aggregated") is not None else sum(x) / len(x))
  if not xs:
    raise ValueError("no labelled rows with scores")
  x, y = torch.tensor(xs, dtype=torch.float64), torch.tensor(ys, dtype=torch.float64)
  w = torch.full((len(RUBRIC),), 1.0 / len(RUBRIC), dtype=torch.float64)
  step = 1.0 / max(1e-9, float(torch.linalg.matrix_norm(x.t() @ x / len(y), ord=2)))
  for _ in range(2000):      # projected gradient: a clipped unconstrained solution is not the constrained optimum
    w = (w - step * (x.t() @ (x @ w - y) / len(y))).clamp(min=0.0)
  w = w / w.sum() if float(w.sum()) > 0 else torch.full_like(w, 1.0 / len(w))
  s = x @ w
  lo, hi = float(torch.quantile(s, target_keep)), float(torch.quantile(s, 1.0 - target_keep))
  cal = Calibration({k: float(v) for k, v in zip(RUBRIC, w)}, tau_drop=min(lo, hi), tau_keep=max(lo, hi))
  return cal, len(xs)


def calibrate(rubric_pred: torch.Tensor, oracle_keep: torch.Tensor, *, keep_precision: float = 0.9,
              drop_recall_loss: float = 0.02) -> Calibration:
  """Fit rubric weights (non-negative least squares by projected gradient onto the oracle keep label)
  and pick thresholds: ``tau_keep`` = lowest score whose keep-precision reaches the target,
  ``tau_drop`` = highest score below which at most ``drop_recall_loss`` of the oracle keeps fall."""
  x = (rubric_pred.float() / 4.0).clamp(0, 1)
  y = oracle_keep.float()
  w = torch.full((x.size(1),), 1.0 / x.size(1))
  for _ in range(500):
    g = x.t() @ (x @ w - y) / len(y)
    w = (w - 0.5 * g).clamp(min=0.0)
  if w.sum() <= 0:
    w = torch.ones_like(w)
  w = w / w.sum()
  s = x @ w
  order = torch.argsort(s, descending=True)
  ys = y[order]
  prec = ys.cumsum(0) / torch.arange(1, len(ys) + 1)
  ok = (prec >= keep_precision).nonzero()
  tau_keep = float(s[order][ok[-1, 0]]) if len(ok) else float(s.max()) + 1e-6
  asc = torch.argsort(s)
  lost = y[asc].cumsum(0) / y.sum().clamp(min=1)
  ok2 = (lost <= drop_recall_loss).nonzero()
  tau_drop = float(s[asc][ok2[-1, 0]]) if len(ok2) else float(s.min())
  tau_drop = min(tau_drop, tau_keep)
  return Calibration({k: float(v) for k, v in zip(RUBRIC, w.tolist())}, tau_drop, tau_keep)


# ---------------------------------------------------------------------------------------------- grading
def pad_batch(token_lists: Sequence[Sequence[int]], max_ctx: int, device) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
  S = min(max_ctx, max(len(t) for t in token_lists))
  ids = torch.zeros(len(token_lists), S, dtype=torch.long)
  mask = torch.zeros(len(token_lists), S, dtype=torch.bool)
  for i, t in enumerate(token_lists):
    t = list(t)[:S]
    ids[i, :len(t)] = torch.tensor(t, dtype=torch.long)
    mask[i, :len(t)] = True
  pos = torch.arange(S).expand(len(token_lists), S).contiguous()
  return ids.to(device), pos.to(device), mask.to(device)


@torch.inference_mode()
def grade(model, probe: Optional[ProbeHead], judge: JudgeHead, docs: Sequence[Sequence[int]], doc_ids: Sequence[str],
          calib: Calibration, *, batch_size: int = 32, max_ctx: int = 4096, early_exit: bool = True) -> List[dict]:
  """Rows ``{doc_id, q_probe, scores, aggregated, decision, early_exit}`` in input order."""
  from ..serve.model import pool_hidden
  if len(docs) != len(doc_ids):
    raise ValueError("docs / doc_ids length mismatch")
  cfg = model.cfg
  dev = model.embed.device
  out: List[Optional[dict]] = [None] * len(docs)
  stats = {"probe_only": 0, "judged": 0}
  for i0 in range(0, len(docs), batch_size):
    chunk = docs[i0:i0 + batch_size]
    ids, pos, mask = pad_batch(chunk, max_ctx, dev)
    _, taps = model(ids, pos, is_prefill=True, up_to_layer=cfg.probe_layer, return_hidden_states=True, no_logits=True)
    h_probe = taps[cfg.probe_layer]
    if probe is not None:
      q_probe = probe(pool_hidden(h_probe, mask))["gate"].float()
    else:
      q_probe = torch.zeros(len(chunk), device=dev)
    need = torch.ones(len(chunk), dtype=torch.bool, device=dev)
    if early_exit and probe is not None:
      need = q_probe >= calib.tau_drop
    qp = q_probe.tolist()
    for j in (~need).nonzero().flatten().tolist():
      out[i0 + j] = {"doc_id": doc_ids[i0 + j], "q_probe": qp[j], "scores": None, "aggregated": qp[j],
                     "decision": "drop", "early_exit": True}
      stats["probe_only"] += 1
    idx = need.nonzero().flatten()
    if len(idx):
      # resume the survivors from the probe layer instead of recomputing the lower blocks
      _, taps2 = model(ids[idx], pos[idx], is_prefill=True, from_layer=cfg.probe_layer, hidden_in=h_probe[idx],
                       up_to_layer=cfg.judge_layer, return_hidden_states=True, no_logits=True)
      rub = judge(taps2[cfg.judge_layer], mask[idx]).float().clamp(0.0, 4.0)
      agg = JudgeHead.aggregate(rub, calib.weight_vector()).tolist()
      for k, j in enumerate(idx.tolist()):
        a = agg[k]
        decision = "keep" if a >= calib.tau_keep else ("drop" if a < calib.tau_drop else "band")
        out[i0 + j] = {"doc_id": doc_ids[i0 + j], "q_probe": qp[j], "scores": dict(zip(RUBRIC, rub[k].tolist())),
                       "aggregated": a, "decision": decision, "early_exit": False}
        stats["judged"] += 1
  grade.last_stats = stats
  return out  # type: ignore[return-value]


def make_flow_grader(model, probe: Optional[ProbeHead], judge: JudgeHead, calib: Calibration, tokenizer, *,
                     max_ctx: int = 4096, batch_size: int = 32) -> Callable[[List[str]], List[float]]:
  """texts -> aggregated scores, the callable a data flow's grading stage filters on
  (``nmoe_b200.data.flow.run_flow(spec, grader=...)``)."""
  def score(texts: List[str]) -> List[float]:
    docs = [tokenizer.encode(t)[:max_ctx] or [0] for t in texts]
    rows = grade(model, probe, judge, docs, [str(i) for i in range(len(docs))], calib, batch_size=batch_size, max_ctx=max_ctx)
    return [float(r["aggregated"]) for r in rows]
  return score


# ---------------------------------------------------------------------------------------------- training
@dataclass
class PhaseConfig:
  phase: str                       # "A" probe on weak labels | "B" judge on oracle labels | "C" probe distilled from judge
  steps: int = 1000
  lr: float = 1e-3
  rank_weight: float = 0.5         # phase B: pairwise ranking term on (better, worse) pairs
  rank_margin: float = 0.1
  log_every: int = 100
  clip: float = 1.0                # gradient-norm clip; backbone states are not normalised, early steps can be huge


Features = Callable[[dict], Tuple[torch.Tensor, torch.Tensor, torch.Tensor]]
"""batch -> (pooled probe-layer state [B,H], judge-layer sequence [B,S,H], mask [B,S]) from the frozen backbone."""


def train_heads(cfg: PhaseConfig, probe: ProbeHead, judge: JudgeHead, batches: Iterator[dict], features: Features,
                log: Optional[Callable[[int, float], None]] = None) -> List[float]:
  """One training phase over frozen backbone features.  Batch keys: phase A ``targets`` (dict of probe
  targets); phase B ``rubric`` [B,5] (NaN = unlabeled) and optional ``pairs`` [P,2] (index of the better,
  index of the worse document); phase C needs nothing but documents."""
  params = list(probe.parameters()) if cfg.phase in ("A", "C") else list(judge.parameters())
  opt = torch.optim.AdamW(params, lr=cfg.lr, weight_decay=0.0)
  losses: List[float] = []
  for step in range(cfg.steps):
    batch = next(batches)
    pooled, seq, mask = features(batch)
    if cfg.phase == "A":
      loss = probe.loss(probe(pooled), batch["targets"])
    elif cfg.phase == "B":
      pred = judge(seq, mask)
      t = batch["rubric"].to(pred.device)
      m = torch.isfinite(t)
      loss = F.mse_loss(pred[m], t[m]) if m.any() else pred.new_zeros(())
      pairs = batch.get("pairs")
      if pairs is not None and len(pairs):
        agg = JudgeHead.aggregate(pred)
        loss = loss + cfg.rank_weight * F.relu(cfg.rank_margin - (agg[pairs[:, 0]] - agg[pairs[:, 1]])).mean()
    elif cfg.phase == "C":
      with torch.no_grad():
        teacher = JudgeHead.aggregate(judge(seq, mask).clamp(0, 4))
      loss = F.mse_loss(probe(pooled)["gate"].float(), teacher)
    else:
      raise ValueError(f"unknown phase {cfg.phase!r}")
    opt.zero_grad(set_to_none=True)
    loss.backward()
    if cfg.clip and cfg.clip > 0:
      torch.nn.utils.clip_grad_norm_(params, cfg.clip)
    opt.step()
    losses.append(float(loss.detach()))
    if log is not None and (step + 1) % cfg.log_every == 0:
      log(step + 1, losses[-1])
  return losses


def save_heads(directory: str, probe: ProbeHead, judge: JudgeHead) -> None:
  p = Path(directory)
  p.mkdir(parents=True, exist_ok=True)
  torch.save({"probe": probe.state_dict(), "tasks": probe.tasks}, p / "probe.pt")
  torch.save({"judge": judge.state_dict()}, p / "judge.pt")


def load_heads(directory: str, hidden_dim: int, device="cpu") -> Tuple[ProbeHead, JudgeHead]:
  p = Path(directory)
  pj = torch.load(p / "probe.pt", map_location=device, weights_only=False)
  probe = ProbeHead(hidden_dim, pj.get("tasks"))
  probe.load_state_dict(pj["probe"])
  jj = torch.load(p / "judge.pt", map_location=device, weights_only=False)
  mid = jj["judge"]["proj.weight"].shape[0]
  judge = JudgeHead(hidden_dim, mid)
  judge.load_state_dict(jj["judge"])
  return probe.to(device), judge.to(device)
