"""Mixture plans: which sources feed which training stage, with how many sequences each.

A plan is resolved from two TOML files -- a mixture file (``[mixtures.<name>]`` with ``sources``
carrying ``tokens_b`` weights) and a flow-profile file (``[flow.<mode>]`` with a token budget and a
stage -> mixture mapping).  Sequence quotas use the largest-remainder method so they sum exactly to
the stage budget; sampling weights are fixed-point integers so that smooth weighted round-robin is
exact integer arithmetic.  The plan hash (sha256 of the canonical JSON) is stored in checkpoints and
a resume with a different plan is refused (nmoe/data/mixture.py:20-286).
"""
from __future__ import annotations

import glob
import hashlib
import json
from dataclasses import dataclass, field
from pathlib import Path
from typing import Dict, List, Optional

from ..config import load_toml

FP_SCALE = 1_000_000
STAGE_ORDER = ("pretrain", "mid", "long")


@dataclass
class HFSource:
  dataset: str
  subset: Optional[str] = None
  split: str = "train"
  valid_split: Optional[str] = None
  text_field: str = "text"
  data_files: Optional[object] = None


@dataclass
class SourcePlan:
  id: str
  weight_fp: int
  quota_sequences: int
  target_tokens: int
  paths: List[str] = field(default_factory=list)
  hf: Optional[HFSource] = None
  max_repetition_ratio: float = 1.0
  max_source_fraction: float = 1.0


@dataclass
class StagePlan:
  stage_id: str
  total_tokens_b: float
  sources: List[SourcePlan]


@dataclass
class MixturePlan:
  plan_id: str
  plan_hash: str
  mixture_id: str
  flow_mode: str
  sample_temperature: float
  seq_len: int
  stages: List[StagePlan]

  def _proto(self, with_paths: bool = True) -> dict:
    return {
      "plan_id": self.plan_id, "mixture_id": self.mixture_id, "flow_mode": self.flow_mode,
      "sample_temperature": self.sample_temperature, "seq_len": self.seq_len,
      "stages": [{"stage_id": s.stage_id, "total_tokens_b": s.total_tokens_b,
                  "sources": [{"id": sp.id, "weight_fp": sp.weight_fp, "quota_sequences": sp.quota_sequences,
                               "target_tokens": sp.target_tokens, "paths": sp.paths if with_paths else [],
                               "max_repetition_ratio": sp.max_repetition_ratio,
                               "max_source_fraction": sp.max_source_fraction} for sp in s.sources]}
                 for s in self.stages],
    }

  def to_json(self) -> str:
    return json.dumps(self._proto(), sort_keys=True)


def largest_remainder_quota(tokens_target: int, seq_len: int, weights: List[float]) -> List[int]:
  total = max(0, tokens_target // seq_len)
  if total == 0 or not weights:
    return [0] * len(weights)
  wsum = sum(weights) or 1.0
  exact = [total * (w / wsum) for w in weights]
  base = [int(x) for x in exact]
  order = sorted(range(len(weights)), key=lambda i: exact[i] - base[i], reverse=True)
  for i in range(total - sum(base)):
    base[order[i % len(order)]] += 1
  return base


def fixed_point_weights(weights: List[float]) -> List[int]:
  wsum = sum(weights) or 1.0
  return [max(1, int(round(w / wsum * FP_SCALE))) for w in weights]


def _dig(d: dict, dotted: str) -> dict:
  for k in dotted.split("."):
    d = d[k]
  return d


def resolve_plan(*, mixture_toml: Path, flow_profiles_toml: Path, flow_section: str, seq_len: int,
                 active_params_b: Optional[float] = None) -> MixturePlan:
  mix = load_toml(mixture_toml)
  flow = _dig(load_toml(flow_profiles_toml), flow_section)
  mode = str(flow.get("mode", ""))
  temperature = float(flow.get("sample_temperature", 1.0))
  scale = flow.get("scale")
  tokens_b = flow.get("tokens_b")
  ratio = flow.get("tokens_b_ratio")
  override: Dict[str, float] = flow.get("tokens_b_override", {})
  stage_map: Dict[str, str] = dict(flow.get("mixture", {}))
  # A mixture file may say itself which of its tables feeds which stage ([profiles]); that is used for a stage of the
  # flow whose named table the file does not have, so that one set of flow profiles serves every mixture file.
  own = {"pretrain": "pretrain_profile", "mid": "midtrain_profile", "long": "longctx_profile"}
  for stage_id in flow.get("stages", list(stage_map)):
    if stage_map.get(stage_id) not in mix.get("mixtures", {}):
      alt = mix.get("profiles", {}).get(own.get(stage_id, ""))
      if alt in mix.get("mixtures", {}):
        stage_map[stage_id] = alt
      elif stage_id in stage_map and "profiles" in mix:
        del stage_map[stage_id]          # the file declares its stages and has none for this one
  if ratio is not None and tokens_b is None:
    if active_params_b is None:
      raise ValueError(f"{flow_section} uses tokens_b_ratio but active_params_b is not set")
    tokens_b = float(ratio) * float(active_params_b)
  if tokens_b is not None and scale is None:
    have = sum(float(_dig(mix, f"mixtures.{stage_map[s]}").get("total_tokens_b", 0.0))
               for s in STAGE_ORDER if stage_map.get(s))
    scale = float(tokens_b) / have if have > 0 else 1.0
  stages: List[StagePlan] = []
  for stage_id in STAGE_ORDER:
    name = stage_map.get(stage_id)
    if not name:
      continue
    sd = _dig(mix, f"mixtures.{name}")
    srcs = sd.get("sources", [])
    stage_b = float(override[stage_id]) if stage_id in override else float(sd.get("total_tokens_b", 0.0)) * (scale or 1.0)
    weights = [float(s.get("tokens_b", 0.0)) for s in srcs]
    quotas = largest_remainder_quota(int(stage_b * 1e9), seq_len, weights)
    wfp = fixed_point_weights(weights)
    plans = []
    for s, q, w in zip(srcs, quotas, wfp):
      hf = None
      if "hf_dataset" in s:
        hf = HFSource(str(s["hf_dataset"]), s.get("hf_subset"), str(s.get("hf_split", "train")),
                      s.get("hf_valid_split"), str(s.get("text_field", "text")), s.get("hf_data_files"))
      plans.append(SourcePlan(id=str(s.get("id")), weight_fp=w, quota_sequences=q,
                              target_tokens=int(float(s.get("tokens_b", 0.0)) * 1e9), hf=hf))
    stages.append(StagePlan(stage_id, stage_b, plans))
  plan = MixturePlan(f"{Path(mixture_toml).stem}:{mode}", "", Path(mixture_toml).stem, mode, temperature, seq_len,
                     stages)
  proto = plan._proto(with_paths=False)
  proto.pop("plan_id")
  plan.plan_hash = hashlib.sha256(json.dumps(proto, sort_keys=True).encode()).hexdigest()
  return plan


def populate_paths(plan: MixturePlan, *, dataset_root: Path, split: str = "train", registry=None) -> None:
  """Fill ``paths`` from ``{dataset_root}/{stage}/{source}/{split}/**/*.npy``.  A source that has nothing there and is a
  task of the corpus registry (``data.registry.Registry``, same id) takes the task's shards instead: corpora built once
  with ``prep --task`` serve every flow without being copied under each flow's directory."""
  for st in plan.stages:
    for sp in st.sources:
      sp.paths = sorted(set(glob.glob(str(Path(dataset_root) / st.stage_id / sp.id / split / "**" / "*.npy"),
                                      recursive=True)))
      if not sp.paths and registry is not None and sp.id in registry.tasks:
        sp.paths = registry.shard_files(sp.id, split)


def single_source_plan(paths: List[str], seq_len: int, total_tokens: int, source_id: str = "data_path") -> MixturePlan:
  sp = SourcePlan(id=source_id, weight_fp=1, quota_sequences=max(1, total_tokens // seq_len),
                  target_tokens=total_tokens, paths=list(paths))
  return MixturePlan("data_path", "0", "data_path", "direct", 1.0, seq_len,
                     [StagePlan("pretrain", total_tokens / 1e9, [sp])])
