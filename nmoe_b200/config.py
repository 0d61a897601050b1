"""Run configuration: one flat dataclass, TOML loading, env/CLI overrides, fingerprint.

The TOML key names are the user contract shared with the reference
(nmoe/config.py:20-193 lists them; nmoe/train.py:211-250 gives the precedence
TOML < NMOE_* environment < ``--key=value``).  This module keeps those keys so
an existing config file loads unchanged, and adds the keys this framework needs
for features the reference does not have (softmax / device-limited routing,
true NVFP4, fused ZeRO-2 selection).  All validation lives in
``Config.validate`` instead of being spread over train/model/opt.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import re
import tomllib
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Dict, Optional

EXPERT_DTYPES = ("bf16", "fp8", "nvfp4", "nvfp4x16")   # nvfp4 = E2M1 + E8M0/32 (the reference's profile), nvfp4x16 = E2M1 + UE4M3/16 + tensor scale
ATTENTION_KINDS = ("mla", "swa", "nsa", "dsa", "kda")
ROUTER_KINDS = ("sigmoid", "softmax")


@dataclass
class Config:
  # ---- meta
  preset: str = "custom"
  experiment_id: str = "default"

  # ---- architecture
  vocab_size: int = 201088
  tokenizer: str = "o200k_harmony"
  eos_token_id: int = 199999
  dim: Optional[int] = None
  n_layers: Optional[int] = None
  n_heads: Optional[int] = None
  inter_dim: Optional[int] = None
  moe_inter_dim: Optional[int] = None
  n_routed_experts: Optional[int] = None
  n_activated_experts: Optional[int] = None
  n_shared_experts: int = 2
  n_dense_layers: int = 1

  # ---- attention
  attn: str = "mla"
  attn_local: str = "swa"
  attn_global_every: int = 1
  attn_local_window: int = 128
  q_lora_rank: int = 1536
  kv_lora_rank: int = 512
  qk_nope_head_dim: int = 128
  qk_rope_head_dim: int = 64
  v_head_dim: int = 128

  # ---- rope
  max_position_embeddings: int = 8192
  rope_theta: float = 50000.0
  rope_scaling_factor: float = 1.0
  rope_ntk_alpha: float = 1.0
  rope_ntk_beta: float = 32.0

  rms_norm_eps: float = 1e-5

  # ---- routing
  router_bias_update_rate: float = 1e-4
  aux_loss_alpha: float = 0.0
  norm_topk_prob: bool = True
  route_scale: float = 1.0
  router_type: str = "sigmoid"        # sigmoid (aux-loss-free bias) | softmax
  route_max_devices: int = 0          # >0: device-limited routing (top-M expert groups per token)
  route_n_groups: int = 0             # number of expert groups for device-limited routing (0 = world size)

  # ---- precision of the expert GEMMs
  dtype: Optional[str] = "bf16"       # bf16 | fp8 (E4M3 + 1x32 E8M0) | nvfp4 (E2M1 + 1x32 E8M0) | nvfp4x16 (E2M1 + 1x16 UE4M3 + tensor scale)
  nvfp4_block: int = 32               # 32: E8M0 scales (reference-compatible); 16: E4M3 scales (true NVFP4)

  # ---- optimizer
  lr_dense: float = 3.4e-4
  lr_router: float = 3.4e-4
  lr_expert: float = 3.4e-4
  weight_decay: float = 0.1
  adam_beta1: float = 0.9
  adam_beta2: float = 0.95
  adam_beta2_expert: float = 0.99
  adam_eps: float = 1e-8
  muon_momentum: float = 0.95
  expert_optimizer: str = "adamw"     # adamw | muon
  zero2_impl: str = "auto"            # auto | nccl | fused   (fused = peer-memory RS+AdamW+AG kernel)
  zero2_bucket_mb: int = 64           # with zero2_overlap: size of one bucket of the flat buffers (MB of bf16 parameters)
  zero2_overlap: str = "auto"         # auto | true | false: step every bucket on a side stream as soon as backward has
                                      # finished its gradients (auto = with more than one rank, where it measured +6 %)
  moe_pipeline: str = "false"         # auto | true | false: run the two halves of every MoE layer's tokens on two streams
                                      # so that one half's dispatch / return overlaps the other half's GEMMs
  rdep_capacity_factor: float = 0.0   # 0 = lossless receive buffers (worst case); > 0 = that multiple of the balanced share

  # ---- schedule (warmup by step, hold by tokens, cosine decay to an absolute floor)
  warmup_steps: int = 500
  hold_tokens: int = 10_000_000_000
  decay_tokens: int = 40_000_000_000
  decay_floor: float = 3e-5

  # ---- training
  steps: int = 10000
  batch_size: int = 8
  seq_len: int = 4096
  seed: int = 42
  log_every: int = 10
  activation_checkpoint: str = "attention"   # attention | none | full
  moe_overlap_shared: str = "auto"  # shared-expert MLP on a second stream: auto (when world > 1) | 1 | 0
  moe_save_h13: bool = False        # keep the experts' up/gate output for backward instead of recomputing it (memory for time)

  # ---- checkpointing
  checkpoint_dir: str = "/data/checkpoints"
  checkpoint_every: int = 1000
  checkpoint_keep_last_n: int = 3
  resume: bool = True

  # ---- data
  data_root: str = "/data"
  data_path: Optional[str] = None
  hf_dataset: Optional[str] = None
  hf_split: str = "train"
  hf_subset: Optional[str] = None
  hf_text_field: str = "text"
  hf_data_files: Optional[str] = None
  mixture_toml: Optional[str] = None
  flow_profiles_toml: Optional[str] = None
  flow_mode: Optional[str] = None
  tasks_toml: Optional[str] = None    # corpus registry: mixture sources without shards under the flow directory resolve as its tasks
  active_params_b: Optional[float] = None

  # ---- metrics
  metrics_dir: str = "/data/metrics"
  experiments_db: str = "/data/experiments.db"

  # ---- dormant sections kept so reference TOMLs load (no code path reads them there either)
  sft_enabled: bool = False
  sft_prompt_format: str = "chatml"
  sft_mask_prompt_loss: bool = True
  sft_packing_enabled: bool = False
  sft_data_path: Optional[str] = None
  rl_enabled: bool = False
  rl_algorithm: str = "grpo"
  grpo_kl_beta: float = 0.001
  grpo_clamp_eps_lower: float = 0.01
  grpo_clamp_eps_upper: float = 0.01
  grpo_group_size: int = 2
  grpo_prompts_per_step: int = 32
  grpo_iterations: int = 2
  grpo_temperature: float = 1.0
  grpo_top_p: float = 0.9
  reward_model_path: Optional[str] = None
  validation_enabled: bool = False
  validation_data_path: Optional[str] = None
  validation_every: int = 500
  validation_steps: int = 100
  profiling_enabled: bool = False
  profiling_steps: int = 10
  profiling_skip: int = 2             # steps of the run that pass before the profiler starts (allocator, caches warm)
  profiling_output_dir: str = "/data/profiles"

  # ---- evaluation
  eval_enabled: bool = False
  eval_mode: str = "reserved_gpu"
  eval_every: int = 0
  eval_tasks: str = "core"
  eval_tasks_file: str = "configs/eval/tasks.toml"
  eval_budget_max_examples: int = 500
  eval_budget_max_time_s: int = 300
  eval_reserved_gpu_id: int = 7

  # ---- per-backend attention knobs
  attn_swa: Dict[str, Any] = field(default_factory=dict)
  attn_nsa: Dict[str, Any] = field(default_factory=dict)
  attn_dsa: Dict[str, Any] = field(default_factory=dict)
  attn_kda: Dict[str, Any] = field(default_factory=dict)

  # ------------------------------------------------------------------ helpers
  @property
  def qk_head_dim(self) -> int:
    return self.qk_nope_head_dim + self.qk_rope_head_dim

  @property
  def has_moe(self) -> bool:
    return self.n_layers is not None and self.n_layers > self.n_dense_layers

  def is_global_layer(self, layer_id: int) -> bool:
    """Global/local interleave rule (nmoe/model.py:148-153)."""
    every = int(self.attn_global_every)
    return every == 1 or ((layer_id + 1) % every) == 0 or layer_id == self.n_layers - 1

  def validate(self, world: int = 1) -> "Config":
    def need(cond: bool, msg: str) -> None:
      if not cond:
        raise ValueError(msg)

    for k in ("dim", "n_layers", "n_heads"):
      need(getattr(self, k) is not None, f"config key '{k}' is required")
    need(self.dtype in EXPERT_DTYPES, f"dtype must be one of {EXPERT_DTYPES}, got {self.dtype!r}")
    need(self.attn in ATTENTION_KINDS, f"attn must be one of {ATTENTION_KINDS}, got {self.attn!r}")
    need(self.attn_local in ATTENTION_KINDS, f"attn_local must be one of {ATTENTION_KINDS}")
    need(self.router_type in ROUTER_KINDS, f"router_type must be one of {ROUTER_KINDS}")
    need(self.nvfp4_block in (16, 32), "nvfp4_block must be 16 or 32")
    need(self.attn_global_every >= 1, f"attn_global_every must be >= 1, got {self.attn_global_every}")
    if self.attn_global_every > 1:
      need(self.attn_local_window > 0, "attn_local_window must be > 0 when local attention layers exist")
    need(self.batch_size > 0, f"batch_size must be > 0 (got {self.batch_size})")
    need(self.seq_len > 0, f"seq_len must be > 0 (got {self.seq_len})")
    need(world < 2 or self.batch_size % world == 0,
         f"batch_size ({self.batch_size}) must be divisible by world_size ({world})")
    if self.has_moe:
      need(self.n_routed_experts is not None and self.n_activated_experts is not None,
           "MoE requires n_routed_experts and n_activated_experts")
      need(0 < self.n_activated_experts <= self.n_routed_experts,
           f"n_activated_experts ({self.n_activated_experts}) must be in (0, n_routed_experts]")
      need(self.n_routed_experts % max(1, world) == 0,
           f"n_routed_experts ({self.n_routed_experts}) must be divisible by world_size ({world})")
      need(self.moe_inter_dim is not None or self.inter_dim is not None, "MoE requires moe_inter_dim")
      if self.dtype != "bf16":
        need(self.dim % 128 == 0 and (self.moe_inter_dim or self.inter_dim) % 128 == 0,
             "block-scaled experts need dim and moe_inter_dim to be multiples of 128")
    if self.n_dense_layers > 0:
      need(self.inter_dim is not None, "dense layers require inter_dim")
    need(self.decay_floor > 0.0, f"decay_floor must be > 0 (got {self.decay_floor})")
    need(self.decay_floor <= self.lr_expert and self.decay_floor <= self.lr_dense,
         f"decay_floor ({self.decay_floor}) must be <= lr_expert and lr_dense")
    return self


def fingerprint(cfg: Config) -> str:
  """sha256 over the canonical JSON of every public field; resume refuses on mismatch."""
  d = {k: v for k, v in dataclasses.asdict(cfg).items() if not k.startswith("_")}
  s = json.dumps(d, sort_keys=True, separators=(",", ":"), ensure_ascii=True)
  return hashlib.sha256(s.encode("utf-8")).hexdigest()


# ------------------------------------------------------------------ TOML with ${VAR} expansion

_ALLOWED_ENV_PREFIXES = ("NMOE_", "HYDRA_")
_PLACEHOLDER = re.compile(r"\$\{([A-Z_][A-Z0-9_]*)(?::-([^}]*))?\}")


class ConfigEnvError(Exception):
  """An environment placeholder in a TOML file could not be expanded."""


def expand_env(obj: Any, source: str = "<config>") -> Any:
  """Expand ``${VAR}`` / ``${VAR:-default}`` inside every string of a parsed TOML tree.

  Only NMOE_* and HYDRA_* variables may be referenced, so a config file cannot
  pull an unrelated secret out of the environment (nmoe/config.py:287-345).
  """
  if isinstance(obj, dict):
    return {k: expand_env(v, source) for k, v in obj.items()}
  if isinstance(obj, list):
    return [expand_env(v, source) for v in obj]
  if not isinstance(obj, str):
    return obj

  def sub(m: re.Match) -> str:
    name, default = m.group(1), m.group(2)
    if not name.startswith(_ALLOWED_ENV_PREFIXES):
      raise ConfigEnvError(f"${{{name}}} in {source}: only {_ALLOWED_ENV_PREFIXES} variables may be referenced")
    val = os.environ.get(name, default)
    if val is None:
      raise ConfigEnvError(f"${{{name}}} in {source} is unset and has no ':-default'")
    return val

  out = _PLACEHOLDER.sub(sub, obj)
  if "${" in out:
    raise ConfigEnvError(f"malformed placeholder left in {source}: {out!r}")
  return out


def load_toml(path: str | Path) -> dict:
  path = Path(path)
  with open(path, "rb") as f:
    return expand_env(tomllib.load(f), str(path))


# ------------------------------------------------------------------ overrides

_ENV_OVERRIDES = {
  "NMOE_DTYPE": "dtype", "NMOE_STEPS": "steps", "NMOE_BATCH_SIZE": "batch_size",
  "NMOE_SEQ_LEN": "seq_len", "NMOE_RESUME": "resume",
}


def _coerce(key: str, raw: str) -> Any:
  """Turn a CLI/env string into the type of the dataclass field it overrides."""
  fields = {f.name: f for f in dataclasses.fields(Config)}
  if key not in fields:
    raise TypeError(f"unknown config key '{key}'")
  default = fields[key].default
  ann = str(fields[key].type)
  low = raw.strip().lower()
  if isinstance(default, bool) or "bool" in ann:
    if low in ("1", "true", "yes", "on"):
      return True
    if low in ("0", "false", "no", "off"):
      return False
    raise ValueError(f"--{key} expects a boolean, got {raw!r}")
  if low in ("none", "null") and "Optional" in ann:
    return None
  if "int" in ann and "float" not in ann:
    return int(float(raw)) if re.fullmatch(r"[-+]?\d+(\.0*)?([eE]\+?\d+)?", raw.strip()) else int(raw)
  if "float" in ann:
    return float(raw)
  if "Dict" in ann:
    return json.loads(raw)
  return raw


def apply_overrides(d: dict, argv: list[str], env: Optional[dict] = None) -> dict:
  """TOML dict < NMOE_* env < ``--key=value`` / ``--key value`` / ``--resume`` / ``--no-resume``."""
  env = os.environ if env is None else env
  out = dict(d)
  for var, key in _ENV_OVERRIDES.items():
    if var in env and env[var] != "":
      out[key] = _coerce(key, env[var])
  i = 0
  while i < len(argv):
    a = argv[i]
    if not a.startswith("--"):
      raise SystemExit(f"unexpected argument {a!r} (overrides look like --key=value)")
    body = a[2:]
    if "=" in body:
      k, v = body.split("=", 1)
    elif body.startswith("no-") and body[3:].replace("-", "_") in {f.name for f in dataclasses.fields(Config)}:
      k, v = body[3:], "false"
    elif i + 1 < len(argv) and not argv[i + 1].startswith("--"):
      k, v = body, argv[i + 1]
      i += 1
    else:
      k, v = body, "true"
    k = k.replace("-", "_")
    out[k] = _coerce(k, v)
    i += 1
  return out


def from_toml(path: str | Path, argv: Optional[list[str]] = None, env: Optional[dict] = None) -> Config:
  with open(path, "rb") as f:
    d = tomllib.load(f)
  return Config(**apply_overrides(d, argv or [], env))
