"""Optimizer construction, WSD schedule and the training-step update.

Parameter groups follow nmoe/opt.py:146-227: experts (rank-local AdamW, beta2 = adam_beta2_expert),
dense_decay, dense_no_decay (biases, norms, embedding, lm_head), router (own LR, no decay).
Dense groups are stepped by ZeRO-2 (``parallel/zero2.py``).  Experts are stepped either after
backward or -- ``fuse_in_backward`` -- inside backward, right after each layer's weight gradient
is produced, so a full set of expert gradients never has to be resident (on one GPU the
16B-parameter model would otherwise hold ~29 GB of them).
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional

import torch
import torch.distributed as dist

from . import ops
from .config import Config
from .parallel import zero2


def wsd_scale(step: int, tokens_seen: int, cfg: Config) -> float:
  """1 during hold, linear (step+1)/warmup before, cosine to 0 over decay_tokens after hold_tokens."""
  if step < cfg.warmup_steps:
    return (step + 1) / max(1, int(cfg.warmup_steps))
  if tokens_seen < cfg.hold_tokens:
    return 1.0
  t = int(tokens_seen - cfg.hold_tokens)
  if t < cfg.decay_tokens:
    return 0.5 * (1.0 + math.cos(math.pi * t / float(max(1, int(cfg.decay_tokens)))))
  return 0.0


def scheduled_lrs(step: int, tokens_seen: int, cfg: Config) -> Dict[str, float]:
  """Per-group learning rates: floor + (peak - floor) * scale, with an absolute floor
  (the router's floor is capped at its own peak) -- nmoe/opt.py:230-287."""
  s = wsd_scale(step, tokens_seen, cfg)
  floor = float(cfg.decay_floor)
  out = {}
  for name, peak in (("expert", cfg.lr_expert), ("dense", cfg.lr_dense), ("router", cfg.lr_router)):
    f = min(floor, float(peak))
    out[name] = f + (float(peak) - f) * s
  return out


class ExpertAdamW:
  """AdamW over rank-local expert tensors with the flat fused kernel (bf16 moments, fp32 math)."""

  def __init__(self, params: List[torch.nn.Parameter], cfg: Config, fuse_in_backward: bool = False):
    self.params = params
    self.lr = float(cfg.lr_expert)
    self.betas = (cfg.adam_beta1, cfg.adam_beta2_expert)
    self.eps, self.wd = cfg.adam_eps, cfg.weight_decay
    self.step_count = 0
    self.state: Dict[int, Dict[str, torch.Tensor]] = {}
    for i, p in enumerate(params):
      self.state[i] = {"exp_avg": torch.zeros_like(p), "exp_avg_sq": torch.zeros_like(p)}
    self.fuse_in_backward = fuse_in_backward
    self.gradnorm_sq: Optional[torch.Tensor] = None
    self._hooks = []
    # In-backward updates run on a side stream: the update of a layer's experts streams 14 bytes per parameter through
    # HBM and uses no tensor core, the backward GEMMs of the layers below it are tensor-bound and do not depend on it,
    # so the two overlap instead of taking turns (NMOE_EXPERT_OPT_SIDE_STREAM=0 keeps them on one stream).
    self.side: Optional[torch.cuda.Stream] = None
    if fuse_in_backward and params and params[0].is_cuda and os.environ.get("NMOE_EXPERT_OPT_SIDE_STREAM", "1") == "1":
      self.side = torch.cuda.Stream(device=params[0].device)
      self._events = [torch.cuda.Event() for _ in params]
    if fuse_in_backward:
      for i, p in enumerate(params):
        self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))

  def _apply(self, i: int, p: torch.Tensor, g: torch.Tensor) -> None:
    st = self.state[i]
    if self.gradnorm_sq is not None:
      ops.sumsq(g.reshape(-1), self.gradnorm_sq)
    qc = getattr(p, "_nmoe_qcache", None)
    if qc is not None and p.is_cuda and g.dtype == p.dtype and g.is_contiguous():
      # block-scaled profile: the same pass writes the quantised copy of the new weights for the next forward
      from .ops.quant import expert_adamw_quant_
      cache, idx = qc
      q, sf, fp4 = cache.target(idx)
      expert_adamw_quant_(p.data, g, st["exp_avg"], st["exp_avg_sq"], q, sf, fp4, lr=self.lr, beta1=self.betas[0],
                          beta2=self.betas[1], eps=self.eps, weight_decay=self.wd, step=self.step_count + 1)
      torch.autograd.graph.increment_version(p)
      cache.mark_fresh(idx, p._version)
      return
    ops.adamw_flat_(p.data.view(-1), g.reshape(-1).to(p.dtype), st["exp_avg"].view(-1), st["exp_avg_sq"].view(-1),
                    lr=self.lr, beta1=self.betas[0], beta2=self.betas[1], eps=self.eps, weight_decay=self.wd,
                    step=self.step_count + 1)
    torch.autograd.graph.increment_version(p)      # the kernel wrote through a raw pointer: let caches notice

  def _make_hook(self, i: int):
    def hook(p: torch.Tensor) -> None:
      if p.grad is None:
        return
      g = p.grad
      with torch.no_grad():
        if self.side is None:
          self._apply(i, p, g)
        else:
          # everything that reads this layer's weights in backward (the dgrad GEMMs inside the MoE function) is already
          # queued on the current stream; the update waits for that point and for the gradient itself
          cur = torch.cuda.current_stream(p.device)
          self._events[i].record(cur)
          with torch.cuda.stream(self.side):
            self.side.wait_event(self._events[i])
            self._apply(i, p, g)
          g.record_stream(self.side)               # the allocator must not hand the gradient's memory out early
      p.grad = None
    return hook

  def begin_step(self, lr: float, gradnorm_sq: Optional[torch.Tensor] = None) -> None:
    """Called before backward so that in-backward updates see this step's learning rate."""
    self.lr = lr
    self.gradnorm_sq = gradnorm_sq

  @torch.no_grad()
  def step(self) -> None:
    if not self.fuse_in_backward:
      for i, p in enumerate(self.params):
        if p.grad is not None:
          self._apply(i, p, p.grad)
          p.grad = None
    if self.side is not None:
      torch.cuda.current_stream(self.params[0].device).wait_stream(self.side)   # the next forward reads the new weights
    self.step_count += 1

  def state_dict(self) -> dict:
    return {"step": self.step_count,
            "state": {i: {k: v for k, v in s.items()} for i, s in self.state.items()}}

  def load_state_dict(self, sd: dict) -> None:
    self.step_count = int(sd["step"])
    for i, s in sd["state"].items():
      for k, v in s.items():
        self.state[int(i)][k].copy_(v)


class _MuonExperts:
  """Adapter giving ``ops.muon.Muon`` the interface the train loop expects from the expert optimizer."""

  def __init__(self, params: List[torch.nn.Parameter], cfg: Config):
    from .ops.muon import Muon
    self.inner = Muon(params, lr=float(cfg.lr_expert), momentum=cfg.muon_momentum, weight_decay=cfg.weight_decay)
    self.params = params
    self.gradnorm_sq: Optional[torch.Tensor] = None

  def begin_step(self, lr: float, gradnorm_sq: Optional[torch.Tensor] = None) -> None:
    self.inner.lr = lr
    self.gradnorm_sq = gradnorm_sq

  def step(self) -> None:
    if self.gradnorm_sq is not None:
      for p in self.params:
        if p.grad is not None:
          ops.sumsq(p.grad.reshape(-1), self.gradnorm_sq)
    self.inner.step()

  @property
  def step_count(self) -> int:
    return self.inner.step_count

  def state_dict(self) -> dict:
    return self.inner.state_dict()

  def load_state_dict(self, sd: dict) -> None:
    self.inner.load_state_dict(sd)


def build_param_groups(model: torch.nn.Module, cfg: Config):
  """Returns (expert_params, dense_groups) with the reference's name-based rules."""
  expert_params, _ = model.param_sets()
  expert_ids = {id(p) for p in expert_params}
  router, decay, no_decay = [], [], []
  for name, p in model.named_parameters():
    if not p.requires_grad or id(p) in expert_ids:
      continue
    if "router" in name:
      router.append(p)
    elif name.endswith("_b") or name.endswith(".bias") or "norm" in name or name.startswith("embedding") \
        or name.startswith("lm_head") or name.endswith("sinks"):
      no_decay.append(p)
    else:
      decay.append(p)
  groups = []
  if decay:
    groups.append({"name": "dense_decay", "params": decay, "lr": cfg.lr_dense, "weight_decay": cfg.weight_decay})
  if no_decay:
    groups.append({"name": "dense_no_decay", "params": no_decay, "lr": cfg.lr_dense, "weight_decay": 0.0})
  if router:
    groups.append({"name": "router", "params": router, "lr": cfg.lr_router, "weight_decay": 0.0})
  return expert_params, groups


class Optimizer:
  """Everything the train loop needs: LR update, in-backward expert updates, ZeRO-2 dense step,
  router-bias update."""

  def __init__(self, model: torch.nn.Module, cfg: Config, *, fuse_expert_in_backward: bool = False,
               group: Optional[dist.ProcessGroup] = None):
    self.model, self.cfg = model, cfg
    expert_params, groups = build_param_groups(model, cfg)
    self.expert = None
    if expert_params and cfg.expert_optimizer == "muon":
      self.expert = _MuonExperts(expert_params, cfg)
    elif expert_params:
      self.expert = ExpertAdamW(expert_params, cfg, fuse_expert_in_backward)
    self.dense = zero2.Zero2(groups, cfg, group=group)
    self.lrs = scheduled_lrs(0, 0, cfg)

  def begin_step(self, step: int, tokens_seen: int, gradnorm_sq: Optional[torch.Tensor] = None) -> float:
    self.lrs = scheduled_lrs(step, tokens_seen, self.cfg)
    if self.expert is not None:
      self.expert.begin_step(self.lrs["expert"], gradnorm_sq)
    self.dense.set_lrs(self.lrs)
    self.dense.zero_grad()
    return self.lrs["dense"]

  @torch.no_grad()
  def step(self) -> None:
    self.dense.step()
    if self.expert is not None:
      self.expert.step()
    loads = self.model.expert_loads() if hasattr(self.model, "expert_loads") else None
    if loads is not None:
      for m, l in zip(self.model.moe_layers(), loads):
        if m.router.kind == "sigmoid":
          m.router.update_bias(l, self.cfg.router_bias_update_rate)
