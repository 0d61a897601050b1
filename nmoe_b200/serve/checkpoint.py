"""Weights of the grading model on disk.

Two directory layouts are read:

  native      ``config.json`` (the ``ServeConfig`` fields) + ``model.pt`` (``state_dict`` of
              ``serve.Transformer``); written by ``save_model``.
  gpt-oss     the published layout: ``config.json`` + ``*.safetensors`` with ``block.N.attn.*`` /
              ``block.N.mlp.*`` tensors, expert matrices as MXFP4 (``*.blocks`` uint8 nibbles, 32 values
              per 16 bytes, low nibble first; ``*.scales`` E8M0 bytes).  Needs ``safetensors``.

MXFP4 expert matrices are expanded to bf16 here; the model re-packs them to E4M3 + the same
E8M0 scales on first use, which is exact.  Reference counterpart: ``Checkpoint`` and
``Transformer.from_checkpoint`` (nmoe/data/model.py:357-383, 563-634).
"""
from __future__ import annotations

import json
from dataclasses import asdict, fields
from pathlib import Path
from typing import Dict

import torch

from .model import ServeConfig, Transformer

FP4_VALUES = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0)


def dequant_mxfp4(blocks: torch.Tensor, scales: torch.Tensor, dtype=torch.bfloat16) -> torch.Tensor:
  """blocks [..., G, 16] uint8 (two E2M1 codes per byte, low nibble = even element), scales [..., G]
  uint8 (E8M0, bias 127) -> [..., G*32]."""
  lut = torch.tensor(FP4_VALUES, dtype=torch.float32, device=blocks.device)
  lo, hi = (blocks & 0x0F).long(), (blocks >> 4).long()
  vals = torch.stack((lut[lo], lut[hi]), dim=-1).flatten(-2)                    # [..., G, 32]
  out = vals * torch.exp2(scales.float() - 127.0).unsqueeze(-1)
  return out.flatten(-2).to(dtype)


def save_model(model: Transformer, directory: str) -> None:
  d = Path(directory)
  d.mkdir(parents=True, exist_ok=True)
  (d / "config.json").write_text(json.dumps(asdict(model.cfg), indent=1))
  torch.save({k: v.detach().cpu() for k, v in model.state_dict().items()}, d / "model.pt")


def _config(d: Path) -> ServeConfig:
  j = json.loads((d / "config.json").read_text())
  known = {f.name for f in fields(ServeConfig)}
  alias = {"num_local_experts": "num_experts", "num_experts_per_tok": "experts_per_token", "rms_norm_eps": "rms_eps"}
  kw = {}
  for k, v in j.items():
    k = alias.get(k, k)
    if k in known:
      kw[k] = v
  rs = j.get("rope_scaling") or {}
  if "factor" in rs:
    kw.setdefault("rope_scaling_factor", rs["factor"])
    kw.setdefault("rope_ntk_alpha", rs.get("beta_slow", 1.0))
    kw.setdefault("rope_ntk_beta", rs.get("beta_fast", 32.0))
    kw.setdefault("initial_context_length", rs.get("original_max_position_embeddings", 4096))
  cfg = ServeConfig(**kw)
  cfg.probe_layer = min(cfg.probe_layer, cfg.num_hidden_layers)
  cfg.judge_layer = min(cfg.judge_layer, cfg.num_hidden_layers)
  return cfg


def _from_gpt_oss(d: Path, cfg: ServeConfig, device) -> Dict[str, torch.Tensor]:
  from safetensors import safe_open  # type: ignore
  raw: Dict[str, torch.Tensor] = {}
  for f in sorted(d.glob("*.safetensors")):
    with safe_open(str(f), framework="pt", device=str(device)) as sf:
      for k in sf.keys():
        raw[k] = sf.get_tensor(k)
  sd: Dict[str, torch.Tensor] = {"embed": raw["embedding.weight"], "norm": raw["norm.scale"], "unembed": raw["unembedding.weight"]}
  for i in range(cfg.num_hidden_layers):
    a, m = f"block.{i}.attn.", f"block.{i}.mlp."
    sd[f"attn.{i}.norm"] = raw[a + "norm.scale"]
    sd[f"attn.{i}.qkv_w"], sd[f"attn.{i}.qkv_b"] = raw[a + "qkv.weight"], raw[a + "qkv.bias"]
    sd[f"attn.{i}.out_w"], sd[f"attn.{i}.out_b"] = raw[a + "out.weight"], raw[a + "out.bias"]
    sd[f"attn.{i}.sinks"] = raw[a + "sinks"]
    sd[f"mlp.{i}.norm"] = raw[m + "norm.scale"]
    sd[f"mlp.{i}.gate_w"], sd[f"mlp.{i}.gate_b"] = raw[m + "gate.weight"], raw[m + "gate.bias"]
    # published expert matrices are [E, out, in/32, 16] blocks: out = 2I for mlp1 (gate/linear interleaved), H for mlp2
    sd[f"mlp.{i}.w1"] = dequant_mxfp4(raw[m + "mlp1_weight.blocks"], raw[m + "mlp1_weight.scales"])
    sd[f"mlp.{i}.b1"] = raw[m + "mlp1_bias"]
    sd[f"mlp.{i}.w2"] = dequant_mxfp4(raw[m + "mlp2_weight.blocks"], raw[m + "mlp2_weight.scales"])
    sd[f"mlp.{i}.b2"] = raw[m + "mlp2_bias"]
  return sd


def load_model(directory: str, device="cuda", dtype=torch.bfloat16, max_tokens: int = 8192) -> Transformer:
  d = Path(directory)
  cfg = _config(d)
  model = Transformer(cfg, dtype=dtype, device=device, max_tokens=max_tokens)
  if (d / "model.pt").exists():
    sd = torch.load(d / "model.pt", map_location="cpu", weights_only=True)
  elif any(d.glob("*.safetensors")):
    sd = _from_gpt_oss(d, cfg, "cpu")
  else:
    raise FileNotFoundError(f"{d} has neither model.pt nor *.safetensors")
  missing, unexpected = model.load_state_dict({k: v.to(dtype) for k, v in sd.items()}, strict=False)
  missing = [k for k in missing if k != "inv_freq"]
  if missing or unexpected:
    raise KeyError(f"checkpoint mismatch: missing {missing[:5]} unexpected {list(unexpected)[:5]}")
  return model
