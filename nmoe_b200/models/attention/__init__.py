"""Attention registry (name in the config -> module class), as in nmoe/model.py:17-31."""
from importlib import import_module

ATTN = {
  "mla": "nmoe_b200.models.attention.mla.MLA",
  "swa": "nmoe_b200.models.attention.swa.SWA",
  "nsa": "nmoe_b200.models.attention.nsa.NSA",
  "dsa": "nmoe_b200.models.attention.dsa.DSA",
  "kda": "nmoe_b200.models.attention.kda.KDA",
}


def get_attention(name: str):
  if name not in ATTN:
    raise ValueError(f"unknown attention '{name}'; expected one of {sorted(ATTN)}")
  mod, cls = ATTN[name].rsplit(".", 1)
  return getattr(import_module(mod), cls)
