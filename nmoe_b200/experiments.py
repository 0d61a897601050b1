"""Experiment tracking in SQLite (nmoe/experiments.py:39-236): tables ``experiments`` and
``runs(id, experiment_id, config_json, git_hash, git_dirty, started_at, ended_at, status, results_json)``,
WAL mode with a busy timeout so several runs on one filesystem can share the database."""
from __future__ import annotations

import dataclasses
import json
import os
import sqlite3
import subprocess
import time
from pathlib import Path
from typing import Optional


def _git(*args: str) -> str:
  try:
    return subprocess.run(["git", *args], capture_output=True, text=True, timeout=5,
                          cwd=Path(__file__).resolve().parent).stdout.strip()
  except (OSError, subprocess.SubprocessError):
    return ""


class ExperimentTracker:
  def __init__(self, cfg, db_path: Optional[str] = None):
    self.cfg = cfg
    path = Path(os.environ.get("NMOE_EXPERIMENTS_DB", db_path or cfg.experiments_db))
    self.db: Optional[sqlite3.Connection] = None
    try:
      path.parent.mkdir(parents=True, exist_ok=True)
      self.db = sqlite3.connect(str(path), timeout=30.0)
      self.db.execute("PRAGMA busy_timeout=30000")
      try:
        self.db.execute("PRAGMA journal_mode=WAL")
      except sqlite3.OperationalError:
        pass   # network filesystems without working locks: keep the default journal
      self.db.executescript(
        "CREATE TABLE IF NOT EXISTS experiments (id TEXT PRIMARY KEY, created_at REAL, description TEXT);"
        "CREATE TABLE IF NOT EXISTS runs (id TEXT PRIMARY KEY, experiment_id TEXT, config_json TEXT, git_hash TEXT,"
        " git_dirty INTEGER, started_at REAL, ended_at REAL, status TEXT, results_json TEXT,"
        " FOREIGN KEY (experiment_id) REFERENCES experiments(id));")
      self.db.commit()
    except (OSError, sqlite3.Error) as e:
      print(f"[experiments] tracking disabled ({e}); if the database lives on NFS, mount with working locks "
            f"or point NMOE_EXPERIMENTS_DB at local disk", flush=True)
      self.db = None

  def start_run(self, run_id: Optional[str] = None) -> str:
    run_id = run_id or f"run_{int(time.time())}_{os.getpid()}"
    if self.db is None:
      return run_id
    exp = self.cfg.experiment_id
    cfg_json = json.dumps({k: v for k, v in dataclasses.asdict(self.cfg).items() if not k.startswith("_")},
                          sort_keys=True, default=str)
    self.db.execute("INSERT OR IGNORE INTO experiments VALUES (?, ?, ?)", (exp, time.time(), ""))
    self.db.execute("INSERT OR REPLACE INTO runs VALUES (?, ?, ?, ?, ?, ?, NULL, 'running', NULL)",
                    (run_id, exp, cfg_json, _git("rev-parse", "HEAD"), int(bool(_git("status", "--porcelain"))),
                     time.time()))
    self.db.commit()
    return run_id

  def end_run(self, run_id: str, status: str, results: Optional[dict] = None) -> None:
    if self.db is None:
      return
    self.db.execute("UPDATE runs SET ended_at = ?, status = ?, results_json = ? WHERE id = ?",
                    (time.time(), status, json.dumps(results) if results is not None else None, run_id))
    self.db.commit()

  def get_run(self, run_id: str) -> Optional[dict]:
    if self.db is None:
      return None
    cur = self.db.execute("SELECT id, experiment_id, git_hash, git_dirty, started_at, ended_at, status, results_json "
                          "FROM runs WHERE id = ?", (run_id,))
    r = cur.fetchone()
    if r is None:
      return None
    keys = ("id", "experiment_id", "git_hash", "git_dirty", "started_at", "ended_at", "status", "results_json")
    return dict(zip(keys, r))

  def close(self) -> None:
    if self.db is not None:
      self.db.close()
      self.db = None
