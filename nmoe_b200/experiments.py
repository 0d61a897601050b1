"""Experiment tracking in SQLite (nmoe/experiments.py:39-236).

The database is shared with the dashboard and, on a cluster that has run the reference framework, with databases that
framework wrote, so the two tables keep its column names and types:

  experiments(id, name, project, description, created_at TEXT)
  runs(id, experiment_id, config_json, git_hash, git_dirty, started_at TEXT, ended_at TEXT, status, results_json)

with ``datetime('now')`` (UTC, ``YYYY-MM-DD HH:MM:SS``) timestamps and the two indices on ``runs``.  A database made by
an earlier version of this module (REAL timestamps, no ``name`` / ``project``) is upgraded in place when it is opened.
WAL mode with a busy timeout lets several runs on one filesystem share the file; on a filesystem without working file
locks tracking switches itself off with a message instead of taking the training job down.
"""
from __future__ import annotations

import dataclasses
import json
import os
import sqlite3
import subprocess
import time
from dataclasses import dataclass
from pathlib import Path
from typing import List, Optional

STATUSES = ("running", "completed", "failed", "killed")

_SCHEMA = """
CREATE TABLE IF NOT EXISTS experiments (
  id TEXT PRIMARY KEY, name TEXT NOT NULL, project TEXT NOT NULL, description TEXT,
  created_at TEXT NOT NULL DEFAULT (datetime('now')));
CREATE TABLE IF NOT EXISTS runs (
  id TEXT PRIMARY KEY, experiment_id TEXT NOT NULL, config_json TEXT NOT NULL, git_hash TEXT, git_dirty INTEGER DEFAULT 0,
  started_at TEXT NOT NULL DEFAULT (datetime('now')), ended_at TEXT, status TEXT NOT NULL DEFAULT 'running',
  results_json TEXT, FOREIGN KEY (experiment_id) REFERENCES experiments(id));
CREATE INDEX IF NOT EXISTS idx_runs_experiment ON runs(experiment_id);
CREATE INDEX IF NOT EXISTS idx_runs_status ON runs(status);
"""


@dataclass
class ExperimentInfo:
  id: str
  name: str
  project: str
  description: str
  created_at: str


@dataclass
class RunInfo:
  id: str
  experiment_id: str
  config_json: str
  git_hash: str
  git_dirty: bool
  started_at: str
  ended_at: Optional[str]
  status: str
  results_json: Optional[str] = None

  def __getitem__(self, key: str):      # rows used to be plain dicts
    return getattr(self, key)


def _git(*args: str) -> str:
  try:
    return subprocess.run(["git", *args], capture_output=True, text=True, timeout=5,
                          cwd=Path(__file__).resolve().parent).stdout.strip()
  except (OSError, subprocess.SubprocessError):
    return ""


def _upgrade(db: sqlite3.Connection) -> None:
  """Bring a database of the earlier layout (REAL timestamps, experiments without name / project) to the current one."""
  cols = {r[1]: (r[2] or "").upper() for r in db.execute("PRAGMA table_info(experiments)")}
  if cols and "name" not in cols:
    db.execute("ALTER TABLE experiments ADD COLUMN name TEXT NOT NULL DEFAULT ''")
    db.execute("ALTER TABLE experiments ADD COLUMN project TEXT NOT NULL DEFAULT 'default'")
    db.execute("UPDATE experiments SET name = id WHERE name = ''")
  if cols.get("created_at") == "REAL":
    # the column keeps its declared type; SQLite stores the text all the same
    db.execute("UPDATE experiments SET created_at = datetime(created_at, 'unixepoch') WHERE typeof(created_at) IN ('real', 'integer')")
  rcols = {r[1]: (r[2] or "").upper() for r in db.execute("PRAGMA table_info(runs)")}
  if rcols.get("started_at") == "REAL":
    for c in ("started_at", "ended_at"):
      db.execute(f"UPDATE runs SET {c} = datetime({c}, 'unixepoch') WHERE typeof({c}) IN ('real', 'integer')")


class ExperimentTracker:
  def __init__(self, cfg, db_path: Optional[str] = None):
    self.cfg = cfg
    path = Path(os.environ.get("NMOE_EXPERIMENTS_DB", db_path or getattr(cfg, "experiments_db", "/data/experiments.db")))
    self.path = path
    self.db: Optional[sqlite3.Connection] = None
    try:
      path.parent.mkdir(parents=True, exist_ok=True)
      self.db = sqlite3.connect(str(path), timeout=30.0)
      self.db.execute("PRAGMA busy_timeout=30000")
      try:
        self.db.execute("PRAGMA journal_mode=WAL")
      except sqlite3.OperationalError:
        self.db.execute("PRAGMA journal_mode=DELETE")   # network filesystems where WAL's shared memory cannot work
      _upgrade(self.db)
      self.db.executescript(_SCHEMA)
      self.db.commit()
    except (OSError, sqlite3.Error) as e:
      print(f"[experiments] tracking disabled ({e}); if the database lives on NFS, mount with working locks "
            f"or point NMOE_EXPERIMENTS_DB at local disk", flush=True)
      self.db = None

  # -- writes
  def create_experiment(self, name: str, project: str, description: str = "") -> str:
    """A new experiment ``{project}_{name}_{unix time}``; returns its id."""
    exp = f"{project}_{name}_{int(time.time())}"
    if self.db is not None:
      self.db.execute("INSERT INTO experiments(id, name, project, description, created_at) VALUES (?, ?, ?, ?, datetime('now'))",
                      (exp, name, project, description))
      self.db.commit()
    return exp

  def _ensure_experiment(self, exp: str) -> None:
    # configs name an experiment id without creating it first: give the runs table's foreign key a row to point at
    self.db.execute("INSERT OR IGNORE INTO experiments(id, name, project, description, created_at) VALUES (?, ?, ?, '', datetime('now'))",
                    (exp, exp, getattr(self.cfg, "project", None) or "default"))

  def start_run(self, run_id: Optional[str] = None) -> str:
    """Record a run of ``cfg.experiment_id`` as running.  A given ``run_id`` is used as is; starting the same id again
    (a job resumed from its checkpoint) re-opens the row rather than failing the job."""
    run_id = run_id or f"run_{int(time.time())}_{os.getpid()}"
    if self.db is None:
      return run_id
    exp = getattr(self.cfg, "experiment_id", "default")
    cfg = dataclasses.asdict(self.cfg) if dataclasses.is_dataclass(self.cfg) else dict(vars(self.cfg))
    cfg_json = json.dumps({k: v for k, v in cfg.items() if not k.startswith("_")}, sort_keys=True, default=str)
    self._ensure_experiment(exp)
    self.db.execute(
      # timestamps are written out rather than left to column defaults: an upgraded database has none
      "INSERT INTO runs(id, experiment_id, config_json, git_hash, git_dirty, status, started_at) VALUES (?, ?, ?, ?, ?, 'running', datetime('now')) "
      "ON CONFLICT(id) DO UPDATE SET config_json = excluded.config_json, git_hash = excluded.git_hash, "
      "git_dirty = excluded.git_dirty, status = 'running', ended_at = NULL",
      (run_id, exp, cfg_json, _git("rev-parse", "HEAD"), int(bool(_git("status", "--porcelain")))))
    self.db.commit()
    return run_id

  def update_results(self, run_id: str, results: dict) -> None:
    """Intermediate results of a run that is still going (an evaluation in mid-training)."""
    if self.db is None:
      return
    self.db.execute("UPDATE runs SET results_json = ? WHERE id = ?", (json.dumps(results, indent=2, default=str), run_id))
    self.db.commit()

  def end_run(self, run_id: str, status: str, results: Optional[dict] = None) -> None:
    if status not in STATUSES[1:]:
      raise ValueError(f"status must be one of {STATUSES[1:]}, not {status!r}")
    if self.db is None:
      return
    if results is not None:
      self.db.execute("UPDATE runs SET ended_at = datetime('now'), status = ?, results_json = ? WHERE id = ?",
                      (status, json.dumps(results, indent=2, default=str), run_id))
    else:
      self.db.execute("UPDATE runs SET ended_at = datetime('now'), status = ? WHERE id = ?", (status, run_id))
    self.db.commit()

  # -- reads
  _RUN_COLS = "id, experiment_id, config_json, git_hash, git_dirty, started_at, ended_at, status, results_json"

  @staticmethod
  def _run(r) -> RunInfo:
    return RunInfo(r[0], r[1], r[2], r[3] or "", bool(r[4]), r[5], r[6], r[7], r[8])

  def get_experiment(self, experiment_id: str) -> Optional[ExperimentInfo]:
    if self.db is None:
      return None
    r = self.db.execute("SELECT id, name, project, description, created_at FROM experiments WHERE id = ?", (experiment_id,)).fetchone()
    return ExperimentInfo(r[0], r[1], r[2], r[3] or "", r[4]) if r else None

  def list_experiments(self, project: Optional[str] = None) -> List[ExperimentInfo]:
    if self.db is None:
      return []
    sql, args = "SELECT id, name, project, description, created_at FROM experiments", ()
    if project:
      sql, args = sql + " WHERE project = ?", (project,)
    return [ExperimentInfo(r[0], r[1], r[2], r[3] or "", r[4]) for r in self.db.execute(sql + " ORDER BY created_at DESC, id", args)]

  def get_run(self, run_id: str) -> Optional[RunInfo]:
    if self.db is None:
      return None
    r = self.db.execute(f"SELECT {self._RUN_COLS} FROM runs WHERE id = ?", (run_id,)).fetchone()
    return self._run(r) if r else None

  def list_runs(self, experiment_id: str, status: Optional[str] = None) -> List[RunInfo]:
    """Runs of an experiment, newest first, optionally only those with the given status."""
    if self.db is None:
      return []
    sql, args = f"SELECT {self._RUN_COLS} FROM runs WHERE experiment_id = ?", [experiment_id]
    if status:
      sql += " AND status = ?"
      args.append(status)
    return [self._run(r) for r in self.db.execute(sql + " ORDER BY started_at DESC, id", args)]

  def close(self) -> None:
    if self.db is not None:
      self.db.close()
      self.db = None
