"""Structured error codes of the data pipeline (pattern E-{CATEGORY}-{SPECIFIC}); every error
carries the action that fixes it (nmoe/data/errors.py:14-133)."""
from __future__ import annotations

import sys
from enum import Enum
from typing import NoReturn, Optional


class ErrorCode(str, Enum):
  MANIFEST_COMMIT = "E-MANIFEST-COMMIT"
  INDEX_MISSING = "E-INDEX-MISSING"
  SHARD_CHECKSUM = "E-SHARD-CHECKSUM"
  SOURCE_NOTFOUND = "E-SOURCE-NOTFOUND"
  TOKENIZER_DRIFT = "E-TOKENIZER-DRIFT"
  RESUME_CURSOR_MISMATCH = "E-RESUME-CURSOR-MISMATCH"

  def __str__(self) -> str:
    return self.value


ACTIONS = {
  ErrorCode.MANIFEST_COMMIT: "atomic rename/write failed; check disk space and permissions",
  ErrorCode.INDEX_MISSING: "the shard has no .idx; run `regenerate-index` or redo the stage",
  ErrorCode.SHARD_CHECKSUM: "checksum differs from the manifest; the shard is corrupt, redo the stage",
  ErrorCode.SOURCE_NOTFOUND: "no input files or invalid split; check the source path/config",
  ErrorCode.TOKENIZER_DRIFT: "tokenizer-derived values differ from the manifest; use one tokenizer throughout",
  ErrorCode.RESUME_CURSOR_MISMATCH: "state file is stale or data changed; delete the state file to restart the stage",
}


class PipelineError(Exception):
  code: ErrorCode = ErrorCode.MANIFEST_COMMIT

  def __init__(self, message: str, details: Optional[str] = None, code: Optional[ErrorCode] = None):
    self.code = code or type(self).code
    self.message, self.details = message, details
    super().__init__(f"[{self.code}]: {message}")

  def exit(self) -> NoReturn:
    print(f"ERROR [{self.code}]: {self.message}", file=sys.stderr)
    if self.details:
      print(f"  Details: {self.details}", file=sys.stderr)
    print(f"  Action: {ACTIONS.get(self.code, '?')}", file=sys.stderr)
    sys.exit(1)


class ManifestCommitError(PipelineError):
  code = ErrorCode.MANIFEST_COMMIT


class IndexMissingError(PipelineError):
  code = ErrorCode.INDEX_MISSING


class ShardChecksumError(PipelineError):
  code = ErrorCode.SHARD_CHECKSUM


class SourceNotFoundError(PipelineError):
  code = ErrorCode.SOURCE_NOTFOUND


class TokenizerDriftError(PipelineError):
  code = ErrorCode.TOKENIZER_DRIFT


class ResumeCursorMismatchError(PipelineError):
  code = ErrorCode.RESUME_CURSOR_MISMATCH
