"""Evaluation: multiple-choice log-likelihood scoring, lockstep generation, sandboxed code checks."""
