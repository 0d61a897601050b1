"""Data platform: deterministic shard loader (training path), shard building, CLI."""
