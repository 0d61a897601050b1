"""Serving engine on CPU: block pool with prefix sharing, continuous batching == one-by-one generation."""
import pytest
import torch

from nmoe_b200.serve import BlockPool, Engine, Sequence, ServeConfig, Transformer


def tiny_cfg():
  return ServeConfig(num_hidden_layers=3, num_experts=4, experts_per_token=2, vocab_size=128, hidden_size=64,
                     intermediate_size=64, head_dim=16, num_attention_heads=4, num_key_value_heads=2, sliding_window=8,
                     initial_context_length=64, rope_scaling_factor=1.0, probe_layer=2, judge_layer=3)


def test_block_pool_prefix_sharing_and_release():
  pool = BlockPool(num_blocks=8, block_size=4)
  a = Sequence(list(range(10)))
  pool.allocate(a)
  assert len(a.block_table) == 3 and a.n_cached == 0 and pool.n_free == 5
  pool.mark_ready(a)
  b = Sequence(list(range(8)) + [99, 98, 97])            # shares the first two full blocks
  pool.allocate(b)
  assert b.block_table[:2] == a.block_table[:2] and b.n_cached == 8 and pool.n_free == 4
  c = Sequence(list(range(8)))                            # identical to the shared prefix: last block must be computed
  pool.allocate(c)
  assert c.n_cached == 4 and c.block_table[0] == a.block_table[0] and c.block_table[1] != a.block_table[1]
  pool.release(a); pool.release(b); pool.release(c)
  assert pool.n_free == 8 and all(r == 0 for r in pool.ref)
  d = Sequence(list(range(9)))                            # freed blocks keep their content until re-used
  pool.allocate(d)
  assert d.n_cached == 8
  # decode appends: new block at a boundary
  d.tokens += [1, 2, 3]
  assert pool.can_append(d)
  s1 = pool.append_slot(d)
  assert s1 == d.block_table[2] * 4 + 3
  d.tokens.append(4)
  s2 = pool.append_slot(d)
  assert len(d.block_table) == 4 and s2 == d.block_table[3] * 4


def test_pool_exhaustion_raises_and_can_allocate_guards():
  pool = BlockPool(num_blocks=2, block_size=4)
  a = Sequence(list(range(8)))
  pool.allocate(a)
  b = Sequence([5, 6, 7])
  assert not pool.can_allocate(b)
  with pytest.raises(RuntimeError):
    pool.allocate(b)


def test_engine_batched_equals_sequential_and_uses_prefix_cache():
  torch.manual_seed(0)
  cfg = tiny_cfg()
  model = Transformer(cfg, dtype=torch.float32)
  model.init_weights(std=0.2)
  shared = [3, 1, 4, 1, 5, 9, 2, 6, 5, 3, 5, 8]
  prompts = [shared + [7, 7], shared + [10, 11, 12, 13, 14], [20, 21, 22], shared[:8] + [30]]
  ref = []
  for p in prompts:
    e1 = Engine(model, max_seq_len=48, max_batch=1, block_size=4)
    ref.append(e1.generate([p], max_new_tokens=6)[0])
  eng = Engine(model, max_seq_len=48, max_batch=2, block_size=4)        # forces two admission waves
  out = eng.generate(prompts, max_new_tokens=6)
  assert out == ref
  assert eng.steps["cached_tokens"] > 0                                 # later prompts reused the shared prefix
  assert eng.pool.n_free == eng.num_blocks
  # early exit: hidden states after two layers, then resume from them
  h, mask = eng.hidden_states(prompts[:2], up_to_layer=2)
  assert h.shape[:2] == mask.shape and h.shape[-1] == cfg.hidden_size
  S = h.size(1)
  pos = torch.arange(S).expand(2, S)
  ids = torch.zeros(2, S, dtype=torch.long)
  for i, p in enumerate(prompts[:2]):
    ids[i, :len(p)] = torch.tensor(p)
  full = model(ids, pos)
  resumed = model(ids, pos, from_layer=2, hidden_in=h)
  assert torch.allclose(full, resumed, atol=1e-5)


def test_engine_preempts_when_cache_is_full():
  torch.manual_seed(1)
  cfg = tiny_cfg()
  model = Transformer(cfg, dtype=torch.float32)
  model.init_weights(std=0.2)
  eng = Engine(model, max_seq_len=32, max_batch=4, block_size=4, num_blocks=7)
  prompts = [[1, 2, 3, 4, 5], [6, 7, 8, 9, 10], [11, 12, 13, 14, 15]]
  out = eng.generate(prompts, max_new_tokens=10)
  assert all(len(o) == 10 for o in out)
  ref = [Engine(model, max_seq_len=32, max_batch=1, block_size=4).generate([p], max_new_tokens=10)[0] for p in prompts]
  assert out == ref
