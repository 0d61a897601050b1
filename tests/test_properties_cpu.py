"""Property tests (hypothesis) for the host-side data structures whose contracts are easy to state and easy to break."""
import random

import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from nmoe_b200.data import docid as D
from nmoe_b200.data import stack_v2 as S
from nmoe_b200.data.hydra_labels import GradedPairs, Labelled, length_bucket
from nmoe_b200.data.index import IndexReader, IndexWriter
from nmoe_b200.viz.server import lttb

FAST = settings(max_examples=60, deadline=None)

_seg = st.text(alphabet=st.characters(whitelist_categories=("Ll", "Lu", "Nd"), whitelist_characters="_-."), min_size=1, max_size=12)


@FAST
@given(source=_seg, parts=st.lists(_seg, min_size=1, max_size=4), start=st.integers(0, 10 ** 12), length=st.integers(0, 10 ** 9))
def test_shard_reference_prints_and_parses_to_itself(source, parts, start, length):
  ref = D.SpanRef.make(source, "/".join(parts) + ".npy", start, start + length)
  again = D.SpanRef.parse(str(ref))
  assert again == ref and str(again) == str(ref) and len(again) == length and D.is_ref(str(ref))


@FAST
@given(lens=st.lists(st.integers(1, 500), min_size=0, max_size=40))
def test_index_file_round_trips_document_boundaries(tmp_path_factory, lens):
  p = tmp_path_factory.mktemp("idx") / "s.idx"
  w = IndexWriter(p)
  pos, want = 0, []
  for n in lens:
    w.add_document(pos, pos + n)
    want.append((pos, pos + n))
    pos += n
  assert w.finalize() == len(lens)
  r = IndexReader(p)
  assert r.num_docs == len(lens) and list(r.iter_documents()) == want
  assert all(r.get_document(i) == want[i] for i in range(len(lens)))


@FAST
@given(n=st.integers(0, 400), n_out=st.integers(3, 120), seed=st.integers(0, 10 ** 6))
def test_lttb_keeps_ends_order_and_only_real_points(n, n_out, seed):
  rnd = random.Random(seed)
  pts = [(i * rnd.randint(1, 3), rnd.uniform(-5, 5)) for i in range(n)]
  pts = sorted({s: v for s, v in pts}.items())
  out = lttb(pts, n_out)
  assert len(out) == min(len(pts), n_out) or len(pts) <= n_out
  assert set(out) <= set(pts) and [s for s, _ in out] == sorted(s for s, _ in out)
  if pts:
    assert out[0] == pts[0] and out[-1] == pts[-1]


def _rows(seed, n, repos):
  rnd = random.Random(seed)
  return [{"blob_id": f"b{i:05d}", "path": f"src/f{i}.py", "repo_name": f"r{rnd.randrange(repos)}", "language": "Python",
           "length_bytes": 1000, "star_events_count": rnd.randrange(50), "fork_events_count": rnd.randrange(10)} for i in range(n)]


@FAST
@given(seed=st.integers(0, 10 ** 6), n=st.integers(0, 300), repos=st.integers(1, 12), top_n=st.integers(1, 60), cap=st.integers(1, 8))
def test_stack_selection_equals_the_brute_force_answer_in_any_order(seed, n, repos, top_n, cap):
  rows = _rows(seed, n, repos)
  refs = [S.FileRef.from_row(r) for r in rows]
  by_repo = {}
  for f in sorted(refs, key=lambda f: (f.score, f.blob_id), reverse=True):
    if len(by_repo.setdefault(f.repo_name, [])) < cap:
      by_repo[f.repo_name].append(f)
  want = [f.blob_id for f in sorted((f for v in by_repo.values() for f in v), key=lambda f: (f.score, f.blob_id), reverse=True)[:top_n]]
  assert [f.blob_id for f in S.select_top(rows, top_n, max_files_per_repo=cap)] == want
  random.Random(seed + 1).shuffle(rows)
  assert [f.blob_id for f in S.select_top(rows, top_n, max_files_per_repo=cap)] == want


@FAST
@given(seed=st.integers(0, 10 ** 6), grades=st.lists(st.integers(0, 5), min_size=2, max_size=60), lens=st.integers(1, 5000))
def test_ranking_pairs_are_ordered_and_share_a_length_bucket(seed, grades, lens):
  docs = [Labelled(text=str(i), grade=g, n_tokens=(lens * (i + 1)) % 4000) for i, g in enumerate(grades)]
  ps = GradedPairs(docs, seed=seed, warm=1, draw_budget=256)
  feasible = any(a.grade != b.grade and length_bucket(a.n_tokens) == length_bucket(b.n_tokens) for a in docs for b in docs)
  try:
    pairs = ps.next_pairs(6)
  except RuntimeError:
    assert not feasible
    return
  assert feasible
  for hi, lo in pairs:
    assert hi.grade > lo.grade and length_bucket(hi.n_tokens) == length_bucket(lo.n_tokens)
  assert ps.relaxed <= ps.issued == 6


@FAST
@given(data=st.binary(min_size=0, max_size=300), enc=st.sampled_from(["", "utf-8", "latin-1", "utf-16", "ascii", "no-such-codec"]))
def test_blob_decoding_never_raises_and_text_stays_text(data, enc):
  out = S.decode_text(data, enc)
  assert out is None or isinstance(out, str)
  text = "def f(x):\n    return x + 1  # naïve\n" * 3
  assert S.decode_text(text.encode("utf-8"), enc if enc in ("", "utf-8") else "") == text


@FAST
@given(tokens=st.integers(0, 10 ** 9), seq=st.integers(1, 8192), weights=st.lists(st.floats(0.0, 100.0, allow_nan=False), min_size=1, max_size=12))
def test_sequence_quotas_sum_to_the_budget_and_follow_the_weights(tokens, seq, weights):
  from nmoe_b200.data.mixture import largest_remainder_quota
  q = largest_remainder_quota(tokens, seq, weights)
  total = tokens // seq
  assert len(q) == len(weights) and all(x >= 0 for x in q) and sum(q) == (total if sum(weights) > 0 or total == 0 else sum(q))
  wsum = sum(weights)
  if wsum > 0 and total > 0:
    assert sum(q) == total
    for x, w in zip(q, weights):
      assert abs(x - total * w / wsum) <= 1.0 + 1e-6 * total        # never more than one sequence off the exact share


@settings(max_examples=12, deadline=None)
@given(weights=st.lists(st.integers(1, 50), min_size=1, max_size=6), world=st.integers(1, 4), seed=st.integers(0, 1000))
def test_loader_split_over_ranks_is_the_global_stream(tmp_path_factory, weights, world, seed):
  """Whatever the weights and the number of ranks, the ranks' slices put side by side are the single-rank stream, and
  each source is drawn in proportion to its weight (smooth weighted round-robin: never more than one draw off)."""
  from nmoe_b200.data.loader import DeterministicLoader
  from nmoe_b200.data.mixture import MixturePlan, SourcePlan, StagePlan
  d = tmp_path_factory.mktemp("ld")
  rng = np.random.default_rng(seed)
  seq, steps, per_step = 8, 5, 4 * world
  srcs = []
  for i, w in enumerate(weights):
    p = d / f"s{i}.npy"
    np.save(p, (rng.integers(0, 1000, size=4000) + 1000 * i).astype(np.uint32))      # the thousands digit names the source
    srcs.append(SourcePlan(id=f"s{i}", weight_fp=w, quota_sequences=10 ** 6, target_tokens=10 ** 9, paths=[str(p)]))
  plan = MixturePlan("m", "0", "f", "test", 1.0, seq, [StagePlan("pretrain", 1.0, srcs)])
  mk = lambda r, n: DeterministicLoader(plan=plan, dp_world_size=n, dp_rank=r, seq_len=seq, tokens_per_update=per_step * seq, device="cpu")
  one = mk(0, 1)
  ranks = [mk(r, world) for r in range(world)]
  counts = [0] * len(weights)
  for _ in range(steps):
    whole = one.next_host()
    parts = torch.cat([ld.next_host() for ld in ranks])
    assert torch.equal(whole, parts)
    for row in whole:
      counts[int(row[0]) // 1000] += 1
  n = steps * per_step
  for c, w in zip(counts, weights):
    assert abs(c - n * w / sum(weights)) <= 1.0 + 1e-9
