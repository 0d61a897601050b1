"""The threaded host model of the RDEP count / data / return epoch protocol (nmoe_b200/parallel/protocol_model.py):
correct delivery under scheduling jitter over consecutive calls, and bounded waits that report a missing peer."""
from nmoe_b200.parallel import protocol_model as PM


def _expected(eids, world, n_experts, c, r):
  n_local = n_experts // world
  return [2.0 * (1000.0 * c + 10.0 * r + 0.001 * i) + (e // n_local) for i, e in enumerate(eids[c][r])]


def test_rows_reach_their_owner_and_return_over_consecutive_calls():
  world, E, calls, pairs = 4, 8, 6, 40
  results, statuses, violations, eids = PM.run_ranks(world, E, calls, pairs, seed=3)
  assert violations == []
  assert all(s.code == 0 for s in statuses)
  for r in range(world):
    assert len(results[r]) == calls
    for c in range(calls):
      assert results[r][c] == _expected(eids, world, E, c, r), (r, c)


def test_skewed_routing_keeps_positions_unique():
  # every pair of every rank goes to expert 0: the owner's segment is filled by rank order without collisions
  world, E = 4, 4
  fabric = PM.Fabric(world, E, align=4, seed=1)
  actors = [PM.RankActor(fabric, r) for r in range(world)]
  import threading
  out = [None] * world
  def body(r):
    out[r] = actors[r].moe_call([0] * 13, payload=lambda i, r=r: r * 100 + i, fn=lambda owner, v: v)
  ts = [threading.Thread(target=body, args=(r,)) for r in range(world)]
  [t.start() for t in ts]; [t.join(20) for t in ts]
  assert [m.violations for m in fabric.mem] == [[]] * world
  for r in range(world):
    assert out[r] == [r * 100 + i for i in range(13)]
  assert sorted(fabric.mem[0].xbuf) == list(range(52))        # 4 ranks x 13 rows, contiguous, rank-major


def test_a_peer_that_never_arrives_runs_out_every_wait_with_a_status():
  world, E = 4, 8
  results, statuses, violations, _ = PM.run_ranks(world, E, 2, 16, absent=(2,), wait_budget_s=0.3)
  assert violations == []                                      # nobody hung, nobody wrote where it should not
  for r in (0, 1, 3):
    assert results[r] == [None]                                # the first call gave up and the rank stopped
    s = statuses[r]
    assert (s.code, s.where, s.a, s.b) == (PM.WAIT_TIMEOUT, PM.WHERE_COUNT, 2, 1)


def test_a_peer_that_stops_after_the_count_exchange_is_caught_by_the_data_wait():
  world, E = 3, 6
  results, statuses, violations, _ = PM.run_ranks(world, E, 1, 10, die_after_counts=(1,), wait_budget_s=0.3)
  assert violations == []
  for r in (0, 2):
    assert results[r] == [None]
    assert (statuses[r].code, statuses[r].where, statuses[r].a) == (PM.WAIT_TIMEOUT, PM.WHERE_DATA, 1)


def test_a_flag_left_from_an_earlier_epoch_does_not_satisfy_a_later_wait():
  s = PM.Status()
  flags = [3, 3, 2]                                            # rank 2 is still one epoch behind
  assert not PM.bounded_wait(flags, 3, 0.05, s, PM.WHERE_RET)
  assert (s.code, s.where, s.a, s.b) == (PM.WAIT_TIMEOUT, PM.WHERE_RET, 2, 3)
  flags[2] = 3
  assert PM.bounded_wait(flags, 3, 0.05, PM.Status(), PM.WHERE_RET)
