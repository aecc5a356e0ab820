"""The synchronisation protocols of the kernels, checked over every interleaving on small instances; each model is also run
in a deliberately broken variant to show that the checker finds the bug it guards against."""
from maxtext_b200.utils import protocol_model as pm


def test_shared_memory_ring_has_no_race_and_no_deadlock():
  for stages, items in ((1, 3), (2, 5), (3, 7), (4, 9)):
    n, err = pm.explore(*pm.ring_model(stages, items))
    assert err is None and n > items, (stages, items, err)


def test_ring_with_the_wrong_initial_parity_deadlocks():
  # a producer that waits `empty` with the un-inverted parity never gets through its first pass
  n, err = pm.explore(*pm.ring_model(2, 4, producer_parity_inverted=False))
  assert err is not None and "deadlock" in err


def test_epoch_flag_barrier_orders_buffer_writes_and_reads():
  for ranks, rounds in ((2, 3), (3, 2)):
    n, err = pm.explore(*pm.epoch_flag_model(ranks, rounds))
    assert err is None, err


def test_reusing_a_buffer_after_a_single_barrier_is_caught():
  n, err = pm.explore(*pm.epoch_flag_model(2, 2, wait_before_overwrite=False))
  assert err is not None and "did not hold" in err
