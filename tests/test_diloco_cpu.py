"""DiLoCo pieces that need one process: fragment assignment, streaming schedule, outer Nesterov step."""
import torch

from helpers import batch_of, make_engine, tiny_config
from maxtext_b200.trainers.diloco import DiLoCoTrainer, fragments_of, nesterov_outer_step, streaming_schedule

EXTRA = ["base_num_decoder_layers=4", "enable_diloco=true", "enable_streaming_diloco=true", "num_diloco_fragments=3", "diloco_sync_period=6"]


def test_fragments_strided_and_sequential():
  cfg = tiny_config(extra=EXTRA)
  eng = make_engine(cfg)
  fr = fragments_of(eng, cfg)
  names = [sorted({u.name.split("#")[0] for u in f}) for f in fr]
  assert names == [["embed", "head"], ["layer_0", "layer_2"], ["layer_1", "layer_3"]]
  cfg2 = tiny_config(extra=EXTRA + ["use_sequential_layers=true"])
  names2 = [sorted({u.name.split("#")[0] for u in f}) for f in fragments_of(make_engine(cfg2), cfg2)]
  assert names2[1:] == [["layer_0", "layer_1"], ["layer_2", "layer_3"]]
  assert streaming_schedule(cfg) == (2, 6)


def test_outer_step_is_optax_nesterov():
  p, tr, g = torch.tensor([1.0, 2.0]), torch.tensor([0.5, -0.5]), torch.tensor([0.1, 0.2])
  nesterov_outer_step(p, tr, g, lr=0.3, momentum=0.9)
  want_tr = torch.tensor([0.1 + 0.45, 0.2 - 0.45])
  assert torch.allclose(tr, want_tr)
  assert torch.allclose(p, torch.tensor([1.0, 2.0]) - 0.3 * (g + 0.9 * want_tr))


def test_streaming_syncs_one_fragment_at_a_time_with_delay_and_alpha():
  cfg = tiny_config(extra=EXTRA + ["num_communication_overlapping_steps=1", "communication_overlapping_alpha=0.5", "diloco_outer_lr=1.0",
                                   "diloco_outer_momentum=0.0"])
  eng = make_engine(cfg)
  tr = DiLoCoTrainer(eng, cfg, None)
  start = eng.store.master.clone()
  b = batch_of(cfg)
  ranges = [tr._ranges(f) for f in tr.frags]
  tr.train_step(b)                      # step 1: nothing
  assert torch.equal(tr.outer, start)
  before = eng.store.master.clone()
  tr.train_step(b)                      # step 2: fragment 1 measured (outer - inner), applied one step later
  assert 1 in tr._inflight and torch.equal(tr.outer, start)
  tr.train_step(b)                      # step 3 = 2 + delay: with lr 1, momentum 0 and one replica outer becomes inner@step2
  assert not tr._inflight
  for lo, hi in ranges[1]:
    assert not torch.equal(tr.outer[lo:hi], start[lo:hi])
  for lo, hi in ranges[0] + ranges[2]:
    assert torch.equal(tr.outer[lo:hi], start[lo:hi])
  del before
